// Mamba-1 selective-scan backward for 16 < d_state <= 256.
//
// Same recomputation scheme as the d_state <= 16 kernels (the state entering each
// block of S steps comes from the forward's saves, the block is rebuilt forward and
// walked backward), with the forward kernel's lane layout for large states: LPC lanes
// own one channel, 8 states each, a warp owns 32 / LPC channels and is its own CTA.
// The states of the block sit in shared memory between the two sweeps.  This is the
// coverage path for state sizes no shipped Mamba-1 model uses (the reference's
// parallel backward goes to 256 as well, kernels/mamba_ssm_parallel.cu:49-50); it is
// written for clarity, with plain loads, and is not tuned.
#include <string.h>

#include "m1_bwd2_kernel.cuh"

namespace mb200 {

template <typename Tact, int LPC>
__global__ void __launch_bounds__(32) sscan_bwd_wide_kernel(const BwdParams p, int softplus) {
    constexpr int CHW = 32 / LPC, NP = 8 * LPC;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int S = p.S;
    float* hs = reinterpret_cast<float*>(smem_raw);   // [S][8][32] state after each step
    float* Bf = hs + S * 8 * 32;                      // [S][NP]
    float* Cf = Bf + S * NP;                          // [S][NP]
    float* dls = Cf + S * NP;                         // [S][CHW] delta (after softplus)
    float* us = dls + S * CHW;                        // [S][CHW] u
    float* gys = us + S * CHW;                        // [S][CHW] dy * gate
    float* raws = gys + S * CHW;                      // [S][CHW][3] raw delta, z, dy
    const int lane = threadIdx.x, colw = lane / LPC, part = lane % LPC;
    const int b = blockIdx.y, tile = blockIdx.x, d0 = tile * CHW, d = d0 + colw;
    const int T = p.T, D = p.D, N = p.N, n0 = part * 8;
    const bool d_ok = d < D;
    const int nblk = (T + S - 1) / S;
    const bool gate = p.z_mode != 0, gate_is_silu = p.z_mode == 1;
    const Tact *gu = static_cast<const Tact*>(p.u), *gdl = static_cast<const Tact*>(p.dl),
               *gz = static_cast<const Tact*>(p.z), *gdy = static_cast<const Tact*>(p.dy),
               *gb = static_cast<const Tact*>(p.bm), *gc = static_cast<const Tact*>(p.cm);
    Tact *o_du = static_cast<Tact*>(p.du), *o_ddl = static_cast<Tact*>(p.ddl), *o_dz = static_cast<Tact*>(p.dz);

    float a2[8], an[8], dh[8], accA[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        an[j] = (d_ok && n0 + j < N) ? p.a_neg[static_cast<long long>(d) * N + n0 + j] : 0.0f;
        a2[j] = an[j] * kLog2e;
        dh[j] = accA[j] = 0.0f;
    }
    const float Dd = d_ok ? p.Dp[d] : 0.0f;
    float accD = 0.0f;

    for (int it = 0; it < nblk; ++it) {
        const int k = nblk - 1 - it, t0 = k * S, nv = min(S, T - t0);
        __syncwarp();
        // ---- tiles of the block ----
        for (int i = lane; i < S * CHW; i += 32) {
            const int r = i / CHW, cc = i - r * CHW, t = t0 + r, dd = d0 + cc;
            float vdl = 0.0f, vu = 0.0f, vz = 0.0f, vdy = 0.0f;
            if (t < T && dd < D) {
                const long long row = static_cast<long long>(b) * T + t;
                vdl = to_f(gdl[row * p.ld_dl + dd]);
                vu = to_f(gu[row * p.ld_u + dd]);
                vdy = to_f(gdy[row * p.ld_dy + dd]);
                if (gate) vz = to_f(gz[row * p.ld_z + dd]);
            }
            raws[i * 3] = vdl; raws[i * 3 + 1] = vz; raws[i * 3 + 2] = vdy;
            dls[i] = softplus ? softplusf_fast(vdl) : vdl;
            us[i] = vu;
            gys[i] = gate ? vdy * (gate_is_silu ? siluf_fast(vz) : vz) : vdy;
        }
        for (int i = lane; i < S * NP; i += 32) {
            const int r = i / NP, n = i - r * NP, t = t0 + r;
            const bool in = t < T && n < N;
            Bf[i] = in ? to_f(gb[(static_cast<long long>(b) * T + t) * p.ld_bc + n]) : 0.0f;
            Cf[i] = in ? to_f(gc[(static_cast<long long>(b) * T + t) * p.ld_bc + n]) : 0.0f;
        }
        __syncwarp();
        // ---- forward sweep from the saved state ----
        float h[8], h_in[8];
        const float* cs = p.chunk_states + b * p.cs_ld_b + k * p.cs_ld_k + static_cast<long long>(d_ok ? d : 0) * N;
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = h_in[j] = (d_ok && n0 + j < N) ? cs[n0 + j] : 0.0f;
        for (int r = 0; r < nv; ++r) {
            const float dlv = dls[r * CHW + colw], duv = dlv * us[r * CHW + colw];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                h[j] = fmaf(ex2(dlv * a2[j]), h[j], duv * Bf[r * NP + n0 + j]);
                hs[(r * 8 + j) * 32 + lane] = h[j];
            }
        }
        // ---- reverse sweep ----
        float* pbc = p.part_bc + ((static_cast<long long>(b) * gridDim.x + tile) * T + t0) * (2 * NP);
        for (int r = nv - 1; r >= 0; --r) {
            const float dlv = dls[r * CHW + colw], uv = us[r * CHW + colw], dyp = gys[r * CHW + colw];
            const float duv = dlv * uv;
            float sB = 0.0f, sA = 0.0f, ys = 0.0f, rB[8], rC[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float e = ex2(dlv * a2[j]);
                const float hc = hs[(r * 8 + j) * 32 + lane];
                const float hp = r > 0 ? hs[((r - 1) * 8 + j) * 32 + lane] : h_in[j];
                const float cn = Cf[r * NP + n0 + j], bn = Bf[r * NP + n0 + j];
                dh[j] = fmaf(dyp, cn, dh[j]);
                sB = fmaf(dh[j], bn, sB);
                const float dhda = dh[j] * e;
                const float w = dhda * hp;
                sA = fmaf(a2[j], w, sA);
                accA[j] = fmaf(dlv, w, accA[j]);
                rB[j] = dh[j] * duv;
                rC[j] = dyp * hc;
                ys = fmaf(hc, cn, ys);
                dh[j] = dhda;
            }
            // sums over the channel's LPC lanes
#pragma unroll
            for (int m = 1; m < LPC; m <<= 1) {
                sB += __shfl_xor_sync(0xffffffffu, sB, m);
                sA += __shfl_xor_sync(0xffffffffu, sA, m);
                ys += __shfl_xor_sync(0xffffffffu, ys, m);
            }
            if (part == 0 && d_ok) {
                const long long grow = static_cast<long long>(b) * T + t0 + r;
                const float raw_dl = raws[(r * CHW + colw) * 3], zv = raws[(r * CHW + colw) * 3 + 1],
                            dyv = raws[(r * CHW + colw) * 3 + 2];
                o_du[grow * p.ld_du + d] = from_f<Tact>(fmaf(dyp, Dd, dlv * sB));
                accD = fmaf(dyp, uv, accD);
                if (gate) {
                    const float sg = sigmoidf_fast(zv);
                    const float dsilu = sg * fmaf(zv, 1.0f - sg, 1.0f);
                    o_dz[grow * p.ld_dz + d] = from_f<Tact>(dyv * fmaf(Dd, uv, ys) * (gate_is_silu ? dsilu : 1.0f));
                }
                float ddl = fmaf(sA, kLn2, uv * sB);
                if (softplus) ddl *= raw_dl > 20.0f ? 1.0f : sigmoidf_fast(raw_dl);
                o_ddl[grow * p.ld_ddl + d] = from_f<Tact>(ddl);
            }
            // dB_t / dC_t: sums over the warp's channels, in a fixed order
#pragma unroll
            for (int m = LPC; m < 32; m <<= 1) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    rB[j] += __shfl_xor_sync(0xffffffffu, rB[j], m);
                    rC[j] += __shfl_xor_sync(0xffffffffu, rC[j], m);
                }
            }
            if (colw == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    pbc[r * 2 * NP + n0 + j] = rB[j];
                    pbc[r * 2 * NP + NP + n0 + j] = rC[j];
                }
            }
        }
    }
    // per-sample parameter-gradient partials
    if (d_ok) {
        if (part == 0) p.part_d[static_cast<long long>(b) * D + d] = accD;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (n0 + j < N) p.part_a[(static_cast<long long>(b) * D + d) * N + n0 + j] = accA[j] * an[j];
    }
}

int bwd_wide_lpc(int N) {
    int lpc = 4;
    while (lpc * 8 < N) lpc *= 2;
    return lpc;
}

size_t bwd_wide_smem(int N, int S) {
    const int lpc = bwd_wide_lpc(N), chw = 32 / lpc, np = 8 * lpc;
    return sizeof(float) * (static_cast<size_t>(S) * 8 * 32 + 2 * static_cast<size_t>(S) * np +
                            6 * static_cast<size_t>(S) * chw);
}

template <typename Tact>
static cudaError_t configure_wide_t() {
    const int lim = 227 * 1024;
    cudaError_t e = cudaFuncSetAttribute(sscan_bwd_wide_kernel<Tact, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sscan_bwd_wide_kernel<Tact, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sscan_bwd_wide_kernel<Tact, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sscan_bwd_wide_kernel<Tact, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    return e;
}

// Raises the dynamic shared-memory limit of every wide kernel (once, at handle creation).
cudaError_t bwd_wide_configure() {
    cudaError_t e = configure_wide_t<float>();
    if (e == cudaSuccess) e = configure_wide_t<__half>();
    if (e == cudaSuccess) e = configure_wide_t<__nv_bfloat16>();
    return e;
}

template <typename Tact>
static cudaError_t launch_wide_t(const BwdParams& p, int softplus, int lpc, dim3 grid, size_t smem,
                                 cudaStream_t st) {
    auto go = [&](auto kern) {
        kern<<<grid, 32, smem, st>>>(p, softplus);
        return cudaGetLastError();
    };
    switch (lpc) {
        case 4: return go(sscan_bwd_wide_kernel<Tact, 4>);
        case 8: return go(sscan_bwd_wide_kernel<Tact, 8>);
        case 16: return go(sscan_bwd_wide_kernel<Tact, 16>);
        default: return go(sscan_bwd_wide_kernel<Tact, 32>);
    }
}

// Launches the wide-state backward; returns the number of channel tiles through *tiles.
cudaError_t launch_bwd_wide(const BwdParams& p, int dtype, int softplus, cudaStream_t st, int* tiles) {
    const int lpc = bwd_wide_lpc(p.N), chw = 32 / lpc;
    *tiles = (p.D + chw - 1) / chw;
    dim3 grid(*tiles, p.B);
    const size_t smem = bwd_wide_smem(p.N, p.S);
    if (dtype == MAMBA_B200_F32) return launch_wide_t<float>(p, softplus, lpc, grid, smem, st);
    if (dtype == MAMBA_B200_F16) return launch_wide_t<__half>(p, softplus, lpc, grid, smem, st);
    return launch_wide_t<__nv_bfloat16>(p, softplus, lpc, grid, smem, st);
}

}  // namespace mb200
