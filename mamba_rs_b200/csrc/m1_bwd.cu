// Mamba-1 fused selective-scan backward (BPTT) for sm_100a, by recomputation.
//
// The training-mode forward saves only the state ENTERING each block of S
// timesteps (S = save_stride, 32 or 64; 32 is the fast setting).  This file
// holds the host entry point, the reducers and the one-lane-per-channel kernel
// used for d_state <= 8; d_state 9..16 runs the two-lane kernel of
// m1_bwd2_kernel.cuh.  In the one-lane kernel one warp owns
// (sample b, 32 channels), one channel per lane with all d_state values in
// registers, and walks the blocks from last to first:
//   1. TMA brings the block's u, delta, z, dy, B, C tiles (double-buffered
//      against the previous block's work);
//   2. a forward sweep over the block rebuilds the state entering each
//      16-step sub-block;
//   3. per sub-block, last to first: a forward sweep stores h_t for its 16
//      steps in shared memory, then the reverse sweep runs the BPTT
//      recurrence dh <- exp(delta a) dh + dy C and emits du, ddelta, dz;
//   4. dB_t[n] and dC_t[n] are sums over channels: a shuffle butterfly reduces
//      them over the warp's 32 channels and the per-tile partial goes to the
//      caller's workspace; a second kernel adds the tiles in a fixed order
//      (no atomics, bit-reproducible), and reduces dA_log / dD over samples.
// Nothing of size B*T*D*N is ever written (the reference saves h for every
// step and per-channel dB/dC partials, kernels/mamba_ssm_parallel.cu:1182-1532).
#include <string.h>

#include <type_traits>

#include <stdlib.h>

#include "common.cuh"
#include "internal.h"
#include "m1_bwd2_kernel.cuh"

namespace mb200 {

// m1_bwd_wide.cu: 16 < d_state <= 256
int bwd_wide_lpc(int N);
size_t bwd_wide_smem(int N, int S);
cudaError_t bwd_wide_configure();
cudaError_t launch_bwd_wide(const BwdParams& p, int dtype, int softplus, cudaStream_t st, int* tiles);


constexpr int kBwdSub = 16;   // sub-block length (h_t kept in shared memory)
constexpr int kBwdSMax = 64;  // largest save_stride

template <typename Tact, int NS>
struct BwdTraits {
    static constexpr int DT = 32;
    static constexpr size_t al(size_t v) { return (v + 127) & ~size_t(127); }
    static constexpr size_t ACT = al(sizeof(Tact) * kBwdSMax * DT);
    static constexpr size_t BC = al(sizeof(Tact) * kBwdSMax * NS);
    static constexpr size_t STAGE = 4 * ACT + 2 * BC;
    static constexpr size_t OFF_HBUF = 2 * STAGE;                                        // f32 [16][NS][32]
    static constexpr size_t OFF_HB = OFF_HBUF + sizeof(float) * kBwdSub * NS * 32;        // f32 [4][NS][32]
    static constexpr size_t OFF_OUT = OFF_HB + sizeof(float) * (kBwdSMax / kBwdSub) * NS * 32;  // 3 x Tact [S][32]
    static constexpr size_t OFF_DLS = OFF_OUT + 3 * ACT;                                   // f32 delta [S][32]
    static constexpr size_t OFF_BAR = OFF_DLS + sizeof(float) * kBwdSMax * 32;
    static constexpr size_t SMEM = OFF_BAR + 128;
};

// FLAGS: bit0 softplus on delta, bit1 gate present.
template <typename Tact, int NS, int FLAGS>
__global__ void __launch_bounds__(32) sscan_bwd_kernel(const __grid_constant__ BwdParams p) {
    using Tr = BwdTraits<Tact, NS>;
    constexpr bool kSoftplus = (FLAGS & 1) != 0, kGate = (FLAGS & 2) != 0;
    constexpr int DT = 32;
    extern __shared__ __align__(128) unsigned char smem[];
    float* hbuf = reinterpret_cast<float*>(smem + Tr::OFF_HBUF);
    float* hb = reinterpret_cast<float*>(smem + Tr::OFF_HB);
    float* dls = reinterpret_cast<float*>(smem + Tr::OFF_DLS);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    const int lane = threadIdx.x;
    const int b = blockIdx.y, tile = blockIdx.x, d0 = tile * DT, d = d0 + lane;
    const int T = p.T, D = p.D, N = p.N, S = p.S;
    const bool d_ok = d < D;
    const int nblk = (T + S - 1) / S;
    const bool gate_is_silu = p.z_mode == 1;

    auto st_u = [&](int s) { return reinterpret_cast<Tact*>(smem + s * Tr::STAGE); };
    auto st_dl = [&](int s) { return reinterpret_cast<Tact*>(smem + s * Tr::STAGE + Tr::ACT); };
    auto st_z = [&](int s) { return reinterpret_cast<Tact*>(smem + s * Tr::STAGE + 2 * Tr::ACT); };
    auto st_dy = [&](int s) { return reinterpret_cast<Tact*>(smem + s * Tr::STAGE + 3 * Tr::ACT); };
    auto st_b = [&](int s) { return reinterpret_cast<Tact*>(smem + s * Tr::STAGE + 4 * Tr::ACT); };
    auto st_c = [&](int s) { return reinterpret_cast<Tact*>(smem + s * Tr::STAGE + 4 * Tr::ACT + Tr::BC); };
    Tact* o_du = reinterpret_cast<Tact*>(smem + Tr::OFF_OUT);
    Tact* o_ddl = reinterpret_cast<Tact*>(smem + Tr::OFF_OUT + Tr::ACT);
    Tact* o_dz = reinterpret_cast<Tact*>(smem + Tr::OFF_OUT + 2 * Tr::ACT);

    const unsigned lm = p.tma_mask;
    uint32_t tx_bytes = 0;
    if (lm & kBU) tx_bytes += sizeof(Tact) * S * DT;
    if (lm & kBDl) tx_bytes += sizeof(Tact) * S * DT;
    if (kGate && (lm & kBZ)) tx_bytes += sizeof(Tact) * S * DT;
    if (lm & kBDy) tx_bytes += sizeof(Tact) * S * DT;
    if (lm & kBB) tx_bytes += sizeof(Tact) * S * N;
    if (lm & kBC) tx_bytes += sizeof(Tact) * S * N;
    const unsigned all_loads = kBU | kBDl | kBZ | kBDy | kBB | kBC;
    const bool any_plain = (lm & all_loads) != all_loads;

    auto issue = [&](int k, int s) {  // lane 0
        const int t0 = k * S;
        if (!tx_bytes) return;
        mbar_expect_tx(&bars[s], tx_bytes);
        if (lm & kBU) tma_load_3d(st_u(s), &p.tm_u, &bars[s], d0, t0, b);
        if (lm & kBDl) tma_load_3d(st_dl(s), &p.tm_dl, &bars[s], d0, t0, b);
        if (kGate && (lm & kBZ)) tma_load_3d(st_z(s), &p.tm_z, &bars[s], d0, t0, b);
        if (lm & kBDy) tma_load_3d(st_dy(s), &p.tm_dy, &bars[s], d0, t0, b);
        if (lm & kBB) tma_load_3d(st_b(s), &p.tm_b, &bars[s], 0, t0, b);
        if (lm & kBC) tma_load_3d(st_c(s), &p.tm_c, &bars[s], 0, t0, b);
    };

    if (lane == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        fence_barrier_init();
    }
    __syncwarp();
    if (lane == 0 && nblk > 0) issue(nblk - 1, 0);

    // per-channel constants
    float a2[NS];
    bool geo_local = true;
#pragma unroll
    for (int j = 0; j < NS; ++j)
        a2[j] = (d_ok && j < N) ? p.a_neg[static_cast<long long>(d) * N + j] * kLog2e : 0.0f;
    {
        const float step = a2[1] - a2[0];
#pragma unroll
        for (int j = 2; j < NS; ++j)
            if (fabsf(a2[j] - fmaf(static_cast<float>(j), step, a2[0])) > 4.8e-7f * fabsf(a2[j]))
                geo_local = false;
    }
    const bool geo = __all_sync(0xffffffffu, geo_local ? 1 : 0) != 0;
    const float a2_step = a2[1] - a2[0];
    const float Dd = d_ok ? p.Dp[d] : 0.0f;

    // exp2(delta * a2[j]) for all j
    auto decay_t = [&](auto geo_tag, float dlv, float* e) {
        if (decltype(geo_tag)::value) {
            const float E = ex2(dlv * a2[0]), R = ex2(dlv * a2_step);
            e[0] = E;
#pragma unroll
            for (int j = 1; j < NS; ++j) e[j] = (j == NS / 2 && NS == 16) ? ex2(dlv * a2[NS / 2]) : e[j - 1] * R;
        } else {
#pragma unroll
            for (int j = 0; j < NS; ++j) e[j] = ex2(dlv * a2[j]);
        }
    };

    // B or C of one step as f32: one or two 128-bit loads when the row fills the
    // lane slice, element loads otherwise.
    const bool vec_bc = N == NS;
    auto load_row = [&](const Tact* row, float* out) {
        if (vec_bc) {
            StateVec<Tact, NS> v;
            v.load(row);
#pragma unroll
            for (int j = 0; j < NS / 2; ++j) {
                const float2 f = v.pair(j);
                out[2 * j] = f.x;
                out[2 * j + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int j = 0; j < NS; ++j) out[j] = j < N ? to_f(row[j]) : 0.0f;
        }
    };

    float dh[NS], accA[NS];
    float accD = 0.0f;
#pragma unroll
    for (int j = 0; j < NS; ++j) dh[j] = accA[j] = 0.0f;

    auto run_blocks = [&](auto geo_tag) {
    auto decay = [&](float dlv, float* e) { decay_t(geo_tag, dlv, e); };
    for (int it = 0; it < nblk; ++it) {
        const int k = nblk - 1 - it, s = it & 1, t0 = k * S;
        const int nv = min(S, T - t0);
        if (lane == 0 && it + 1 < nblk) issue(k - 1, s ^ 1);
        if (any_plain) {
            if (!(lm & kBU)) bwd_load_plain(st_u(s), static_cast<const Tact*>(p.u), p.ld_u, b, T, t0, d0, D, S, DT);
            if (!(lm & kBDl)) bwd_load_plain(st_dl(s), static_cast<const Tact*>(p.dl), p.ld_dl, b, T, t0, d0, D, S, DT);
            if (kGate && !(lm & kBZ)) bwd_load_plain(st_z(s), static_cast<const Tact*>(p.z), p.ld_z, b, T, t0, d0, D, S, DT);
            if (!(lm & kBDy)) bwd_load_plain(st_dy(s), static_cast<const Tact*>(p.dy), p.ld_dy, b, T, t0, d0, D, S, DT);
            if (!(lm & kBB)) bwd_load_plain(st_b(s), static_cast<const Tact*>(p.bm), p.ld_bc, b, T, t0, 0, N, S, N);
            if (!(lm & kBC)) bwd_load_plain(st_c(s), static_cast<const Tact*>(p.cm), p.ld_bc, b, T, t0, 0, N, S, N);
        }
        if (lane == 0) tma_wait_read0();  // output tiles of the previous block fully read
        if (tx_bytes) mbar_wait(&bars[s], (it >> 1) & 1, p.status);
        __syncwarp();

        const Tact* ru = st_u(s) + lane;
        const Tact* rd = st_dl(s) + lane;
        const Tact* rz = st_z(s) + lane;
        const Tact* rdy = st_dy(s) + lane;
        const Tact* rb = st_b(s);
        const Tact* rc = st_c(s);

        // softplus(delta) of the whole block once (three sweeps read it)
#pragma unroll 4
        for (int r = 0; r < nv; ++r) {
            const float v = to_f(rd[r * DT]);
            dls[r * 32 + lane] = kSoftplus ? softplusf_fast(v) : v;
        }
        auto delta_at = [&](int r) { return dls[r * 32 + lane]; };

        // ---- 2. state entering each sub-block ----
        float h[NS];
        {
#pragma unroll
            for (int j = 0; j < NS; ++j)
                h[j] = (d_ok && j < N)
                           ? p.chunk_states[b * p.cs_ld_b + k * p.cs_ld_k + static_cast<long long>(d) * N + j]
                           : 0.0f;
        }
        const int nsub = (nv + kBwdSub - 1) / kBwdSub;
        for (int sb = 0; sb < nsub; ++sb) {
#pragma unroll
            for (int j = 0; j < NS; ++j) hb[(sb * NS + j) * 32 + lane] = h[j];
            if (sb + 1 == nsub) break;
#pragma unroll 2
            for (int r = sb * kBwdSub; r < (sb + 1) * kBwdSub; ++r) {
                const float dlv = delta_at(r), duv = dlv * to_f(ru[r * DT]);
                float e[NS], Bv[NS];
                decay(dlv, e);
                load_row(rb + r * N, Bv);
#pragma unroll
                for (int j = 0; j < NS; ++j) h[j] = fmaf(e[j], h[j], duv * Bv[j]);
            }
        }

        // ---- 3. sub-blocks, last to first ----
        for (int sb = nsub - 1; sb >= 0; --sb) {
            const int r_lo = sb * kBwdSub, r_hi = min(nv, r_lo + kBwdSub);
#pragma unroll
            for (int j = 0; j < NS; ++j) h[j] = hb[(sb * NS + j) * 32 + lane];
#pragma unroll 2
            for (int r = r_lo; r < r_hi; ++r) {  // forward: keep h_t
                const float dlv = delta_at(r), duv = dlv * to_f(ru[r * DT]);
                float e[NS], Bv[NS];
                decay(dlv, e);
                load_row(rb + r * N, Bv);
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    h[j] = fmaf(e[j], h[j], duv * Bv[j]);
                    hbuf[((r - r_lo) * NS + j) * 32 + lane] = h[j];
                }
            }
            for (int r = r_hi - 1; r >= r_lo; --r) {  // reverse: BPTT
                const float uv = to_f(ru[r * DT]);
                const float raw = to_f(rd[r * DT]);
                const float dlv = delta_at(r);
                const float dyv = to_f(rdy[r * DT]);
                float e[NS], hc[NS], hp[NS], Bv[NS], Cv[NS];
                decay(dlv, e);
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    hc[j] = hbuf[((r - r_lo) * NS + j) * 32 + lane];
                    hp[j] = r > r_lo ? hbuf[((r - r_lo - 1) * NS + j) * 32 + lane]
                                     : hb[(sb * NS + j) * 32 + lane];
                }
                load_row(rb + r * N, Bv);
                load_row(rc + r * N, Cv);
                // pre-gate output and the gate, kernels/elementwise.cu:191-233
                float ys = Dd * uv;
#pragma unroll
                for (int j = 0; j < NS; ++j) ys = fmaf(hc[j], Cv[j], ys);
                float dyp = dyv, dzv = 0.0f;
                if (kGate) {
                    const float zv = to_f(rz[r * DT]);
                    const float sg = sigmoidf_fast(zv);
                    const float gsilu = zv * sg;
                    const float dsilu = sg * fmaf(zv, 1.0f - sg, 1.0f);
                    dyp = dyv * (gate_is_silu ? gsilu : zv);
                    dzv = dyv * ys * (gate_is_silu ? dsilu : 1.0f);
                }
                accD = fmaf(dyp, uv, accD);
                float sB = 0.0f, sA = 0.0f;
                float red[2 * NS];  // dB_t[n] | dC_t[n] contributions of this channel
                const float duv = dlv * uv;
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    dh[j] = fmaf(dyp, Cv[j], dh[j]);
                    sB = fmaf(dh[j], Bv[j], sB);
                    const float dhda = dh[j] * e[j];
                    const float w = dhda * hp[j];
                    sA = fmaf(a2[j], w, sA);
                    accA[j] = fmaf(dlv, w, accA[j]);
                    red[j] = dh[j] * duv;
                    red[NS + j] = dyp * hc[j];
                    dh[j] = dhda;
                }
                const float du_out = fmaf(dyp, Dd, dlv * sB);
                float ddl = fmaf(sA, kLn2, uv * sB);
                if (kSoftplus) ddl *= raw > 20.0f ? 1.0f : sigmoidf_fast(raw);  // activations.cu:68-104
                o_du[r * DT + lane] = from_f<Tact>(du_out);
                o_ddl[r * DT + lane] = from_f<Tact>(ddl);
                if (kGate) o_dz[r * DT + lane] = from_f<Tact>(dzv);
                // sum over the warp's 32 channels: recursive-halving butterfly; lane l
                // ends with element l / (32 / (2 NS)) of the reduced vector.
                {
                    constexpr int V = 2 * NS;
                    int len = V;
#pragma unroll
                    for (int m = 16; m >= 1; m >>= 1) {
                        if (len > 1) {
                            const int half = len / 2;
                            const bool upper = (lane & m) != 0;
#pragma unroll
                            for (int i = 0; i < V / 2; ++i) {
                                if (i < half) {
                                    const float send = upper ? red[i] : red[i + half];
                                    const float keep = upper ? red[i + half] : red[i];
                                    red[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
                                }
                            }
                            len = half;
                        } else {
                            red[0] += __shfl_xor_sync(0xffffffffu, red[0], m);
                        }
                    }
                    constexpr int REP = 32 / V;  // lanes holding the same element
                    if ((lane % REP) == 0 && d0 < D)
                        p.part_bc[(((static_cast<long long>(b) * gridDim.x + tile) * T) + t0 + r) * V + lane / REP] = red[0];
                }
            }
        }

        // ---- store du / ddelta / dz of the block ----
        fence_proxy_async();
        __syncwarp();
        const unsigned sm = lm & (kBDu | kBDdl | kBDz);
        if (lane == 0) {
            if (sm & kBDu) tma_store_3d(&p.tm_du, o_du, d0, t0, b);
            if (sm & kBDdl) tma_store_3d(&p.tm_ddl, o_ddl, d0, t0, b);
            if (kGate && (sm & kBDz)) tma_store_3d(&p.tm_dz, o_dz, d0, t0, b);
            tma_commit();
        }
        auto plain_store = [&](Tact* dst, long long ld, const Tact* src) {
            for (int i = lane; i < nv * DT; i += 32) {
                const int r = i / DT, c = i - r * DT;
                if (d0 + c < D) dst[(static_cast<long long>(b) * T + t0 + r) * ld + d0 + c] = src[i];
            }
        };
        if (!(sm & kBDu)) plain_store(static_cast<Tact*>(p.du), p.ld_du, o_du);
        if (!(sm & kBDdl)) plain_store(static_cast<Tact*>(p.ddl), p.ld_ddl, o_ddl);
        if (kGate && !(sm & kBDz)) plain_store(static_cast<Tact*>(p.dz), p.ld_dz, o_dz);
        __syncwarp();
    }
    };
    if (geo) run_blocks(std::true_type{});
    else run_blocks(std::false_type{});

    // per-sample parameter-gradient partials
    if (d_ok) {
        p.part_d[static_cast<long long>(b) * D + d] = accD;
#pragma unroll
        for (int j = 0; j < NS; ++j)
            if (j < N)
                p.part_a[(static_cast<long long>(b) * D + d) * N + j] =
                    accA[j] * p.a_neg[static_cast<long long>(d) * N + j];
    }
    if (lane == 0) tma_wait_read0();
}

// dB / dC: add the channel tiles in index order.  part [B][tiles][T][2N] -> dB, dC [B,T,N].
// A thread owns four adjacent values of one (sample, step) and keeps eight 16-byte
// loads in flight; the sum still runs in tile order.
__global__ void __launch_bounds__(256) bwd_reduce_bc_kernel(const float* __restrict__ part, float* __restrict__ dB,
                                                            float* __restrict__ dC, int B, int T, int N, int NSv,
                                                            int tiles, int vec_out) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const int V = 2 * NSv, V4 = V / 4;
    if (i >= static_cast<long long>(B) * T * V4) return;
    const int v = static_cast<int>(i % V4) * 4;
    const long long bt = i / V4;
    const long long bb = bt / T, t = bt % T;
    const long long stride = static_cast<long long>(T) * V;
    const float* src = part + (bb * tiles * T + t) * V + v;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int k = 0;
    for (; k + 8 <= tiles; k += 8) {
        float4 q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = __ldcs(reinterpret_cast<const float4*>(src + (k + j) * stride));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc.x += q[j].x; acc.y += q[j].y; acc.z += q[j].z; acc.w += q[j].w;
        }
    }
    for (; k < tiles; ++k) {
        const float4 q = __ldcs(reinterpret_cast<const float4*>(src + k * stride));
        acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    float* dst = v < NSv ? dB : dC;
    const int n = v % NSv;
    const float out[4] = {acc.x, acc.y, acc.z, acc.w};
    if (vec_out && n + 3 < N) {
        *reinterpret_cast<float4*>(dst + bt * N + n) = acc;
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (n + j < N) dst[bt * N + n + j] = out[j];
    }
}

// dA_log[D,N] += sum_b part_a, dD[D] += sum_b part_d, in sample order
// (kernels/mamba_ssm.cu:703-715, :750-763).
__global__ void bwd_reduce_params_kernel(const float* __restrict__ part_a,
                                         const float* __restrict__ part_d, float* __restrict__ dA,
                                         float* __restrict__ dD, int B, int D, int N) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < D * N) {
        float acc = 0.0f;
        for (int b = 0; b < B; ++b) acc += part_a[static_cast<long long>(b) * D * N + i];
        dA[i] += acc;
    }
    if (i < D) {
        float acc = 0.0f;
        for (int b = 0; b < B; ++b) acc += part_d[static_cast<long long>(b) * D + i];
        dD[i] += acc;
    }
}

// States entering every 32-step block from states saved every 64 steps: one
// warp per (sample, 64-step block, 16 channels), two lanes per channel as in the
// two-lane backward, 32 forward steps from the saved state.  Lets a stride-64
// save run the stride-32 backward (whose CTAs all fit the GPU at once).
template <typename Tact>
__global__ void __launch_bounds__(32) sscan_densify_kernel(const BwdParams p, float* __restrict__ dense,
                                                           int softplus) {
    const int lane = threadIdx.x, part = lane >> 4, chl = lane & 15;
    const int d = blockIdx.x * 16 + chl, k = blockIdx.y, b = blockIdx.z, n0 = part * 8;
    const int T = p.T, D = p.D, N = p.N;
    if (d >= D) return;
    const int nb64 = (T + 63) / 64, nb32 = (T + 31) / 32;
    float h[8], a2[8];
    const float* cs = p.chunk_states + b * p.cs_ld_b + k * p.cs_ld_k + static_cast<long long>(d) * N;
    float* o0 = dense + ((static_cast<long long>(b) * nb32 + 2 * k) * D + d) * N;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const bool ok = n0 + j < N;
        h[j] = ok ? cs[n0 + j] : 0.0f;
        a2[j] = ok ? p.a_neg[static_cast<long long>(d) * N + n0 + j] * kLog2e : 0.0f;
        if (ok) o0[n0 + j] = h[j];
    }
    const int t0 = 64 * k;
    if (t0 + 32 >= T) return;  // no second 32-step block inside this one
    const Tact* ub = static_cast<const Tact*>(p.u) + (static_cast<long long>(b) * T + t0) * p.ld_u + d;
    const Tact* db = static_cast<const Tact*>(p.dl) + (static_cast<long long>(b) * T + t0) * p.ld_dl + d;
    const Tact* bb = static_cast<const Tact*>(p.bm) + (static_cast<long long>(b) * T + t0) * p.ld_bc + n0;
    // arithmetic-progression rows of a_neg (the S4D init): two exp2 per step instead of eight
    bool geo = true;
    const float step = a2[1] - a2[0];
#pragma unroll
    for (int j = 2; j < 8; ++j)
        if (fabsf(a2[j] - fmaf(static_cast<float>(j), step, a2[0])) > 4.8e-7f * fabsf(a2[j])) geo = false;
    geo = __all_sync(__activemask(), geo ? 1 : 0) != 0;
    const bool vec_b = N == 16 && (p.ld_bc % 8) == 0 && (reinterpret_cast<uintptr_t>(p.bm) % 16) == 0;
#pragma unroll 4
    for (int r = 0; r < 32; ++r) {
        float dl = to_f(db[static_cast<long long>(r) * p.ld_dl]);
        if (softplus) dl = softplusf_fast(dl);
        const float du = dl * to_f(ub[static_cast<long long>(r) * p.ld_u]);
        float bv[8], e[8];
        if (vec_b) {
            StateVec<Tact, 8> q;
            q.load(bb + static_cast<long long>(r) * p.ld_bc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = q.pair(j);
                bv[2 * j] = f.x;
                bv[2 * j + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) bv[j] = n0 + j < N ? to_f(bb[static_cast<long long>(r) * p.ld_bc + j]) : 0.0f;
        }
        if (geo) {
            const float R = ex2(dl * step);
            e[0] = ex2(dl * a2[0]);
#pragma unroll
            for (int j = 1; j < 8; ++j) e[j] = e[j - 1] * R;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = ex2(dl * a2[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = fmaf(e[j], h[j], du * bv[j]);
    }
    float* o1 = o0 + static_cast<long long>(D) * N;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (n0 + j < N) o1[n0 + j] = h[j];
}

template <typename Tact, int NS>
static void fill_bwd(BwdKernelFn* f, size_t* smem) {
    f[0] = sscan_bwd_kernel<Tact, NS, 0>;
    f[1] = sscan_bwd_kernel<Tact, NS, 1>;
    f[2] = sscan_bwd_kernel<Tact, NS, 2>;
    f[3] = sscan_bwd_kernel<Tact, NS, 3>;
    *smem = BwdTraits<Tact, NS>::SMEM;
}

struct BwdTable {
    BwdKernelFn fn[3][3][4];  // dtype, NS index (4, 8, 16), flags
    size_t smem[3][3];
};

// Built once, under the thread-safe initialisation of a function-local static.
static const BwdTable& bwd_table() {
    static const BwdTable table = [] {
        BwdTable t;
        memset(&t, 0, sizeof(t));
        fill_bwd<float, 4>(t.fn[0][0], &t.smem[0][0]);
        fill_bwd<float, 8>(t.fn[0][1], &t.smem[0][1]);
        fill_bwd<float, 16>(t.fn[0][2], &t.smem[0][2]);
        fill_bwd<__half, 4>(t.fn[1][0], &t.smem[1][0]);
        fill_bwd<__half, 8>(t.fn[1][1], &t.smem[1][1]);
        fill_bwd<__half, 16>(t.fn[1][2], &t.smem[1][2]);
        fill_bwd<__nv_bfloat16, 4>(t.fn[2][0], &t.smem[2][0]);
        fill_bwd<__nv_bfloat16, 8>(t.fn[2][1], &t.smem[2][1]);
        fill_bwd<__nv_bfloat16, 16>(t.fn[2][2], &t.smem[2][2]);
        return t;
    }();
    return table;
}

// Two-lane kernels (8 < d_state <= 16): [dtype][stride index][flags].
struct Bwd2Table {
    BwdKernelFn fn[3][2][4];
    size_t smem[3][2];
};

static const Bwd2Table& bwd2_table() {
    static const Bwd2Table table = [] {
        Bwd2Table t;
        memset(&t, 0, sizeof(t));
        bwd2_kernels_f32(t.fn[MAMBA_B200_F32], t.smem[MAMBA_B200_F32]);
        bwd2_kernels_f16(t.fn[MAMBA_B200_F16], t.smem[MAMBA_B200_F16]);
        bwd2_kernels_bf16(t.fn[MAMBA_B200_BF16], t.smem[MAMBA_B200_BF16]);
        return t;
    }();
    return table;
}

int m1_bwd_configure(Ctx* c) {
    MB200_CUDA_CHECK(c, bwd_wide_configure());
    const Bwd2Table& t2 = bwd2_table();
    for (int dt = 0; dt < 3; ++dt)
        for (int si = 0; si < 2; ++si)
            for (int f = 0; f < 4; ++f) {
                MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(t2.fn[dt][si][f]),
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                         static_cast<int>(t2.smem[dt][si])));
                // many small CTAs per SM: ask for the largest shared-memory carve-out
                MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(t2.fn[dt][si][f]),
                                                         cudaFuncAttributePreferredSharedMemoryCarveout,
                                                         cudaSharedmemCarveoutMaxShared));
            }
    const BwdTable& t = bwd_table();
    for (int dt = 0; dt < 3; ++dt)
        for (int v = 0; v < 3; ++v)
            for (int f = 0; f < 4; ++f)
                MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(t.fn[dt][v][f]),
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                         static_cast<int>(t.smem[dt][v])));
    return MAMBA_B200_OK;
}

static int bwd_ns(int N) { return N <= 4 ? 4 : (N <= 8 ? 8 : 16); }


static void bwd_ws_layout(int B, int T, int D, int N, size_t* off_a, size_t* off_d, size_t* off_dense,
                          size_t* total) {
    // channel tiles of the dB/dC partials: 16 channels per CTA for the two-lane
    // kernel (d_state > 8), 32 for the one-lane kernel
    size_t tiles = N > 8 ? (D + 15) / 16 : (D + 31) / 32, V = 2 * bwd_ns(N);
    if (N > 16) {  // wide-state kernel: 32 / LPC channels per warp, rows of 2 * (8 * LPC) partials
        const int lpc = bwd_wide_lpc(N);
        tiles = (D + 32 / lpc - 1) / (32 / lpc);
        V = 2 * 8 * lpc;
    }
    size_t bc = sizeof(float) * static_cast<size_t>(B) * tiles * T * V;
    bc = (bc + 255) & ~size_t(255);
    size_t a = sizeof(float) * static_cast<size_t>(B) * D * N;
    a = (a + 255) & ~size_t(255);
    const size_t dd = sizeof(float) * static_cast<size_t>(B) * D;
    *off_a = bc;
    *off_d = bc + a;
    *off_dense = bc + a + ((dd + 255) & ~size_t(255));
    // states every 32 steps, rebuilt from a stride-64 save (two-lane kernel only)
    const size_t dense = (N > 8 && N <= 16) ? sizeof(float) * static_cast<size_t>(B) * ((T + 31) / 32) * D * N : 0;
    *total = *off_dense + ((dense + 255) & ~size_t(255));
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API long long mamba_b200_sscan_bwd_workspace_bytes(int B, int T, int D, int N) {
    if (B <= 0 || T <= 0 || D <= 0 || N <= 0 || N > 256) return 0;
    size_t a, d, dn, total;
    bwd_ws_layout(B, T, D, N, &a, &d, &dn, &total);
    return static_cast<long long>(total);
}

static int launch_bwd(Ctx* c, void* stream, const mamba_b200_sscan_bwd_args& a, long long cs_ld_b,
                      long long cs_ld_k) {
    if (!dtype_ok(a.dtype)) return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: bad dtype %d", a.dtype);
    if (a.B < 0 || a.T < 0 || a.D <= 0 || a.N <= 0)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: bad dims B=%d T=%d D=%d N=%d", a.B, a.T, a.D, a.N);
    if (a.N > 256) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_bwd: d_state %d > 256", a.N);
    if (a.B == 0 || a.T == 0) return MAMBA_B200_OK;
    if (a.B > 65535) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_bwd: batch %d > 65535", a.B);
    if (!a.u || !a.delta || !a.Bm || !a.Cm || !a.a_neg || !a.Dp || !a.dy || !a.chunk_states || !a.d_u ||
        !a.d_delta || !a.dBm || !a.dCm || !a.dA_log || !a.dD || !a.workspace)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: null required pointer");
    if (a.z_mode < 0 || a.z_mode > 2 || (a.z_mode && (!a.z || !a.d_z)))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: z_mode %d needs z and d_z", a.z_mode);
    if (a.save_stride != 32 && a.save_stride != 64)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: save_stride %d must be 32 or 64", a.save_stride);
    if (a.ld_u < a.D || a.ld_delta < a.D || a.ld_dy < a.D || a.ld_bc < a.N || a.ld_du < a.D ||
        a.ld_ddelta < a.D || (a.z_mode && (a.ld_z < a.D || a.ld_dz < a.D)))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: a row stride is smaller than its row");
    size_t off_a, off_d, off_dense, total;
    bwd_ws_layout(a.B, a.T, a.D, a.N, &off_a, &off_d, &off_dense, &total);
    if (a.workspace_bytes < static_cast<long long>(total))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: workspace %lld < %zu bytes", a.workspace_bytes, total);
    if (reinterpret_cast<uintptr_t>(a.workspace) % 256)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: workspace must be 256-byte aligned");

    const int ns = bwd_ns(a.N), vi = ns == 4 ? 0 : (ns == 8 ? 1 : 2);
    BwdParams p;
    memset(&p, 0, sizeof(p));
    p.u = a.u; p.dl = a.delta; p.z = a.z_mode ? a.z : nullptr; p.dy = a.dy; p.bm = a.Bm; p.cm = a.Cm;
    p.du = a.d_u; p.ddl = a.d_delta; p.dz = a.z_mode ? a.d_z : nullptr;
    p.ld_u = a.ld_u; p.ld_dl = a.ld_delta; p.ld_z = a.ld_z; p.ld_dy = a.ld_dy; p.ld_bc = a.ld_bc;
    p.ld_du = a.ld_du; p.ld_ddl = a.ld_ddelta; p.ld_dz = a.ld_dz;
    p.a_neg = a.a_neg; p.Dp = a.Dp; p.chunk_states = a.chunk_states;
    p.cs_ld_k = cs_ld_k ? cs_ld_k : static_cast<long long>(a.D) * a.N;
    p.cs_ld_b = cs_ld_b ? cs_ld_b : p.cs_ld_k * ((a.T + a.save_stride - 1) / a.save_stride);
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    p.part_bc = reinterpret_cast<float*>(ws);
    const int bc_vec = a.N % 4 == 0 && (reinterpret_cast<uintptr_t>(a.dBm) | reinterpret_cast<uintptr_t>(a.dCm)) % 16 == 0;
    p.part_a = reinterpret_cast<float*>(ws + off_a);
    p.part_d = reinterpret_cast<float*>(ws + off_d);
    p.B = a.B; p.T = a.T; p.D = a.D; p.N = a.N; p.S = a.save_stride; p.z_mode = a.z_mode;
    p.status = c->d_status;
    cudaStream_t stw = static_cast<cudaStream_t>(stream);
    if (a.N > 16) {
        if (bwd_wide_smem(a.N, a.save_stride) > 227 * 1024)
            return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_bwd: d_state %d with save_stride %d needs more shared memory "
                        "than an SM has; save every 32 steps", a.N, a.save_stride);
        int wtiles = 0;
        cudaError_t e = launch_bwd_wide(p, a.dtype, a.delta_softplus, stw, &wtiles);
        if (e != cudaSuccess) return fail(c, MAMBA_B200_ERR_CUDA, "sscan_bwd (wide): %s", cudaGetErrorString(e));
        const int np = 8 * bwd_wide_lpc(a.N);
        const long long nbcw = static_cast<long long>(a.B) * a.T * 2 * np / 4;
        bwd_reduce_bc_kernel<<<static_cast<unsigned>((nbcw + 255) / 256), 256, 0, stw>>>(
            p.part_bc, a.dBm, a.dCm, a.B, a.T, a.N, np, wtiles, bc_vec);
        MB200_CUDA_CHECK(c, cudaGetLastError());
        const int npar = a.D * a.N;
        bwd_reduce_params_kernel<<<(npar + 255) / 256, 256, 0, stw>>>(p.part_a, p.part_d, a.dA_log, a.dD, a.B, a.D,
                                                                    a.N);
        MB200_CUDA_CHECK(c, cudaGetLastError());
        return MAMBA_B200_OK;
    }
    // one lane per channel for d_state <= 8, two lanes above
    const bool two_lane = a.N > 8;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int S = a.save_stride;
    if (two_lane && S == 64) {
        // rebuild the states at the odd 32-step boundaries, then run the stride-32 kernel
        float* dense = reinterpret_cast<float*>(ws + off_dense);
        dim3 dg((a.D + 15) / 16, (a.T + 63) / 64, a.B);
        if (a.dtype == MAMBA_B200_F32) sscan_densify_kernel<float><<<dg, 32, 0, st>>>(p, dense, a.delta_softplus);
        else if (a.dtype == MAMBA_B200_F16) sscan_densify_kernel<__half><<<dg, 32, 0, st>>>(p, dense, a.delta_softplus);
        else sscan_densify_kernel<__nv_bfloat16><<<dg, 32, 0, st>>>(p, dense, a.delta_softplus);
        MB200_CUDA_CHECK(c, cudaGetLastError());
        p.chunk_states = dense;
        p.S = S = 32;
        p.cs_ld_k = static_cast<long long>(a.D) * a.N;
        p.cs_ld_b = p.cs_ld_k * ((a.T + 31) / 32);
    }
    const int DT = two_lane ? 16 : 32;  // channels per CTA
    unsigned m = 0;
    if (make_tmap_3d(c, &p.tm_u, a.dtype, a.u, a.ld_u, a.D, a.T, a.B, DT, S)) m |= kBU;
    if (make_tmap_3d(c, &p.tm_dl, a.dtype, a.delta, a.ld_delta, a.D, a.T, a.B, DT, S)) m |= kBDl;
    if (!a.z_mode || make_tmap_3d(c, &p.tm_z, a.dtype, a.z, a.ld_z, a.D, a.T, a.B, DT, S)) m |= kBZ;
    if (make_tmap_3d(c, &p.tm_dy, a.dtype, a.dy, a.ld_dy, a.D, a.T, a.B, DT, S)) m |= kBDy;
    if (make_tmap_3d(c, &p.tm_b, a.dtype, a.Bm, a.ld_bc, a.N, a.T, a.B, a.N, S)) m |= kBB;
    if (make_tmap_3d(c, &p.tm_c, a.dtype, a.Cm, a.ld_bc, a.N, a.T, a.B, a.N, S)) m |= kBC;
    if (!two_lane) {  // the two-lane kernel stores its outputs from registers
        if (make_tmap_3d(c, &p.tm_du, a.dtype, a.d_u, a.ld_du, a.D, a.T, a.B, DT, S)) m |= kBDu;
        if (make_tmap_3d(c, &p.tm_ddl, a.dtype, a.d_delta, a.ld_ddelta, a.D, a.T, a.B, DT, S)) m |= kBDdl;
        if (!a.z_mode || make_tmap_3d(c, &p.tm_dz, a.dtype, a.d_z, a.ld_dz, a.D, a.T, a.B, DT, S)) m |= kBDz;
    }
    p.tma_mask = m;

    const BwdTable& t = bwd_table();
    const int flags = (a.delta_softplus ? 1 : 0) | (a.z_mode ? 2 : 0);
    const int tiles = (a.D + DT - 1) / DT;
    dim3 grid(tiles, a.B);
    if (two_lane) {
        const Bwd2Table& t2 = bwd2_table();
        const int si = S == 32 ? 0 : 1;
        t2.fn[a.dtype][si][flags]<<<grid, 32, t2.smem[a.dtype][si], st>>>(p);
    } else {
        t.fn[a.dtype][vi][flags]<<<grid, 32, t.smem[a.dtype][vi], st>>>(p);
    }
    MB200_CUDA_CHECK(c, cudaGetLastError());
    const long long nbc = static_cast<long long>(a.B) * a.T * 2 * ns / 4;
    bwd_reduce_bc_kernel<<<static_cast<unsigned>((nbc + 255) / 256), 256, 0, st>>>(
        p.part_bc, a.dBm, a.dCm, a.B, a.T, a.N, ns, tiles, bc_vec);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    const int np = a.D * a.N;
    bwd_reduce_params_kernel<<<(np + 255) / 256, 256, 0, st>>>(p.part_a, p.part_d, a.dA_log, a.dD, a.B,
                                                             a.D, a.N);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API int mamba_b200_sscan_bwd(void* handle, void* stream,
                                                   const mamba_b200_sscan_bwd_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "sscan_bwd: null args");
    return launch_bwd(c, stream, *ap, 0, 0);
}

extern "C" MAMBA_B200_API int mamba_b200_ssm_scan_bwd(void* handle, void* stream, int dtype, const float* h_saved,
                                                      const void* delta, const void* u, const void* B,
                                                      const void* C, const float* a_neg, const float* D,
                                                      const void* dy, void* d_delta, void* d_u, float* d_B,
                                                      float* d_C, float* d_D, float* d_a_log, int batch, int T,
                                                      int d_inner, int d_state, void* workspace,
                                                      long long workspace_bytes) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    mamba_b200_sscan_bwd_args a;
    memset(&a, 0, sizeof(a));
    a.dtype = dtype; a.B = batch; a.T = T; a.D = d_inner; a.N = d_state;
    a.u = u; a.ld_u = d_inner; a.delta = delta; a.ld_delta = d_inner; a.delta_softplus = 0;
    a.Bm = B; a.Cm = C; a.ld_bc = d_state; a.z_mode = 0;
    a.a_neg = a_neg; a.Dp = D;
    a.chunk_states = h_saved; a.save_stride = 32;  // rows 0, 32, 64, ... of h_saved [batch, T+1, d_inner, d_state]
    a.dy = dy; a.ld_dy = d_inner;
    a.d_u = d_u; a.ld_du = d_inner; a.d_delta = d_delta; a.ld_ddelta = d_inner;
    a.dBm = d_B; a.dCm = d_C; a.dA_log = d_a_log; a.dD = d_D;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    const long long row = static_cast<long long>(d_inner) * d_state;
    return launch_bwd(c, stream, a, row * (static_cast<long long>(T) + 1), 32 * row);
}
