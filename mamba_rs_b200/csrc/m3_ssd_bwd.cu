// Mamba-3 SISO SSD scan backward (chunked form, CUDA cores, f32).
//
// One CTA per (sample, head) walks 32-step chunks twice:
//   A. forward over the chunks, parking the state S_in[c] that ENTERS each chunk
//      in the caller's workspace (the only O(T) scratch: [B,nh,T/32,hd,N] f32);
//   B. backward over the chunks with the running gradient dS of the state.
// Per chunk (local t, s; E_t = exp(dA_t), Lh_ts = exp(dA_t - dA_s), w_t = scale_t exp(dA_end - dA_t)):
//   G = Q K^T, P = dY V^T, R = dY S_in, U = V dS, W = K dS^T
//   dV_s = sum_{t>s} scale_s Lh_ts G_ts dY_t + (gamma_s G_ss + D) dY_s + w_s W_s
//   dQ_t = sum_{s<t} scale_s Lh_ts P_ts K_s + gamma_t P_tt K_t + E_t R_t
//   dK_s = sum_{t>s} scale_s Lh_ts P_ts Q_t + gamma_s P_ss Q_s + w_s U_s
//   d(dA_t) = sum_{s<t} X_ts - sum_{r>t} X_rt + E_t <Q_t, R_t> - w_t Z_t,  X_ts = scale_s Lh_ts G_ts P_ts,
//             Z_t = <K_t, U_t>;  d(dA_end) += sum_t w_t Z_t + E_end <dS, S_in>
//   dscale_s = sum_{t>s} Lh_ts G_ts P_ts + exp(dA_end - dA_s) Z_s;  dgamma_t = G_tt P_tt;  dD += P_tt
//   dS_in = E_end dS + (E o dY)^T Q
// d(adt) is the in-chunk reverse cumulative sum of d(dA); a second, elementwise
// kernel turns (dgamma, dscale) into d(dt), d(trap) (scale_t = gamma_t +
// dt_{t+1}(1 - trap_{t+1}) couples neighbouring steps) and adds dD over samples.
// It replaces m3_extract_da_cs_sum, m3_dqkv (+ its dD reduce), and the parts of
// m3_ddt_dtrap / m3_final_grads that belong to the scan
// (kernels/mamba3_chunked.cu:439-1035; src/mamba3_siso/gpu/backward.rs:235-457).
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

constexpr int kM3C = 32;  // chunk length of the backward

struct M3BwdParams {
    const void *x, *K, *Q, *dy;
    const float *dt, *trap, *adt, *Dh;
    void* dx;
    float *dK, *dQ, *d_adt, *d_dt, *d_trap, *dD;
    float *ws_states;  // [B,nh,nc,hd,N]
    float *ws_dgam;    // [B,T,nh] dgamma (diagonal part)
    float *ws_dscl;    // [B,T,nh] dscale
    float *ws_dD;      // [B,nh]
    int B, T, nh, hd, N;
};

template <typename Tact>
__global__ void __launch_bounds__(256) m3_ssd_bwd_kernel(const M3BwdParams p) {
    extern __shared__ float sm[];
    const int tid = threadIdx.x, NT = 256;
    const int h = blockIdx.x, b = blockIdx.y;
    const int T = p.T, nh = p.nh, hd = p.hd, N = p.N;
    const int LQ = N + 1, LV = hd + 1, LG = kM3C + 1;
    float* Qs = sm;                    // [32][LQ]
    float* Ks = Qs + kM3C * LQ;        // [32][LQ]
    float* Rs = Ks + kM3C * LQ;        // [32][LQ]  R, then U
    float* Vs = Rs + kM3C * LQ;        // [32][LV]
    float* Ys = Vs + kM3C * LV;        // [32][LV]  dY
    float* Ws = Ys + kM3C * LV;        // [32][LV]  W
    float* Gs = Ws + kM3C * LV;        // [32][LG]
    float* Ps = Gs + kM3C * LG;        // [32][LG]
    float* Ss = Ps + kM3C * LG;        // [hd][LQ]  S_in
    float* dS = Ss + hd * LQ;          // [hd][LQ]  running dS
    float* vec = dS + hd * LQ;         // per-step scalars, 12 x 32
    float *dA = vec, *Ee = vec + 32, *scl = vec + 64, *gam = vec + 96, *wv = vec + 128, *ddA = vec + 160,
          *Zv = vec + 192, *dgm = vec + 224, *dsc = vec + 256, *lend = vec + 288, *red = vec + 320;
    const Tact* xg = static_cast<const Tact*>(p.x);
    const Tact* Kg = static_cast<const Tact*>(p.K);
    const Tact* Qg = static_cast<const Tact*>(p.Q);
    const Tact* dyg = static_cast<const Tact*>(p.dy);
    Tact* dxg = static_cast<Tact*>(p.dx);
    const int nc = (T + kM3C - 1) / kM3C;
    const float Dv = p.Dh[h];
    const long long st_base = (static_cast<long long>(b) * nh + h) * nc;

    auto load_scalars = [&](int t0, int len) {
        if (tid < kM3C) {
            float a = 0.0f, g = 0.0f, s = 0.0f;
            if (tid < len) {
                const long long th = (static_cast<long long>(b) * T + t0 + tid) * nh + h;
                a = p.adt[th];
                g = p.dt[th] * p.trap[th];
                s = g;
                if (t0 + tid + 1 < T) s += p.dt[th + nh] * (1.0f - p.trap[th + nh]);
            }
            float run = a;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const float o = __shfl_up_sync(0xffffffffu, run, m);
                if (tid >= m) run += o;
            }
            const float aend = __shfl_sync(0xffffffffu, run, len - 1);
            dA[tid] = run;
            Ee[tid] = ex2(run * kLog2e);
            scl[tid] = s;
            gam[tid] = g;
            lend[tid] = tid < len ? ex2((aend - run) * kLog2e) : 0.0f;  // exp(dA_end - dA_t)
            wv[tid] = lend[tid] * s;
        }
    };
    auto load_tile = [&](float* dst, int ld, const Tact* src, long long row_stride, long long base, int cols,
                         int t0, int len) {
        for (int i = tid; i < kM3C * cols; i += NT) {
            const int r = i / cols, c = i - r * cols;
            dst[r * ld + c] = r < len ? to_f(src[base + (static_cast<long long>(t0 + r)) * row_stride + c]) : 0.0f;
        }
    };
    const long long qk_base = (static_cast<long long>(b) * T * nh + h) * N;   // + t*nh*N
    const long long x_base = static_cast<long long>(b) * T * nh * hd + static_cast<long long>(h) * hd;

    // ---------------- A. forward: states entering each chunk ----------------
    for (int i = tid; i < hd * LQ; i += NT) Ss[i] = 0.0f;
    __syncthreads();
    for (int c = 0; c < nc; ++c) {
        const int t0 = c * kM3C, len = min(kM3C, T - t0);
        load_scalars(t0, len);
        load_tile(Ks, LQ, Kg, static_cast<long long>(nh) * N, qk_base, N, t0, len);
        load_tile(Vs, LV, xg, static_cast<long long>(nh) * hd, x_base, hd, t0, len);
        __syncthreads();
        const float e_end = Ee[len - 1];
        for (int i = tid; i < hd * N; i += NT) {
            const int pp = i / N, n = i - pp * N;
            const float sv = Ss[pp * LQ + n];
            p.ws_states[(st_base + c) * hd * N + i] = sv;
            float acc = e_end * sv;
            for (int t = 0; t < len; ++t) acc = fmaf(wv[t] * Vs[t * LV + pp], Ks[t * LQ + n], acc);
            Ss[pp * LQ + n] = acc;
        }
        __syncthreads();
    }

    // ---------------- B. backward over the chunks ----------------
    for (int i = tid; i < hd * LQ; i += NT) dS[i] = 0.0f;
    float dD_acc = 0.0f;  // thread 0..31 partials
    __syncthreads();
    for (int c = nc - 1; c >= 0; --c) {
        const int t0 = c * kM3C, len = min(kM3C, T - t0);
        load_scalars(t0, len);
        load_tile(Qs, LQ, Qg, static_cast<long long>(nh) * N, qk_base, N, t0, len);
        load_tile(Ks, LQ, Kg, static_cast<long long>(nh) * N, qk_base, N, t0, len);
        load_tile(Vs, LV, xg, static_cast<long long>(nh) * hd, x_base, hd, t0, len);
        load_tile(Ys, LV, dyg, static_cast<long long>(nh) * hd, x_base, hd, t0, len);
        for (int i = tid; i < hd * N; i += NT)
            Ss[(i / N) * LQ + (i % N)] = p.ws_states[(st_base + c) * hd * N + i];
        __syncthreads();
        // G = Q K^T, P = dY V^T
        for (int i = tid; i < kM3C * kM3C; i += NT) {
            const int t = i / kM3C, s = i - t * kM3C;
            float g = 0.0f, pv = 0.0f;
            for (int n = 0; n < N; ++n) g = fmaf(Qs[t * LQ + n], Ks[s * LQ + n], g);
            for (int q = 0; q < hd; ++q) pv = fmaf(Ys[t * LV + q], Vs[s * LV + q], pv);
            Gs[t * LG + s] = g;
            Ps[t * LG + s] = pv;
        }
        // R = dY S_in  [32 x N]
        for (int i = tid; i < kM3C * N; i += NT) {
            const int t = i / N, n = i - t * N;
            float acc = 0.0f;
            for (int q = 0; q < hd; ++q) acc = fmaf(Ys[t * LV + q], Ss[q * LQ + n], acc);
            Rs[t * LQ + n] = acc;
        }
        // W = K dS^T  [32 x hd]
        for (int i = tid; i < kM3C * hd; i += NT) {
            const int s = i / hd, q = i - s * hd;
            float acc = 0.0f;
            for (int n = 0; n < N; ++n) acc = fmaf(Ks[s * LQ + n], dS[q * LQ + n], acc);
            Ws[s * LV + q] = acc;
        }
        __syncthreads();
        // dQ (needs R), and the <Q_t, R_t> part of d(dA)
        for (int i = tid; i < kM3C * N; i += NT) {
            const int t = i / N, n = i - t * N;
            if (t < len) {
                float acc = Ee[t] * Rs[t * LQ + n] + gam[t] * Ps[t * LG + t] * Ks[t * LQ + n];
                for (int s = 0; s < t; ++s)
                    acc = fmaf(scl[s] * ex2((dA[t] - dA[s]) * kLog2e) * Ps[t * LG + s], Ks[s * LQ + n], acc);
                p.dQ[qk_base + static_cast<long long>(t0 + t) * nh * N + n] = acc;
            }
        }
        // dV (needs W)
        for (int i = tid; i < kM3C * hd; i += NT) {
            const int s = i / hd, q = i - s * hd;
            if (s < len) {
                float acc = fmaf(gam[s], Gs[s * LG + s], Dv) * Ys[s * LV + q] + wv[s] * Ws[s * LV + q];
                for (int t = s + 1; t < len; ++t)
                    acc = fmaf(scl[s] * ex2((dA[t] - dA[s]) * kLog2e) * Gs[t * LG + s], Ys[t * LV + q], acc);
                dxg[x_base + static_cast<long long>(t0 + s) * nh * hd + q] = from_f<Tact>(acc);
            }
        }
        // per-step scalars: d(dA) pieces, dscale, dgamma, dD
        if (tid < kM3C) {
            const int t = tid;
            float qr = 0.0f;
            for (int n = 0; n < N; ++n) qr = fmaf(Qs[t * LQ + n], Rs[t * LQ + n], qr);
            float rowX = 0.0f, colX = 0.0f, dsl = 0.0f;
            for (int s = 0; s < t; ++s)
                rowX = fmaf(scl[s] * ex2((dA[t] - dA[s]) * kLog2e), Gs[t * LG + s] * Ps[t * LG + s], rowX);
            for (int r = t + 1; r < len; ++r) {
                const float lh = ex2((dA[r] - dA[t]) * kLog2e) * Gs[r * LG + t] * Ps[r * LG + t];
                dsl += lh;
                colX = fmaf(scl[t], lh, colX);
            }
            ddA[t] = rowX - colX + Ee[t] * qr;
            dsc[t] = dsl;
            dgm[t] = t < len ? Gs[t * LG + t] * Ps[t * LG + t] : 0.0f;
            if (t < len) dD_acc += Ps[t * LG + t];
        }
        __syncthreads();
        // U = V dS  [32 x N]  (R is no longer needed)
        for (int i = tid; i < kM3C * N; i += NT) {
            const int s = i / N, n = i - s * N;
            float acc = 0.0f;
            for (int q = 0; q < hd; ++q) acc = fmaf(Vs[s * LV + q], dS[q * LQ + n], acc);
            Rs[s * LQ + n] = acc;
        }
        // <dS, S_in> for d(dA_end)
        {
            float part = 0.0f;
            for (int i = tid; i < hd * N; i += NT) part = fmaf(dS[(i / N) * LQ + (i % N)], Ss[(i / N) * LQ + (i % N)], part);
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
            if ((tid & 31) == 0) red[tid >> 5] = part;
        }
        __syncthreads();
        // dK (needs U), Z_t = <K_t, U_t>
        for (int i = tid; i < kM3C * N; i += NT) {
            const int s = i / N, n = i - s * N;
            if (s < len) {
                float acc = wv[s] * Rs[s * LQ + n] + gam[s] * Ps[s * LG + s] * Qs[s * LQ + n];
                for (int t = s + 1; t < len; ++t)
                    acc = fmaf(scl[s] * ex2((dA[t] - dA[s]) * kLog2e) * Ps[t * LG + s], Qs[t * LQ + n], acc);
                p.dK[qk_base + static_cast<long long>(t0 + s) * nh * N + n] = acc;
            }
        }
        if (tid < kM3C) {
            float z = 0.0f;
            for (int n = 0; n < N; ++n) z = fmaf(Ks[tid * LQ + n], Rs[tid * LQ + n], z);
            Zv[tid] = z;
        }
        __syncthreads();
        // finish the per-step scalars and write them
        if (tid < kM3C) {
            const int t = tid;
            float v = tid < len ? ddA[t] - wv[t] * Zv[t] : 0.0f;
            float wz = tid < len ? wv[t] * Zv[t] : 0.0f;
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) wz += __shfl_xor_sync(0xffffffffu, wz, m);
            float ds_dot = 0.0f;
            for (int w = 0; w < NT / 32; ++w) ds_dot += red[w];
            if (t == len - 1) v += wz + Ee[len - 1] * ds_dot;  // dA_end is the last dA of the chunk
            // d(adt_r) = sum_{t >= r} d(dA_t): reverse inclusive scan
            float run = v;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const float o = __shfl_down_sync(0xffffffffu, run, m);
                if (tid + m < 32) run += o;
            }
            if (t < len) {
                const long long th = (static_cast<long long>(b) * T + t0 + t) * nh + h;
                p.d_adt[th] = run;
                p.ws_dgam[th] = dgm[t];
                p.ws_dscl[th] = dsc[t] + lend[t] * Zv[t];
            }
        }
        // dS <- E_end dS + (E o dY)^T Q
        {
            const float e_end = Ee[len - 1];
            for (int i = tid; i < hd * N; i += NT) {
                const int q = i / N, n = i - q * N;
                float acc = e_end * dS[q * LQ + n];
                for (int t = 0; t < len; ++t) acc = fmaf(Ee[t] * Ys[t * LV + q], Qs[t * LQ + n], acc);
                dS[q * LQ + n] = acc;
            }
        }
        __syncthreads();
    }
    if (tid < 32) {
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) dD_acc += __shfl_xor_sync(0xffffffffu, dD_acc, m);
        if (tid == 0) p.ws_dD[static_cast<long long>(b) * nh + h] = dD_acc;
    }
}

// scale_t = gamma_t + dt_{t+1}(1 - trap_{t+1}), gamma_t = dt_t trap_t:
//   d_dt[t]   = dgt[t] trap[t] + dscale[t-1] (1 - trap[t]),  dgt = dgamma + dscale
//   d_trap[t] = dgt[t] dt[t]   - dscale[t-1] dt[t]
// and dD[h] += sum_b partial[b,h] in sample order.
__global__ void m3_bwd_finish_kernel(const M3BwdParams p) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long total = static_cast<long long>(p.B) * p.T * p.nh;
    if (i < total) {
        const long long t = (i / p.nh) % p.T;
        const float dgt = p.ws_dgam[i] + p.ws_dscl[i];
        const float dsp = t > 0 ? p.ws_dscl[i - p.nh] : 0.0f;
        p.d_dt[i] = dgt * p.trap[i] + dsp * (1.0f - p.trap[i]);
        p.d_trap[i] = dgt * p.dt[i] - dsp * p.dt[i];
    }
    if (i < p.nh) {
        float acc = 0.0f;
        for (int b = 0; b < p.B; ++b) acc += p.ws_dD[static_cast<long long>(b) * p.nh + i];
        p.dD[i] += acc;
    }
}

static size_t m3_bwd_smem(int hd, int N) {
    const size_t LQ = N + 1, LV = hd + 1, LG = kM3C + 1;
    return sizeof(float) * (3 * kM3C * LQ + 3 * kM3C * LV + 2 * kM3C * LG + 2 * hd * LQ + 12 * 32);
}

static void m3_bwd_ws(int B, int T, int nh, int hd, int N, size_t* o_g, size_t* o_s, size_t* o_d, size_t* total) {
    const size_t nc = (T + kM3C - 1) / kM3C;
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t st = al(sizeof(float) * static_cast<size_t>(B) * nh * nc * hd * N);
    const size_t v = al(sizeof(float) * static_cast<size_t>(B) * T * nh);
    *o_g = st; *o_s = st + v; *o_d = st + 2 * v;
    *total = st + 2 * v + al(sizeof(float) * static_cast<size_t>(B) * nh);
}

int m3_bwd_configure(Ctx* c) {
    const int smem = static_cast<int>(m3_bwd_smem(64, 128));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(m3_ssd_bwd_kernel<float>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(m3_ssd_bwd_kernel<__half>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(m3_ssd_bwd_kernel<__nv_bfloat16>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API long long mamba_b200_m3_ssd_bwd_workspace_bytes(int B, int T, int nh, int hd, int N) {
    if (B <= 0 || T <= 0 || nh <= 0 || hd <= 0 || N <= 0) return 0;
    size_t a, b2, d, total;
    m3_bwd_ws(B, T, nh, hd, N, &a, &b2, &d, &total);
    return static_cast<long long>(total);
}

extern "C" MAMBA_B200_API int mamba_b200_m3_ssd_bwd(void* handle, void* stream,
                                                    const mamba_b200_m3_ssd_bwd_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: null args");
    const mamba_b200_m3_ssd_bwd_args& a = *ap;
    if (!dtype_ok(a.dtype)) return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: bad dtype %d", a.dtype);
    if (a.B < 0 || a.T < 0 || a.nh <= 0 || a.hd <= 0 || a.N <= 0)
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: bad dims");
    if (a.hd > 64 || a.N > 128)
        return fail(c, MAMBA_B200_ERR_SHAPE, "m3_ssd_bwd: headdim %d > 64 or d_state %d > 128", a.hd, a.N);
    if (a.B == 0 || a.T == 0) return MAMBA_B200_OK;
    if (a.B > 65535) return fail(c, MAMBA_B200_ERR_SHAPE, "m3_ssd_bwd: batch %d > 65535", a.B);
    if (!a.x || !a.K || !a.Q || !a.dt || !a.trap || !a.adt || !a.Dh || !a.dy || !a.dx || !a.dK || !a.dQ ||
        !a.d_adt || !a.d_dt || !a.d_trap || !a.dD || !a.workspace)
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: null required pointer");
    size_t o_g, o_s, o_d, total;
    m3_bwd_ws(a.B, a.T, a.nh, a.hd, a.N, &o_g, &o_s, &o_d, &total);
    if (a.workspace_bytes < static_cast<long long>(total))
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: workspace %lld < %zu bytes", a.workspace_bytes, total);
    if (reinterpret_cast<uintptr_t>(a.workspace) % 256)
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: workspace must be 256-byte aligned");
    M3BwdParams p;
    memset(&p, 0, sizeof(p));
    p.x = a.x; p.K = a.K; p.Q = a.Q; p.dy = a.dy; p.dt = a.dt; p.trap = a.trap; p.adt = a.adt; p.Dh = a.Dh;
    p.dx = a.dx; p.dK = a.dK; p.dQ = a.dQ; p.d_adt = a.d_adt; p.d_dt = a.d_dt; p.d_trap = a.d_trap; p.dD = a.dD;
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    p.ws_states = reinterpret_cast<float*>(ws);
    p.ws_dgam = reinterpret_cast<float*>(ws + o_g);
    p.ws_dscl = reinterpret_cast<float*>(ws + o_s);
    p.ws_dD = reinterpret_cast<float*>(ws + o_d);
    p.B = a.B; p.T = a.T; p.nh = a.nh; p.hd = a.hd; p.N = a.N;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(a.nh, a.B);
    const size_t smem = m3_bwd_smem(a.hd, a.N);
    if (a.dtype == MAMBA_B200_F32) m3_ssd_bwd_kernel<float><<<grid, 256, smem, st>>>(p);
    else if (a.dtype == MAMBA_B200_F16) m3_ssd_bwd_kernel<__half><<<grid, 256, smem, st>>>(p);
    else m3_ssd_bwd_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    const long long total_e = static_cast<long long>(a.B) * a.T * a.nh;
    m3_bwd_finish_kernel<<<static_cast<unsigned>((total_e + 255) / 256), 256, 0, st>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}
