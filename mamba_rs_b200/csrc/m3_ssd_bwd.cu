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
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "internal.h"
#include "m3_tc.cuh"

namespace mb200 {

constexpr int kM3C = 32;  // chunk length of the backward

struct M3BwdParams {
    // tensor-core kernel: adt, dt, trap [B,T,nh] f32 as boxes of 4 heads x 129 rows (valid when
    // sc_tma; needs nheads % 4 == 0)
    CUtensorMap tm_adt, tm_dt, tm_trap;
    // tensor-core kernel: Q, K, x, dy as [128 x 64] swizzled sub-tile maps
    CUtensorMap tm_q, tm_k, tm_x, tm_dy;
    int sc_tma;
    int wide_st;  // dK and dQ are 32-byte aligned: their rows leave as 256-bit stores
    int wide_dx;  // the same for dx (headdim a multiple of 16)
    const void *x, *K, *Q, *dy;
    const float *dt, *trap, *adt, *Dh;
    void* dx;
    float *dK, *dQ, *d_adt, *d_dt, *d_trap, *dD;
    float *ws_states;  // [B,nh,nc,hd,N]
    float *ws_dgam;    // [B,T,nh] dgamma (diagonal part)
    float *ws_dscl;    // [B,T,nh] dscale
    float *ws_dD;      // [B,nh]
    int B, T, nh, hd, N;
    int* status;
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

// ---------------------------------------------------------------------------
// Tensor-core backward (16-bit storage, headdim 64, d_state 128): the same
// chunked formulas with 128-step chunks, every product on tcgen05 with f32
// accumulators in TMEM.  One CTA of 128 threads per (sample, head); thread t
// owns step t of the chunk and TMEM lane t.
//   A. forward over the chunks: S^T[n][p] lives in TMEM; a 16-bit copy of the
//      state entering each chunk goes to the workspace in operand-tile order.
//   B. backward over the chunks, three MMA groups per chunk:
//      1. G = Q K^T, P = dY V^T, R' = (E o dY) S_in, W = K dS^T
//         -> rows of M1 = mask(scale L o P), M2 = mask(scale L o G) to shared
//            memory, row sums of X, <Q_t, R'_t>, W rows scaled by w in place,
//            dS decayed by exp(dA_end) in place
//      2. G^T, P^T (column sums of X and dscale), dQ = R' + M1 K, dV = wW + M2^T dY
//      3. dK = M1^T Q, U = V dS, dS += Q^T (E o dY)
// Operands are rounded to the storage dtype (M1, M2, E o dY, the state copies),
// so results carry 16-bit rounding like the forward's tensor-core path.
namespace tcb {
using namespace tc;

// Eight consecutive floats: one 256-bit store (a whole 32-byte sector per request) when the
// destination allows it, else two 128-bit stores.
__device__ __forceinline__ void store8(float* dst, const float* o, bool wide) {
    if (wide) {
        asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "f"(o[0]), "f"(o[1]), "f"(o[2]),
                     "f"(o[3]), "f"(o[4]), "f"(o[5]), "f"(o[6]), "f"(o[7])
                     : "memory");
    } else {
        reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
}

constexpr int CS = 128, HD = 64, NS = 128;
constexpr uint32_t kQ = 0, kK = 32768, kV = 65536, kDY = 81920, kSin = 98304, kDS = 114688, kM1 = 131072,
                   kM2 = 163840, kEdY = 196608, kVec = 212992;
// f32 vectors: dA, scl, gam, red (scratch), gdv, pdv, part[5], dA*log2(e)
// staging of the per-row scalars of one chunk: [3][129 rows][4 heads] f32, each array on a
// 128-byte boundary (TMA destinations)
constexpr uint32_t kStage = kVec + 12 * 128 * 4, kStageArr = 17 * 128;
static_assert(kStage % 128 == 0 && kStageArr >= 129 * 16, "scalar staging");
constexpr uint32_t kBar = kStage + 3 * kStageArr, kTmemSlot = kBar + 64, kSmem = kTmemSlot + 16;
static_assert(kSmem <= 227 * 1024, "shared memory");
constexpr uint32_t c0 = 0, c1 = 128, c2 = 256, c3 = 384, cDS = 448, kTmemCols = 512;
constexpr uint32_t kStateTile = NS * HD * 2;  // bytes of one 16-bit state copy

template <typename Th>
__global__ void __launch_bounds__(256) m3_ssd_bwd_tc_kernel(const __grid_constant__ M3BwdParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // two threads per step: (row tid, half) share TMEM lane tid and split its columns
    const int tid = threadIdx.x & 127, half = threadIdx.x >> 7, warp = (threadIdx.x >> 5) & 3, lane = tid & 31;
    const int h = blockIdx.x, b = blockIdx.y;
    const int T = p.T, nh = p.nh;
    // headdim <= 64, d_state <= 128 (multiples of 8): full-size tiles, missing columns zero-filled
    const int hdv = p.hd, nsv = p.N;
    constexpr uint32_t fmt = std::is_same<Th, __nv_bfloat16>::value ? 1u : 0u;
    float* dA = reinterpret_cast<float*>(smem + kVec);
    float* scl = dA + 128;
    float* gam = dA + 256;
    float* red = dA + 384;
    float* gdv = dA + 512;
    float* pdv = dA + 640;
    float* part = dA + 768;  // [5][128]: partial sums of the upper-half threads
    float* dAl = dA + 1408;  // dA * log2(e)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBar);
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + kTmemSlot);
    const uint32_t sbase = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);  // 5, 6: a chunk's tiles have landed (TMA)
        fence_barrier_init();
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tslot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tslot;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);

    const Th* xg = static_cast<const Th*>(p.x);
    const Th* Kg = static_cast<const Th*>(p.K);
    const Th* Qg = static_cast<const Th*>(p.Q);
    const Th* dyg = static_cast<const Th*>(p.dy);
    Th* dxg = static_cast<Th*>(p.dx);
    const float Dv = p.Dh[h];
    const int nc = (T + CS - 1) / CS;
    unsigned char* ws_st = reinterpret_cast<unsigned char*>(p.ws_states) +
                           (static_cast<size_t>(b) * nh + h) * nc * kStateTile;
    uint32_t ph[4] = {0, 0, 0, 0};
    bool ok = true;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // The per-row adt, dt, trap of a chunk come as three TMA boxes issued before the tile
    // copies (so they land while those are being issued) instead of 128-byte-strided register
    // loads with their latency exposed; without the maps (nheads % 4 != 0) the loads remain.
    uint32_t scph = 0;
    const int hcol = h & 3;
    auto issue_scalars_now = [&](int t0) {  // one thread
        if (p.sc_tma) {
            mbar_expect_tx(&bars[4], 3 * 129 * 16);
            tma_load_3d(smem + kStage, &p.tm_adt, &bars[4], h & ~3, t0, b);
            tma_load_3d(smem + kStage + kStageArr, &p.tm_dt, &bars[4], h & ~3, t0, b);
            tma_load_3d(smem + kStage + 2 * kStageArr, &p.tm_trap, &bars[4], h & ~3, t0, b);
        }
    };
    auto issue_scalars = [&](int t0) {
        if (threadIdx.x == 0) issue_scalars_now(t0);
    };
    // per-row scalars of chunk c -> dA (inclusive cumsum), scl, gam in shared memory
    auto load_scalars = [&](int t0, int nv, float& run_o, float& g_o, float& s_o) {
        const int t = t0 + tid;
        float a = 0.0f, g = 0.0f, s = 0.0f;
        if (p.sc_tma) {
            ok = mbar_wait(&bars[4], scph, p.status) && ok;
            scph ^= 1;
            const float* stg = reinterpret_cast<const float*>(smem + kStage) + tid * 4 + hcol;
            if (tid < nv) {  // rows past T arrive as zeros
                a = stg[0];
                g = stg[kStageArr / 4] * stg[2 * kStageArr / 4];
                s = g + stg[kStageArr / 4 + 4] * (1.0f - stg[2 * kStageArr / 4 + 4]);
            }
        } else if (tid < nv) {
            const long long th = (static_cast<long long>(b) * T + t) * nh + h;
            a = p.adt[th];
            g = p.dt[th] * p.trap[th];
            s = g;
            if (t + 1 < T) s += p.dt[th + nh] * (1.0f - p.trap[th + nh]);
        }
        float run = a;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const float o = __shfl_up_sync(0xffffffffu, run, m);
            if (lane >= m) run += o;
        }
        if (lane == 31) red[warp] = run;
        gam[tid] = g;
        scl[tid] = s;
        __syncthreads();
        float off = 0.0f;
        for (int w = 0; w < warp; ++w) off += red[w];
        run += off;
        dA[tid] = run;
        dAl[tid] = run * kLog2e;
        __syncthreads();
        run_o = run; g_o = g; s_o = s;
    };
    auto wait_bar = [&](int i) {
        ok = mbar_wait(&bars[i], ph[i], p.status) && ok;
        ph[i] ^= 1;
        fence_after();
    };
    // sum over the CTA of one float per thread (result to every thread)
    auto block_sum = [&](float v) {  // callers pass 0 from the upper-half threads
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
        __syncthreads();
        if (lane == 0 && half == 0) red[warp] = v;
        __syncthreads();
        return red[0] + red[1] + red[2] + red[3];
    };

    // Tiles come by TMA (one thread; rows past T and columns past the head's width arrive as
    // zeros), the 16-bit state copy of a chunk by one contiguous bulk copy.
    // barrier 5 for the backward pass and the even chunks of the state pass, 6 for its odd
    // chunks (two requests are in flight there)
    uint32_t tfph[2] = {0, 0};
    auto load_qk = [&](uint32_t tile, const CUtensorMap* map, int t0, int bi) {
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
            tma_load_4d(smem + tile + sub * kSwSub, map, &bars[5 + bi], 64 * sub, h, t0, b);
    };
    auto wait_tiles = [&](int bi) {
        ok = mbar_wait(&bars[5 + bi], tfph[bi], p.status) && ok;
        tfph[bi] ^= 1;
    };

    // ---------------- A. forward: 16-bit copies of the entering states ----------------
    // K and V of chunk c + 1 are requested while chunk c is worked on; the pass needs few tiles,
    // so odd chunks simply use the tiles the backward pass calls M1 and S_in.
    auto request_kv = [&](int c) {  // one thread
        const int t0 = c * CS;
        mbar_expect_tx(&bars[5 + (c & 1)], 2 * kSwSub + kSwSub);
        load_qk((c & 1) ? kM1 : kK, &p.tm_k, t0, c & 1);
        tma_load_4d(smem + ((c & 1) ? kSin : kV), &p.tm_x, &bars[5 + (c & 1)], 0, h, t0, b);
    };
    if (threadIdx.x == 0 && nc > 1) {
        issue_scalars_now(0);
        request_kv(0);
    }
    for (int c = 0; c < nc; ++c) {
        const int t0 = c * CS, nv = min(CS, T - t0);
        const bool last = c + 1 == nc;
        const uint32_t tKa = (c & 1) ? kM1 : kK, tVa = (c & 1) ? kSin : kV;
        float run = 0.0f, g = 0.0f, s = 0.0f;
        if (!last) {
            if (threadIdx.x == 0 && c + 2 < nc) request_kv(c + 1);  // its tiles were last read by chunk c - 1
            load_scalars(t0, nv, run, g, s);
            if (threadIdx.x == 0 && c + 2 < nc) issue_scalars_now(t0 + CS);  // the staging was read just above
            const float dA_end = dA[nv - 1];
            const float wt = tid < nv ? ex2((dA_end - run) * kLog2e) * s : 0.0f;
            wait_tiles(c & 1);
#pragma unroll
            for (int j = half * (HD / 16); j < (half + 1) * (HD / 16); ++j) {
                const uint4 v = *reinterpret_cast<const uint4*>(smem + tVa + sw_chunk(tid, j));
                uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float2 f = unpack2<Th>(w4[q4]);
                    w4[q4] = pack2<Th>(f.x * wt, f.y * wt);
                }
                *reinterpret_cast<uint4*>(smem + kDY + sw_chunk(tid, j)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
        }
        if (c > 0) {  // state entering chunk c: copy out, then decay for the update
            const float e_end = last ? 0.0f : ex2(dA[nv - 1] * kLog2e);
            {
                const int q2 = half;
                float sv[32];
                tmem_ld32(lane_addr + cDS + q2 * 32, sv);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(ws_st + static_cast<size_t>(c) * kStateTile + sw_chunk(tid, q2 * 4 + j)) =
                        make_uint4(pack2<Th>(sv[8 * j], sv[8 * j + 1]), pack2<Th>(sv[8 * j + 2], sv[8 * j + 3]),
                                   pack2<Th>(sv[8 * j + 4], sv[8 * j + 5]), pack2<Th>(sv[8 * j + 6], sv[8 * j + 7]));
                if (!last) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) sv[i] *= e_end;
                    tmem_st32(lane_addr + cDS + q2 * 32, sv);
                }
            }
        }
        if (last) break;
        fence_proxy_async();
        fence_before();
        __syncthreads();
        if (threadIdx.x == 0) {
            fence_after();
            const uint32_t idS = instr_desc(fmt, 1, 1, 64);
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // S^T[n][p] += sum_t K[t][n] (w V)[t][p]
                mma(tmem + cDS, desc_sw_mn(sbase + tKa, k), desc_sw_mn(sbase + kDY, k), idS, c > 0 || k > 0);
            commit(&bars[3]);
        }
        wait_bar(3);
    }
    // the state copies of this CTA (generic stores) are read back below by bulk copies
    asm volatile("fence.proxy.async;" ::: "memory");
    fence_before();
    __syncthreads();
    fence_after();

    // ---------------- B. backward over the chunks ----------------
    bool has_ds = false;
    float dD_acc = 0.0f;
    // The tiles of a chunk are requested while the previous chunk's last epilogue runs: as soon
    // as its last MMA group is done, Q and K of the next chunk go where this chunk's M1 and M2
    // were (the two pairs of tiles swap places every chunk, so nothing is double-buffered), V, dY
    // and the entering state go to their own tiles.
    auto request_tiles = [&](int c, uint32_t q_tile, uint32_t k_tile) {  // one thread
        const int t0 = c * CS;
        issue_scalars_now(t0);
        mbar_expect_tx(&bars[5], 4 * kSwSub + 2 * kSwSub + (c > 0 ? kStateTile : 0));
        load_qk(q_tile, &p.tm_q, t0, 0);
        load_qk(k_tile, &p.tm_k, t0, 0);
        tma_load_4d(smem + kV, &p.tm_x, &bars[5], 0, h, t0, b);
        tma_load_4d(smem + kDY, &p.tm_dy, &bars[5], 0, h, t0, b);
        if (c > 0) bulk_load(smem + kSin, ws_st + static_cast<size_t>(c) * kStateTile, kStateTile, &bars[5]);
    };
    if (threadIdx.x == 0 && nc > 0) request_tiles(nc - 1, kQ, kK);
    for (int c = nc - 1, it = 0; c >= 0; --c, ++it) {
        const bool par = (it & 1) != 0;
        const uint32_t tQ = par ? kM1 : kQ, tK = par ? kM2 : kK, tM1 = par ? kQ : kM1, tM2 = par ? kK : kM2;
        const int t0 = c * CS, nv = min(CS, T - t0);
        const int t = t0 + tid;
        const bool row_ok = tid < nv;
        const bool has_sin = c > 0;
        float run, g_t, s_t;
        load_scalars(t0, nv, run, g_t, s_t);
        const float dA_t = run, dA_end = dA[nv - 1];
        const float e_t = ex2(dA_t * kLog2e), e_end = ex2(dA_end * kLog2e);
        const float lend_t = row_ok ? ex2((dA_end - dA_t) * kLog2e) : 0.0f;
        const float w_t = lend_t * s_t;
        const long long qk_row = ((static_cast<long long>(b) * T + t) * nh + h) * nsv;
        const long long x_row = (static_cast<long long>(b) * T + t) * nh * hdv + h * hdv;
        wait_tiles(0);
        // E o dY from the landed dY tile (own row, own half of the columns)
#pragma unroll
        for (int j = half * (HD / 16); j < (half + 1) * (HD / 16); ++j) {
            const uint4 dyv = *reinterpret_cast<const uint4*>(smem + kDY + sw_chunk(tid, j));
            uint32_t w4[4] = {dyv.x, dyv.y, dyv.z, dyv.w};
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const float2 f = unpack2<Th>(w4[q4]);
                w4[q4] = pack2<Th>(f.x * e_t, f.y * e_t);
            }
            *reinterpret_cast<uint4*>(smem + kEdY + sw_chunk(tid, j)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
        fence_proxy_async();
        fence_before();
        __syncthreads();
        // ---- group 1 ----
        if (threadIdx.x == 0) {
            fence_after();
            const uint32_t idKK = instr_desc(fmt, 0, 0, 128), idW = instr_desc(fmt, 0, 1, 64);
#pragma unroll
            for (int k = 0; k < NS / 16; ++k)  // G[t][s] = sum_n Q[t][n] K[s][n]
                mma(tmem + c0, desc_sw_k(sbase + tQ, k), desc_sw_k(sbase + tK, k), idKK, k > 0);
#pragma unroll
            for (int k = 0; k < HD / 16; ++k)  // P[t][s] = sum_p dY[t][p] V[s][p]
                mma(tmem + c1, desc_sw_k(sbase + kDY, k), desc_sw_k(sbase + kV, k), idKK, k > 0);
            if (has_sin) {
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)  // R'[t][n] = sum_p (E dY)[t][p] S_in^T[n][p]
                    mma(tmem + c2, desc_sw_k(sbase + kEdY, k), desc_sw_k(sbase + kSin, k), idKK, k > 0);
            }
            if (has_ds) {
#pragma unroll
                for (int k = 0; k < NS / 16; ++k)  // W[s][p] = sum_n K[s][n] dS^T[n][p]
                    mma(tmem + c3, desc_sw_k(sbase + tK, k), desc_sw_mn(sbase + kDS, k), idW, k > 0);
            }
            commit(&bars[0]);
        }
        wait_bar(0);
        // ---- epilogue 1 ----
        float rowX = 0.0f, gd = 0.0f, pd = 0.0f, qr = 0.0f, ds_part = 0.0f;
        // One 32-column block of row `tid` of M1 = scale L o P and M2 = scale L o G.  Blocks
        // left of the diagonal block need no mask; rows and columns past the end of the
        // sequence come out as exact zeros (their Q, dY rows and scale are zero).
        const float dAl_t = dAl[tid];
        auto mask_block = [&](auto diag_tag, int q4) {
            constexpr bool DIAG = decltype(diag_tag)::value;
            float gv[32], pv[32];
            tmem_ld32x2(lane_addr + c0 + q4 * 32, gv, lane_addr + c1 + q4 * 32, pv);
            uint32_t pk1[16], pk2[16];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 da4 = *reinterpret_cast<const float4*>(dAl + q4 * 32 + i);
                const float4 sc4 = *reinterpret_cast<const float4*>(scl + q4 * 32 + i);
                const float dav[4] = {da4.x, da4.y, da4.z, da4.w}, scv[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
                float m1[4], m2[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float f = scv[u] * ex2(dAl_t - dav[u]);
                    if (DIAG) {
                        const int s = q4 * 32 + i + u;
                        if (s >= tid) f = 0.0f;
                        if (s == tid) {
                            gd = gv[i + u];
                            pd = pv[i + u];
                        }
                    }
                    m1[u] = f * pv[i + u];
                    m2[u] = f * gv[i + u];
                    rowX = fmaf(m1[u], gv[i + u], rowX);
                }
                pk1[i / 2] = pack2<Th>(m1[0], m1[1]);
                pk1[i / 2 + 1] = pack2<Th>(m1[2], m1[3]);
                pk2[i / 2] = pack2<Th>(m2[0], m2[1]);
                pk2[i / 2 + 1] = pack2<Th>(m2[2], m2[3]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                *reinterpret_cast<uint4*>(smem + tM1 + sw_chunk(tid, q4 * 4 + j)) =
                    make_uint4(pk1[4 * j], pk1[4 * j + 1], pk1[4 * j + 2], pk1[4 * j + 3]);
                *reinterpret_cast<uint4*>(smem + tM2 + sw_chunk(tid, q4 * 4 + j)) =
                    make_uint4(pk2[4 * j], pk2[4 * j + 1], pk2[4 * j + 2], pk2[4 * j + 3]);
            }
        };
        for (int q4 = 2 * half; q4 < 2 * half + 2; ++q4) {
            if (q4 > warp) {  // wholly above the diagonal for every row of this warp
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    *reinterpret_cast<uint4*>(smem + tM1 + sw_chunk(tid, q4 * 4 + j)) = zero4;
                    *reinterpret_cast<uint4*>(smem + tM2 + sw_chunk(tid, q4 * 4 + j)) = zero4;
                }
            } else if (q4 == warp) {
                mask_block(std::true_type{}, q4);
            } else {
                mask_block(std::false_type{}, q4);
            }
        }
        if ((tid >> 6) == half) {  // the diagonal lies in this thread's columns
            gdv[tid] = row_ok ? gd : 0.0f;
            pdv[tid] = row_ok ? pd : 0.0f;
        }
        if (has_sin) {  // <Q_t, R'_t> (E_t is already inside R')
            for (int q4 = 2 * half; q4 < 2 * half + 2; ++q4) {
                float rv[32];
                tmem_ld32(lane_addr + c2 + q4 * 32, rv);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 qv = *reinterpret_cast<const uint4*>(smem + tQ + sw_chunk(tid, q4 * 4 + j));
                    const uint32_t w4[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float2 f = unpack2<Th>(w4[u]);
                        qr = fmaf(f.x, rv[8 * j + 2 * u], qr);
                        qr = fmaf(f.y, rv[8 * j + 2 * u + 1], qr);
                    }
                }
            }
        }
        if (has_ds) {
            {
                const int q2 = half;
                float wv[32], dv[32];
                // W row s = tid -> w_s W;  dS^T row n = tid
                tmem_ld32x2(lane_addr + c3 + q2 * 32, wv, lane_addr + cDS + q2 * 32, dv);
#pragma unroll
                for (int i = 0; i < 32; ++i) wv[i] *= w_t;
                tmem_st32(lane_addr + c3 + q2 * 32, wv);
                if (has_sin) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 sv = *reinterpret_cast<const uint4*>(smem + kSin + sw_chunk(tid, q2 * 4 + j));
                        const uint32_t w4[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float2 f = unpack2<Th>(w4[u]);
                            ds_part = fmaf(f.x, dv[8 * j + 2 * u], ds_part);
                            ds_part = fmaf(f.y, dv[8 * j + 2 * u + 1], ds_part);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) dv[i] *= e_end;
                tmem_st32(lane_addr + cDS + q2 * 32, dv);
            }
        }
        fence_proxy_async();
        fence_before();
        __syncthreads();
        // ---- group 2 ----
        if (threadIdx.x == 0) {
            fence_after();
            const uint32_t idKK = instr_desc(fmt, 0, 0, 128), idQ = instr_desc(fmt, 0, 1, 128),
                           idV = instr_desc(fmt, 1, 1, 64);
#pragma unroll
            for (int k = 0; k < NS / 16; ++k)  // G^T[s][t]
                mma(tmem + c0, desc_sw_k(sbase + tK, k), desc_sw_k(sbase + tQ, k), idKK, k > 0);
#pragma unroll
            for (int k = 0; k < HD / 16; ++k)  // P^T[s][t]
                mma(tmem + c1, desc_sw_k(sbase + kV, k), desc_sw_k(sbase + kDY, k), idKK, k > 0);
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // dQ[t][n] (+)= sum_s M1[t][s] K[s][n]
                mma(tmem + c2, desc_sw_k(sbase + tM1, k), desc_sw_mn(sbase + tK, k), idQ, has_sin || k > 0);
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // dV[s][p] (+)= sum_t M2[t][s] dY[t][p]
                mma(tmem + c3, desc_sw_mn(sbase + tM2, k), desc_sw_mn(sbase + kDY, k), idV, has_ds || k > 0);
            commit(&bars[1]);
        }
        wait_bar(1);
        // ---- epilogue 2 ----
        gd = gdv[tid];
        pd = pdv[tid];
        float dsc = 0.0f;
        auto colsum_block = [&](auto diag_tag, int q4) {
            constexpr bool DIAG = decltype(diag_tag)::value;
            float gv[32], pv[32];
            tmem_ld32x2(lane_addr + c0 + q4 * 32, gv, lane_addr + c1 + q4 * 32, pv);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 da4 = *reinterpret_cast<const float4*>(dAl + q4 * 32 + i);
                const float dav[4] = {da4.x, da4.y, da4.z, da4.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float f = ex2(dav[u] - dAl_t);
                    if (DIAG && q4 * 32 + i + u <= tid) f = 0.0f;
                    dsc = fmaf(f * gv[i + u], pv[i + u], dsc);
                }
            }
        };
        for (int q4 = 2 * half; q4 < 2 * half + 2; ++q4) {  // only later steps (tt > s) contribute
            if (q4 == warp) colsum_block(std::true_type{}, q4);
            else if (q4 > warp) colsum_block(std::false_type{}, q4);
        }
        {
            const float gp = g_t * pd;  // gamma_t P_tt
            for (int q4 = 2 * half; q4 < 2 * half + 2; ++q4) {
                float av[32];
                tmem_ld32(lane_addr + c2 + q4 * 32, av);
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 kv = *reinterpret_cast<const uint4*>(smem + tK + sw_chunk(tid, q4 * 4 + j));
                        const uint32_t w4[4] = {kv.x, kv.y, kv.z, kv.w};
                        float o[8];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float2 f = unpack2<Th>(w4[u]);
                            o[2 * u] = fmaf(gp, f.x, av[8 * j + 2 * u]);
                            o[2 * u + 1] = fmaf(gp, f.y, av[8 * j + 2 * u + 1]);
                        }
                        if (q4 * 32 + 8 * j < nsv) store8(p.dQ + qk_row + q4 * 32 + 8 * j, o, p.wide_st != 0);
                    }
                }
            }
            const float dcoef = fmaf(g_t, gd, Dv);  // gamma_s G_ss + D
            {
                const int q2 = half;
                float av[32];
                tmem_ld32(lane_addr + c3 + q2 * 32, av);
                if (row_ok) {
                    uint4 ox[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 yv = *reinterpret_cast<const uint4*>(smem + kDY + sw_chunk(tid, q2 * 4 + j));
                        const uint32_t w4[4] = {yv.x, yv.y, yv.z, yv.w};
                        uint32_t o[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float2 f = unpack2<Th>(w4[u]);
                            o[u] = pack2<Th>(fmaf(dcoef, f.x, av[8 * j + 2 * u]), fmaf(dcoef, f.y, av[8 * j + 2 * u + 1]));
                        }
                        ox[j] = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    if (p.wide_dx) {  // headdim a multiple of 16, dx 32-byte aligned
#pragma unroll
                        for (int j = 0; j < 4; j += 2)
                            if (q2 * 32 + 8 * j < hdv) store32b(dxg + x_row + q2 * 32 + 8 * j, ox[j], ox[j + 1], true);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (q2 * 32 + 8 * j < hdv) *reinterpret_cast<uint4*>(dxg + x_row + q2 * 32 + 8 * j) = ox[j];
                    }
                }
            }
        }
        fence_before();
        __syncthreads();
        // ---- group 3 ----
        if (threadIdx.x == 0) {
            fence_after();
            const uint32_t idK = instr_desc(fmt, 1, 1, 128), idU = instr_desc(fmt, 0, 0, 128),
                           idS = instr_desc(fmt, 1, 1, 64);
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // dK[s][n] = sum_t M1[t][s] Q[t][n]
                mma(tmem + c0, desc_sw_mn(sbase + tM1, k), desc_sw_mn(sbase + tQ, k), idK, k > 0);
            if (has_ds) {
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)  // U[s][n] = sum_p V[s][p] dS^T[n][p]
                    mma(tmem + c1, desc_sw_k(sbase + kV, k), desc_sw_k(sbase + kDS, k), idU, k > 0);
            }
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // dS^T[n][p] (+)= sum_t Q[t][n] (E dY)[t][p]
                mma(tmem + cDS, desc_sw_mn(sbase + tQ, k), desc_sw_mn(sbase + kEdY, k), idS, has_ds || k > 0);
            commit(&bars[2]);
        }
        wait_bar(2);
        if (threadIdx.x == 0 && c > 0) request_tiles(c - 1, tM1, tM2);
        // ---- epilogue 3 ----
        // 16-bit copy of the new dS for the next (earlier) chunk
        if (c > 0) {
            {
                const int q2 = half;
                float sv[32];
                tmem_ld32(lane_addr + cDS + q2 * 32, sv);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(smem + kDS + sw_chunk(tid, q2 * 4 + j)) =
                        make_uint4(pack2<Th>(sv[8 * j], sv[8 * j + 1]), pack2<Th>(sv[8 * j + 2], sv[8 * j + 3]),
                                   pack2<Th>(sv[8 * j + 4], sv[8 * j + 5]), pack2<Th>(sv[8 * j + 6], sv[8 * j + 7]));
            }
        }
        // The proxy fence this copy needs comes before the dK rows are stored: a fence waits for
        // the thread's outstanding global stores, and stored after it the 64 KB of dK drain
        // under the next chunk's tile copies instead of at the end of this one.
        fence_proxy_async();
        float zw = 0.0f;  // w_s <K_s, U_s>
        {
            const float gp = g_t * pd;
            for (int q4 = 2 * half; q4 < 2 * half + 2; ++q4) {
                float av[32], uv[32];
                if (has_ds) tmem_ld32x2(lane_addr + c0 + q4 * 32, av, lane_addr + c1 + q4 * 32, uv);
                else tmem_ld32(lane_addr + c0 + q4 * 32, av);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 qv = *reinterpret_cast<const uint4*>(smem + tQ + sw_chunk(tid, q4 * 4 + j));
                    const uint4 kv = *reinterpret_cast<const uint4*>(smem + tK + sw_chunk(tid, q4 * 4 + j));
                    const uint32_t q4w[4] = {qv.x, qv.y, qv.z, qv.w};
                    const uint32_t k4w[4] = {kv.x, kv.y, kv.z, kv.w};
                    float o[8];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float2 fq = unpack2<Th>(q4w[u]);
                        const float2 fk = unpack2<Th>(k4w[u]);
                        float o0 = fmaf(gp, fq.x, av[8 * j + 2 * u]), o1 = fmaf(gp, fq.y, av[8 * j + 2 * u + 1]);
                        if (has_ds) {
                            const float u0 = w_t * uv[8 * j + 2 * u], u1 = w_t * uv[8 * j + 2 * u + 1];
                            o0 += u0;
                            o1 += u1;
                            zw = fmaf(fk.x, u0, zw);
                            zw = fmaf(fk.y, u1, zw);
                        }
                        o[2 * u] = o0;
                        o[2 * u + 1] = o1;
                    }
                    if (row_ok && q4 * 32 + 8 * j < nsv) store8(p.dK + qk_row + q4 * 32 + 8 * j, o, p.wide_st != 0);
                }
            }
        }
        // ---- per-step scalars ----
        if (!row_ok) zw = 0.0f;
        // fold the upper-half threads' partial sums into the lower-half thread of the row
        if (half == 1) {
            part[tid] = rowX; part[128 + tid] = qr; part[256 + tid] = dsc; part[384 + tid] = zw; part[512 + tid] = ds_part;
        }
        __syncthreads();
        if (half == 0) {
            rowX += part[tid]; qr += part[128 + tid]; dsc += part[256 + tid]; zw += part[384 + tid]; ds_part += part[512 + tid];
        }
        const float sum_zw = block_sum(half == 0 ? zw : 0.0f);
        const float ds_dot = block_sum(half == 0 ? ds_part : 0.0f);
        float v = (row_ok && half == 0) ? rowX - s_t * dsc + qr - zw : 0.0f;
        if (tid == nv - 1 && half == 0) v += sum_zw + e_end * ds_dot;
        // d(adt_r) = sum_{t >= r} d(dA_t): reverse inclusive scan over the CTA
        float rs = v;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const float o = __shfl_down_sync(0xffffffffu, rs, m);
            if (lane + m < 32) rs += o;
        }
        __syncthreads();
        if (lane == 0 && half == 0) red[warp] = rs;
        __syncthreads();
        for (int w = warp + 1; w < 4; ++w) rs += red[w];
        if (row_ok && half == 0) {
            const long long th = (static_cast<long long>(b) * T + t) * nh + h;
            p.d_adt[th] = rs;
            p.ws_dgam[th] = gd * pd;
            p.ws_dscl[th] = dsc + (s_t > 0.0f ? zw / s_t : 0.0f);
            dD_acc += pd;
        }
        has_ds = true;
        fence_before();
        __syncthreads();
        fence_after();
    }
    {
        const float tot = block_sum(half == 0 ? dD_acc : 0.0f);
        if (threadIdx.x == 0) p.ws_dD[static_cast<long long>(b) * nh + h] = tot;
    }
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    (void)ok;
}

}  // namespace tcb

static size_t m3_bwd_smem(int hd, int N) {
    const size_t LQ = N + 1, LV = hd + 1, LG = kM3C + 1;
    return sizeof(float) * (3 * kM3C * LQ + 3 * kM3C * LV + 2 * kM3C * LG + 2 * hd * LQ + 12 * 32);
}

// Tensor-core geometry: 16-bit storage, headdim <= 64, d_state <= 128, both multiples of 8.
static bool m3_bwd_tc_shape(int dtype, int hd, int N) {
    return dtype != MAMBA_B200_F32 && hd <= tcb::HD && hd % 8 == 0 && N <= tcb::NS && N % 8 == 0;
}

// States first (f32 every 32 steps for the CUDA-core kernel; 16-bit tiles every 128
// steps for the tensor-core kernel), then dgamma, dscale [B,T,nh] and dD partials.
static void m3_bwd_ws(bool tc, int B, int T, int nh, int hd, int N, size_t* o_g, size_t* o_s, size_t* o_d,
                      size_t* total) {
    const size_t nc = (T + kM3C - 1) / kM3C;
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t st = tc ? al(static_cast<size_t>(B) * nh * ((T + tcb::CS - 1) / tcb::CS) * tcb::kStateTile)
                         : al(sizeof(float) * static_cast<size_t>(B) * nh * nc * hd * N);
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
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(tcb::m3_ssd_bwd_tc_kernel<__half>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, tcb::kSmem));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(tcb::m3_ssd_bwd_tc_kernel<__nv_bfloat16>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, tcb::kSmem));
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API long long mamba_b200_m3_ssd_bwd_workspace_bytes(int B, int T, int nh, int hd, int N) {
    if (B <= 0 || T <= 0 || nh <= 0 || hd <= 0 || N <= 0) return 0;
    size_t a, b2, d, total;
    m3_bwd_ws(false, B, T, nh, hd, N, &a, &b2, &d, &total);
    return static_cast<long long>(total);
}

extern "C" MAMBA_B200_API long long mamba_b200_m3_ssd_bwd_workspace_bytes_for(int dtype, int B, int T, int nh,
                                                                              int hd, int N) {
    if (B <= 0 || T <= 0 || nh <= 0 || hd <= 0 || N <= 0) return 0;
    size_t a, b2, d, total;
    m3_bwd_ws(m3_bwd_tc_shape(dtype, hd, N), B, T, nh, hd, N, &a, &b2, &d, &total);
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
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    M3BwdParams p;
    memset(&p, 0, sizeof(p));
    // the tensor-core kernel needs its four tile maps; without them (no encoder, a stride beyond
    // its range) the CUDA-core kernel takes the call
    const bool tensor_core = m3_bwd_tc_shape(a.dtype, a.hd, a.N) && al16(a.x) && al16(a.K) &&
                             al16(a.Q) && al16(a.dy) && al16(a.dx) && al16(a.dK) && al16(a.dQ) &&
                             make_tmap_head_tile(c, &p.tm_q, a.dtype, a.Q, a.N, a.nh, a.T, a.B) &&
                             make_tmap_head_tile(c, &p.tm_k, a.dtype, a.K, a.N, a.nh, a.T, a.B) &&
                             make_tmap_head_tile(c, &p.tm_x, a.dtype, a.x, a.hd, a.nh, a.T, a.B) &&
                             make_tmap_head_tile(c, &p.tm_dy, a.dtype, a.dy, a.hd, a.nh, a.T, a.B);
    size_t o_g, o_s, o_d, total;
    // a misaligned tensor-core-shaped call falls back to the CUDA-core kernel and its larger scratch
    m3_bwd_ws(tensor_core, a.B, a.T, a.nh, a.hd, a.N, &o_g, &o_s, &o_d, &total);
    if (a.workspace_bytes < static_cast<long long>(total))
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: workspace %lld < %zu bytes", a.workspace_bytes, total);
    if (reinterpret_cast<uintptr_t>(a.workspace) % 256)
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_bwd: workspace must be 256-byte aligned");
    p.x = a.x; p.K = a.K; p.Q = a.Q; p.dy = a.dy; p.dt = a.dt; p.trap = a.trap; p.adt = a.adt; p.Dh = a.Dh;
    p.dx = a.dx; p.dK = a.dK; p.dQ = a.dQ; p.d_adt = a.d_adt; p.d_dt = a.d_dt; p.d_trap = a.d_trap; p.dD = a.dD;
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    p.ws_states = reinterpret_cast<float*>(ws);
    p.ws_dgam = reinterpret_cast<float*>(ws + o_g);
    p.ws_dscl = reinterpret_cast<float*>(ws + o_s);
    p.ws_dD = reinterpret_cast<float*>(ws + o_d);
    p.B = a.B; p.T = a.T; p.nh = a.nh; p.hd = a.hd; p.N = a.N;
    p.status = c->d_status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(a.nh, a.B);
    const size_t smem = m3_bwd_smem(a.hd, a.N);
    if (tensor_core) {
        p.wide_st = (reinterpret_cast<uintptr_t>(a.dK) | reinterpret_cast<uintptr_t>(a.dQ)) % 32 == 0;
        p.wide_dx = a.hd % 16 == 0 && reinterpret_cast<uintptr_t>(a.dx) % 32 == 0;
        p.sc_tma = a.nh % 4 == 0 &&
                   make_tmap_3d(c, &p.tm_adt, MAMBA_B200_F32, a.adt, a.nh, a.nh, a.T, a.B, 4, 129) &&
                   make_tmap_3d(c, &p.tm_dt, MAMBA_B200_F32, a.dt, a.nh, a.nh, a.T, a.B, 4, 129) &&
                   make_tmap_3d(c, &p.tm_trap, MAMBA_B200_F32, a.trap, a.nh, a.nh, a.T, a.B, 4, 129);
        if (a.dtype == MAMBA_B200_F16) tcb::m3_ssd_bwd_tc_kernel<__half><<<grid, 256, tcb::kSmem, st>>>(p);
        else tcb::m3_ssd_bwd_tc_kernel<__nv_bfloat16><<<grid, 256, tcb::kSmem, st>>>(p);
    } else if (a.dtype == MAMBA_B200_F32) m3_ssd_bwd_kernel<float><<<grid, 256, smem, st>>>(p);
    else if (a.dtype == MAMBA_B200_F16) m3_ssd_bwd_kernel<__half><<<grid, 256, smem, st>>>(p);
    else m3_ssd_bwd_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    const long long total_e = static_cast<long long>(a.B) * a.T * a.nh;
    m3_bwd_finish_kernel<<<static_cast<unsigned>((total_e + 255) / 256), 256, 0, st>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}
