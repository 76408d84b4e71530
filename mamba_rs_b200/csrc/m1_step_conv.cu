// Decode step (T = 1) and the standalone depthwise causal conv1d kernels.
//
// All three are memory-bound streaming kernels: lanes map to consecutive
// channels so every global access is a contiguous row segment, the conv window
// lives in registers, and each element of x / u / d_u / d_x is read or written
// once (plus a K-1 row halo per time chunk).
#include <string.h>

#include <atomic>
#include <initializer_list>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

constexpr int kStepKMax = 8;

// ---------------------------------------------------------------------------
// T = 1: conv step + SiLU, softplus(delta), SSM step, D skip, gate.
// Replaces conv1d_step_forward_silu_{dt} (kernels/conv1d.cu:85-115), the
// softplus pass and ssm_step_forward_gather_gate_{dt} (kernels/mamba_ssm.cu:180-227).
// ---------------------------------------------------------------------------
struct StepParams {
    const void *x, *dl, *bm, *cm, *z;
    void *y, *u_out;
    long long ld_x, ld_dl, ld_bc, ld_z, ld_y, ld_u;
    const float *a_neg, *Dp, *conv_w, *conv_b;
    float *conv_state, *ssm_state;
    int B, D, N, K, delta_softplus, z_mode;
    int vec_state;  // a_neg and ssm_state rows may be moved as float4 (N % 4 == 0, 16-byte aligned bases)
};

template <typename Tact>
__global__ void __launch_bounds__(128) sscan_step_kernel(const StepParams p) {
    const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (idx >= static_cast<long long>(p.B) * p.D) return;
    const int b = static_cast<int>(idx / p.D), d = static_cast<int>(idx % p.D);
    const Tact* x = static_cast<const Tact*>(p.x);
    float u = to_f(x[b * p.ld_x + d]);
    if (p.conv_w) {
        // shift, insert, bias-first dot product (kernels/conv1d.cu:100-112)
        float* st = p.conv_state + (static_cast<long long>(b) * p.D + d) * p.K;
        float win[kStepKMax];
        for (int k = 0; k + 1 < p.K; ++k) win[k] = st[k + 1];
        win[p.K - 1] = u;
        float acc = p.conv_b[d];
        for (int k = 0; k < p.K; ++k) {
            acc = fmaf(win[k], p.conv_w[static_cast<long long>(d) * p.K + k], acc);
            st[k] = win[k];
        }
        u = siluf_fast(acc);
        if (p.u_out) static_cast<Tact*>(p.u_out)[b * p.ld_u + d] = from_f<Tact>(u);
    }
    float dl = to_f(static_cast<const Tact*>(p.dl)[b * p.ld_dl + d]);
    if (p.delta_softplus) dl = softplusf_fast(dl);
    const float du = dl * u;
    const Tact* Bv = static_cast<const Tact*>(p.bm) + b * p.ld_bc;
    const Tact* Cv = static_cast<const Tact*>(p.cm) + b * p.ld_bc;
    float* h = p.ssm_state + (static_cast<long long>(b) * p.D + d) * p.N;
    const float* a = p.a_neg + static_cast<long long>(d) * p.N;
    float y = 0.0f;
    int n = 0;
    if (p.vec_state) {
        for (; n < p.N; n += 4) {
            float4 hv = *reinterpret_cast<float4*>(h + n);
            const float4 av = *reinterpret_cast<const float4*>(a + n);
            hv.x = fmaf(ex2(dl * av.x * kLog2e), hv.x, du * to_f(Bv[n]));
            hv.y = fmaf(ex2(dl * av.y * kLog2e), hv.y, du * to_f(Bv[n + 1]));
            hv.z = fmaf(ex2(dl * av.z * kLog2e), hv.z, du * to_f(Bv[n + 2]));
            hv.w = fmaf(ex2(dl * av.w * kLog2e), hv.w, du * to_f(Bv[n + 3]));
            y = fmaf(hv.x, to_f(Cv[n]), y);
            y = fmaf(hv.y, to_f(Cv[n + 1]), y);
            y = fmaf(hv.z, to_f(Cv[n + 2]), y);
            y = fmaf(hv.w, to_f(Cv[n + 3]), y);
            *reinterpret_cast<float4*>(h + n) = hv;
        }
    }
    for (; n < p.N; ++n) {
        const float hn = fmaf(ex2(dl * a[n] * kLog2e), h[n], du * to_f(Bv[n]));
        h[n] = hn;
        y = fmaf(hn, to_f(Cv[n]), y);
    }
    y = fmaf(p.Dp[d], u, y);
    if (p.z_mode) {
        const float zv = to_f(static_cast<const Tact*>(p.z)[b * p.ld_z + d]);
        y *= p.z_mode == 1 ? siluf_fast(zv) : zv;
    }
    static_cast<Tact*>(p.y)[b * p.ld_y + d] = from_f<Tact>(y);
}

// ---------------------------------------------------------------------------
// Sequence conv1d + SiLU forward.  Replaces conv1d_burnin_forward[_nosave]_{dt}
// (kernels/conv1d.cu:161-359).  grid = (channel tiles, time chunks, B).
// ---------------------------------------------------------------------------
constexpr int kConvTT = 64;  // timesteps per thread

struct ConvParams {
    const void *x, *du;
    void *u, *dx;
    long long ld_x, ld_u, ld_du, ld_dx;
    const float *w, *bias;
    const float* state_in;  // entering window [B,D,K] or null (zeros)
    float* state_out;       // window after the sequence [B,D,K] or null (may alias state_in)
    float* part;            // backward: [B][chunks][D][K+1] partial dW | db
    int B, T, D, K;
};

// x[t] for t in [-K, T): negative t reads the entering window (slot K + t).
template <typename Tact>
__device__ __forceinline__ float conv_x_at(const ConvParams& p, const Tact* xb, int b, int d, int t) {
    if (t >= 0) return to_f(xb[static_cast<long long>(t) * p.ld_x]);
    return p.state_in ? p.state_in[(static_cast<long long>(b) * p.D + d) * p.K + p.K + t] : 0.0f;
}

template <typename Tact>
__global__ void __launch_bounds__(128) conv1d_fwd_kernel(const ConvParams p) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = blockIdx.y * kConvTT, b = blockIdx.z;
    if (d >= p.D) return;
    const int K = p.K;
    const Tact* xb = static_cast<const Tact*>(p.x) + static_cast<long long>(b) * p.T * p.ld_x + d;
    Tact* ub = static_cast<Tact*>(p.u) + static_cast<long long>(b) * p.T * p.ld_u + d;
    float w[kStepKMax], win[kStepKMax];
#pragma unroll
    for (int k = 0; k < kStepKMax; ++k) {
        w[k] = k < K ? p.w[static_cast<long long>(d) * K + k] : 0.0f;
        // window right-aligned in win[kStepKMax-K .. kStepKMax): history before t0
        const int kk = k - (kStepKMax - K);
        win[k] = kk >= 0 ? conv_x_at(p, xb, b, d, t0 - K + kk) : 0.0f;
    }
    const float bias = p.bias[d];
    const int t1 = min(p.T, t0 + kConvTT);
    for (int t = t0; t < t1; ++t) {
#pragma unroll
        for (int k = 0; k < kStepKMax - 1; ++k) win[k] = win[k + 1];
        win[kStepKMax - 1] = to_f(xb[static_cast<long long>(t) * p.ld_x]);
        float acc = bias;
#pragma unroll
        for (int k = 0; k < kStepKMax; ++k) {
            const int kk = k - (kStepKMax - K);
            if (kk >= 0) acc = fmaf(win[k], w[kk], acc);
        }
        ub[static_cast<long long>(t) * p.ld_u] = from_f<Tact>(siluf_fast(acc));
    }
}

// Window after the sequence: the last K inputs (older slots come from the
// entering window when T < K).  Runs after the forward kernel, which reads the
// entering window, so updating the state in place cannot race with it.
template <typename Tact>
__global__ void conv1d_state_kernel(const ConvParams p) {
    const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (idx >= static_cast<long long>(p.B) * p.D) return;
    const int b = static_cast<int>(idx / p.D), d = static_cast<int>(idx % p.D);
    const Tact* xb = static_cast<const Tact*>(p.x) + static_cast<long long>(b) * p.T * p.ld_x + d;
    float nw[kStepKMax];
    for (int k = 0; k < p.K; ++k) nw[k] = conv_x_at(p, xb, b, d, p.T - p.K + k);
    float* so = p.state_out + (static_cast<long long>(b) * p.D + d) * p.K;
    for (int k = 0; k < p.K; ++k) so[k] = nw[k];
}

// ---------------------------------------------------------------------------
// conv1d + SiLU backward by recomputation.  Replaces conv1d_burnin_backward_{dt}
// and its two reduce_sum_axis0 launches (kernels/conv1d.cu:373-515,
// kernels/elementwise.cu:89-114).  d_x[t] = sum_k w[k] dco[t + K-1-k],
// dco = d_u * SiLU'(conv pre-activation); dW / db partials per (b, time chunk).
// ---------------------------------------------------------------------------
template <typename Tact>
__global__ void __launch_bounds__(128) conv1d_bwd_kernel(const ConvParams p) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    const int chunk = blockIdx.y, t0 = chunk * kConvTT, b = blockIdx.z;
    if (d >= p.D) return;
    const int K = p.K, T = p.T;
    const Tact* xb = static_cast<const Tact*>(p.x) + static_cast<long long>(b) * T * p.ld_x + d;
    const Tact* gb = static_cast<const Tact*>(p.du) + static_cast<long long>(b) * T * p.ld_du + d;
    Tact* dxb = static_cast<Tact*>(p.dx) + static_cast<long long>(b) * T * p.ld_dx + d;
    float w[kStepKMax], win[kStepKMax], dco[kStepKMax], dW[kStepKMax];
#pragma unroll
    for (int k = 0; k < kStepKMax; ++k) {
        w[k] = k < K ? p.w[static_cast<long long>(d) * K + k] : 0.0f;
        dco[k] = 0.0f;
        dW[k] = 0.0f;
    }
    const float bias = p.bias[d];
    float db = 0.0f;
    const int t1 = min(T, t0 + kConvTT);
    // Walk backwards from t1 + K - 2 (future steps whose dco reaches into this
    // chunk) down to t0.  win holds x[t-K+1 .. t] right-aligned; dco[j] holds
    // dco[t + j + 1] for the K-1 steps ahead of t.
    const int t_start = min(T - 1, t1 + K - 2);
#pragma unroll
    for (int k = 0; k < kStepKMax; ++k) {
        const int kk = k - (kStepKMax - K);
        win[k] = kk >= 0 ? conv_x_at(p, xb, b, d, t_start - (K - 1) + kk) : 0.0f;
    }
    for (int t = t_start; t >= t0; --t) {
        float acc = bias;
#pragma unroll
        for (int k = 0; k < kStepKMax; ++k) {
            const int kk = k - (kStepKMax - K);
            if (kk >= 0) acc = fmaf(win[k], w[kk], acc);
        }
        const float sg = sigmoidf_fast(acc);
        const float g = to_f(gb[static_cast<long long>(t) * p.ld_du]) * sg * fmaf(acc, 1.0f - sg, 1.0f);
        if (t < t1) {
            db += g;
            float dx = g * w[K - 1];
#pragma unroll
            for (int k = 0; k < kStepKMax; ++k) {
                const int kk = k - (kStepKMax - K);
                if (kk >= 0) dW[kk] = fmaf(g, win[k], dW[kk]);
            }
            // future steps: dco[j] = dco[t + 1 + j] meets tap K-2-j
#pragma unroll
            for (int j = 0; j < kStepKMax - 1; ++j)
                if (j < K - 1) dx = fmaf(dco[j], w[K - 2 - j], dx);
            dxb[static_cast<long long>(t) * p.ld_dx] = from_f<Tact>(dx);
        }
#pragma unroll
        for (int j = kStepKMax - 1; j > 0; --j) dco[j] = dco[j - 1];
        dco[0] = g;
        // slide the window one step back in time
#pragma unroll
        for (int k = kStepKMax - 1; k > 0; --k) win[k] = win[k - 1];
        win[kStepKMax - K] = conv_x_at(p, xb, b, d, t - K);
    }
    const int chunks = gridDim.y;
    float* pt = p.part + ((static_cast<long long>(b) * chunks + chunk) * p.D + d) * (K + 1);
    for (int k = 0; k < K; ++k) pt[k] = dW[k];
    pt[K] = db;
}

// ---------------------------------------------------------------------------
// Vector variants (d_conv <= 4, rows and pointers aligned to the vector): a
// thread owns VEC adjacent channels and moves them with one 4- to 16-byte access
// per step, kConvUnr steps of loads in flight.  Same arithmetic, in the same
// order per channel, as the scalar kernels above.  The defaults (8-byte accesses
// forward, 2 channels backward, 32-step forward chunks, 2 steps in flight) are the
// fastest of the combinations timed at B 16, L 2048, D 1536, bf16: wider vectors
// and deeper unrolling cost more in registers (occupancy) than they save.
// ---------------------------------------------------------------------------
constexpr int kConvKV = 4;     // widest d_conv of the vector kernels
constexpr int kConvFwdTT = 32;      // timesteps per thread, forward
constexpr int kConvUnr = 2;         // steps of loads in flight per thread
constexpr int kConvFwdBytes = 8;    // bytes one forward thread moves per step
// (a backward thread owns 2 channels with 16-bit storage, 4 with f32)

template <typename Tact, int VEC>
__device__ __forceinline__ void load_vec(const Tact* ptr, float* out) {
    constexpr int BYTES = sizeof(Tact) * VEC;
    static_assert(BYTES == 16 || BYTES == 8 || BYTES == 4, "vector access of 4, 8 or 16 bytes");
    uint32_t w[BYTES / 4];
    if constexpr (BYTES == 16) {
        const uint4 v = *reinterpret_cast<const uint4*>(ptr);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (BYTES == 8) {
        const uint2 v = *reinterpret_cast<const uint2*>(ptr);
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = *reinterpret_cast<const uint32_t*>(ptr);
    }
#pragma unroll
    for (int i = 0; i < BYTES / 4; ++i) {
        if (sizeof(Tact) == 4) {
            out[i] = __uint_as_float(w[i]);
        } else {
            const Tact* h = reinterpret_cast<const Tact*>(&w[i]);
            out[2 * i] = to_f(h[0]);
            out[2 * i + 1] = to_f(h[1]);
        }
    }
}
template <typename Tact, int VEC>
__device__ __forceinline__ void store_vec(Tact* ptr, const float* v) {
    constexpr int BYTES = sizeof(Tact) * VEC;
    __align__(16) Tact tmp[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) tmp[i] = from_f<Tact>(v[i]);
    if (BYTES == 16) *reinterpret_cast<uint4*>(ptr) = *reinterpret_cast<const uint4*>(tmp);
    else if (BYTES == 8) *reinterpret_cast<uint2*>(ptr) = *reinterpret_cast<const uint2*>(tmp);
    else *reinterpret_cast<uint32_t*>(ptr) = *reinterpret_cast<const uint32_t*>(tmp);
}

// Taps of VEC adjacent channels, right-aligned in KV slots (absent taps zero), and bias.
template <int VEC>
__device__ __forceinline__ void conv_load_taps(const ConvParams& p, int d, float (*w)[VEC], float* bias) {
    constexpr int KV = kConvKV;
    const int K = p.K;
    if (VEC % 4 == 0) {
#pragma unroll
        for (int v = 0; v + 3 < VEC; v += 4) {
            const float4 bv = *reinterpret_cast<const float4*>(p.bias + d + v);
            bias[v] = bv.x; bias[v + 1] = bv.y; bias[v + 2] = bv.z; bias[v + 3] = bv.w;
        }
    } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) bias[v] = p.bias[d + v];
    }
    if (K == KV) {  // one 16-byte load per channel
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const float4 wv = *reinterpret_cast<const float4*>(p.w + static_cast<long long>(d + v) * KV);
            w[0][v] = wv.x; w[1][v] = wv.y; w[2][v] = wv.z; w[3][v] = wv.w;
        }
    } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v)
#pragma unroll
            for (int k = 0; k < KV; ++k) {
                const int kk = k - (KV - K);
                w[k][v] = kk >= 0 ? p.w[static_cast<long long>(d + v) * K + kk] : 0.0f;
            }
    }
}

template <typename Tact>
__global__ void __launch_bounds__(64) conv1d_fwd_vec_kernel(const ConvParams p) {
    constexpr int VEC = kConvFwdBytes / sizeof(Tact), KV = kConvKV;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    const int t0 = blockIdx.y * kConvFwdTT, b = blockIdx.z;
    if (d >= p.D) return;
    const int K = p.K;
    const Tact* xb = static_cast<const Tact*>(p.x) + static_cast<long long>(b) * p.T * p.ld_x + d;
    Tact* ub = static_cast<Tact*>(p.u) + static_cast<long long>(b) * p.T * p.ld_u + d;
    // taps right-aligned: w[KV-1] meets x[t], absent taps are zero
    float w[KV][VEC], win[KV - 1][VEC], bias[VEC];
    conv_load_taps<VEC>(p, d, w, bias);
    if (t0 >= KV - 1) {  // history rows lie in x: whole-vector loads (absent taps have zero weight)
#pragma unroll
        for (int k = 0; k < KV - 1; ++k)
            load_vec<Tact, VEC>(xb + static_cast<long long>(t0 - (KV - 1) + k) * p.ld_x, win[k]);
    } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v)
#pragma unroll
            for (int k = 0; k < KV - 1; ++k)
                win[k][v] = k - (KV - K) >= 0 ? conv_x_at(p, xb + v, b, d + v, t0 - (KV - 1) + k) : 0.0f;
    }
    const int t1 = min(p.T, t0 + kConvFwdTT);
    for (int tb = t0; tb < t1; tb += kConvUnr) {
        float cur[kConvUnr][VEC];
#pragma unroll
        for (int i = 0; i < kConvUnr; ++i) {
            if (tb + i < t1) load_vec<Tact, VEC>(xb + static_cast<long long>(tb + i) * p.ld_x, cur[i]);
        }
#pragma unroll
        for (int i = 0; i < kConvUnr; ++i) {
            if (tb + i < t1) {
                float o[VEC];
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    float acc = bias[v];
#pragma unroll
                    for (int k = 0; k < KV - 1; ++k) acc = fmaf(win[k][v], w[k][v], acc);
                    acc = fmaf(cur[i][v], w[KV - 1][v], acc);
                    o[v] = siluf_fast(acc);
#pragma unroll
                    for (int k = 0; k < KV - 2; ++k) win[k][v] = win[k + 1][v];
                    win[KV - 2][v] = cur[i][v];
                }
                store_vec<Tact, VEC>(ub + static_cast<long long>(tb + i) * p.ld_u, o);
            }
        }
    }
}

template <typename Tact>
__global__ void __launch_bounds__(64) conv1d_bwd_vec_kernel(const ConvParams p) {
    constexpr int VEC = sizeof(Tact) == 2 ? 2 : 4, KV = kConvKV;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    const int chunk = blockIdx.y, t0 = chunk * kConvTT, b = blockIdx.z;
    if (d >= p.D) return;
    const int K = p.K, T = p.T;
    const Tact* xb = static_cast<const Tact*>(p.x) + static_cast<long long>(b) * T * p.ld_x + d;
    const Tact* gb = static_cast<const Tact*>(p.du) + static_cast<long long>(b) * T * p.ld_du + d;
    Tact* dxb = static_cast<Tact*>(p.dx) + static_cast<long long>(b) * T * p.ld_dx + d;
    // right-aligned taps as in the forward; win[k] = x[t - (KV-1) + k]
    float w[KV][VEC], win[KV][VEC], dco[KV - 1][VEC], dW[KV][VEC], bias[VEC], db[VEC];
    const int t1 = min(T, t0 + kConvTT);
    const int t_start = min(T - 1, t1 + K - 2);
    conv_load_taps<VEC>(p, d, w, bias);
    if (t_start >= KV - 1) {
#pragma unroll
        for (int k = 0; k < KV; ++k)
            load_vec<Tact, VEC>(xb + static_cast<long long>(t_start - (KV - 1) + k) * p.ld_x, win[k]);
    } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v)
#pragma unroll
            for (int k = 0; k < KV; ++k)
                win[k][v] = k - (KV - K) >= 0 ? conv_x_at(p, xb + v, b, d + v, t_start - (KV - 1) + k) : 0.0f;
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        db[v] = 0.0f;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            dW[k][v] = 0.0f;
            if (k < KV - 1) dco[k][v] = 0.0f;
        }
    }
    for (int tb = t_start; tb >= t0; tb -= kConvUnr) {
        // loads of four steps: d_u[t] and the input that enters the window when it
        // slides back past t (x[t - K], from the entering state when negative)
        float g4[kConvUnr][VEC], xin[kConvUnr][VEC];
#pragma unroll
        for (int i = 0; i < kConvUnr; ++i) {
            const int t = tb - i;
            if (t >= t0) {
                load_vec<Tact, VEC>(gb + static_cast<long long>(t) * p.ld_du, g4[i]);
                if (t - K >= 0) {
                    load_vec<Tact, VEC>(xb + static_cast<long long>(t - K) * p.ld_x, xin[i]);
                } else {
#pragma unroll
                    for (int v = 0; v < VEC; ++v) xin[i][v] = conv_x_at(p, xb + v, b, d + v, t - K);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kConvUnr; ++i) {
            const int t = tb - i;
            if (t >= t0) {
                float dxv[VEC];
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    float acc = bias[v];
#pragma unroll
                    for (int k = 0; k < KV; ++k) acc = fmaf(win[k][v], w[k][v], acc);
                    const float sg = sigmoidf_fast(acc);
                    const float g = g4[i][v] * sg * fmaf(acc, 1.0f - sg, 1.0f);
                    if (t < t1) {
                        db[v] += g;
                        float dx = g * w[KV - 1][v];
#pragma unroll
                        for (int k = 0; k < KV; ++k) dW[k][v] = fmaf(g, win[k][v], dW[k][v]);
                        // future steps: dco[j] = dco[t + 1 + j] meets tap KV-2-j
#pragma unroll
                        for (int j = 0; j < KV - 1; ++j) dx = fmaf(dco[j][v], w[KV - 2 - j][v], dx);
                        dxv[v] = dx;
                    }
#pragma unroll
                    for (int j = KV - 2; j > 0; --j) dco[j][v] = dco[j - 1][v];
                    dco[0][v] = g;
#pragma unroll
                    for (int k = KV - 1; k > 0; --k) win[k][v] = win[k - 1][v];
                    // x[t - K] enters at the oldest tap that exists (slot KV - K)
#pragma unroll
                    for (int k = 0; k < KV; ++k)
                        if (k == KV - K) win[k][v] = xin[i][v];
                }
                if (t < t1) store_vec<Tact, VEC>(dxb + static_cast<long long>(t) * p.ld_dx, dxv);
            }
        }
    }
    const int chunks = gridDim.y;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        float* pt = p.part + ((static_cast<long long>(b) * chunks + chunk) * p.D + d + v) * (K + 1);
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int kk = k - (KV - K);
            if (kk >= 0) pt[kk] = dW[k][v];
        }
        pt[K] = db[v];
    }
}

// ---------------------------------------------------------------------------
// conv1d + SiLU backward from shared-memory tiles (16-bit storage, d_conv <= 4, rows on
// 16-byte boundaries).  The register kernels above are bound by instruction issue and load
// latency (146 warp-instructions per step of two channels, each thread waiting on its own
// 4-byte loads); here a CTA of 128 threads first brings the x and d_u rows of its 64 steps
// (plus the halo) into shared memory with 16-byte loads that are all in flight together, then
// thread = channel walks the steps out of shared memory with the same arithmetic in the same
// order, and d_x leaves through a tile and 16-byte stores.
// ---------------------------------------------------------------------------
constexpr int kConvTileD = 128;
constexpr int kConvTileXRows = kConvTT + 2 * kConvKV - 1;  // x[t0 - K .. t1 + K - 2]
constexpr int kConvTileGRows = kConvTT + kConvKV - 1;      // d_u[t0 .. t1 + K - 2]
template <typename Tact>
constexpr size_t conv_tile_smem() {
    return sizeof(Tact) * kConvTileD * (kConvTileXRows + kConvTileGRows + kConvTT) + sizeof(float) * kConvKV * kConvTileD;
}

template <typename Tact>
__global__ void __launch_bounds__(kConvTileD) conv1d_bwd_tile_kernel(const ConvParams p) {
    static_assert(sizeof(Tact) == 2, "16-bit storage");
    constexpr int KV = kConvKV, DT = kConvTileD, PIECES = DT / 8;  // 16-byte pieces per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Tact* xs = reinterpret_cast<Tact*>(smem_raw);            // [kConvTileXRows][DT], row r = step xt0 + r
    Tact* gs = xs + kConvTileXRows * DT;                     // [kConvTileGRows][DT], row r = step t0 + r
    Tact* dxs = gs + kConvTileGRows * DT;                    // [kConvTT][DT]
    float* xneg = reinterpret_cast<float*>(dxs + kConvTT * DT);  // [K][DT]: x[-K .. -1] (chunk 0 only)
    const int d0 = blockIdx.x * DT, chunk = blockIdx.y, t0 = chunk * kConvTT, b = blockIdx.z;
    const int K = p.K, T = p.T, D = p.D;
    const int t1 = min(T, t0 + kConvTT), t_start = min(T - 1, t1 + K - 2);
    // row r of xs is step xt0 + r; rows of negative steps (first chunk) stay unused
    const int xt0 = t0 - K, nx = t_start - xt0 + 1, ng = t_start - t0 + 1;
    const Tact* xb = static_cast<const Tact*>(p.x) + static_cast<long long>(b) * T * p.ld_x + d0;
    const Tact* gb = static_cast<const Tact*>(p.du) + static_cast<long long>(b) * T * p.ld_du + d0;
    Tact* dxb = static_cast<Tact*>(p.dx) + static_cast<long long>(b) * T * p.ld_dx + d0;
    const int tid = threadIdx.x;
    const uint4 z4 = make_uint4(0, 0, 0, 0);
    for (int i = tid; i < nx * PIECES; i += DT) {
        const int r = i / PIECES, pc = i - r * PIECES;
        const bool in = d0 + pc * 8 < D && xt0 + r >= 0;
        reinterpret_cast<uint4*>(xs)[i] = in ? *reinterpret_cast<const uint4*>(xb + static_cast<long long>(xt0 + r) * p.ld_x + pc * 8) : z4;
    }
    for (int i = tid; i < ng * PIECES; i += DT) {
        const int r = i / PIECES, pc = i - r * PIECES;
        const bool in = d0 + pc * 8 < D;
        reinterpret_cast<uint4*>(gs)[i] = in ? *reinterpret_cast<const uint4*>(gb + static_cast<long long>(t0 + r) * p.ld_du + pc * 8) : z4;
    }
    const int d = d0 + tid;
    const bool d_ok = d < D;
    const bool has_neg = t0 < K;  // only the first chunk reaches the entering window
    if (has_neg) {
        for (int k = 0; k < K; ++k)
            xneg[k * DT + tid] = (p.state_in && d_ok) ? p.state_in[(static_cast<long long>(b) * D + d) * K + k] : 0.0f;
    }
    __syncthreads();
    // x[t] for t in [-K, T)
    auto xat = [&](int t) { return (has_neg && t < 0) ? xneg[(K + t) * DT + tid] : to_f(xs[(t - xt0) * DT + tid]); };
    float w[KV], win[KV], dco[KV - 1], dW[KV], bias = 0.0f, db = 0.0f;
#pragma unroll
    for (int k = 0; k < KV; ++k) {
        const int kk = k - (KV - K);
        w[k] = (kk >= 0 && d_ok) ? p.w[static_cast<long long>(d) * K + kk] : 0.0f;
        win[k] = kk >= 0 ? xat(t_start - (KV - 1) + k) : 0.0f;
        dW[k] = 0.0f;
        if (k < KV - 1) dco[k] = 0.0f;
    }
    if (d_ok) bias = p.bias[d];
    // One step back in time: gv = d_u[t], xin = x[t - K] (enters the window), OUT: t < t1.
    auto step = [&](auto out_tag, float gv, float xin, Tact* dst) {
        float acc = bias;
#pragma unroll
        for (int k = 0; k < KV; ++k) acc = fmaf(win[k], w[k], acc);
        const float sg = sigmoidf_fast(acc);
        const float g = gv * sg * fmaf(acc, 1.0f - sg, 1.0f);
        if (decltype(out_tag)::value) {
            db += g;
            float dx = g * w[KV - 1];
#pragma unroll
            for (int k = 0; k < KV; ++k) dW[k] = fmaf(g, win[k], dW[k]);
            // future steps: dco[j] = dco[t + 1 + j] meets tap KV-2-j
#pragma unroll
            for (int j = 0; j < KV - 1; ++j) dx = fmaf(dco[j], w[KV - 2 - j], dx);
            *dst = from_f<Tact>(dx);
        }
#pragma unroll
        for (int j = KV - 2; j > 0; --j) dco[j] = dco[j - 1];
        dco[0] = g;
#pragma unroll
        for (int k = KV - 1; k > 0; --k) win[k] = win[k - 1];
        // x[t - K] enters at the oldest tap that exists (slot KV - K)
#pragma unroll
        for (int k = 0; k < KV; ++k)
            if (k == KV - K) win[k] = xin;
    };
    // the halo steps after the chunk feed dco only
    for (int t = t_start; t >= t1; --t) step(std::false_type{}, to_f(gs[(t - t0) * DT + tid]), xat(t - K), dxs);
    const int n = t1 - t0;
    const Tact* gp = gs + (n - 1) * DT + tid;
    Tact* dp = dxs + (n - 1) * DT + tid;
    if (has_neg) {
        for (int i = n - 1; i >= 0; --i, gp -= DT, dp -= DT) step(std::true_type{}, to_f(*gp), xat(t0 + i - K), dp);
    } else {
        const Tact* xp = xs + (n - 1) * DT + tid;  // x[t - K] sits K rows below x[t]: row (t - K) - xt0 = t - t0
        int i = n;
        for (; i >= 8; i -= 8) {
#pragma unroll
            for (int u = 0; u < 8; ++u) step(std::true_type{}, to_f(gp[-u * DT]), to_f(xp[-u * DT]), dp - u * DT);
            gp -= 8 * DT; xp -= 8 * DT; dp -= 8 * DT;
        }
        for (; i > 0; --i, gp -= DT, xp -= DT, dp -= DT) step(std::true_type{}, to_f(*gp), to_f(*xp), dp);
    }
    if (d_ok) {
        float* pt = p.part + ((static_cast<long long>(b) * gridDim.y + chunk) * D + d) * (K + 1);
#pragma unroll
        for (int k = 0; k < KV; ++k) {
            const int kk = k - (KV - K);
            if (kk >= 0) pt[kk] = dW[k];
        }
        pt[K] = db;
    }
    __syncthreads();
    for (int i = tid; i < (t1 - t0) * PIECES; i += DT) {
        const int r = i / PIECES, pc = i - r * PIECES;
        if (d0 + pc * 8 < D)
            *reinterpret_cast<uint4*>(dxb + static_cast<long long>(t0 + r) * p.ld_dx + pc * 8) = reinterpret_cast<const uint4*>(dxs)[i];
    }
}

int conv_configure(Ctx* c) {
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(conv1d_bwd_tile_kernel<__half>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, conv_tile_smem<__half>()));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(conv1d_bwd_tile_kernel<__nv_bfloat16>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             conv_tile_smem<__nv_bfloat16>()));
    return MAMBA_B200_OK;
}

// The vector kernels need d_conv <= 4 and every row start on a vector boundary.
static bool conv_vec_ok(int K, int D, int vec, size_t esize, std::initializer_list<const void*> ptrs,
                        std::initializer_list<long long> lds) {
    if (K > kConvKV || D % vec) return false;
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) % (vec * esize)) return false;
    for (long long ld : lds)
        if (ld % vec) return false;
    return true;
}

// dW[D,K] += sum over (b, chunk) partials; db[D] likewise.  A block owns 32
// consecutive outputs; warp w adds the groups g = w, w+8, ... (coalesced
// 128-byte rows, several loads in flight) and the eight warp sums are added
// in warp order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) conv1d_bwd_reduce_kernel(const float* __restrict__ part,
                                                                float* __restrict__ dW, float* __restrict__ db,
                                                                int groups, int D, int K) {
    __shared__ float sums[8][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + lane, n = D * (K + 1);
    float acc = 0.0f;
    if (i < n) {
        const long long stride = static_cast<long long>(n);
        int g = w;
        for (; g + 24 < groups; g += 32) {
            const float a0 = part[g * stride + i], a1 = part[(g + 8) * stride + i];
            const float a2 = part[(g + 16) * stride + i], a3 = part[(g + 24) * stride + i];
            acc += a0;
            acc += a1;
            acc += a2;
            acc += a3;
        }
        for (; g < groups; g += 8) acc += part[g * stride + i];
    }
    sums[w][lane] = acc;
    __syncthreads();
    if (w == 0 && i < n) {
        float t = sums[0][lane];
#pragma unroll
        for (int k = 1; k < 8; ++k) t += sums[k][lane];
        const int d = i / (K + 1), kk = i % (K + 1);
        if (kk < K) dW[d * K + kk] += t;
        else db[d] += t;
    }
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API int mamba_b200_sscan_step(void* handle, void* stream,
                                                    const mamba_b200_sscan_step_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "sscan_step: null args");
    const mamba_b200_sscan_step_args& a = *ap;
    if (!dtype_ok(a.dtype)) return fail(c, MAMBA_B200_ERR_ARG, "sscan_step: bad dtype %d", a.dtype);
    if (a.B < 0 || a.D <= 0 || a.N <= 0)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_step: bad dims B=%d D=%d N=%d", a.B, a.D, a.N);
    if (a.B == 0) return MAMBA_B200_OK;
    if (!a.x || !a.delta || !a.Bm || !a.Cm || !a.a_neg || !a.Dp || !a.y || !a.ssm_state)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_step: null required pointer");
    if (a.z_mode < 0 || a.z_mode > 2 || (a.z_mode && !a.z))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_step: z_mode %d needs z", a.z_mode);
    if (a.conv_w && (!a.conv_b || !a.conv_state || a.K < 1 || a.K > kStepKMax))
        return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_step: d_conv %d outside 1..%d, or null bias/state", a.K,
                    kStepKMax);
    StepParams p;
    memset(&p, 0, sizeof(p));
    p.x = a.x; p.dl = a.delta; p.bm = a.Bm; p.cm = a.Cm; p.z = a.z_mode ? a.z : nullptr;
    p.y = a.y; p.u_out = a.u_out;
    p.ld_x = a.ld_x; p.ld_dl = a.ld_delta; p.ld_bc = a.ld_bc; p.ld_z = a.ld_z; p.ld_y = a.ld_y; p.ld_u = a.ld_u;
    p.a_neg = a.a_neg; p.Dp = a.Dp; p.conv_w = a.conv_w; p.conv_b = a.conv_b;
    p.conv_state = a.conv_state; p.ssm_state = a.ssm_state;
    p.B = a.B; p.D = a.D; p.N = a.N; p.K = a.conv_w ? a.K : 0;
    p.delta_softplus = a.delta_softplus; p.z_mode = a.z_mode;
    // f32 slices of a flat weight / state arena are only 4-byte aligned in general:
    // the float4 path needs 16-byte bases (rows are then aligned since N % 4 == 0).
    p.vec_state = (a.N % 4 == 0) && reinterpret_cast<uintptr_t>(a.a_neg) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(a.ssm_state) % 16 == 0;
    const long long n = static_cast<long long>(a.B) * a.D;
    const unsigned blocks = static_cast<unsigned>((n + 127) / 128);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a.dtype == MAMBA_B200_F32) sscan_step_kernel<float><<<blocks, 128, 0, st>>>(p);
    else if (a.dtype == MAMBA_B200_F16) sscan_step_kernel<__half><<<blocks, 128, 0, st>>>(p);
    else sscan_step_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

static int conv_check(Ctx* c, const char* who, const mamba_b200_conv1d_args& a, bool bwd) {
    if (!dtype_ok(a.dtype)) return fail(c, MAMBA_B200_ERR_ARG, "%s: bad dtype %d", who, a.dtype);
    if (a.B < 0 || a.T < 0 || a.D <= 0) return fail(c, MAMBA_B200_ERR_ARG, "%s: bad dims", who);
    if (a.K < 1 || a.K > kStepKMax) return fail(c, MAMBA_B200_ERR_SHAPE, "%s: d_conv %d outside 1..%d", who, a.K, kStepKMax);
    if (a.B > 65535) return fail(c, MAMBA_B200_ERR_SHAPE, "%s: batch %d > 65535", who, a.B);
    if (!a.x || !a.conv_w || !a.conv_b) return fail(c, MAMBA_B200_ERR_ARG, "%s: null required pointer", who);
    if (!bwd && !a.u) return fail(c, MAMBA_B200_ERR_ARG, "%s: null output", who);
    if (bwd && (!a.d_u || !a.d_x || !a.dconv_w || !a.dconv_b || !a.workspace))
        return fail(c, MAMBA_B200_ERR_ARG, "%s: null gradient or workspace pointer", who);
    if (a.ld_x < a.D || (!bwd && a.ld_u < a.D) || (bwd && (a.ld_du < a.D || a.ld_dx < a.D)))
        return fail(c, MAMBA_B200_ERR_ARG, "%s: a row stride is smaller than its row", who);
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API int mamba_b200_conv1d_fwd(void* handle, void* stream,
                                                    const mamba_b200_conv1d_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "conv1d_fwd: null args");
    const mamba_b200_conv1d_args& a = *ap;
    int rc = conv_check(c, "conv1d_fwd", a, false);
    if (rc) return rc;
    if (a.B == 0 || a.T == 0) return MAMBA_B200_OK;
    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.x = a.x; p.u = a.u; p.ld_x = a.ld_x; p.ld_u = a.ld_u; p.w = a.conv_w; p.bias = a.conv_b;
    p.state_in = a.conv_state; p.state_out = a.conv_state;
    p.B = a.B; p.T = a.T; p.D = a.D; p.K = a.K;
    const int chunks = (a.T + kConvTT - 1) / kConvTT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((a.D + 127) / 128, chunks, a.B);
    const unsigned sb = static_cast<unsigned>((static_cast<long long>(a.B) * a.D + 127) / 128);
    const size_t es = a.dtype == MAMBA_B200_F32 ? 4 : 2;
    const int vec = static_cast<int>(kConvFwdBytes / es);
    const bool use_vec = conv_vec_ok(a.K, a.D, vec, es, {a.x, a.u}, {a.ld_x, a.ld_u}) &&
                         reinterpret_cast<uintptr_t>(a.conv_w) % 16 == 0 && reinterpret_cast<uintptr_t>(a.conv_b) % 16 == 0;
    dim3 vgrid((a.D / vec + 63) / 64, (a.T + kConvFwdTT - 1) / kConvFwdTT, a.B);
    if (a.dtype == MAMBA_B200_F32) {
        if (use_vec) conv1d_fwd_vec_kernel<float><<<vgrid, 64, 0, st>>>(p);
        else conv1d_fwd_kernel<float><<<grid, 128, 0, st>>>(p);
        if (a.conv_state) conv1d_state_kernel<float><<<sb, 128, 0, st>>>(p);
    } else if (a.dtype == MAMBA_B200_F16) {
        if (use_vec) conv1d_fwd_vec_kernel<__half><<<vgrid, 64, 0, st>>>(p);
        else conv1d_fwd_kernel<__half><<<grid, 128, 0, st>>>(p);
        if (a.conv_state) conv1d_state_kernel<__half><<<sb, 128, 0, st>>>(p);
    } else {
        if (use_vec) conv1d_fwd_vec_kernel<__nv_bfloat16><<<vgrid, 64, 0, st>>>(p);
        else conv1d_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(p);
        if (a.conv_state) conv1d_state_kernel<__nv_bfloat16><<<sb, 128, 0, st>>>(p);
    }
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API long long mamba_b200_conv1d_bwd_workspace_bytes(int B, int T, int D, int K) {
    if (B <= 0 || T <= 0 || D <= 0 || K <= 0) return 0;
    const long long chunks = (T + kConvTT - 1) / kConvTT;
    return static_cast<long long>(sizeof(float)) * B * chunks * D * (K + 1);
}

extern "C" MAMBA_B200_API int mamba_b200_conv1d_bwd(void* handle, void* stream,
                                                    const mamba_b200_conv1d_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "conv1d_bwd: null args");
    const mamba_b200_conv1d_args& a = *ap;
    int rc = conv_check(c, "conv1d_bwd", a, true);
    if (rc) return rc;
    if (a.B == 0 || a.T == 0) return MAMBA_B200_OK;
    const int chunks = (a.T + kConvTT - 1) / kConvTT;
    const long long need = static_cast<long long>(sizeof(float)) * a.B * chunks * a.D * (a.K + 1);
    if (a.workspace_bytes < need)
        return fail(c, MAMBA_B200_ERR_ARG, "conv1d_bwd: workspace %lld < %lld bytes", a.workspace_bytes, need);
    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.x = a.x; p.du = a.d_u; p.dx = a.d_x; p.ld_x = a.ld_x; p.ld_du = a.ld_du; p.ld_dx = a.ld_dx;
    p.w = a.conv_w; p.bias = a.conv_b; p.state_in = a.conv_state;
    p.part = static_cast<float*>(a.workspace);
    p.B = a.B; p.T = a.T; p.D = a.D; p.K = a.K;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((a.D + 127) / 128, chunks, a.B);
    const size_t es = a.dtype == MAMBA_B200_F32 ? 4 : 2;
    const int bvec = es == 2 ? 2 : 4;
    const bool use_vec = conv_vec_ok(a.K, a.D, bvec, es, {a.x, a.d_u, a.d_x}, {a.ld_x, a.ld_du, a.ld_dx}) &&
                         reinterpret_cast<uintptr_t>(a.conv_w) % 16 == 0 && reinterpret_cast<uintptr_t>(a.conv_b) % 16 == 0;
    dim3 vgrid((a.D / bvec + 63) / 64, chunks, a.B);
    // 16-bit storage with rows on 16-byte boundaries: the shared-memory tile kernel
    const bool use_tile = es == 2 && conv_vec_ok(a.K, a.D, 8, es, {a.x, a.d_u, a.d_x}, {a.ld_x, a.ld_du, a.ld_dx});
    if (use_tile) {
        dim3 tgrid((a.D + kConvTileD - 1) / kConvTileD, chunks, a.B);
        if (a.dtype == MAMBA_B200_F16)
            conv1d_bwd_tile_kernel<__half><<<tgrid, kConvTileD, conv_tile_smem<__half>(), st>>>(p);
        else
            conv1d_bwd_tile_kernel<__nv_bfloat16><<<tgrid, kConvTileD, conv_tile_smem<__nv_bfloat16>(), st>>>(p);
    } else if (a.dtype == MAMBA_B200_F32) {
        if (use_vec) conv1d_bwd_vec_kernel<float><<<vgrid, 64, 0, st>>>(p);
        else conv1d_bwd_kernel<float><<<grid, 128, 0, st>>>(p);
    } else if (a.dtype == MAMBA_B200_F16) {
        if (use_vec) conv1d_bwd_vec_kernel<__half><<<vgrid, 64, 0, st>>>(p);
        else conv1d_bwd_kernel<__half><<<grid, 128, 0, st>>>(p);
    } else {
        if (use_vec) conv1d_bwd_vec_kernel<__nv_bfloat16><<<vgrid, 64, 0, st>>>(p);
        else conv1d_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(p);
    }
    MB200_CUDA_CHECK(c, cudaGetLastError());
    const int n = a.D * (a.K + 1);
    conv1d_bwd_reduce_kernel<<<(n + 31) / 32, 256, 0, st>>>(p.part, a.dconv_w, a.dconv_b, a.B * chunks,
                                                             a.D, a.K);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

// ---------------------------------------------------------------------------
// conv1d backward with built-in scratch: an entry point that allocates nothing.
// ---------------------------------------------------------------------------
namespace mb200 {

// 16 MiB of partial-sum scratch that lives in the library image.  Every GPU
// that loads the library carries it until the process exits.
constexpr long long kStaticScratchFloats = 4ll * 1024 * 1024;
static __device__ __align__(256) float g_conv_bwd_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
// Device address of g_conv_bwd_scratch per device ordinal.  In host code the
// symbol itself is only a stand-in; the address a kernel may dereference comes
// from cudaGetSymbolAddress, asked once per device with that device current.
// Host threads may make their first call on a device at the same time: the slot is
// an atomic, and two racing look-ups store the same address.
static std::atomic<float*> g_scratch_addr[kMaxDevices];

static int static_scratch_for_current_device(float** out, int* device) {
    if (cudaGetDevice(device) != cudaSuccess) return MAMBA_B200_ERR_CUDA;
    if (*device < 0 || *device >= kMaxDevices) return MAMBA_B200_ERR_DEVICE;
    float* ptr = g_scratch_addr[*device].load(std::memory_order_acquire);
    if (!ptr) {
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_conv_bwd_scratch) != cudaSuccess || !ptr)
            return MAMBA_B200_ERR_CUDA;
        g_scratch_addr[*device].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return MAMBA_B200_OK;
}

}  // namespace mb200

extern "C" MAMBA_B200_API long long mamba_b200_conv1d_bwd_static_max_bytes(void) {
    return kStaticScratchFloats * static_cast<long long>(sizeof(float));
}

extern "C" MAMBA_B200_API int mamba_b200_conv1d_bwd_static(void* handle, void* stream,
                                                           const mamba_b200_conv1d_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);  // may be null: then failures are reported by code only
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "conv1d_bwd_static: null args");
    mamba_b200_conv1d_args a = *ap;
    const long long need = mamba_b200_conv1d_bwd_workspace_bytes(a.B, a.T, a.D, a.K);
    if (need > mamba_b200_conv1d_bwd_static_max_bytes())
        return fail(c, MAMBA_B200_ERR_SHAPE,
                    "conv1d_bwd_static: B=%d T=%d D=%d K=%d needs %lld bytes of scratch, the built-in "
                    "array holds %lld; use mamba_b200_conv1d_bwd with a caller workspace",
                    a.B, a.T, a.D, a.K, need, mamba_b200_conv1d_bwd_static_max_bytes());
    float* scratch = nullptr;
    int device = -1;
    int rc = static_scratch_for_current_device(&scratch, &device);
    if (rc) return fail(c, rc, "conv1d_bwd_static: cannot resolve the scratch address on device %d", device);
    if (c && c->device != device)
        return fail(c, MAMBA_B200_ERR_DEVICE,
                    "conv1d_bwd_static: the handle belongs to device %d but device %d is current", c->device,
                    device);
    a.workspace = scratch;
    a.workspace_bytes = mamba_b200_conv1d_bwd_static_max_bytes();
    // Every partial the reduction reads is written by this call's first kernel,
    // so nothing left over from an earlier call needs clearing.
    Ctx local;
    return mamba_b200_conv1d_bwd(c ? c : &local, stream, &a);
}

extern "C" MAMBA_B200_API int mamba_b200_conv1d_fwd_nosave(void* handle, void* stream, int dtype, void* u_out,
                                                           float* state, const void* x_branch, const float* weight,
                                                           const float* bias, int batch, int T, int d_inner,
                                                           int d_conv) {
    mamba_b200_conv1d_args a;
    memset(&a, 0, sizeof(a));
    a.dtype = dtype; a.B = batch; a.T = T; a.D = d_inner; a.K = d_conv;
    a.x = x_branch; a.ld_x = d_inner; a.conv_w = weight; a.conv_b = bias; a.conv_state = state;
    a.u = u_out; a.ld_u = d_inner;
    return mamba_b200_conv1d_fwd(handle, stream, &a);
}
