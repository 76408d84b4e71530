// Streaming kernels either side of the backbone in a training step: token-embedding
// gather into the f32 residual stream, softmax cross-entropy (loss and d_logits in
// one pass over the logits), and the fused AdamW update.
//
// The reference trainer takes its inputs and the output gradient from the host
// (src/mamba_ssm/gpu/trainer.rs:437-481) and runs AdamW, the master -> compute cast
// and the a_neg refresh as three passes over the parameters (trainer.rs:1453-1475,
// kernels/adamw.cu:30-61); its language-model wrapper computes logits with one
// GEMM on a [vocab, d_model] table (src/module/gpu_lm.rs:560-679).  These kernels put
// the embedding row gather, the loss and the optimiser tail on the device: all are
// bandwidth-bound, one read and at most one write per element.
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

// out[r, :] (f32 residual stream) = table[ids[r], :]; ids outside [0, vocab) give zeros.
template <typename Tact>
__global__ void __launch_bounds__(256) embedding_gather_kernel(const Tact* __restrict__ table,
                                                               const int* __restrict__ ids, float* __restrict__ out,
                                                               long long rows, int dim, int vocab) {
    const int per_row = (dim + 3) / 4;
    const long long total = rows * per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / per_row;
        const int c = static_cast<int>(i - r * per_row) * 4;
        const int id = ids[r];
        const bool ok = id >= 0 && id < vocab;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (ok && c + j < dim) v[j] = to_f(table[static_cast<long long>(id) * dim + c + j]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (c + j < dim) out[r * dim + c + j] = v[j];
    }
}

// One CTA per row of logits.  loss[r] = log(sum exp(l)) - l[target]; d_logits =
// (softmax(l) - onehot(target)) * grad_scale.  target < 0 marks a row that does not
// count: loss 0, zero gradient.  The row is kept in shared memory in its storage
// dtype between the two passes when it fits, so the logits are read once.
template <typename Tact, bool VEC>
__global__ void __launch_bounds__(512) softmax_xent_kernel(const Tact* __restrict__ logits,
                                                           const int* __restrict__ targets, float* __restrict__ loss,
                                                           Tact* __restrict__ dlogits, float grad_scale, int V,
                                                           long long ld, int cache_row) {
    extern __shared__ __align__(16) unsigned char xsm[];
    __shared__ float red_m[16], red_s[16];
    constexpr int W = 16 / sizeof(Tact);  // elements per 16-byte access
    Tact* row_c = reinterpret_cast<Tact*>(xsm);
    const long long r = blockIdx.x;
    const Tact* row = logits + r * ld;
    const int tgt = targets[r];
    const int tid = threadIdx.x;
    // online max / sum of exponentials
    float m = -INFINITY, s = 0.0f;
    auto take = [&](float v) {
        if (v > m) {
            s = s * ex2((m - v) * kLog2e) + 1.0f;
            m = v;
        } else {
            s += ex2((v - m) * kLog2e);
        }
    };
    auto widen = [&](const uint4& q, float* f) {
        if constexpr (sizeof(Tact) == 2) {
            const float2 a = unpack2<Tact>(q.x), b = unpack2<Tact>(q.y), c2 = unpack2<Tact>(q.z), d2 = unpack2<Tact>(q.w);
            f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c2.x; f[5] = c2.y; f[6] = d2.x; f[7] = d2.y;
        } else {
            f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
        }
    };
    if (VEC) {
        for (int i = tid * W; i < V; i += blockDim.x * W) {
            const uint4 q = *reinterpret_cast<const uint4*>(row + i);
            if (cache_row) *reinterpret_cast<uint4*>(row_c + i) = q;
            float f[W];
            widen(q, f);
#pragma unroll
            for (int j = 0; j < W; ++j) take(f[j]);
        }
    } else {
        for (int i = tid; i < V; i += blockDim.x) {
            const Tact raw = row[i];
            if (cache_row) row_c[i] = raw;
            take(to_f(raw));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float mm = fmaxf(m, m2);
        s = (m == -INFINITY ? 0.0f : s * ex2((m - mm) * kLog2e)) + (m2 == -INFINITY ? 0.0f : s2 * ex2((m2 - mm) * kLog2e));
        m = mm;
    }
    const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
    if (lane == 0) {
        red_m[warp] = m;
        red_s[warp] = s;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < nw; ++w) M = fmaxf(M, red_m[w]);
    float S = 0.0f;
    for (int w = 0; w < nw; ++w)
        if (red_m[w] != -INFINITY) S += red_s[w] * ex2((red_m[w] - M) * kLog2e);
    const bool counted = tgt >= 0 && tgt < V;
    if (tid == 0) loss[r] = counted ? (M + lg2(S) * kLn2) - to_f(row[tgt]) : 0.0f;
    if (!dlogits) return;
    const float inv = counted ? grad_scale / S : 0.0f;
    Tact* drow = dlogits + r * ld;
    const Tact* src = cache_row ? row_c : row;
    const float Ml = M * kLog2e;
    if (VEC) {
        for (int i = tid * W; i < V; i += blockDim.x * W) {
            const uint4 q = *reinterpret_cast<const uint4*>(src + i);
            float f[W];
            widen(q, f);
#pragma unroll
            for (int j = 0; j < W; ++j) {
                f[j] = ex2(fmaf(f[j], kLog2e, -Ml)) * inv;
                if (i + j == tgt && counted) f[j] -= grad_scale;
            }
            uint4 o;
            if constexpr (sizeof(Tact) == 2) {
                o = make_uint4(pack2<Tact>(f[0], f[1]), pack2<Tact>(f[2], f[3]), pack2<Tact>(f[4], f[5]),
                               pack2<Tact>(f[6], f[7]));
            } else {
                o = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
            }
            *reinterpret_cast<uint4*>(drow + i) = o;
        }
    } else {
        for (int i = tid; i < V; i += blockDim.x) {
            float g = ex2(fmaf(to_f(src[i]), kLog2e, -Ml)) * inv;
            if (i == tgt && counted) g -= grad_scale;
            drow[i] = from_f<Tact>(g);
        }
    }
}

// AdamW with decoupled weight decay, the arithmetic of adamw_step_f32_capturable
// (kernels/adamw.cu:30-61): bias corrections come from a 2-element device buffer so the
// launch can sit in a captured graph.  Optionally writes the compute-dtype copy of the
// updated parameter in the same pass (the reference's separate master -> compute cast).
template <typename Tlp>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ param, const float* __restrict__ grad,
                                                    float* __restrict__ m, float* __restrict__ v, float lr,
                                                    float beta1, float beta2, float eps, float wd,
                                                    const float* __restrict__ bias_factors, Tlp* __restrict__ lp,
                                                    long long n) {
    const float bc1 = bias_factors[0], bc2 = bias_factors[1];
    const float omb1 = 1.f - beta1, omb2 = 1.f - beta2, decay = 1.f - lr * wd;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float g = grad[i], p = param[i];
        const float mi = m[i] * beta1 + omb1 * g;
        const float vi = v[i] * beta2 + omb2 * g * g;
        m[i] = mi;
        v[i] = vi;
        const float pn = decay * p - lr * (mi * bc1) / (sqrtf(vi * bc2) + eps);
        param[i] = pn;
        if (lp) lp[i] = from_f<Tlp>(pn);
    }
}

int train_ops_configure(Ctx* c) {
    const int lim = 208 * 1024;
#define MB200_XENT_ATTR(T, V)                                                                                      \
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(softmax_xent_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim))
    MB200_XENT_ATTR(float, true); MB200_XENT_ATTR(float, false);
    MB200_XENT_ATTR(__half, true); MB200_XENT_ATTR(__half, false);
    MB200_XENT_ATTR(__nv_bfloat16, true); MB200_XENT_ATTR(__nv_bfloat16, false);
#undef MB200_XENT_ATTR
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API int mamba_b200_embedding_gather(void* handle, void* stream, int dtype, const void* table,
                                                          const int* ids, float* out, long long rows, int dim,
                                                          int vocab) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!dtype_ok(dtype)) return fail(c, MAMBA_B200_ERR_ARG, "embedding_gather: bad dtype %d", dtype);
    if (rows < 0 || dim <= 0 || vocab <= 0) return fail(c, MAMBA_B200_ERR_ARG, "embedding_gather: bad dims");
    if (rows == 0) return MAMBA_B200_OK;
    if (!table || !ids || !out) return fail(c, MAMBA_B200_ERR_ARG, "embedding_gather: null pointer");
    const long long work = rows * ((dim + 3) / 4);
    const int grid = static_cast<int>(work / 256 + 1 < 148ll * 16 ? work / 256 + 1 : 148ll * 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == MAMBA_B200_F32)
        embedding_gather_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(table), ids, out, rows, dim, vocab);
    else if (dtype == MAMBA_B200_F16)
        embedding_gather_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(table), ids, out, rows, dim, vocab);
    else
        embedding_gather_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(table), ids, out, rows, dim, vocab);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API int mamba_b200_softmax_xent(void* handle, void* stream, int dtype, const void* logits,
                                                      const int* targets, float* loss_rows, void* dlogits,
                                                      float grad_scale, long long rows, int V, long long ld) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!dtype_ok(dtype)) return fail(c, MAMBA_B200_ERR_ARG, "softmax_xent: bad dtype %d", dtype);
    if (rows < 0 || V <= 0 || ld < V) return fail(c, MAMBA_B200_ERR_ARG, "softmax_xent: bad dims");
    if (rows == 0) return MAMBA_B200_OK;
    if (rows > 2147483647ll) return fail(c, MAMBA_B200_ERR_SHAPE, "softmax_xent: too many rows");
    if (!logits || !targets || !loss_rows) return fail(c, MAMBA_B200_ERR_ARG, "softmax_xent: null pointer");
    const size_t bytes = static_cast<size_t>(V) * dtype_size(dtype);
    const int cache = bytes <= 208 * 1024 - 256 && dlogits != nullptr;
    const size_t smem = cache ? bytes : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>(rows);
    const size_t es = dtype_size(dtype);
    const int w16 = static_cast<int>(16 / es);
    auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const bool vec = V % w16 == 0 && ld % w16 == 0 && al16(logits) && (!dlogits || al16(dlogits));
#define MB200_XENT(T)                                                                                              \
    do {                                                                                                           \
        if (vec)                                                                                                   \
            softmax_xent_kernel<T, true><<<grid, 512, smem, st>>>(static_cast<const T*>(logits), targets, loss_rows, \
                                                                  static_cast<T*>(dlogits), grad_scale, V, ld, cache); \
        else                                                                                                       \
            softmax_xent_kernel<T, false><<<grid, 512, smem, st>>>(static_cast<const T*>(logits), targets, loss_rows, \
                                                                   static_cast<T*>(dlogits), grad_scale, V, ld, cache); \
    } while (0)
    if (dtype == MAMBA_B200_F32) MB200_XENT(float);
    else if (dtype == MAMBA_B200_F16) MB200_XENT(__half);
    else MB200_XENT(__nv_bfloat16);
#undef MB200_XENT
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API int mamba_b200_adamw_step(void* handle, void* stream, float* param, const float* grad,
                                                    float* m, float* v, float lr, float beta1, float beta2,
                                                    float eps, float weight_decay, const float* bias_factors,
                                                    void* param_lp, int lp_dtype, long long n) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (n < 0) return fail(c, MAMBA_B200_ERR_ARG, "adamw_step: negative length");
    if (n == 0) return MAMBA_B200_OK;
    if (!param || !grad || !m || !v || !bias_factors) return fail(c, MAMBA_B200_ERR_ARG, "adamw_step: null pointer");
    if (param_lp && lp_dtype != MAMBA_B200_F16 && lp_dtype != MAMBA_B200_BF16)
        return fail(c, MAMBA_B200_ERR_ARG, "adamw_step: the compute copy is f16 or bf16");
    const int grid = static_cast<int>(n / 256 + 1 < 148ll * 16 ? n / 256 + 1 : 148ll * 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (param_lp && lp_dtype == MAMBA_B200_F16)
        adamw_kernel<__half><<<grid, 256, 0, st>>>(param, grad, m, v, lr, beta1, beta2, eps, weight_decay, bias_factors,
                                                   static_cast<__half*>(param_lp), n);
    else
        adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(param, grad, m, v, lr, beta1, beta2, eps, weight_decay,
                                                          bias_factors, static_cast<__nv_bfloat16*>(param_lp), n);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}
