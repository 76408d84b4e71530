// Residual add + RMSNorm, forward and backward, one pass each.
//
// Between two Mamba layers the reference runs residual_add_f32_{dt} (the out_proj
// output, 16-bit, is added to the f32 residual stream; kernels/elementwise.cu:367-377)
// and then rmsnorm_forward_f32in_{dt} on the result (kernels/norms.cu:126-168): the
// residual is written and read straight back.  Here one kernel reads the residual row
// and the branch output, writes the new residual, the normalised row in the GEMM's
// dtype and the row's rms: every element is read once and written once.  The backward
// (rmsnorm_backward_f32in_{dt}, kernels/norms.cu:323-367, plus the reference's
// [rows, dim] d_scale partials and reduce_sum_axis0) adds dx into the residual
// gradient in place and reduces d_scale over a CTA's rows before it touches memory.
//
// Memory-bound streaming kernels: a CTA walks rows with a grid stride, a row sits in
// shared memory between the reduction and the output pass, 128-bit accesses where the
// row length and the pointers allow.
#include <string.h>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

constexpr int kNormThreads = 256;
constexpr int kNormMaxDim = 16384;  // a row of f32 in shared memory (64 KB)

struct NormParams {
    float* residual;        // [rows, dim] f32: in (old residual), out (residual + branch)
    const void* branch;     // [rows, dim] storage dtype, or null (plain RMSNorm of the residual)
    const float* scale;     // [dim]
    void* y;                // [rows, dim] storage dtype: rmsnorm(residual) * scale
    float* rms_out;         // [rows] or null
    // backward
    const void* dy;         // [rows, dim] storage dtype
    const float* x;         // [rows, dim] f32: the residual the forward normalised
    const float* rms_saved; // [rows]
    float* d_residual;      // [rows, dim] f32, += dx
    float* part;            // [ctas, dim] d_scale partials
    int rows, dim;
    float eps;
};

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // red may still be read from the previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) t += red[w];  // same order in every thread
    return t;
}

template <typename Tact, bool VEC>
__global__ void __launch_bounds__(kNormThreads) residual_rmsnorm_fwd_kernel(const NormParams p) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[kNormThreads / 32];
    const int dim = p.dim, tid = threadIdx.x;
    const Tact* br = static_cast<const Tact*>(p.branch);
    Tact* yo = static_cast<Tact*>(p.y);
    for (long long r = blockIdx.x; r < p.rows; r += gridDim.x) {
        float* res = p.residual + r * dim;
        float ss = 0.0f;
        if (VEC) {
            for (int i = tid * 4; i < dim; i += kNormThreads * 4) {
                float4 v = *reinterpret_cast<const float4*>(res + i);
                if (br) {
                    float bv[4];
                    if constexpr (sizeof(Tact) == 2) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(br + r * dim + i);
                        const float2 lo = unpack2<Tact>(raw.x), hi = unpack2<Tact>(raw.y);
                        bv[0] = lo.x; bv[1] = lo.y; bv[2] = hi.x; bv[3] = hi.y;
                    } else {
                        const float4 raw = *reinterpret_cast<const float4*>(br + r * dim + i);
                        bv[0] = raw.x; bv[1] = raw.y; bv[2] = raw.z; bv[3] = raw.w;
                    }
                    v.x += bv[0]; v.y += bv[1]; v.z += bv[2]; v.w += bv[3];
                    *reinterpret_cast<float4*>(res + i) = v;
                }
                *reinterpret_cast<float4*>(row + i) = v;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        } else {
            for (int i = tid; i < dim; i += kNormThreads) {
                float v = res[i];
                if (br) {
                    v += to_f(br[r * dim + i]);
                    res[i] = v;
                }
                row[i] = v;
                ss += v * v;
            }
        }
        const float tot = block_sum(ss, red);
        float rms = sqrtf(tot / static_cast<float>(dim) + p.eps);
        if (!isfinite(rms) || rms < 1e-20f) rms = 1.0f;  // the reference's guard, kernels/norms.cu:152-159
        if (tid == 0 && p.rms_out) p.rms_out[r] = rms;
        const float inv = 1.0f / rms;
        if (VEC) {
            for (int i = tid * 4; i < dim; i += kNormThreads * 4) {
                const float4 v = *reinterpret_cast<const float4*>(row + i);
                const float4 s = *reinterpret_cast<const float4*>(p.scale + i);
                const float o0 = v.x * inv * s.x, o1 = v.y * inv * s.y, o2 = v.z * inv * s.z, o3 = v.w * inv * s.w;
                if constexpr (sizeof(Tact) == 2) {
                    *reinterpret_cast<uint2*>(yo + r * dim + i) = make_uint2(pack2<Tact>(o0, o1), pack2<Tact>(o2, o3));
                } else {
                    *reinterpret_cast<float4*>(yo + r * dim + i) = make_float4(o0, o1, o2, o3);
                }
            }
        } else {
            for (int i = tid; i < dim; i += kNormThreads) yo[r * dim + i] = from_f<Tact>(row[i] * inv * p.scale[i]);
        }
        __syncthreads();  // the row buffer is rewritten by the next iteration
    }
}

// dx = (scale * dy - x_hat * mean(dy * y_hat)) / rms, added into d_residual;
// d_scale[i] += sum over rows of dy * x_hat (per-CTA partial, reduced afterwards in
// CTA order).
template <typename Tact, bool VEC>
__global__ void __launch_bounds__(kNormThreads) residual_rmsnorm_bwd_kernel(const NormParams p) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[kNormThreads / 32];
    const int dim = p.dim, tid = threadIdx.x;
    float* xh = sm;          // x_hat of the row
    float* dyv = sm + dim;   // dy of the row
    float* acc = sm + 2 * dim;  // d_scale partial of this CTA
    const Tact* dy = static_cast<const Tact*>(p.dy);
    for (int i = tid; i < dim; i += kNormThreads) acc[i] = 0.0f;
    for (long long r = blockIdx.x; r < p.rows; r += gridDim.x) {
        const float inv = 1.0f / p.rms_saved[r];
        float s = 0.0f;
        if (VEC) {
            for (int i = tid * 4; i < dim; i += kNormThreads * 4) {
                float4 xv = *reinterpret_cast<const float4*>(p.x + r * dim + i);
                xv.x *= inv; xv.y *= inv; xv.z *= inv; xv.w *= inv;
                float4 g;
                if constexpr (sizeof(Tact) == 2) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(dy + r * dim + i);
                    const float2 lo = unpack2<Tact>(raw.x), hi = unpack2<Tact>(raw.y);
                    g = make_float4(lo.x, lo.y, hi.x, hi.y);
                } else {
                    g = *reinterpret_cast<const float4*>(dy + r * dim + i);
                }
                const float4 sc = *reinterpret_cast<const float4*>(p.scale + i);
                *reinterpret_cast<float4*>(xh + i) = xv;
                *reinterpret_cast<float4*>(dyv + i) = g;
                s = fmaf(g.x, xv.x * sc.x, s);
                s = fmaf(g.y, xv.y * sc.y, s);
                s = fmaf(g.z, xv.z * sc.z, s);
                s = fmaf(g.w, xv.w * sc.w, s);
            }
        } else {
            for (int i = tid; i < dim; i += kNormThreads) {
                const float xv = p.x[r * dim + i] * inv, g = to_f(dy[r * dim + i]);
                xh[i] = xv;
                dyv[i] = g;
                s = fmaf(g, xv * p.scale[i], s);
            }
        }
        const float mean = block_sum(s, red) / static_cast<float>(dim);
        if (VEC) {
            for (int i = tid * 4; i < dim; i += kNormThreads * 4) {
                const float4 xv = *reinterpret_cast<const float4*>(xh + i), g = *reinterpret_cast<const float4*>(dyv + i);
                const float4 sc = *reinterpret_cast<const float4*>(p.scale + i);
                float4 dr = *reinterpret_cast<const float4*>(p.d_residual + r * dim + i);
                dr.x += (sc.x * g.x - xv.x * mean) * inv;
                dr.y += (sc.y * g.y - xv.y * mean) * inv;
                dr.z += (sc.z * g.z - xv.z * mean) * inv;
                dr.w += (sc.w * g.w - xv.w * mean) * inv;
                *reinterpret_cast<float4*>(p.d_residual + r * dim + i) = dr;
                float4 a = *reinterpret_cast<const float4*>(acc + i);  // elements i..i+3 are always this thread's
                a.x = fmaf(g.x, xv.x, a.x); a.y = fmaf(g.y, xv.y, a.y); a.z = fmaf(g.z, xv.z, a.z); a.w = fmaf(g.w, xv.w, a.w);
                *reinterpret_cast<float4*>(acc + i) = a;
            }
        } else {
            for (int i = tid; i < dim; i += kNormThreads) {
                const float xv = xh[i], g = dyv[i];
                p.d_residual[r * dim + i] += (p.scale[i] * g - xv * mean) * inv;
                acc[i] = fmaf(g, xv, acc[i]);  // element i is always this thread's
            }
        }
        __syncthreads();
    }
    for (int i = tid; i < dim; i += kNormThreads) p.part[static_cast<long long>(blockIdx.x) * dim + i] = acc[i];
}

__global__ void norm_dscale_reduce_kernel(const float* __restrict__ part, float* __restrict__ d_scale, int ctas,
                                          int dim) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    float a = 0.0f;
    for (int k = 0; k < ctas; ++k) a += part[static_cast<long long>(k) * dim + i];
    d_scale[i] += a;
}

static int norm_ctas(const Ctx* c, int rows) {
    const int want = 4 * (c->sm_count > 0 ? c->sm_count : 148);
    return rows < want ? rows : want;
}

int norm_configure(Ctx* c) {
    const int lim = 3 * kNormMaxDim * 4;
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_bwd_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_bwd_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_bwd_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_bwd_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_bwd_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_bwd_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    const int limf = kNormMaxDim * 4;
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_fwd_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, limf));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_fwd_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, limf));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_fwd_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, limf));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_fwd_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, limf));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_fwd_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, limf));
    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(residual_rmsnorm_fwd_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, limf));
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API int mamba_b200_residual_rmsnorm_fwd(void* handle, void* stream, int dtype, float* residual,
                                                              const void* branch, const float* scale, void* y,
                                                              float* rms_out, int rows, int dim, float eps) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!dtype_ok(dtype)) return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_fwd: bad dtype %d", dtype);
    if (rows < 0 || dim <= 0) return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_fwd: bad dims");
    if (dim > kNormMaxDim) return fail(c, MAMBA_B200_ERR_SHAPE, "residual_rmsnorm_fwd: dim %d > %d", dim, kNormMaxDim);
    if (rows == 0) return MAMBA_B200_OK;
    if (!residual || !scale || !y) return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_fwd: null required pointer");
    NormParams p;
    memset(&p, 0, sizeof(p));
    p.residual = residual; p.branch = branch; p.scale = scale; p.y = y; p.rms_out = rms_out;
    p.rows = rows; p.dim = dim; p.eps = eps;
    auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
    const size_t es = dtype_size(dtype);
    const bool vec = dim % 4 == 0 && al(residual, 16) && al(scale, 16) && al(y, 4 * es) && (!branch || al(branch, 4 * es));
    const int grid = norm_ctas(c, rows);
    const size_t smem = sizeof(float) * dim;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define MB200_NORM_FWD(T)                                                                      \
    do {                                                                                       \
        if (vec) residual_rmsnorm_fwd_kernel<T, true><<<grid, kNormThreads, smem, st>>>(p);    \
        else residual_rmsnorm_fwd_kernel<T, false><<<grid, kNormThreads, smem, st>>>(p);       \
    } while (0)
    if (dtype == MAMBA_B200_F32) MB200_NORM_FWD(float);
    else if (dtype == MAMBA_B200_F16) MB200_NORM_FWD(__half);
    else MB200_NORM_FWD(__nv_bfloat16);
#undef MB200_NORM_FWD
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API long long mamba_b200_residual_rmsnorm_bwd_workspace_bytes(int rows, int dim) {
    if (rows <= 0 || dim <= 0) return 0;
    const long long ctas = rows < 4 * 148 ? rows : 4 * 148;
    return ctas * dim * static_cast<long long>(sizeof(float));
}

extern "C" MAMBA_B200_API int mamba_b200_residual_rmsnorm_bwd(void* handle, void* stream, int dtype, const void* dy,
                                                              const float* x, const float* scale,
                                                              const float* rms_saved, float* d_residual,
                                                              float* d_scale, int rows, int dim, void* workspace,
                                                              long long workspace_bytes) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!dtype_ok(dtype)) return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_bwd: bad dtype %d", dtype);
    if (rows < 0 || dim <= 0) return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_bwd: bad dims");
    if (dim > kNormMaxDim) return fail(c, MAMBA_B200_ERR_SHAPE, "residual_rmsnorm_bwd: dim %d > %d", dim, kNormMaxDim);
    if (rows == 0) return MAMBA_B200_OK;
    if (!dy || !x || !scale || !rms_saved || !d_residual || !d_scale || !workspace)
        return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_bwd: null required pointer");
    int grid = norm_ctas(c, rows);
    if (grid > 4 * 148) grid = 4 * 148;  // what the workspace query promises
    if (workspace_bytes < static_cast<long long>(grid) * dim * 4)
        return fail(c, MAMBA_B200_ERR_ARG, "residual_rmsnorm_bwd: workspace %lld < %lld bytes", workspace_bytes,
                    static_cast<long long>(grid) * dim * 4);
    NormParams p;
    memset(&p, 0, sizeof(p));
    p.dy = dy; p.x = x; p.scale = scale; p.rms_saved = rms_saved; p.d_residual = d_residual;
    p.part = static_cast<float*>(workspace);
    p.rows = rows; p.dim = dim;
    const size_t smem = sizeof(float) * 3 * dim;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
    const bool vec = dim % 4 == 0 && al(x, 16) && al(scale, 16) && al(d_residual, 16) && al(dy, 4 * dtype_size(dtype));
#define MB200_NORM_BWD(T)                                                                        \
    do {                                                                                         \
        if (vec) residual_rmsnorm_bwd_kernel<T, true><<<grid, kNormThreads, smem, st>>>(p);      \
        else residual_rmsnorm_bwd_kernel<T, false><<<grid, kNormThreads, smem, st>>>(p);         \
    } while (0)
    if (dtype == MAMBA_B200_F32) MB200_NORM_BWD(float);
    else if (dtype == MAMBA_B200_F16) MB200_NORM_BWD(__half);
    else MB200_NORM_BWD(__nv_bfloat16);
#undef MB200_NORM_BWD
    MB200_CUDA_CHECK(c, cudaGetLastError());
    norm_dscale_reduce_kernel<<<(dim + 255) / 256, 256, 0, st>>>(p.part, d_scale, grid, dim);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}
