// Shared device helpers for the sm_100a selective-scan kernels: storage-dtype
// conversion, the activation math conventions, packed f32x2 arithmetic and
// the mbarrier / TMA (cp.async.bulk.tensor) PTX wrappers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Device-visible status word values (first error wins).
enum : int { kStatusOk = 0, kStatusBarrierTimeout = 1, kStatusBadShape = 2 };

// ---- storage dtypes --------------------------------------------------------
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// Two adjacent storage elements -> float2 (one 32/64-bit shared or global load).
__device__ __forceinline__ float2 ld_pair(const float* p) {
    return *reinterpret_cast<const float2*>(p);
}
__device__ __forceinline__ float2 ld_pair(const __nv_bfloat16* p) {
    uint32_t r = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(r << 16), __uint_as_float(r & 0xffff0000u));
}
__device__ __forceinline__ float2 ld_pair(const __half* p) {
    return __half22float2(*reinterpret_cast<const __half2*>(p));
}
__device__ __forceinline__ void st_pair(float* p, float2 v) {
    *reinterpret_cast<float2*>(p) = v;
}
__device__ __forceinline__ void st_pair(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v);
}
__device__ __forceinline__ void st_pair(__half* p, float2 v) {
    *reinterpret_cast<__half2*>(p) = __float22half2_rn(v);
}

// Two f32 values <-> one 32-bit word of two 16-bit storage elements.
template <typename Th> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <typename Th> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
}

// ---- math conventions -------------------------------------------------------
// exp2 on the MUFU pipe (2 ulp); every exp of the path is exp2(x * log2 e), the
// convention of the reference's device code (kernels/_typed_prelude.cuh:20-32).
__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float lg2(float x) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rcp(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// sigmoid(v) = 1 / (1 + exp(-v))
__device__ __forceinline__ float sigmoidf_fast(float v) { return rcp(1.0f + ex2(-v * kLog2e)); }
// SiLU, kernels/activations.cu:12-30.
__device__ __forceinline__ float siluf_fast(float v) { return v * sigmoidf_fast(v); }
// softplus with threshold 20 (kernels/activations.cu:34-52).  log1p(e) is the
// degree-5 series below e = 1/32 (relative error < 1e-8) and ln(1 + e) above,
// so a small delta keeps its relative precision.
__device__ __forceinline__ float softplusf_fast(float v) {
    float e = ex2(fminf(v, 20.0f) * kLog2e);
    float big = lg2(1.0f + e) * kLn2;
    float p = fmaf(e, 0.2f, -0.25f);
    p = fmaf(p, e, 0.33333334f);
    p = fmaf(p, e, -0.5f);
    p = fmaf(p, e, 1.0f);
    float small = p * e;
    float r = e < 0.03125f ? small : big;
    return v > 20.0f ? v : r;
}

// ---- packed f32x2 arithmetic (one issue slot for two lanes of FP32 work) ----
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

// ---- B / C vectors ------------------------------------------------------------
// NS consecutive B or C values of one timestep, held in registers in their
// storage dtype and widened to f32 pairs at the point of use.
template <typename Tact, int NS>
struct StateVec;
template <int NS>
struct StateVec<float, NS> {
    float4 q[NS / 4];
    __device__ __forceinline__ void load(const float* p) {
#pragma unroll
        for (int j = 0; j < NS / 4; ++j) q[j] = *reinterpret_cast<const float4*>(p + 4 * j);
    }
    __device__ __forceinline__ float2 pair(int j) const {
        return (j & 1) ? make_float2(q[j / 2].z, q[j / 2].w) : make_float2(q[j / 2].x, q[j / 2].y);
    }
};
template <typename Th, int NS>
struct StateVecHalf {
    uint32_t w[NS / 2];  // two 16-bit elements per word
    __device__ __forceinline__ void load(const Th* p) {
        if (NS % 8 == 0) {
#pragma unroll
            for (int j = 0; j < NS / 8; ++j) {
                const uint4 v = *reinterpret_cast<const uint4*>(p + 8 * j);
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < NS / 4; ++j) {
                const uint2 v = *reinterpret_cast<const uint2*>(p + 4 * j);
                w[2 * j] = v.x; w[2 * j + 1] = v.y;
            }
        }
    }
};
template <int NS>
struct StateVec<__nv_bfloat16, NS> : StateVecHalf<__nv_bfloat16, NS> {
    __device__ __forceinline__ float2 pair(int j) const {
        return make_float2(__uint_as_float(this->w[j] << 16), __uint_as_float(this->w[j] & 0xffff0000u));
    }
};
template <int NS>
struct StateVec<__half, NS> : StateVecHalf<__half, NS> {
    __device__ __forceinline__ float2 pair(int j) const {
        return __half22float2(*reinterpret_cast<const __half2*>(&this->w[j]));
    }
};

// ---- mbarrier + TMA ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait: gives up after max_polls polls (each poll suspends for a
// hardware-chosen time), records kStatusBarrierTimeout and returns false so the
// kernel can run to its end instead of hanging.
constexpr int kMbarMaxPolls = 1 << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status,
                                          int max_polls = kMbarMaxPolls) {
    uint32_t ok = 0;
    for (int it = 0; it < max_polls; ++it) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    if (status) atomicCAS(status, kStatusOk, kStatusBarrierTimeout);
    return false;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 3-D tiled TMA load global -> this CTA's own shared memory.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Asks for `bytes` (a multiple of 16, from a 16-byte aligned address) to be brought into L2.
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Contiguous bulk copy global -> this CTA's own shared memory (both addresses 16-byte aligned,
// size a multiple of 16), completion counted on an mbarrier.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// 4-D tiled TMA load global -> this CTA's own shared memory (no multicast).
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 3-D tiled TMA store shared -> global (clipped at the tensor bounds).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0,
                                             int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::
                     "l"(map),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
// 4-D tiled TMA store shared -> global (clipped at the tensor bounds).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1,
                                             int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::
                     "l"(map),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until every committed bulk store has finished READING shared memory.
__device__ __forceinline__ void tma_wait_read0() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Wait until every committed bulk store is complete (visible in global memory).
__device__ __forceinline__ void tma_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

}  // namespace mb200
