// tcgen05 / TMEM helpers shared by the Mamba-3 SSD tensor-core kernels.
//
// Shared-memory operand tiles are 8-row x 16-byte core matrices without
// swizzle: a tile of R rows x C 16-bit columns keeps core (r/8, c/8) at
// (r/8)*(C/8)*128 + (c/8)*128 bytes, row r%8 at +16*(r%8).  With that layout
//   * an operand whose K dimension runs along the tile's COLUMNS (K-major) is
//     described, for the k-th 16-element step, by start = tile + k*256,
//     LBO = 128, SBO = (C/8)*128;
//   * an operand whose K dimension runs along the tile's ROWS (MN-major) by
//     start = tile + k*2*(C/8)*128, LBO = (C/8)*128, SBO = 128.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace mb200 {
namespace tc {

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start >> 4 [0,14) | LBO >> 4 [16,30) | SBO >> 4 [32,46) | version 1 [46,48) | no swizzle
    return static_cast<uint64_t>((addr & 0x3FFFF) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46);
}
// kind::f16 instruction descriptor: f32 accumulate, 16-bit A/B of format `fmt`
// (0 = f16, 1 = bf16), majors (0 = K-major, 1 = MN-major), M = 128.
__device__ __forceinline__ uint32_t instr_desc(uint32_t fmt, uint32_t a_mn, uint32_t b_mn, uint32_t n) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) |
           ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive f32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"
        "%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,"
        "%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Two 32-column loads in flight, one wait.
__device__ __forceinline__ void tmem_ld32x2(uint32_t ta, float* va, uint32_t tb, float* vb) {
    uint32_t ra[32], rb[32];
    tmem_ld32_issue(ta, ra);
    tmem_ld32_issue(tb, rb);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        va[i] = __uint_as_float(ra[i]);
        vb[i] = __uint_as_float(rb[i]);
    }
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Byte offset of the 16-byte chunk (row r, 8-column group j) in a tile of C columns.
__device__ __forceinline__ uint32_t chunk_off(int r, int j, int C) {
    return static_cast<uint32_t>((r >> 3) * (C >> 3) * 128 + j * 128 + (r & 7) * 16);
}


// 16-byte asynchronous copy global -> shared; `valid` false writes zeros.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(valid ? 16u : 0u)
                 : "memory");
}
// Thirty-two consecutive bytes: one 256-bit store (a whole sector per request) when the
// destination is 32-byte aligned, else two 128-bit stores.
__device__ __forceinline__ void store32b(void* dst, const uint4& a, const uint4& b, bool wide) {
    if (wide) {
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(a.x), "r"(a.y), "r"(a.z),
                     "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                     : "memory");
    } else {
        reinterpret_cast<uint4*>(dst)[0] = a;
        reinterpret_cast<uint4*>(dst)[1] = b;
    }
}
// One arrival on an mbarrier of this CTA (release at CTA scope).
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 4-byte asynchronous copy global -> shared.
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Descriptors of the k-th 16-element step of a tile with C columns (see top).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int k, int C) {
    return smem_desc(tile + k * 256, 128, (C >> 3) * 128);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int k, int C) {
    return smem_desc(tile + k * 2 * (C >> 3) * 128, (C >> 3) * 128, 128);
}

// ---- 128-byte-swizzled tiles (what a TMA copy with CU_TENSOR_MAP_SWIZZLE_128B writes) ----
// A tile of R rows x 64 16-bit columns is R rows of 128 bytes, the 16-byte piece j of row r
// stored at piece j ^ (r % 8); a 128-column tile is two such sub-tiles, kSwSub bytes apart
// (128 rows).  Descriptor fields found by comparing every operand form against a host
// product: layout type 2; stride byte offset 1024 (eight rows); a K-major operand advances
// 32 bytes per 16-element K step inside a sub-tile (the leading byte offset is unused); an
// MN-major operand advances 2048 bytes (sixteen rows) per K step and its leading byte offset
// is the distance between the 64-column sub-tiles.
constexpr uint32_t kSwSub = 16384;
__device__ __forceinline__ uint32_t sw_chunk(int r, int j) {
    return static_cast<uint32_t>((j >> 3) * kSwSub + r * 128 + (((j & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint64_t smem_desc_sw(uint32_t addr, uint32_t lbo_bytes) {
    return static_cast<uint64_t>((addr & 0x3FFFF) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_sw_k(uint32_t tile, int k) {
    return smem_desc_sw(tile + (k >> 2) * kSwSub + (k & 3) * 32, 16);
}
__device__ __forceinline__ uint64_t desc_sw_mn(uint32_t tile, int k) {
    return smem_desc_sw(tile + k * 2048, kSwSub);
}

}  // namespace tc
}  // namespace mb200
