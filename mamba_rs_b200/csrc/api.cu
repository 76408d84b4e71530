// Handle life-cycle, error reporting and the TMA tensor-map builder.
#include <string.h>

#include <new>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_tmap_3d(Ctx* c, CUtensorMap* map, int dtype, const void* base, long long ld, int cols,
                  int T, int B, int box_cols, int box_rows) {
    if (!c->encode_tiled || !base) return false;
    const size_t es = dtype_size(dtype);
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
    if ((static_cast<size_t>(ld) * es) % 16 != 0) return false;
    if ((static_cast<size_t>(box_cols) * es) % 16 != 0) return false;
    if (box_cols > 256 || box_rows > 256 || box_cols < 1 || box_rows < 1) return false;
    if (ld < cols) return false;
    CUtensorMapDataType dt = dtype == MAMBA_B200_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == MAMBA_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(T),
                          static_cast<cuuint64_t>(B)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es,
                             static_cast<cuuint64_t>(ld) * es * static_cast<cuuint64_t>(T)};
    if (strides[1] >= (1ull << 40)) return false;
    cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(c->encode_tiled)(
        map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_tmap_head_tile(Ctx* c, CUtensorMap* map, int dtype, const void* base, int cols, int heads, int T,
                         int B) {
    if (!c->encode_tiled || !base || dtype == MAMBA_B200_F32) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || cols % 8 != 0 || cols < 8 || heads < 1) return false;
    const cuuint64_t rs = static_cast<cuuint64_t>(heads) * cols * 2;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(heads),
                          static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(cols) * 2, rs, rs * static_cast<cuuint64_t>(T)};
    if (strides[2] >= (1ull << 40)) return false;
    cuuint32_t box[4] = {64, 1, 128, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(c->encode_tiled)(
        map, dtype == MAMBA_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

int m1_fwd_configure(Ctx* c);   // m1_fwd.cu: raises dynamic shared-memory limits
int m1_bwd_configure(Ctx* c);   // m1_bwd.cu
int m3_configure(Ctx* c);       // m3_ssd.cu
int m3_bwd_configure(Ctx* c);   // m3_ssd_bwd.cu
int norm_configure(Ctx* c);     // norm.cu
int conv_configure(Ctx* c);     // m1_step_conv.cu
int train_ops_configure(Ctx* c);  // train_ops.cu

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API int mamba_b200_init(int device, void** handle) {
    if (!handle) return MAMBA_B200_ERR_ARG;
    *handle = nullptr;
    Ctx* c = new (std::nothrow) Ctx();
    if (!c) return MAMBA_B200_ERR_CUDA;
    *handle = c;  // returned even on failure so last_error() can be read
    c->device = device;
    MB200_CUDA_CHECK(c, cudaSetDevice(device));
    cudaDeviceProp prop;
    MB200_CUDA_CHECK(c, cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(c, MAMBA_B200_ERR_DEVICE,
                    "device %d is sm_%d%d; this library holds sm_100a code only", device,
                    prop.major, prop.minor);
    c->sm_count = prop.multiProcessorCount;
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
        c->encode_tiled = fn;
    MB200_CUDA_CHECK(c, cudaMalloc(&c->d_status, sizeof(int)));
    MB200_CUDA_CHECK(c, cudaMemset(c->d_status, 0, sizeof(int)));
    int rc = MAMBA_B200_OK;
    rc = m1_fwd_configure(c);
    if (rc) return rc;
    rc = m1_bwd_configure(c);
    if (rc) return rc;
    rc = m3_configure(c);
    if (rc) return rc;
    rc = m3_bwd_configure(c);
    if (rc) return rc;
    rc = norm_configure(c);
    if (rc) return rc;
    rc = conv_configure(c);
    if (rc) return rc;
    rc = train_ops_configure(c);
    if (rc) return rc;
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API int mamba_b200_destroy(void* handle) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_OK;
    if (c->d_status) {
        cudaSetDevice(c->device);
        cudaFree(c->d_status);
    }
    delete c;
    return MAMBA_B200_OK;
}

extern "C" MAMBA_B200_API const char* mamba_b200_last_error(void* handle) {
    Ctx* c = static_cast<Ctx*>(handle);
    return c ? c->err : "null handle";
}

extern "C" MAMBA_B200_API int mamba_b200_check_status(void* handle, void* stream) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    int cur = -1;
    MB200_CUDA_CHECK(c, cudaGetDevice(&cur));
    if (cur != c->device)
        return fail(c, MAMBA_B200_ERR_DEVICE, "check_status: the handle belongs to device %d but device %d is current",
                    c->device, cur);
    int st = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MB200_CUDA_CHECK(c, cudaMemcpyAsync(&st, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    MB200_CUDA_CHECK(c, cudaStreamSynchronize(s));
    if (st != kStatusOk) {
        cudaMemsetAsync(c->d_status, 0, sizeof(int), s);
        return fail(c, MAMBA_B200_ERR_KERNEL, "a kernel gave up a bounded wait (status %d)", st);
    }
    return MAMBA_B200_OK;
}

namespace mb200 {
// One thread waits on an mbarrier that nothing ever arrives on, with a small poll
// limit: the wait gives up, records the time-out in the status word and the kernel
// returns normally.
__global__ void wait_timeout_selftest_kernel(int* status, int max_polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_barrier_init();
        mbar_wait(&bar, 0, status, max_polls);
    }
}
}  // namespace mb200

extern "C" MAMBA_B200_API int mamba_b200_selftest_wait_timeout(void* handle, void* stream, int max_polls) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (max_polls < 1 || max_polls > 100000)
        return fail(c, MAMBA_B200_ERR_ARG, "selftest_wait_timeout: max_polls %d outside 1..100000", max_polls);
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c->d_status, max_polls);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}
