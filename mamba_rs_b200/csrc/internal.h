// Host-side internals shared by the entry points: the per-device handle, error
// reporting and the TMA tensor-map builder.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/mamba_b200.h"

namespace mb200 {

struct Ctx {
    int device = -1;
    int sm_count = 0;
    int* d_status = nullptr;  // device status word (bounded-wait timeouts)
    char err[512] = {0};
    void* encode_tiled = nullptr;  // cuTensorMapEncodeTiled, resolved through the runtime
};

inline int fail(Ctx* c, int code, const char* fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof(c->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

inline size_t dtype_size(int dtype) { return dtype == MAMBA_B200_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) {
    return dtype == MAMBA_B200_F32 || dtype == MAMBA_B200_F16 || dtype == MAMBA_B200_BF16;
}

// Describes a [B, T, cols] tensor with row stride ld (elements) as a 3-D TMA
// tensor (cols innermost) and a box of [1, box_rows, box_cols].  Returns false
// when the layout breaks a TMA rule (16-byte base / stride / inner-box size),
// in which case the caller uses the plain-load path for that tensor.
bool make_tmap_3d(Ctx* c, CUtensorMap* map, int dtype, const void* base, long long ld, int cols,
                  int T, int B, int box_cols, int box_rows);

// Describes a 16-bit [B, T, heads, cols] tensor (contiguous) as a 4-D TMA tensor with a box
// of 64 columns x 1 head x 128 rows and 128-byte swizzle: one copy lands a [128 x 64]
// sub-tile of the Mamba-3 tensor-core kernels; columns past `cols` and rows past T read as
// zeros.
bool make_tmap_head_tile(Ctx* c, CUtensorMap* map, int dtype, const void* base, int cols, int heads, int T,
                         int B);

#define MB200_CUDA_CHECK(ctx, expr)                                                          \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return ::mb200::fail(ctx, MAMBA_B200_ERR_CUDA, "%s failed: %s", #expr,           \
                                 cudaGetErrorString(_e));                                    \
    } while (0)

}  // namespace mb200
