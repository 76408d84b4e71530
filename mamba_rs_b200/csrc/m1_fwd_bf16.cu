// Instantiates the fused selective-scan forward kernels for bf16 storage.
#include "m1_fwd_kernel.cuh"

namespace mb200 {
int fwd_variants_bf16(FwdVariant* v) { return build_fwd_variants<__nv_bfloat16>(v); }
}  // namespace mb200
