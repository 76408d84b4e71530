// Instantiates the fused selective-scan forward kernels for f32 storage.
#include "m1_fwd_kernel.cuh"

namespace mb200 {
int fwd_variants_f32(FwdVariant* v) { return build_fwd_variants<float>(v); }
}  // namespace mb200
