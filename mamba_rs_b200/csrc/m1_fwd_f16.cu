// Instantiates the fused selective-scan forward kernels for f16 storage.
#include "m1_fwd_kernel.cuh"

namespace mb200 {
int fwd_variants_f16(FwdVariant* v) { return build_fwd_variants<__half>(v); }
}  // namespace mb200
