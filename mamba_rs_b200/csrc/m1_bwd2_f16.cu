// Instantiates the two-lane selective-scan backward kernels for f16 storage.
#include "m1_bwd2_kernel.cuh"

namespace mb200 {
void bwd2_kernels_f16(BwdKernelFn (*fn)[4], size_t* smem) { fill_bwd2<__half>(fn, smem); }
}  // namespace mb200
