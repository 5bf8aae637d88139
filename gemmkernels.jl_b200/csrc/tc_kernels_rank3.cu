// tcgen05 GEMM instances for plain matrices (3-D tensor maps).
#include "tc_kernels.cuh"

namespace gk {
template const void* tc_kernel_select_r<false>(int cg, int planes, bool tf32, bool dbg);
}
