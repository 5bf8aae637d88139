// tcgen05 GEMM instances for tensor contractions (5-D tensor maps).
#include "tc_kernels.cuh"

namespace gk {
template const void* tc_kernel_select_r<true>(int cg, int planes, bool tf32, bool dbg);
}
