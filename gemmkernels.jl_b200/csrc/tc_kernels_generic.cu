// tcgen05 GEMM instance whose producers use bounds-checked loads instead of TMA (operands whose base
// or leading dimension is not a multiple of 16 bytes).
#include "tc_gemm.cuh"

namespace gk {
const void* tc_kernel_generic(bool dbg) {
  return dbg ? reinterpret_cast<const void*>(&tc_gemm_kernel<1, 1, false, false, true, true>)
             : reinterpret_cast<const void*>(&tc_gemm_kernel<1, 1, false, false, true, false>);
}
}  // namespace gk
