// Kernel-instance table of the tcgen05 GEMM: included by the two translation units that instantiate it.
#pragma once
#include "tc_gemm.cuh"
#include "tc_plan.h"

namespace gk {

template <int CG, int PLANES, bool TF32, bool RANK5>
static const void* tc_kernel_ptr(bool dbg) {
  return dbg ? reinterpret_cast<const void*>(&tc_gemm_kernel<CG, PLANES, TF32, RANK5, false, true>)
             : reinterpret_cast<const void*>(&tc_gemm_kernel<CG, PLANES, TF32, RANK5, false, false>);
}

template <bool RANK5>
const void* tc_kernel_select_r(int cg, int planes, bool tf32, bool dbg) {
  if (cg == 1) {
    if (planes == 1) return tf32 ? tc_kernel_ptr<1, 1, true, RANK5>(dbg) : tc_kernel_ptr<1, 1, false, RANK5>(dbg);
    return tf32 ? tc_kernel_ptr<1, 2, true, RANK5>(dbg) : tc_kernel_ptr<1, 2, false, RANK5>(dbg);
  }
  if (planes == 1) return tf32 ? tc_kernel_ptr<2, 1, true, RANK5>(dbg) : tc_kernel_ptr<2, 1, false, RANK5>(dbg);
  return tf32 ? tc_kernel_ptr<2, 2, true, RANK5>(dbg) : tc_kernel_ptr<2, 2, false, RANK5>(dbg);
}

}  // namespace gk
