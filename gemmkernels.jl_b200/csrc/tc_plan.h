// Launch description of the tcgen05 path (host side).
#pragma once
#include <string>

#include "common.h"
#include "tc_gemm.cuh"

namespace gk {

struct TcLaunch {
  TcParams params;
  const void* kernel = nullptr;
  int cg = 1, planes = 1;
  bool tf32 = false;
  int grid = 0;
  int smem_bytes = 0;
};

// True when the descriptor (and, if given, the operand addresses) can go through TMA + tcgen05.
bool tc_eligible(const gk_gemm_desc& d, const void* a, const void* b, std::string* why);
// Fills everything but the tensor maps (tile choice, descriptors, grid, epilogue).
gk_status tc_plan(gk_handle h, const gk_gemm_desc& d, const gk_epilogue_desc* epi, const void* a,
                  const void* b, const void* c, void* dd, TcLaunch* out);
// Encodes the TMA tensor maps of A and B for the planned tile.
gk_status tc_encode_maps(gk_handle h, const gk_gemm_desc& d, const void* a, const void* b, TcLaunch* L);
gk_status tc_launch(const TcLaunch& L, cudaStream_t stream);

}  // namespace gk
