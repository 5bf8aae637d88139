// Launch description of the tcgen05 path (host side).
#pragma once
#include <string>

#include "common.h"
#include "tc_gemm.cuh"

namespace gk {

// An operand of the product as the tcgen05 path sees it.  An index (M or N, and K) may be split in
// two modes: index = in + ext[0] * out, with its own stride per mode (tensor contractions); plain
// matrices have ext[1] == 1.
struct TcOperand {
  const void* ptr = nullptr;
  int32_t dtype = 0;
  bool mn_major = false;         // the stride-1 index is the M/N index (else the K index)
  int64_t mn_ext[2] = {1, 1}, mn_str[2] = {0, 0};
  int64_t k_ext[2] = {1, 1}, k_str[2] = {0, 0};
  int64_t plane_stride = 0;      // complex / dual: elements between the two planes
};

struct TcProblem {
  int64_t M = 0, N = 0, K = 0;
  int32_t number = GK_REAL;
  TcOperand A, B;
  bool rank5 = false;            // operands need the two-mode split (5-D tensor maps)
  bool generic = false;          // operands are not TMA-addressable (alignment): producers use bounds-checked loads
  // output / C: two-mode split of M and N with strides per mode
  const void* C = nullptr;
  void* D = nullptr;
  bool has_c = false;            // the epilogue reads C (beta != 0 and C is not Layout.Zero), whether or not the pointer is known yet
  int32_t dtype_c = GK_F32, dtype_d = GK_F32;
  int64_t m_ext0 = 0, n_ext0 = 0;           // inner extents (== M, N for plain matrices)
  int64_t c_sm[2] = {1, 0}, c_sn[2] = {0, 0}, d_sm[2] = {1, 0}, d_sn[2] = {0, 0};
  int64_t c_plane = 0, d_plane = 0;
  double alpha = 1.0, beta = 0.0;
  const gk_epilogue_desc* epi = nullptr;
  int32_t tile_n = 0, cta_group = 0, stages = 0, raster = 0, raster_group = 0, max_ctas = 0, debug = 0;
  int32_t kps = 0;               // k-blocks per pipeline stage (0 = choose)
  // split-K: number of contiguous runs the k-blocks are cut into (0 or 1 = none); with k_split > 1, D must be an
  // FP32 workspace of k_split planes, split_stride elements apart, and C, bias and activation are left out
  int32_t k_split = 0;
  int64_t split_stride = 0;
  // strided-batched real products (plain matrices only): operand strides in elements, 0 = shared
  int32_t batch = 1;
  int64_t batch_a = 0, batch_b = 0, batch_c = 0, batch_d = 0;
};

// How many runs to cut K into for this problem on this GPU: 1 unless the tiles fill less than half of the
// CTA slots and K is long.  `L` is the plan without splitting.
struct TcLaunch;
int tc_choose_k_split(const TcProblem& pr, const TcLaunch& L, int sm_count);

struct TcLaunch {
  TcParams params;
  const void* kernel = nullptr;
  int cg = 1, planes = 1;
  bool tf32 = false, rank5 = false, generic = false;
  int grid = 0;
  int smem_bytes = 0;
};

// True when the descriptor (and, if given, the operand addresses) can go through TMA + tcgen05.
bool tc_eligible(const gk_gemm_desc& d, const void* a, const void* b, std::string* why);
// True when the only obstacle to tc_eligible is TMA's alignment rule (base address, leading dimension,
// batch stride) and the product is one the generic-load form of the kernel takes: real, 16-bit operands.
bool tc_eligible_generic(const gk_gemm_desc& d, std::string* why);
// gk_gemm_desc -> TcProblem (plain matrices).
void tc_problem_from_gemm(const gk_gemm_desc& d, const gk_epilogue_desc* epi, const void* a, const void* b,
                          const void* c, void* dd, TcProblem* out);
// Tile choice, descriptors, grid, epilogue and (when `encode`) the TMA tensor maps.
gk_status tc_plan(gk_handle h, const TcProblem& pr, bool encode, TcLaunch* out);
gk_status tc_launch(const TcLaunch& L, cudaStream_t stream);
// Runs the planned product `L` of `pr`.  Given a 256-byte aligned workspace, a product with few output
// tiles and a long K is cut into K-runs over the otherwise idle SMs: FP32 partial sums go to the
// workspace (as many runs as it holds) and a reduction pass applies alpha, beta, bias and activation
// and writes D the way the one-pass epilogue would.  Without one (or when nothing is gained) `L` runs as is.
gk_status tc_run(gk_handle h, const TcProblem& pr, const TcLaunch& L, void* workspace, int64_t workspace_bytes,
                 cudaStream_t stream);
// Bytes of workspace with which tc_run would cut K for this problem (0: it would not).
int64_t tc_split_workspace_bytes(gk_handle h, const TcProblem& pr, const TcLaunch& L);

}  // namespace gk
