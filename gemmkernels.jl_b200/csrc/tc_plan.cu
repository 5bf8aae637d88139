// Host side of the tcgen05 path: eligibility, tile choice, TMA tensor maps, launch.
#include <cstdlib>
#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.h"
#include "tc_gemm.cuh"
#include "splitk_reduce.cuh"
#include "tc_plan.h"

namespace gk {

static int tc_dtype_of(int32_t dt) {
  switch (dt) {
    case GK_F16: return TC_F16;
    case GK_BF16: return TC_BF16;
    case GK_F32: return TC_F32;
    default: return -1;
  }
}

// Everything tc_eligible asks for except TMA's alignment rules.
static bool tc_eligible_types(const gk_gemm_desc& d, std::string* why) {
  auto no = [&](const char* s) { if (why) *why = s; return false; };
  if (d.layout_a != GK_LAYOUT_DENSE || d.layout_b != GK_LAYOUT_DENSE)
    return no("operand layout is not dense");
  if (d.dtype_a != d.dtype_b) return no("A and B element types differ");
  const int32_t comp = d.compute;
  if (d.dtype_a == GK_F16) { if (comp != GK_F16) return no("Float16 operands need compute = F16"); }
  else if (d.dtype_a == GK_BF16) { if (comp != GK_BF16) return no("BFloat16 operands need compute = BF16"); }
  else if (d.dtype_a == GK_F32) { if (comp != GK_TF32) return no("Float32 operands reach the tensor cores only as TF32"); }
  else return no("element type has no tensor-core path");
  if (tc_dtype_of(d.dtype_c) < 0 || tc_dtype_of(d.dtype_d) < 0)
    return no("C/D element type must be Float16, BFloat16 or Float32");
  if (d.m < 1 || d.n < 1 || d.k < 1) return no("empty dimension");
  if (d.m > INT32_MAX / 2 || d.n > INT32_MAX / 2 || d.k > INT32_MAX / 2) return no("dimension too large");
  return true;
}

bool tc_eligible_generic(const gk_gemm_desc& d, std::string* why) {
  if (!tc_eligible_types(d, why)) return false;
  auto no = [&](const char* s) { if (why) *why = s; return false; };
  if (d.number != GK_REAL) return no("complex and dual operands must be 16-byte aligned planes");
  if (dtype_size(d.dtype_a) != 2) return no("32-bit operands must be 16-byte aligned");
  return true;
}

bool tc_eligible(const gk_gemm_desc& d, const void* a, const void* b, std::string* why) {
  if (!tc_eligible_types(d, why)) return false;
  auto no = [&](const char* s) { if (why) *why = s; return false; };
  const int es = dtype_size(d.dtype_a);
  // TMA: 16-byte aligned base, strides that are multiples of 16 bytes.
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
    return no("operand base address is not 16-byte aligned");
  if ((d.lda * es) % 16 || (d.ldb * es) % 16) return no("leading dimension is not a multiple of 16 bytes");
  if (d.batch > 1 && ((d.batch_stride_a * es) % 16 || (d.batch_stride_b * es) % 16))
    return no("batch stride is not a multiple of 16 bytes");
  if (d.number != GK_REAL) {
    if (d.plane_a == 0 || d.plane_b == 0) return no("interleaved complex operands need the split pre-pass");
    if ((d.plane_a * es) % 16 || (d.plane_b * es) % 16) return no("plane stride is not a multiple of 16 bytes");
  }
  return true;
}

// Plain matrix operand -> 3-D tensor map {contiguous, strided, plane}.
static gk_status encode_plain(gk_handle h, CUtensorMap* tm, const TcOperand& op, int planes, int box_contig,
                              int box_other, CUtensorMapSwizzle swizzle, int batch = 1, int64_t batch_stride = 0) {
  const int es = dtype_size(op.dtype);
  CUtensorMapDataType tdt = op.dtype == GK_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                            : op.dtype == GK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const int64_t c_ext = op.mn_major ? op.mn_ext[0] : op.k_ext[0];
  const int64_t o_ext = op.mn_major ? op.k_ext[0] : op.mn_ext[0];
  const int64_t o_str = op.mn_major ? op.k_str[0] : op.mn_str[0];
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(c_ext), static_cast<cuuint64_t>(o_ext), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2];
  strides[0] = static_cast<cuuint64_t>(o_str) * es;
  strides[1] = planes > 1 ? static_cast<cuuint64_t>(op.plane_stride) * es : strides[0] * dims[1];
  if (planes == 1 && batch > 1 && batch_stride > 0) {   // the third mode walks the products of a batch
    dims[2] = static_cast<cuuint64_t>(batch);
    strides[1] = static_cast<cuuint64_t>(batch_stride) * es;
  }
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_contig), static_cast<cuuint32_t>(box_other), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = h->encode_tiled(tm, tdt, 3, const_cast<void*>(op.ptr), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(GK_ERR_INVALID_CONFIG, "cuTensorMapEncodeTiled failed (%d): extents (%llu, %llu, %llu) box (%u, %u)",
                     static_cast<int>(r), (unsigned long long)dims[0], (unsigned long long)dims[1],
                     (unsigned long long)dims[2], box[0], box[1]);
  return GK_OK;
}

// Two-mode operands (contractions) use 5-D tensor maps whose modes are listed in the order in which a box
// is to lie in shared memory, not by stride (TMA adds coordinate x stride per mode; nothing asks for
// nested or increasing strides):
//   MN-major: mn_in (contiguous), k_in, k_out, mn_out  - spans of the contiguous mode, each with its K rows in order
//   K-major : k_in (contiguous), mn_in, mn_out, k_out  - the tile's rows in order, 128 bytes of K each
// and the plane last.  order[i] = which of (0 mn_in, 1 mn_out, 2 k_in, 3 k_out) sits at position i; *perm
// packs the position of each of the four, 3 bits apiece.
static void plan_modes(const TcOperand& op, int order[4], int32_t* perm) {
  static const int mn_first[4] = {0, 2, 3, 1}, k_first[4] = {2, 0, 1, 3};
  for (int i = 0; i < 4; ++i) order[i] = op.mn_major ? mn_first[i] : k_first[i];
  *perm = 0;
  for (int i = 0; i < 4; ++i) *perm |= i << (3 * order[i]);
}

// mode_box[m] = extent of a box along mode m (numbered as above); the plane has box 1.
static gk_status encode_modes(gk_handle h, CUtensorMap* tm, const TcOperand& op, int planes, const int mode_box[4],
                              CUtensorMapSwizzle swizzle) {
  const int es = dtype_size(op.dtype);
  CUtensorMapDataType tdt = op.dtype == GK_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                            : op.dtype == GK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const int64_t ext[4] = {op.mn_ext[0], op.mn_ext[1], op.k_ext[0], op.k_ext[1]};
  const int64_t str[4] = {op.mn_str[0], op.mn_str[1], op.k_str[0], op.k_str[1]};
  int order[4];
  int32_t perm;
  plan_modes(op, order, &perm);
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
  cuuint64_t covered = 16;   // bytes spanned by the modes: the stride given to unit modes (any multiple of 16 would do)
  for (int m = 0; m < 4; ++m)
    if (ext[m] > 1) covered = std::max<cuuint64_t>(covered, static_cast<cuuint64_t>(str[m]) * es * ext[m]);
  covered = (covered + 15) / 16 * 16;
  for (int i = 0; i < 4; ++i) {
    const int m = order[i];
    dims[i] = static_cast<cuuint64_t>(ext[m]);
    if (i > 0) strides[i - 1] = ext[m] > 1 ? static_cast<cuuint64_t>(str[m]) * es : covered;
    box[i] = static_cast<cuuint32_t>(std::max(1, mode_box[m]));
  }
  dims[4] = static_cast<cuuint64_t>(planes);
  strides[3] = planes > 1 ? static_cast<cuuint64_t>(op.plane_stride) * es : covered;
  box[4] = 1;
  CUresult r = h->encode_tiled(tm, tdt, 5, const_cast<void*>(op.ptr), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(GK_ERR_INVALID_CONFIG,
                     "cuTensorMapEncodeTiled failed (%d): extents (%llu, %llu, %llu, %llu) box (%u, %u, %u, %u)",
                     static_cast<int>(r), (unsigned long long)dims[0], (unsigned long long)dims[1],
                     (unsigned long long)dims[2], (unsigned long long)dims[3], box[0], box[1], box[2], box[3]);
  return GK_OK;
}

// The kernel instances are compiled in two translation units of their own (tc_kernels_rank3.cu,
// tc_kernels_rank5.cu), which is what makes the build parallel.
template <bool RANK5>
const void* tc_kernel_select_r(int cg, int planes, bool tf32, bool dbg);
extern template const void* tc_kernel_select_r<false>(int cg, int planes, bool tf32, bool dbg);
extern template const void* tc_kernel_select_r<true>(int cg, int planes, bool tf32, bool dbg);

const void* tc_kernel_generic(bool dbg);   // tc_kernels_generic.cu: <1, 1, false, false, GENERIC, dbg>

// dbg: the instance that honours the descriptor's diagnostic bits (the production instance compiles them out)
static const void* tc_kernel_select(int cg, int planes, bool tf32, bool rank5, bool dbg) {
  return rank5 ? tc_kernel_select_r<true>(cg, planes, tf32, dbg) : tc_kernel_select_r<false>(cg, planes, tf32, dbg);
}

static constexpr int kSmemBudget = 232448;  // 227 KiB opt-in limit per CTA on sm_100
static constexpr int kCtrlBytes = 256;
static constexpr double kWideEff = 1.08;   // measured gain of the single-stage 512-column tiles on large products

static int stage_bytes_for(int cg, int bn, int n_sub, int a_planes, int b_planes) {
  return a_planes * kTcTileM * kTcKBytes + n_sub * b_planes * (bn / cg) * kTcKBytes;
}

// Can a box of `total` elements starting at multiples of `total` be cut from an index whose inner
// mode has extent ext0 (and whose outer mode continues it)?
static bool box_fits(int64_t ext0, int64_t ext1, int total) {
  if (ext1 <= 1) return true;                 // single mode: TMA clips at the end
  if (ext0 >= total) return ext0 % total == 0;
  return total % ext0 == 0 && total / ext0 <= 256;
}

// Picks (cta_group, tile_n): fewest "tile-time" units over the persistent grid, where a larger
// tile is worth more per unit time (operand reuse) but quantises worse on small problems.
// A tile is n_sub column blocks of bn columns (bn = the MMA's N, <= 256).  Tiles whose accumulators
// fill all 512 TMEM columns (n_sub * planes * bn == 512) run with one accumulator stage: their
// epilogue is not overlapped, which the efficiency figure accounts for; they pay off on large
// problems, where the main loop is limited by the operand feed from L2 rather than by the MMAs.
static void choose_tile(const TcProblem& pr, int sm_count, int planes, int* cg_out, int* bn_out, int* nsub_out) {
  // an N-contiguous B is loaded in boxes of 128 bytes of N per CTA
  int n_unit = pr.B.mn_major ? kTcKBytes / dtype_size(pr.B.dtype) : 8;
  if (pr.rank5 && pr.B.mn_major && pr.B.mn_ext[1] > 1 && pr.B.mn_ext[0] < n_unit) n_unit = static_cast<int>(pr.B.mn_ext[0]);
  struct Cand { int cg, bn, n_sub; double eff; };
  static const Cand cands[] = {{2, 256, 2, kWideEff}, {2, 256, 1, 1.00}, {1, 256, 1, 0.92}, {2, 128, 1, 0.80},
                               {1, 128, 1, 0.74},     {1, 64, 1, 0.50},  {1, 32, 1, 0.24}};   // 32 columns: only when it saves a round (512x512x2048: 11.9 us against 9.5 with 64)
  double best = 1e300;
  int bcg = 1, bbn = 128, bns = 1;
  for (const Cand& c : cands) {
    if (c.n_sub * planes * c.bn > 512) continue;  // accumulators of one tile must fit 512 TMEM columns
    if (c.n_sub > 1 && pr.rank5) continue;
    if (pr.generic && (c.cg != 1 || c.n_sub != 1)) continue;
    if ((c.bn / c.cg) % n_unit) continue;
    if (pr.cta_group && c.cg != pr.cta_group) continue;
    if (pr.tile_n && c.bn * c.n_sub != pr.tile_n) continue;
    if (!pr.B.mn_major && !box_fits(pr.B.mn_ext[0], pr.B.mn_ext[1], c.bn / c.cg)) continue;
    if (!pr.B.mn_major && pr.B.mn_ext[1] > 1 && pr.B.mn_ext[0] < c.bn / c.cg && (c.bn / c.cg) / pr.B.mn_ext[0] > 16) continue;
    if (pr.n_ext0 < pr.N && (pr.n_ext0 % 32 != 0)) continue;
    const int64_t tm = (pr.M + 128 * c.cg - 1) / (128 * c.cg);
    const int64_t tn = (pr.N + c.bn * c.n_sub - 1) / (c.bn * c.n_sub);
    const int64_t slots = std::max(1, sm_count / c.cg);
    const int64_t waves = (tm * tn * std::max(1, pr.batch) + slots - 1) / slots;
    // a single accumulator stage exposes the epilogue: worth it only when the main loop is long
    double eff = c.eff;
    if (planes == 2) {
      // Two-plane products issue three or four MMAs per k-step on the same operands, so a 128-column tile
      // already keeps the tensor pipe as busy as a real 512-column tile does, and its two planes leave room
      // for a second accumulator stage.  Measured (4096^3, planar): complex 374 -> 357 us, dual 381 -> 303 us
      // against 256-column tiles, whose single stage exposes the two-plane epilogue; level at 2048^3 and 8192^3.
      eff = c.bn == 256 ? 0.90 : (c.bn == 128 ? (c.cg == 2 ? 1.00 : 0.90) : c.eff);
    } else if (c.n_sub * planes * c.bn > 256) {
      // an epilogue that also reads C (or writes through the general path) is several times
      // longer; exposed, it eats the gain
      const bool light = !pr.has_c;
      eff = pr.K >= 1024 ? (light ? kWideEff : 0.85) : 0.5;
    }
    const double t = static_cast<double>(waves) * c.bn * c.n_sub / eff;
    if (t < best) { best = t; bcg = c.cg; bbn = c.bn; bns = c.n_sub; }
  }
  if (best == 1e300) {  // overrides that match no candidate: honour them if they are valid
    bcg = pr.generic ? 1 : pr.cta_group ? pr.cta_group : 1;
    bbn = pr.tile_n ? pr.tile_n : 128;
    if (bbn == 512) { bbn = 256; bns = 2; }
  }
  *cg_out = bcg;
  *bn_out = bbn;
  *nsub_out = bns;
}

// Tile choices measured on B200 by the tuning sweep (generated file; see tuning.emit_table).
static const gk_tuning_entry kBuiltinTuning[] = {
#include "tuned_table.inc"
    {-1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}   // terminator
};

// Nearest measured entry for this problem (see gk_tuning_entry), or nullptr.
static const gk_tuning_entry* tuning_lookup(gk_handle h, const TcProblem& pr, gk_tuning_entry* copy) {
  if (pr.rank5 || pr.generic || pr.number != GK_REAL || pr.batch > 1 || pr.k_split > 1) return nullptr;
  const int has_c = pr.has_c ? 1 : 0;
  const int ta = pr.A.mn_major ? 0 : 1, tb = pr.B.mn_major ? 1 : 0;
  double best = 1e30;
  const gk_tuning_entry* hit = nullptr;
  auto consider = [&](const gk_tuning_entry& e) {
    if (e.dtype != pr.A.dtype || e.trans_a != ta || e.trans_b != tb || e.has_c != has_c) return;
    if (e.m < 1 || e.n < 1 || e.k < 1) return;
    double dist = 0.0;
    const double have[3] = {static_cast<double>(pr.M), static_cast<double>(pr.N), static_cast<double>(pr.K)};
    const double want[3] = {static_cast<double>(e.m), static_cast<double>(e.n), static_cast<double>(e.k)};
    for (int i = 0; i < 3; ++i) {
      const double r = have[i] / want[i];
      if (r > 1.5 || r < 1.0 / 1.5) return;
      dist += std::fabs(std::log2(r));
    }
    if (dist < best) { best = dist; hit = &e; }
  };
  {
    std::lock_guard<std::mutex> lock(h->mu);
    for (const gk_tuning_entry& e : h->tuning) consider(e);
    if (hit) { *copy = *hit; hit = copy; }       // the vector may be replaced once the lock is gone
  }
  for (const gk_tuning_entry* e = kBuiltinTuning; e->dtype >= 0; ++e) consider(*e);
  return hit;
}

void tc_problem_from_gemm(const gk_gemm_desc& d, const gk_epilogue_desc* epi, const void* a, const void* b,
                          const void* c, void* dd, TcProblem* out) {
  TcProblem& pr = *out;
  pr = TcProblem{};
  pr.M = d.m; pr.N = d.n; pr.K = d.k; pr.number = d.number;
  pr.A.ptr = a; pr.A.dtype = d.dtype_a; pr.A.mn_major = d.trans_a == 0;  // column-major M x K: M contiguous
  pr.A.mn_ext[0] = d.m; pr.A.k_ext[0] = d.k;
  pr.A.mn_str[0] = pr.A.mn_major ? 1 : d.lda; pr.A.k_str[0] = pr.A.mn_major ? d.lda : 1;
  pr.A.plane_stride = d.plane_a;
  pr.B.ptr = b; pr.B.dtype = d.dtype_b; pr.B.mn_major = d.trans_b != 0;  // column-major K x N: K contiguous
  pr.B.mn_ext[0] = d.n; pr.B.k_ext[0] = d.k;
  pr.B.mn_str[0] = pr.B.mn_major ? 1 : d.ldb; pr.B.k_str[0] = pr.B.mn_major ? d.ldb : 1;
  pr.B.plane_stride = d.plane_b;
  pr.C = (d.layout_c == GK_LAYOUT_ZERO) ? nullptr : c; pr.D = dd;
  pr.dtype_c = d.dtype_c; pr.dtype_d = d.dtype_d;
  pr.m_ext0 = d.m; pr.n_ext0 = d.n;
  pr.c_sm[0] = 1; pr.c_sn[0] = d.ldc; pr.d_sm[0] = 1; pr.d_sn[0] = d.ldd;
  pr.c_plane = d.plane_c; pr.d_plane = d.plane_d;
  pr.has_c = d.layout_c != GK_LAYOUT_ZERO && d.beta != 0.0;
  pr.alpha = d.alpha; pr.beta = d.beta; pr.epi = epi;
  pr.tile_n = d.tile_n; pr.cta_group = d.cta_group; pr.stages = d.stages; pr.raster = d.raster;
  pr.raster_group = d.raster_group; pr.max_ctas = d.max_ctas; pr.debug = d.debug;
  pr.kps = d.k_blocks_per_stage;
  if (d.batch > 1) {
    pr.batch = d.batch;
    pr.batch_a = d.batch_stride_a; pr.batch_b = d.batch_stride_b; pr.batch_c = d.batch_stride_c; pr.batch_d = d.batch_stride_d;
  }
}

static int32_t clamp_div(int64_t ext0, int64_t ext1) {
  if (ext1 <= 1 || ext0 >= INT32_MAX) return INT32_MAX;
  return static_cast<int32_t>(ext0);
}

gk_status tc_plan(gk_handle h, const TcProblem& pr_in, bool encode, TcLaunch* out) {
  TcProblem pr_tuned;
  const TcProblem* prp = &pr_in;
  if (pr_in.tile_n == 0 && pr_in.cta_group == 0) {
    gk_tuning_entry copy;
    if (const gk_tuning_entry* e = tuning_lookup(h, pr_in, &copy)) {
      pr_tuned = pr_in;
      pr_tuned.tile_n = e->tile_n; pr_tuned.cta_group = e->cta_group;
      if (pr_tuned.stages == 0) pr_tuned.stages = e->stages;
      if (pr_tuned.raster_group == 0 && pr_tuned.raster == GK_RASTER_AUTO) pr_tuned.raster_group = e->raster_group;
      if (pr_tuned.kps == 0) pr_tuned.kps = e->k_blocks_per_stage;
      prp = &pr_tuned;
    }
  }
  const TcProblem& pr = *prp;
  TcParams& p = out->params;
  std::memset(&p, 0, sizeof(p));
  const int es = dtype_size(pr.A.dtype);
  const bool tf32 = pr.A.dtype == GK_F32;
  const int planes = pr.number == GK_REAL ? 1 : 2;

  int cg, bn, n_sub;
  choose_tile(pr, h->sm_count, planes, &cg, &bn, &n_sub);
  if (cg != 1 && cg != 2)
    return set_error(GK_ERR_INVALID_CONFIG, "cta_group must be 1 or 2, got %d", cg);
  if (pr.generic && (cg != 1 || n_sub != 1 || planes != 1 || tf32 || pr.rank5))
    return set_error(GK_ERR_INVALID_CONFIG, "operands that are not 16-byte aligned run one CTA per tile (cta_group = 1, "
                     "tile_n <= 256), real 16-bit types only");
  if (bn < 32 || bn > 256 || bn % 32 || n_sub * planes * bn > 512 || (cg == 2 && bn % 64))
    return set_error(GK_ERR_INVALID_CONFIG,
                     "tile_n = %d is not usable (multiple of 32 (64 for CTA pairs), <= %d)", bn * n_sub,
                     512 / planes);
  const int acc_stages = n_sub * planes * bn > 256 ? 1 : 2;

  p.M = static_cast<int32_t>(pr.M);
  p.N = static_cast<int32_t>(pr.N);
  p.K = static_cast<int32_t>(pr.K);
  p.bn = bn;
  p.n_sub = n_sub;
  p.acc_stages = acc_stages;
  p.bk = kTcKBytes / es;
  p.k_blocks = (p.K + p.bk - 1) / p.bk;
  p.k_split = 1; p.kb_per_split = std::max(1, p.k_blocks); p.split_stride = 0;
  if (pr.k_split > 1) {
    if (pr.dtype_d != GK_F32 || pr.C != nullptr || pr.epi != nullptr || pr.alpha != 1.0 || pr.m_ext0 < pr.M || pr.n_ext0 < pr.N)
      return set_error(GK_ERR_INVALID_ARGUMENT, "split-K writes raw partial sums into a plain FP32 workspace");
    p.kb_per_split = (p.k_blocks + pr.k_split - 1) / pr.k_split;
    p.k_split = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;   // no empty runs
    p.split_stride = pr.split_stride;
  }
  p.batch = 1;
  if (pr.batch > 1) {
    if (planes != 1 || pr.rank5 || pr.k_split > 1)
      return set_error(GK_ERR_INVALID_CONFIG, "batched products are plain real products without split-K");
    p.batch = pr.batch;
    p.a_batched = pr.batch_a > 0 ? 1 : 0; p.b_batched = pr.batch_b > 0 ? 1 : 0;
    p.c_batch = pr.batch_c; p.d_batch = pr.batch_d;
  }
  p.tiles_m = (p.M + kTcTileM * cg - 1) / (kTcTileM * cg);
  p.tiles_n = (p.N + bn * n_sub - 1) / (bn * n_sub);
  p.a_planes = p.b_planes = planes;
  p.a_mn_major = pr.A.mn_major ? 1 : 0;
  p.b_mn_major = pr.B.mn_major ? 1 : 0;
  const int bn_cta = bn / cg;
  p.a_plane_bytes = kTcTileM * kTcKBytes;
  p.b_plane_bytes = bn_cta * kTcKBytes;
  // MN-major operands are staged in boxes of one swizzle span of M/N by one k-block.  The span is
  // 128 bytes, except for a contraction whose contiguous mode is only 64 or 32 bytes long: the box
  // then is exactly that mode and the swizzle shrinks with it (a box is never narrower than its
  // swizzle span).  Atoms are 8 k rows of one span (16-bit types); 32-bit types must use the
  // 128-byte swizzle with 32-byte units (atoms of 4 k rows).  One MMA consumes 32 / es rows of K.
  struct MnGeom { uint32_t span, box_mn, box_bytes, sbo, swz, kadv; CUtensorMapSwizzle tma; bool ok; };
  auto mn_geom = [&](const TcOperand& op) {
    MnGeom g{};
    const int64_t inner_bytes = op.mn_ext[0] * es;
    uint32_t span = 128;
    if (pr.rank5 && op.mn_ext[1] > 1 && inner_bytes % 128 != 0) span = inner_bytes % 64 == 0 ? 64 : (inner_bytes % 32 == 0 ? 32 : 0);
    g.ok = span != 0 && !(es == 4 && span != 128);
    if (!g.ok) return g;
    g.span = span; g.box_mn = span / es; g.box_bytes = span * p.bk;
    if (es == 4) { g.sbo = 512; g.swz = 1; g.tma = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B; }
    else {
      g.sbo = 8 * span;
      g.swz = span == 128 ? 2 : (span == 64 ? 4 : 6);
      g.tma = span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (span == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    }
    g.kadv = (32 / es) * span;
    return g;
  };
  CUtensorMapSwizzle a_tma = CU_TENSOR_MAP_SWIZZLE_128B, b_tma = CU_TENSOR_MAP_SWIZZLE_128B;
  p.a_box_mn = p.b_box_mn = p.bk;
  if (p.a_mn_major) {
    const MnGeom g = mn_geom(pr.A);
    if (!g.ok) return set_error(GK_ERR_INVALID_CONFIG, "contiguous mode of A does not fill a swizzle span");
    p.a_box_mn = g.box_mn; p.a_boxes = kTcTileM / g.box_mn; p.a_box_bytes = g.box_bytes;
    p.a_lbo = g.box_bytes; p.a_sbo = g.sbo; p.a_kadv = g.kadv; p.a_swz = g.swz; a_tma = g.tma;
  } else {
    p.a_boxes = 1; p.a_box_bytes = p.a_plane_bytes;
    p.a_lbo = 16; p.a_sbo = 1024; p.a_kadv = 32; p.a_swz = 2;
  }
  if (p.b_mn_major) {
    const MnGeom g = mn_geom(pr.B);
    if (!g.ok) return set_error(GK_ERR_INVALID_CONFIG, "contiguous mode of B does not fill a swizzle span");
    if (bn_cta % g.box_mn)
      return set_error(GK_ERR_INVALID_CONFIG, "tile_n = %d too small for a transposed B of this type", bn);
    p.b_box_mn = g.box_mn; p.b_boxes = bn_cta / g.box_mn; p.b_box_bytes = g.box_bytes;
    p.b_lbo = g.box_bytes; p.b_sbo = g.sbo; p.b_kadv = g.kadv; p.b_swz = g.swz; b_tma = g.tma;
  } else {
    p.b_boxes = 1; p.b_box_bytes = p.b_plane_bytes;
    p.b_lbo = 16; p.b_sbo = 1024; p.b_kadv = 32; p.b_swz = 2;
  }
  if (pr.kps < 0 || pr.kps > 2) return set_error(GK_ERR_INVALID_CONFIG, "k_blocks_per_stage must be 1 or 2 (0 = choose), got %d", pr.kps);
  // Two-mode operands.  The modes of a tensor map are listed in shared-memory order, so one box can walk
  // both modes of an index: an MN-major box is one swizzle span of the contiguous mode by the k-block's rows
  // (inner contracted mode, then steps of the outer one), and when the contiguous mode is exactly one span
  // long the tile's spans - consecutive values of the outer M/N mode - join the same box, which then is the
  // operand's whole k-block; a K-major box is 128 bytes of K by the tile's rows (inner M/N mode, then steps
  // of the outer one).
  int a_box[4] = {1, 1, 1, 1}, b_box[4] = {1, 1, 1, 1};
  p.a_sub = p.b_sub = 1;
  p.a_sub_step = p.b_sub_step = 0; p.a_sub_bytes = p.b_sub_bytes = 0;
  if (pr.rank5) {
    auto plan_box = [&](const TcOperand& op, bool mn_major, int tile_rows, int box_mn, int32_t* boxes, int mode_box[4]) -> bool {
      const int need = mn_major ? p.bk : tile_rows;       // rows of one box
      const int64_t* e = mn_major ? op.k_ext : op.mn_ext;
      int rows, rows2 = 1;
      if (e[1] <= 1 || e[0] % need == 0) rows = need;
      else if (need % e[0] == 0) { rows = static_cast<int>(e[0]); rows2 = need / rows; }
      else return false;
      if (rows > 256 || rows2 > 256) return false;
      if (mn_major) {
        // the span must be cut from the inner mode
        if (op.mn_ext[1] > 1 && op.mn_ext[0] % box_mn != 0) return false;
        int spans = 1;
        if (op.mn_ext[1] > 1 && op.mn_ext[0] == box_mn) { spans = *boxes; *boxes = 1; }
        mode_box[0] = box_mn; mode_box[1] = spans; mode_box[2] = rows; mode_box[3] = rows2;
      } else {
        // K-major operands need whole 128-byte runs of their inner contracted mode
        if (op.k_ext[1] > 1 && op.k_ext[0] % p.bk != 0) return false;
        mode_box[0] = rows; mode_box[1] = rows2; mode_box[2] = p.bk; mode_box[3] = 1;
      }
      return true;
    };
    int order[4];
    const bool ok = plan_box(pr.A, p.a_mn_major != 0, kTcTileM, p.a_box_mn, &p.a_boxes, a_box) &&
                    plan_box(pr.B, p.b_mn_major != 0, bn_cta, p.b_box_mn, &p.b_boxes, b_box);
    if (!ok)
      return set_error(GK_ERR_INVALID_CONFIG, "tensor modes do not tile into TMA boxes (extents or strides)");
    plan_modes(pr.A, order, &p.a_perm);
    plan_modes(pr.B, order, &p.b_perm);
  }
  if (planes * (p.a_boxes * p.a_sub + n_sub * p.b_boxes * p.b_sub) > 32)
    return set_error(GK_ERR_INVALID_CONFIG, "too many TMA boxes per k-block for one producer warp");
  p.a_mn_div = clamp_div(pr.A.mn_ext[0], pr.A.mn_ext[1]);
  p.a_k_div = clamp_div(pr.A.k_ext[0], pr.A.k_ext[1]);
  p.b_mn_div = clamp_div(pr.B.mn_ext[0], pr.B.mn_ext[1]);
  p.b_k_div = clamp_div(pr.B.k_ext[0], pr.B.k_ext[1]);

  // terms of the product
  auto term = [](int ap, int bp, int acc, int neg, int first) {
    TcTerm t{}; t.a_plane = ap; t.b_plane = bp; t.acc_plane = acc; t.negate_a = neg; t.first = first;
    return t;
  };
  if (pr.number == GK_REAL) {
    p.n_terms = 1; p.terms[0] = term(0, 0, 0, 0, 1);
  } else if (pr.number == GK_COMPLEX) {
    // re = a_re b_re - a_im b_im ; im = a_re b_im + a_im b_re   (src/operator.jl:301-314)
    p.n_terms = 4;
    p.terms[0] = term(0, 0, 0, 0, 1); p.terms[1] = term(1, 1, 0, 1, 0);
    p.terms[2] = term(0, 1, 1, 0, 1); p.terms[3] = term(1, 0, 1, 0, 0);
  } else if (pr.number == GK_DUAL) {
    // re = a_re b_re ; du = a_re b_du + a_du b_re               (src/operator.jl:360-372)
    p.n_terms = 3;
    p.terms[0] = term(0, 0, 0, 0, 1);
    p.terms[1] = term(0, 1, 1, 0, 1); p.terms[2] = term(1, 0, 1, 0, 0);
  } else {
    return set_error(GK_ERR_INVALID_CONFIG, "unknown number system %d", pr.number);
  }

  const uint32_t fmt = pr.A.dtype == GK_F16 ? 0u : pr.A.dtype == GK_BF16 ? 1u : 2u;
  uint32_t idesc = 0;
  idesc |= 1u << 4;                                   // accumulate in FP32
  idesc |= fmt << 7;                                  // A format
  idesc |= fmt << 10;                                 // B format
  idesc |= static_cast<uint32_t>(p.a_mn_major) << 15;
  idesc |= static_cast<uint32_t>(p.b_mn_major) << 16;
  idesc |= static_cast<uint32_t>(bn >> 3) << 17;      // N
  idesc |= static_cast<uint32_t>((kTcTileM * cg) >> 4) << 24;  // M
  p.idesc = idesc;
  p.idesc_neg = idesc | (1u << 13);                   // negate A

  // Every pipeline stage costs the producer and MMA warps a fixed amount of barrier waits, votes and loop
  // bookkeeping (a few hundred cycles), which the MMAs of a narrow tile's k-block do not cover: a 128-column
  // tile's four take ≈130 ns.  Tiles up to 128 columns therefore put two k-blocks in a stage (1024^3: 10.7 ->
  // 8.7 us).  For 256-column tiles it was worth 8-12 % while the MMA warp still branched around every MMA;
  // since that loop became straight-line code the deeper ring of single k-blocks is 1-2 % ahead again
  // (2048^3: 17.2 against 17.5 us, 8192 x 4096 x 8192: 369 against 375 us), and a 256 x 512 tile's MMAs
  // outlast the fixed cost by far.
  const int kblock_bytes = stage_bytes_for(cg, bn, n_sub, planes, planes);
  const int boxes_per_kblock = planes * (p.a_boxes * p.a_sub + n_sub * p.b_boxes * p.b_sub);   // one lane each in a producer warp
  const int mma_cycles_per_kblock = 2 * bn * n_sub * p.n_terms;
  int kps = pr.kps;
  if (kps == 0)
    kps = (mma_cycles_per_kblock < 512 && (kSmemBudget - 1024 - kCtrlBytes) / (2 * kblock_bytes) >= 3 && p.k_blocks >= 8 &&
           2 * boxes_per_kblock <= 32) ? 2 : 1;
  if (kps * boxes_per_kblock > 32) kps = 1;
  p.kps = kps;
  const int stage_bytes = kps * kblock_bytes;
  int stages = (kSmemBudget - 1024 - kCtrlBytes) / stage_bytes;
  stages = std::min(stages, 8);
  if (pr.stages) stages = std::min(stages, pr.stages);
  stages = std::min(stages, std::max(2, (p.k_blocks + kps - 1) / kps));
  if (stages < 2)
    return set_error(GK_ERR_INVALID_CONFIG, "Requested too much shared memory: one pipeline stage needs %d bytes", stage_bytes);
  p.stages = stages;
  // Skewed schedule of 512-column tiles (tc_gemm.cuh): every work unit must hold at least two rings of k-blocks.
  p.skew = (n_sub == 2 && acc_stages == 1 && planes == 1 && kps == 1 && !pr.generic && pr.k_split <= 1 &&
            p.k_blocks >= 2 * stages && !(pr.debug & 32)) ? 1 : 0;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(acc_stages * n_sub * planes * bn)) cols <<= 1;
  p.tmem_cols = cols;

  // raster
  const int slots_guess = std::max(1, h->sm_count / cg);
  int group = pr.raster_group;
  if (pr.raster == GK_RASTER_IDENTITY) group = p.tiles_m;
  if (group <= 0)
    group = static_cast<int>(std::lround(std::sqrt(static_cast<double>(slots_guess) * bn * n_sub / (kTcTileM * cg))));
  p.raster_group = std::max(1, std::min(group, p.tiles_m));
  p.raster_kind = 0;
  if (pr.raster == GK_RASTER_HORIZONTAL) {
    p.raster_kind = 1;
    p.raster_group = std::max(1, std::min(pr.raster_group > 0 ? pr.raster_group : group, p.tiles_n));
  } else if (pr.raster == GK_RASTER_LEBESGUE) {
    // the Z-order curve needs power-of-two extents in tiles; other grids keep the band raster
    auto log2_exact = [](int x) { int b = 0; while ((1 << b) < x) ++b; return (1 << b) == x ? b : -1; };
    const int bm = log2_exact(p.tiles_m), bnn = log2_exact(p.tiles_n);
    if (bm >= 0 && bnn >= 0) { p.raster_kind = 2; p.z_bits = std::min(bm, bnn); }
  }

  // epilogue
  if (pr.n_ext0 < pr.N && pr.n_ext0 % 32 != 0)
    return set_error(GK_ERR_INVALID_CONFIG, "inner N mode of the output must be a multiple of 32 elements");
  p.C = pr.C; p.D = pr.D;
  p.m_div = clamp_div(pr.m_ext0, pr.m_ext0 < pr.M ? 2 : 1);
  p.n_div = clamp_div(pr.n_ext0, pr.n_ext0 < pr.N ? 2 : 1);
  p.c_sm0 = pr.c_sm[0]; p.c_sm1 = pr.c_sm[1]; p.c_sn0 = pr.c_sn[0]; p.c_sn1 = pr.c_sn[1];
  p.d_sm0 = pr.d_sm[0]; p.d_sm1 = pr.d_sm[1]; p.d_sn0 = pr.d_sn[0]; p.d_sn1 = pr.d_sn[1];
  p.c_plane = pr.c_plane; p.d_plane = pr.d_plane;
  p.dtype_c = tc_dtype_of(pr.dtype_c); p.dtype_d = tc_dtype_of(pr.dtype_d);
  p.alpha = static_cast<float>(pr.alpha);
  p.beta = pr.C == nullptr ? 0.0f : static_cast<float>(pr.beta);
  p.bias = nullptr; p.bias_axis = TC_BIAS_NONE; p.act = TC_ACT_NONE;
  if (pr.epi) {
    if (pr.epi->bias_axis != GK_BIAS_NONE) {
      if (!pr.epi->bias && encode) return set_error(GK_ERR_INVALID_ARGUMENT, "bias axis set but bias pointer is NULL");
      p.bias = pr.epi->bias; p.bias_axis = pr.epi->bias_axis;
    }
    if (pr.epi->activation < GK_ACT_NONE || pr.epi->activation > GK_ACT_GELU)
      return set_error(GK_ERR_UNSUPPORTED, "activation %d is not one of none/ReLU/GELU", pr.epi->activation);
    p.act = pr.epi->activation;
  }
  p.status = h->status_dev;
  p.debug = pr.debug;
  p.dbg_out = nullptr;

  out->cg = cg;
  out->planes = planes;
  out->tf32 = tf32;
  out->rank5 = pr.rank5;
  out->generic = pr.generic;
  out->smem_bytes = stages * stage_bytes + kCtrlBytes + 1024;
  // One CTA of this kernel per SM, whatever the stage count: a CTA allocates up to all 512 TMEM columns
  // without a bound on that wait, and with dependent launch the next kernel's CTAs arrive while this one's
  // are still draining.  Asking for more than half of an SM's shared memory makes two tcgen05 CTAs on one
  // SM impossible, so two CTA pairs can never each hold one SM's tensor memory and wait for the other's.
  out->smem_bytes = std::max(out->smem_bytes, kSmemBudget / 2 + 2048);
  const bool dbg = pr.debug != 0;
  out->kernel = pr.generic ? tc_kernel_generic(dbg) : tc_kernel_select(cg, planes, tf32, pr.rank5, dbg);
  if (pr.generic) {
    p.ga = pr.A.ptr; p.gb = pr.B.ptr;
    p.g_lda = pr.A.mn_major ? pr.A.k_str[0] : pr.A.mn_str[0];
    p.g_ldb = pr.B.mn_major ? pr.B.k_str[0] : pr.B.mn_str[0];
    p.g_a_batch = pr.batch_a; p.g_b_batch = pr.batch_b;
  }

  // persistent grid
  const int64_t tiles64 = static_cast<int64_t>(p.tiles_m) * p.tiles_n * p.k_split * p.batch;
  if (tiles64 > INT32_MAX) return set_error(GK_ERR_INVALID_CONFIG, "too many work units (%lld)", (long long)tiles64);
  const int tiles = static_cast<int>(tiles64);
  int slots;
  {
    std::lock_guard<std::mutex> lock(h->mu);
    bool& set = pr.generic ? h->attr_set_generic[dbg ? 1 : 0]
                           : h->attr_set[dbg ? 1 : 0][cg - 1][planes - 1][(tf32 ? 1 : 0) + (pr.rank5 ? 2 : 0)];
    if (!set) {
      GK_CUDA_CHECK(cudaFuncSetAttribute(out->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
      set = true;
    }
    if (cg == 1) {
      slots = h->sm_count;
    } else {
      int& cached = h->max_clusters[planes - 1][(tf32 ? 1 : 0) + (pr.rank5 ? 2 : 0)];
      if (cached == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (h->sm_count / 2));
        cfg.blockDim = dim3(tc_threads(planes));
        cfg.dynamicSmemBytes = kSmemBudget;
        cudaLaunchAttribute at{};
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
        cfg.attrs = &at; cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, out->kernel, &cfg);
        if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = h->sm_count / 2; }
        cached = n;
      }
      slots = cached;
    }
  }
  if (pr.max_ctas > 0) slots = std::max(1, std::min(slots, pr.max_ctas / cg));
  out->grid = cg * std::min(tiles, slots);

  if (encode && !pr.generic) {
    gk_status s;
    if (pr.rank5) {
      s = encode_modes(h, &p.tm_a, pr.A, planes, a_box, a_tma);
      if (s != GK_OK) return s;
      s = encode_modes(h, &p.tm_b, pr.B, planes, b_box, b_tma);
    } else {
      s = encode_plain(h, &p.tm_a, pr.A, planes, p.a_mn_major ? p.a_box_mn : p.bk, p.a_mn_major ? p.bk : kTcTileM, a_tma,
                       pr.batch, pr.batch_a);
      if (s != GK_OK) return s;
      s = encode_plain(h, &p.tm_b, pr.B, planes, p.b_mn_major ? p.b_box_mn : p.bk, p.b_mn_major ? p.bk : bn_cta, b_tma,
                       pr.batch, pr.batch_b);
    }
    if (s != GK_OK) return s;
  }
  return GK_OK;
}

int tc_choose_k_split(const TcProblem& pr, const TcLaunch& L, int sm_count) {
  const TcParams& p = L.params;
  if (p.k_split != 1 || p.batch != 1) return 1;
  const int tiles = p.tiles_m * p.tiles_n;
  const int slots = std::max(1, sm_count / L.cg);
  if (tiles * 2 > slots || p.k_blocks < 16) return 1;
  // as many runs as there are idle slots per tile, each at least 8 k-blocks long, 64 at most
  const int s = std::min({64, slots / tiles, p.k_blocks / 8});
  (void)pr;
  return s >= 2 ? s : 1;
}

gk_status tc_launch(const TcLaunch& L, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(L.grid);
  cfg.blockDim = dim3(tc_threads(L.planes));
  cfg.dynamicSmemBytes = L.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute at[2]{};
  int n_at = 0;
  if (L.cg == 2) {
    at[n_at].id = cudaLaunchAttributeClusterDimension;
    at[n_at].val.clusterDim.x = 2; at[n_at].val.clusterDim.y = 1; at[n_at].val.clusterDim.z = 1;
    ++n_at;
  }
  // programmatic dependent launch: the kernel's set-up may overlap the tail of the kernel before it in the
  // stream; its producers and epilogue wait (griddepcontrol.wait) before their first global access
  at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[n_at].val.programmaticStreamSerializationAllowed = 1;
  ++n_at;
  cfg.attrs = at; cfg.numAttrs = n_at;
  void* args[1] = {const_cast<TcParams*>(&L.params)};
  GK_CUDA_CHECK(cudaLaunchKernelExC(&cfg, L.kernel, args));
  return GK_OK;
}

// Split-K decision for a planned product: the plan's own tiles if they leave at least half of the CTA
// slots idle; otherwise, when the tile shape was left to the library, 256 x 256 pair tiles cut along K
// (small tiles were chosen to fill the SMs in one round, which a long K makes slow: every tile then
// streams all of K with little operand reuse).  Returns the number of runs (1 = no split) and may
// replace *pr's tile choice.
// Does cutting K pay?  Measured with bound launches (512^2, 1024^2, 256^2, 2048 x 1024 outputs, K = 2048 .. 16384):
// an unsplit product of few tiles costs ≈0.18 us per k-block; split, ≈40 % of that, plus a second kernel and the
// partial planes' trip through memory: ≈6 us + 0.19 us per MB of partial sums.
static bool split_pays(const TcProblem& pr, int k_blocks, int splits, int planes) {
  const double saved_us = 0.11 * k_blocks;
  const double cost_us = 6.0 + 0.19 * (static_cast<double>(splits) * planes * pr.M * pr.N * 4.0 / 1.0e6);
  return saved_us > cost_us;
}

static int plan_k_split(gk_handle h, TcProblem* pr, const TcLaunch& L) {
  if (pr->tile_n == 0 && pr->cta_group == 0) {
    TcProblem alt = *pr;
    alt.tile_n = pr->number == GK_REAL ? 256 : 128; alt.cta_group = 2;
    TcLaunch La;
    if (tc_plan(h, alt, false, &La) == GK_OK) {
      // worth it only for a long K (32 k-blocks or more): below that the second pass costs more than the
      // large tiles save (measured: the 1024^3 contraction took 25 us this way against 13 us unsplit)
      const int splits = La.params.k_blocks >= 32 ? tc_choose_k_split(alt, La, h->sm_count) : 1;
      if (splits > 1 && split_pays(*pr, La.params.k_blocks, splits, La.planes)) { pr->tile_n = alt.tile_n; pr->cta_group = 2; return splits; }
      if (splits > 1) return 1;
    } else {
      clear_error();
    }
  }
  const int splits = tc_choose_k_split(*pr, L, h->sm_count);
  return splits > 1 && split_pays(*pr, L.params.k_blocks, splits, L.planes) ? splits : 1;
}

int64_t tc_split_workspace_bytes(gk_handle h, const TcProblem& pr, const TcLaunch& L) {
  TcProblem q = pr;
  const int splits = plan_k_split(h, &q, L);
  return splits > 1 ? static_cast<int64_t>(splits) * L.planes * pr.M * pr.N * 4 : 0;
}

gk_status tc_run(gk_handle h, const TcProblem& pr_in, const TcLaunch& L, void* workspace, int64_t workspace_bytes,
                 cudaStream_t st) {
  if (!workspace || workspace_bytes <= 0) return tc_launch(L, st);
  TcProblem pr = pr_in;
  const int64_t set_bytes = static_cast<int64_t>(L.planes) * pr.M * pr.N * 4;     // the planes of one K-run
  int splits = plan_k_split(h, &pr, L);
  if (splits > 1 && splits * set_bytes > workspace_bytes) splits = static_cast<int>(workspace_bytes / set_bytes);
  if (splits <= 1) return tc_launch(L, st);
  if (reinterpret_cast<uintptr_t>(workspace) & 255)
    return set_error(GK_ERR_INVALID_ARGUMENT, "the split-K workspace must be 256-byte aligned");
  TcProblem ps = pr;
  ps.C = nullptr; ps.has_c = false; ps.D = workspace; ps.dtype_c = GK_F32; ps.dtype_d = GK_F32;
  ps.m_ext0 = pr.M; ps.n_ext0 = pr.N;
  ps.c_sm[0] = 1; ps.c_sm[1] = 0; ps.d_sm[0] = 1; ps.d_sm[1] = 0;
  ps.c_sn[0] = pr.M; ps.c_sn[1] = 0; ps.d_sn[0] = pr.M; ps.d_sn[1] = 0;
  ps.c_plane = ps.d_plane = pr.M * pr.N;
  ps.alpha = 1.0; ps.beta = 0.0; ps.epi = nullptr;
  if (pr.tile_n == 0) { ps.tile_n = L.params.bn * L.params.n_sub; ps.cta_group = L.cg; }   // same tile as planned
  ps.k_split = splits; ps.split_stride = set_bytes / 4;
  TcLaunch Ls;
  gk_status s = tc_plan(h, ps, true, &Ls);
  if (s != GK_OK) return s;
  if ((s = tc_launch(Ls, st)) != GK_OK) return s;
  SplitKReduceParams r{};
  r.partial = static_cast<const float*>(workspace); r.splits = Ls.params.k_split; r.planes = L.planes; r.stride = ps.split_stride;
  r.M = static_cast<int>(pr.M); r.N = static_cast<int>(pr.N);
  r.alpha = static_cast<float>(pr.alpha);
  r.beta = (pr.C != nullptr) ? static_cast<float>(pr.beta) : 0.0f;
  r.C = pr.C; r.dtype_c = tc_dtype_of(pr.dtype_c);
  r.D = pr.D; r.dtype_d = tc_dtype_of(pr.dtype_d);
  r.m_div = clamp_div(pr.m_ext0, pr.m_ext0 < pr.M ? 2 : 1); r.n_div = clamp_div(pr.n_ext0, pr.n_ext0 < pr.N ? 2 : 1);
  r.c_sm0 = pr.c_sm[0]; r.c_sm1 = pr.c_sm[1]; r.c_sn0 = pr.c_sn[0]; r.c_sn1 = pr.c_sn[1]; r.c_plane = pr.c_plane;
  r.d_sm0 = pr.d_sm[0]; r.d_sm1 = pr.d_sm[1]; r.d_sn0 = pr.d_sn[0]; r.d_sn1 = pr.d_sn[1]; r.d_plane = pr.d_plane;
  if (pr.epi) { r.bias = pr.epi->bias; r.bias_axis = pr.epi->bias_axis; r.act = pr.epi->activation; }
  const bool plain = L.planes == 1 && pr.m_ext0 >= pr.M && pr.n_ext0 >= pr.N && pr.d_sm[0] == 1 && (pr.C == nullptr || pr.c_sm[0] == 1);
  const bool vec = plain && pr.M % 4 == 0;
  const int64_t units = (vec ? pr.M / 4 : pr.M) * pr.N;
  const int blocks = static_cast<int>(std::min<int64_t>((units + 255) / 256, 8 * h->sm_count));
  GK_CUDA_CHECK(launch_dependent(vec ? splitk_reduce_kernel<true> : splitk_reduce_kernel<false>, dim3(blocks), dim3(256), 0, st, r));
  return GK_OK;
}

}  // namespace gk
