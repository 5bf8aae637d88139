// Host side of the tcgen05 path: eligibility, tile choice, TMA tensor maps, launch.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.h"
#include "tc_gemm.cuh"
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

bool tc_eligible(const gk_gemm_desc& d, const void* a, const void* b, std::string* why) {
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
  const int es = dtype_size(d.dtype_a);
  // TMA: 16-byte aligned base, strides that are multiples of 16 bytes.
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
    return no("operand base address is not 16-byte aligned");
  if ((d.lda * es) % 16 || (d.ldb * es) % 16) return no("leading dimension is not a multiple of 16 bytes");
  if (d.number != GK_REAL) {
    if (d.plane_a == 0 || d.plane_b == 0) return no("interleaved complex operands need the split pre-pass");
    if ((d.plane_a * es) % 16 || (d.plane_b * es) % 16) return no("plane stride is not a multiple of 16 bytes");
  }
  return true;
}

static gk_status encode_operand(gk_handle h, CUtensorMap* tm, const void* base, int32_t dt,
                                int64_t contiguous_extent, int64_t strided_extent, int64_t ld,
                                int planes, int64_t plane_stride, int box_contig, int box_strided,
                                bool atom32) {
  const int es = dtype_size(dt);
  CUtensorMapDataType tdt = dt == GK_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                            : dt == GK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                            : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(contiguous_extent),
                        static_cast<cuuint64_t>(strided_extent), static_cast<cuuint64_t>(planes)};
  cuuint64_t plane_bytes = planes > 1 ? static_cast<cuuint64_t>(plane_stride) * es
                                      : static_cast<cuuint64_t>(ld) * es * strided_extent;
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es, plane_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_contig), static_cast<cuuint32_t>(box_strided), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = h->encode_tiled(tm, tdt, 3, const_cast<void*>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE,
                               atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(GK_ERR_INVALID_CONFIG,
                     "cuTensorMapEncodeTiled failed (%d): extents (%lld, %lld, %d) ld %lld box (%d, %d)",
                     static_cast<int>(r), static_cast<long long>(contiguous_extent),
                     static_cast<long long>(strided_extent), planes, static_cast<long long>(ld),
                     box_contig, box_strided);
  return GK_OK;
}

template <int CG, int PLANES, bool TF32>
static const void* tc_kernel_ptr() {
  return reinterpret_cast<const void*>(&tc_gemm_kernel<CG, PLANES, TF32>);
}

static const void* tc_kernel_select(int cg, int planes, bool tf32) {
  if (cg == 1) {
    if (planes == 1) return tf32 ? tc_kernel_ptr<1, 1, true>() : tc_kernel_ptr<1, 1, false>();
    return tf32 ? tc_kernel_ptr<1, 2, true>() : tc_kernel_ptr<1, 2, false>();
  }
  if (planes == 1) return tf32 ? tc_kernel_ptr<2, 1, true>() : tc_kernel_ptr<2, 1, false>();
  return tf32 ? tc_kernel_ptr<2, 2, true>() : tc_kernel_ptr<2, 2, false>();
}

static constexpr int kSmemBudget = 232448;  // 227 KiB opt-in limit per CTA on sm_100
static constexpr int kCtrlBytes = 256;

static int stage_bytes_for(int cg, int bn, int a_planes, int b_planes) {
  return a_planes * kTcTileM * kTcKBytes + b_planes * (bn / cg) * kTcKBytes;
}

// Picks (cta_group, tile_n): fewest "tile-time" units over the persistent grid, where a larger
// tile is worth more per unit time (operand reuse) but quantises worse on small problems.
static void choose_tile(const gk_gemm_desc& d, int sm_count, int planes, int* cg_out, int* bn_out) {
  // a transposed (N-contiguous) B is loaded in boxes of 128 bytes of N per CTA
  const int n_unit = d.trans_b ? kTcKBytes / dtype_size(d.dtype_b) : 8;
  struct Cand { int cg, bn; double eff; };
  static const Cand cands[] = {{2, 256, 1.00}, {1, 256, 0.92}, {2, 128, 0.80},
                               {1, 128, 0.74}, {1, 64, 0.50},  {1, 32, 0.30}};
  double best = 1e300;
  int bcg = 1, bbn = 128;
  for (const Cand& c : cands) {
    if (planes * c.bn > 256) continue;  // two accumulator stages must fit 512 TMEM columns
    if ((c.bn / c.cg) % n_unit) continue;
    if (d.cta_group && c.cg != d.cta_group) continue;
    if (d.tile_n && c.bn != d.tile_n) continue;
    const int64_t tm = (d.m + 128 * c.cg - 1) / (128 * c.cg);
    const int64_t tn = (d.n + c.bn - 1) / c.bn;
    const int64_t slots = std::max(1, sm_count / c.cg);
    const int64_t waves = (tm * tn + slots - 1) / slots;
    const double t = static_cast<double>(waves) * c.bn / c.eff;
    if (t < best) { best = t; bcg = c.cg; bbn = c.bn; }
  }
  if (best == 1e300) {  // overrides that match no candidate: honour them if they are valid
    bcg = d.cta_group ? d.cta_group : 1;
    bbn = d.tile_n ? d.tile_n : 128;
  }
  *cg_out = bcg;
  *bn_out = bbn;
}

gk_status tc_plan(gk_handle h, const gk_gemm_desc& d, const gk_epilogue_desc* epi, const void* a,
                  const void* b, const void* c, void* dd, TcLaunch* out) {
  std::string why;
  if (!tc_eligible(d, a ? a : reinterpret_cast<const void*>(16), b ? b : reinterpret_cast<const void*>(16), &why))
    return set_error(GK_ERR_INVALID_CONFIG, "TCGen05Operator cannot take this GEMM: %s", why.c_str());

  TcParams& p = out->params;
  std::memset(&p, 0, sizeof(p));
  const int es = dtype_size(d.dtype_a);
  const bool tf32 = d.dtype_a == GK_F32;
  const int planes = d.number == GK_REAL ? 1 : 2;

  int cg, bn;
  choose_tile(d, h->sm_count, planes, &cg, &bn);
  if (cg != 1 && cg != 2)
    return set_error(GK_ERR_INVALID_CONFIG, "cta_group must be 1 or 2, got %d", cg);
  if (bn < 32 || bn > 256 || bn % 32 || planes * bn > 256 || (cg == 2 && bn % 64))
    return set_error(GK_ERR_INVALID_CONFIG,
                     "tile_n = %d is not usable (multiple of 32 (64 for CTA pairs), <= %d)", bn,
                     256 / planes);

  p.M = static_cast<int32_t>(d.m);
  p.N = static_cast<int32_t>(d.n);
  p.K = static_cast<int32_t>(d.k);
  p.bn = bn;
  p.bk = kTcKBytes / es;
  p.k_blocks = (p.K + p.bk - 1) / p.bk;
  p.tiles_m = (p.M + kTcTileM * cg - 1) / (kTcTileM * cg);
  p.tiles_n = (p.N + bn - 1) / bn;
  p.a_planes = p.b_planes = planes;
  p.a_mn_major = d.trans_a ? 0 : 1;  // column-major M x K: M is contiguous
  p.b_mn_major = d.trans_b ? 1 : 0;  // column-major K x N: K is contiguous
  const int bn_cta = bn / cg;
  const int mn_box_bytes = p.bk * p.bk * es;  // MN-major box: 128 B of M/N by one k-block
  p.a_plane_bytes = kTcTileM * kTcKBytes;
  p.b_plane_bytes = bn_cta * kTcKBytes;
  // MN-major operands: 16-bit types use the plain 128-byte swizzle (atoms of 8 k rows, 1024 B);
  // 32-bit types must use the 128-byte swizzle with 32-byte units (atoms of 4 k rows, 512 B).
  // Either way one MMA consumes 32 / es rows of K, i.e. 2048 B (16-bit) or 1024 B (32-bit).
  const uint32_t mn_sbo = es == 4 ? 512 : 1024;
  const uint32_t mn_swz = es == 4 ? 1 : 2;
  const uint32_t mn_kadv = (32 / es) * 128;
  if (p.a_mn_major) {
    p.a_boxes = kTcTileM / p.bk; p.a_box_bytes = mn_box_bytes;
    p.a_lbo = mn_box_bytes; p.a_sbo = mn_sbo; p.a_kadv = mn_kadv; p.a_swz = mn_swz;
  } else {
    p.a_boxes = 1; p.a_box_bytes = p.a_plane_bytes;
    p.a_lbo = 16; p.a_sbo = 1024; p.a_kadv = 32; p.a_swz = 2;
  }
  if (p.b_mn_major) {
    if (bn_cta % p.bk)
      return set_error(GK_ERR_INVALID_CONFIG, "tile_n = %d too small for a transposed B of this type", bn);
    p.b_boxes = bn_cta / p.bk; p.b_box_bytes = mn_box_bytes;
    p.b_lbo = mn_box_bytes; p.b_sbo = mn_sbo; p.b_kadv = mn_kadv; p.b_swz = mn_swz;
  } else {
    p.b_boxes = 1; p.b_box_bytes = p.b_plane_bytes;
    p.b_lbo = 16; p.b_sbo = 1024; p.b_kadv = 32; p.b_swz = 2;
  }

  // terms of the product
  auto term = [](int ap, int bp, int acc, int neg, int first) {
    TcTerm t{}; t.a_plane = ap; t.b_plane = bp; t.acc_plane = acc; t.negate_a = neg; t.first = first;
    return t;
  };
  if (d.number == GK_REAL) {
    p.n_terms = 1; p.terms[0] = term(0, 0, 0, 0, 1);
  } else if (d.number == GK_COMPLEX) {
    // re = a_re b_re - a_im b_im ; im = a_re b_im + a_im b_re   (src/operator.jl:301-314)
    p.n_terms = 4;
    p.terms[0] = term(0, 0, 0, 0, 1); p.terms[1] = term(1, 1, 0, 1, 0);
    p.terms[2] = term(0, 1, 1, 0, 1); p.terms[3] = term(1, 0, 1, 0, 0);
  } else if (d.number == GK_DUAL) {
    // re = a_re b_re ; du = a_re b_du + a_du b_re               (src/operator.jl:360-372)
    p.n_terms = 3;
    p.terms[0] = term(0, 0, 0, 0, 1);
    p.terms[1] = term(0, 1, 1, 0, 1); p.terms[2] = term(1, 0, 1, 0, 0);
  } else {
    return set_error(GK_ERR_INVALID_CONFIG, "unknown number system %d", d.number);
  }

  const uint32_t fmt = d.dtype_a == GK_F16 ? 0u : d.dtype_a == GK_BF16 ? 1u : 2u;
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

  const int stage_bytes = stage_bytes_for(cg, bn, planes, planes);
  int stages = (kSmemBudget - 1024 - kCtrlBytes) / stage_bytes;
  stages = std::min(stages, 8);
  if (d.stages) stages = std::min(stages, d.stages);
  stages = std::min(stages, std::max(2, p.k_blocks));
  if (stages < 2)
    return set_error(GK_ERR_INVALID_CONFIG, "Requested too much shared memory: one pipeline stage needs %d bytes", stage_bytes);
  p.stages = stages;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(2 * planes * bn)) cols <<= 1;
  p.tmem_cols = cols;

  // raster
  const int slots_guess = std::max(1, h->sm_count / cg);
  int group = d.raster_group;
  if (d.raster == GK_RASTER_IDENTITY) group = p.tiles_m;
  if (group <= 0)
    group = static_cast<int>(std::lround(std::sqrt(static_cast<double>(slots_guess) * bn / (kTcTileM * cg))));
  p.raster_group = std::max(1, std::min(group, p.tiles_m));

  // epilogue
  p.C = c; p.D = dd;
  p.ldc = d.ldc; p.ldd = d.ldd;
  p.c_plane = d.plane_c; p.d_plane = d.plane_d;
  p.dtype_c = tc_dtype_of(d.dtype_c); p.dtype_d = tc_dtype_of(d.dtype_d);
  p.alpha = static_cast<float>(d.alpha);
  p.beta = (d.layout_c == GK_LAYOUT_ZERO || c == nullptr) ? 0.0f : static_cast<float>(d.beta);
  p.bias = nullptr; p.bias_axis = TC_BIAS_NONE; p.act = TC_ACT_NONE;
  if (epi) {
    if (epi->bias_axis != GK_BIAS_NONE) {
      if (!epi->bias && a) return set_error(GK_ERR_INVALID_ARGUMENT, "bias axis set but bias pointer is NULL");
      p.bias = epi->bias; p.bias_axis = epi->bias_axis;
    }
    if (epi->activation < GK_ACT_NONE || epi->activation > GK_ACT_GELU)
      return set_error(GK_ERR_UNSUPPORTED, "activation %d is not one of none/ReLU/GELU", epi->activation);
    p.act = epi->activation;
  }
  p.status = h->status_dev;
  p.debug = d.reserved[0];
  p.dbg_out = nullptr;

  out->cg = cg;
  out->planes = planes;
  out->tf32 = tf32;
  out->smem_bytes = stages * stage_bytes + kCtrlBytes + 1024;
  out->kernel = tc_kernel_select(cg, planes, tf32);

  // persistent grid
  const int tiles = p.tiles_m * p.tiles_n;
  int slots;
  {
    std::lock_guard<std::mutex> lock(h->mu);
    bool& set = h->attr_set[cg - 1][planes - 1][tf32 ? 1 : 0];
    if (!set) {
      GK_CUDA_CHECK(cudaFuncSetAttribute(out->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
      set = true;
    }
    if (cg == 1) {
      slots = h->sm_count;
    } else {
      int& cached = h->max_clusters[planes - 1][tf32 ? 1 : 0][0];
      if (cached == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * (h->sm_count / 2));
        cfg.blockDim = dim3(kTcThreads);
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
  if (d.max_ctas > 0) slots = std::max(1, std::min(slots, d.max_ctas / cg));
  out->grid = cg * std::min(tiles, slots);
  return GK_OK;
}

gk_status tc_launch(const TcLaunch& L, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(L.grid);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = L.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute at{};
  if (L.cg == 2) {
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
  }
  void* args[1] = {const_cast<TcParams*>(&L.params)};
  GK_CUDA_CHECK(cudaLaunchKernelExC(&cfg, L.kernel, args));
  return GK_OK;
}

gk_status tc_encode_maps(gk_handle h, const gk_gemm_desc& d, const void* a, const void* b, TcLaunch* L) {
  TcParams& p = L->params;
  const int planes = L->planes;
  const int bn_cta = p.bn / L->cg;
  gk_status s;
  if (p.a_mn_major)
    s = encode_operand(h, &p.tm_a, a, d.dtype_a, d.m, d.k, d.lda, planes, d.plane_a, p.bk, p.bk, p.a_swz == 1);
  else
    s = encode_operand(h, &p.tm_a, a, d.dtype_a, d.k, d.m, d.lda, planes, d.plane_a, p.bk, kTcTileM, false);
  if (s != GK_OK) return s;
  if (p.b_mn_major)
    s = encode_operand(h, &p.tm_b, b, d.dtype_b, d.n, d.k, d.ldb, planes, d.plane_b, p.bk, p.bk, p.b_swz == 1);
  else
    s = encode_operand(h, &p.tm_b, b, d.dtype_b, d.k, d.n, d.ldb, planes, d.plane_b, p.bk, bn_cta, false);
  return s;
}

}  // namespace gk
