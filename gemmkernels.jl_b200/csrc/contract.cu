// Tensor contraction entry point (GETT): D[modes_c] = alpha * sum_K A[modes_a] * B[modes_b] + beta * C.
//
// The reference has no contraction function in src/; its only material is the benchmark that maps one
// contraction onto the GEMM kernels through custom layouts with per-load div/mod
// (benchmarks/tensor-contractions/run.jl:21-131).  Here the modes are classified as M (in A and C),
// N (in B and C) and K (in A and B), and the contraction runs
//   * on the tcgen05 kernel when every index splits into at most two modes that tile into TMA boxes
//     (5-D tensor maps address the tensors in place: no transposing or packing pass), or
//   * on a gather kernel that reads through per-index offset tables built in the caller's workspace.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.h"
#include "simt_gemm.cuh"
#include "tc_plan.h"

namespace gk {

struct ModeInfo {
  int label;
  int64_t extent;
  int64_t sa, sb, sc, sd;  // stride in each tensor (0 if absent)
};

struct Groups {
  std::vector<ModeInfo> m, n, k, b;   // free modes of A, of B, contracted modes, batch modes (in A, B and C)
  int64_t M = 1, N = 1, K = 1, Bt = 1;
};

static int find_mode(const int32_t* modes, int rank, int label) {
  for (int i = 0; i < rank; ++i) if (modes[i] == label) return i;
  return -1;
}

static gk_status classify(const gk_contract_desc& d, Groups* g) {
  if (d.rank_a < 1 || d.rank_b < 1 || d.rank_c < 1 || d.rank_a > GK_MAX_MODES || d.rank_b > GK_MAX_MODES ||
      d.rank_c > GK_MAX_MODES)
    return set_error(GK_ERR_INVALID_CONFIG, "tensor ranks must be between 1 and %d", GK_MAX_MODES);
  auto dup = [](const int32_t* m, int r) {
    for (int i = 0; i < r; ++i) for (int j = i + 1; j < r; ++j) if (m[i] == m[j]) return true;
    return false;
  };
  if (dup(d.modes_a, d.rank_a) || dup(d.modes_b, d.rank_b) || dup(d.modes_c, d.rank_c))
    return set_error(GK_ERR_INVALID_CONFIG, "a mode label appears twice in one tensor");
  auto add = [&](int label) -> gk_status {
    const int ia = find_mode(d.modes_a, d.rank_a, label), ib = find_mode(d.modes_b, d.rank_b, label),
              ic = find_mode(d.modes_c, d.rank_c, label);
    ModeInfo mi{};
    mi.label = label;
    int64_t e = -1;
    for (auto [idx, ext] : {std::pair<int, const int64_t*>{ia, d.extents_a}, {ib, d.extents_b}, {ic, d.extents_c}}) {
      if (idx < 0) continue;
      if (e >= 0 && ext[idx] != e)
        return set_error(GK_ERR_DIMENSION_MISMATCH, "Dimensions do not match: mode '%c' has extents %lld and %lld",
                         label, (long long)e, (long long)ext[idx]);
      e = ext[idx];
    }
    if (e < 1) return set_error(GK_ERR_DIMENSION_MISMATCH, "Dimensions do not match: mode '%c' is empty", label);
    mi.extent = e;
    mi.sa = ia >= 0 ? d.strides_a[ia] : 0; mi.sb = ib >= 0 ? d.strides_b[ib] : 0;
    mi.sc = ic >= 0 ? d.strides_c[ic] : 0; mi.sd = ic >= 0 ? d.strides_d[ic] : 0;
    if (ia >= 0 && ib >= 0 && ic >= 0) { g->b.push_back(mi); g->Bt *= e; }   // a batch mode: one contraction per index value
    else if (ia >= 0 && ic >= 0) { g->m.push_back(mi); g->M *= e; }
    else if (ib >= 0 && ic >= 0) { g->n.push_back(mi); g->N *= e; }
    else if (ia >= 0 && ib >= 0) { g->k.push_back(mi); g->K *= e; }
    else return set_error(GK_ERR_INVALID_CONFIG, "mode '%c' appears in one tensor only", label);
    return GK_OK;
  };
  // every label once, in order of first appearance (C, then A, then B)
  std::vector<int> seen;
  auto visit = [&](const int32_t* modes, int rank) -> gk_status {
    for (int i = 0; i < rank; ++i) {
      if (std::find(seen.begin(), seen.end(), modes[i]) != seen.end()) continue;
      seen.push_back(modes[i]);
      gk_status s = add(modes[i]);
      if (s != GK_OK) return s;
    }
    return GK_OK;
  };
  gk_status s;
  if ((s = visit(d.modes_c, d.rank_c)) != GK_OK) return s;
  if ((s = visit(d.modes_a, d.rank_a)) != GK_OK) return s;
  if ((s = visit(d.modes_b, d.rank_b)) != GK_OK) return s;
  if (g->m.empty() || g->n.empty() || g->k.empty())
    return set_error(GK_ERR_UNSUPPORTED, "the contraction needs at least one free mode of A, one of B and one contracted mode");
  return GK_OK;
}

// Orders a group so that `first` (a label, or -1) leads and the rest ascends by the given stride,
// then fuses neighbours that are contiguous in every tensor that holds them.
static void order_and_fuse(std::vector<ModeInfo>* grp, int first, int64_t ModeInfo::*key) {
  std::stable_sort(grp->begin(), grp->end(), [&](const ModeInfo& x, const ModeInfo& y) {
    if ((x.label == first) != (y.label == first)) return x.label == first;
    return x.*key < y.*key;
  });
  std::vector<ModeInfo> out;
  for (const ModeInfo& m : *grp) {
    if (!out.empty()) {
      ModeInfo& p = out.back();
      auto cont = [&](int64_t sp, int64_t sm) { return sp == 0 && sm == 0 ? true : sm == sp * p.extent; };
      if (cont(p.sa, m.sa) && cont(p.sb, m.sb) && cont(p.sc, m.sc) && cont(p.sd, m.sd)) {
        p.extent *= m.extent;
        continue;
      }
    }
    out.push_back(m);
  }
  *grp = out;
}

static int stride1_label(const std::vector<ModeInfo>& a, const std::vector<ModeInfo>& b, int64_t ModeInfo::*s) {
  for (const auto* g : {&a, &b})
    for (const ModeInfo& m : *g)
      if (m.*s == 1) return m.label;
  return -1;
}

static bool in_group(const std::vector<ModeInfo>& g, int label) {
  for (const ModeInfo& m : g) if (m.label == label) return true;
  return false;
}

// Tries to express the contraction as a TcProblem.  Returns false (with a reason) when the tensors
// cannot be addressed by two-mode TMA boxes.
static bool build_tc_problem(const gk_contract_desc& d, Groups g, const void* a, const void* b, const void* c,
                             void* dd, TcProblem* pr, std::string* why) {
  auto no = [&](const char* s) { *why = s; return false; };
  if (d.dtype_a != d.dtype_b) return no("A and B element types differ");
  const bool okc = (d.dtype_a == GK_F16 && d.compute == GK_F16) || (d.dtype_a == GK_BF16 && d.compute == GK_BF16) ||
                   (d.dtype_a == GK_F32 && d.compute == GK_TF32);
  if (!okc) return no("element/compute types have no tensor-core path");
  if (!(d.dtype_d == GK_F32 || d.dtype_d == GK_F16 || d.dtype_d == GK_BF16)) return no("output type");
  const int es = dtype_size(d.dtype_a);
  const int la = stride1_label(g.m, g.k, &ModeInfo::sa);   // A's contiguous mode
  const int lb = stride1_label(g.n, g.k, &ModeInfo::sb);
  if (la < 0 || lb < 0) return no("an operand has no stride-1 mode");
  const bool a_mn = in_group(g.m, la), b_mn = in_group(g.n, lb);
  if (!a_mn && !b_mn && la != lb) return no("A and B are contiguous along different contracted modes");
  order_and_fuse(&g.m, a_mn ? la : -1, a_mn ? &ModeInfo::sa : &ModeInfo::sd);
  order_and_fuse(&g.n, b_mn ? lb : -1, b_mn ? &ModeInfo::sb : &ModeInfo::sd);
  order_and_fuse(&g.k, !a_mn ? la : (!b_mn ? lb : -1), &ModeInfo::sa);
  if (g.m.size() > 2 || g.n.size() > 2 || g.k.size() > 2) return no("an index splits into more than two modes");
  auto aligned = [&](int64_t stride) { return stride == 1 || (stride * es) % 16 == 0; };
  for (const auto* grp : {&g.m, &g.k}) for (const ModeInfo& m : *grp) if (!aligned(m.sa)) return no("stride of A not a multiple of 16 bytes");
  for (const auto* grp : {&g.n, &g.k}) for (const ModeInfo& m : *grp) if (!aligned(m.sb)) return no("stride of B not a multiple of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return no("operand base not 16-byte aligned");
  if (g.M > INT32_MAX / 2 || g.N > INT32_MAX / 2 || g.K > INT32_MAX / 2) return no("index too large");

  *pr = TcProblem{};
  pr->M = g.M; pr->N = g.N; pr->K = g.K; pr->number = GK_REAL;
  pr->rank5 = true;
  auto fill = [](const std::vector<ModeInfo>& grp, int64_t ModeInfo::*s, int64_t* ext, int64_t* str) {
    ext[0] = grp[0].extent; str[0] = grp[0].*s;
    ext[1] = grp.size() > 1 ? grp[1].extent : 1; str[1] = grp.size() > 1 ? grp[1].*s : 0;
  };
  pr->A.ptr = a; pr->A.dtype = d.dtype_a; pr->A.mn_major = a_mn;
  fill(g.m, &ModeInfo::sa, pr->A.mn_ext, pr->A.mn_str); fill(g.k, &ModeInfo::sa, pr->A.k_ext, pr->A.k_str);
  pr->B.ptr = b; pr->B.dtype = d.dtype_b; pr->B.mn_major = b_mn;
  fill(g.n, &ModeInfo::sb, pr->B.mn_ext, pr->B.mn_str); fill(g.k, &ModeInfo::sb, pr->B.k_ext, pr->B.k_str);
  if ((a_mn ? pr->A.mn_str[0] : pr->A.k_str[0]) != 1 || (b_mn ? pr->B.mn_str[0] : pr->B.k_str[0]) != 1)
    return no("contiguous mode is not first after ordering");
  // the 128-byte inner box must be cut from whole modes
  if ((pr->A.mn_major ? pr->A.mn_ext[0] : pr->A.k_ext[0]) * es % 16 || (pr->B.mn_major ? pr->B.mn_ext[0] : pr->B.k_ext[0]) * es % 16)
    return no("contiguous mode is not a multiple of 16 bytes");
  pr->C = (d.beta != 0.0) ? c : nullptr; pr->D = dd;
  pr->has_c = d.beta != 0.0;
  pr->dtype_c = d.dtype_c; pr->dtype_d = d.dtype_d;
  pr->m_ext0 = g.m[0].extent; pr->n_ext0 = g.n[0].extent;
  int64_t e2[2];
  fill(g.m, &ModeInfo::sc, e2, pr->c_sm); fill(g.n, &ModeInfo::sc, e2, pr->c_sn);
  fill(g.m, &ModeInfo::sd, e2, pr->d_sm); fill(g.n, &ModeInfo::sd, e2, pr->d_sn);
  if (g.n.size() > 1 && g.n[0].extent % 32) return no("inner N mode is not a multiple of 32");
  pr->alpha = d.alpha; pr->beta = d.beta;
  pr->tile_n = d.tile_n; pr->cta_group = d.cta_group; pr->stages = d.stages;
  pr->debug = d.debug;
  return true;
}

// ------------------------------------------------------------------------------------------------
// gather path: offset tables in workspace + SIMT kernel
// ------------------------------------------------------------------------------------------------
struct TableSpec {
  int n_modes;
  int64_t extent[GK_MAX_MODES];
  int64_t stride[GK_MAX_MODES];
};

struct TablesParams {
  TableSpec spec[8];   // Am, Ak, Bk, Bn, Cm, Cn, Dm, Dn
  int64_t length[8];
  int64_t* table[8];
};

__global__ void contract_tables_kernel(const TablesParams p) {
  const int t = blockIdx.y;
  const TableSpec& sp = p.spec[t];
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < p.length[t];
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, off = 0;
    for (int q = 0; q < sp.n_modes; ++q) {
      off += (rem % sp.extent[q]) * sp.stride[q];
      rem /= sp.extent[q];
    }
    p.table[t][i] = off;
  }
}

struct GatherParams {
  const void* A; const void* B; const void* C; void* D;
  int64_t M, N, K;
  const int64_t *am, *ak, *bk, *bn, *cm, *cn, *dm, *dn;
  float alpha, beta;
  int has_c;
};

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kSimtThreads) gather_contract_kernel(const GatherParams p) {
  __shared__ float As[kSimtK][kSimtTile + 1];
  __shared__ float Bs[kSimtK][kSimtTile + 1];
  const TIn* A = static_cast<const TIn*>(p.A);
  const TIn* B = static_cast<const TIn*>(p.B);
  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * kSimtTile, n0 = static_cast<int64_t>(blockIdx.y) * kSimtTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < p.K; k0 += kSimtK) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int e = threadIdx.x + r * kSimtThreads;
      const int xx = e & 63, kk = e >> 6;
      const int64_t k = k0 + kk;
      float va = 0.0f, vb = 0.0f;
      if (k < p.K) {
        if (m0 + xx < p.M) va = simt_cvt_in<float, TIn>(A[p.am[m0 + xx] + p.ak[k]]);
        if (n0 + xx < p.N) vb = simt_cvt_in<float, TIn>(B[p.bn[n0 + xx] + p.bk[k]]);
      }
      As[kk][xx] = va;
      Bs[kk][xx] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tx + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][ty + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  const TOut* C = static_cast<const TOut*>(p.C);
  TOut* D = static_cast<TOut*>(p.D);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t m = m0 + tx + 16 * i, n = n0 + ty + 16 * j;
      if (m < p.M && n < p.N) {
        float v = p.alpha * acc[i][j];
        if (p.has_c) v += p.beta * simt_cvt_in<float, TOut>(C[p.cm[m] + p.cn[n]]);
        D[p.dm[m] + p.dn[n]] = simt_cvt_out<TOut, float>(v);
      }
    }
}

static int64_t gather_workspace_bytes(const Groups& g) {
  return static_cast<int64_t>(sizeof(int64_t)) * (3 * g.M + 3 * g.N + 2 * g.K);
}

static void fill_spec(const std::vector<ModeInfo>& grp, int64_t ModeInfo::*s, TableSpec* sp) {
  sp->n_modes = static_cast<int>(grp.size());
  for (size_t i = 0; i < grp.size(); ++i) { sp->extent[i] = grp[i].extent; sp->stride[i] = grp[i].*s; }
}

static gk_status launch_gather(const gk_contract_desc& d, const Groups& g, const void* a, const void* b,
                               const void* c, void* dd, int64_t* tables, cudaStream_t stream) {
  if (d.dtype_a != d.dtype_b || (d.beta != 0.0 && d.dtype_c != d.dtype_d))
    return set_error(GK_ERR_UNSUPPORTED, "gather path needs A/B of one type and C/D of one type");
  TablesParams tp{};
  fill_spec(g.m, &ModeInfo::sa, &tp.spec[0]); fill_spec(g.k, &ModeInfo::sa, &tp.spec[1]);
  fill_spec(g.k, &ModeInfo::sb, &tp.spec[2]); fill_spec(g.n, &ModeInfo::sb, &tp.spec[3]);
  fill_spec(g.m, &ModeInfo::sc, &tp.spec[4]); fill_spec(g.n, &ModeInfo::sc, &tp.spec[5]);
  fill_spec(g.m, &ModeInfo::sd, &tp.spec[6]); fill_spec(g.n, &ModeInfo::sd, &tp.spec[7]);
  const int64_t len[8] = {g.M, g.K, g.K, g.N, g.M, g.N, g.M, g.N};
  int64_t* cur = tables;
  int64_t longest = 1;
  for (int t = 0; t < 8; ++t) { tp.length[t] = len[t]; tp.table[t] = cur; cur += len[t]; longest = std::max(longest, len[t]); }
  const unsigned bx = static_cast<unsigned>(std::min<int64_t>((longest + 255) / 256, 1024));
  contract_tables_kernel<<<dim3(bx, 8), 256, 0, stream>>>(tp);
  GK_CUDA_CHECK(cudaGetLastError());
  GatherParams gp{};
  gp.A = a; gp.B = b; gp.C = c; gp.D = dd; gp.M = g.M; gp.N = g.N; gp.K = g.K;
  gp.am = tp.table[0]; gp.ak = tp.table[1]; gp.bk = tp.table[2]; gp.bn = tp.table[3];
  gp.cm = tp.table[4]; gp.cn = tp.table[5]; gp.dm = tp.table[6]; gp.dn = tp.table[7];
  gp.alpha = static_cast<float>(d.alpha); gp.beta = static_cast<float>(d.beta);
  gp.has_c = (c != nullptr && d.beta != 0.0) ? 1 : 0;
  const dim3 grid(static_cast<unsigned>((g.M + kSimtTile - 1) / kSimtTile), static_cast<unsigned>((g.N + kSimtTile - 1) / kSimtTile));
  if (grid.y > 65535u) return set_error(GK_ERR_INVALID_CONFIG, "N too large for the gather kernel");
  const int ti = d.dtype_a, to = d.dtype_d;
  if (ti == GK_F16 && to == GK_F32) gather_contract_kernel<__half, float><<<grid, kSimtThreads, 0, stream>>>(gp);
  else if (ti == GK_F16 && to == GK_F16) gather_contract_kernel<__half, __half><<<grid, kSimtThreads, 0, stream>>>(gp);
  else if (ti == GK_BF16 && to == GK_F32) gather_contract_kernel<__nv_bfloat16, float><<<grid, kSimtThreads, 0, stream>>>(gp);
  else if (ti == GK_F32 && to == GK_F32) gather_contract_kernel<float, float><<<grid, kSimtThreads, 0, stream>>>(gp);
  else return set_error(GK_ERR_UNSUPPORTED, "no gather kernel for element types A/B %s, C/D %s", dtype_name(ti), dtype_name(to));
  GK_CUDA_CHECK(cudaGetLastError());
  return GK_OK;
}

// One contraction without batch modes (one index value of each batch mode of the caller's).
static gk_status contract_one(gk_handle h, const gk_contract_desc* desc, const Groups& g, const void* a, const void* b,
                              const void* c, void* dd, void* workspace, int64_t workspace_bytes, cudaStream_t stream,
                              gk_gemm_plan* plan_only) {
  gk_status s = GK_OK;
  TcProblem pr;
  std::string why;
  const void* a_chk = plan_only ? reinterpret_cast<const void*>(16) : a;
  const void* b_chk = plan_only ? reinterpret_cast<const void*>(16) : b;
  const bool want_tc = desc->compute == GK_F16 || desc->compute == GK_BF16 || desc->compute == GK_TF32;
  if (want_tc && !desc->force_gather && build_tc_problem(*desc, g, a_chk, b_chk, c, dd, &pr, &why)) {
    TcLaunch L;
    s = tc_plan(h, pr, plan_only == nullptr, &L);
    if (s == GK_OK) {
      if (plan_only) {
        std::memset(plan_only, 0, sizeof(*plan_only));
        plan_only->kernel = 1; plan_only->grid = L.grid; plan_only->block = tc_threads(L.planes); plan_only->cluster = L.cg;
        plan_only->smem_bytes = L.smem_bytes; plan_only->tmem_columns = static_cast<int32_t>(L.params.tmem_cols);
        plan_only->tile_m = kTcTileM * L.cg; plan_only->tile_n = L.params.bn * L.params.n_sub; plan_only->tile_k = L.params.bk * L.params.kps;
        plan_only->stages = L.params.stages;
        plan_only->workspace_bytes = tc_split_workspace_bytes(h, pr, L);   // optional: enables split-K
        return GK_OK;
      }
      if (L.params.debug & 8) {
        if (!workspace || workspace_bytes < static_cast<int64_t>(L.grid) * 16 * 8)
          return set_error(GK_ERR_INVALID_ARGUMENT, "debug counters need a workspace of %lld bytes", (long long)L.grid * 16 * 8);
        L.params.dbg_out = static_cast<long long*>(workspace);
        return tc_launch(L, stream);
      }
      // a 256-byte aligned workspace lets a contraction with few output tiles and a long K be cut along K
      const bool ws_ok = workspace && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0;
      return tc_run(h, pr, L, ws_ok ? workspace : nullptr, workspace_bytes, stream);
    }
    why = gk_last_error_message();   // planning refused (e.g. box shapes): use the gather path
    clear_error();
  }
  if (desc->compute == GK_TF32)
    return set_error(GK_ERR_INVALID_CONFIG, "TF32 contraction cannot use the tensor cores here (%s) and an FP32 gather result is not a TF32 result", why.c_str());
  const int64_t need = gather_workspace_bytes(g);
  if (plan_only) {
    std::memset(plan_only, 0, sizeof(*plan_only));
    plan_only->kernel = 5;
    plan_only->grid = static_cast<int32_t>(((g.M + kSimtTile - 1) / kSimtTile) * ((g.N + kSimtTile - 1) / kSimtTile));
    plan_only->block = kSimtThreads; plan_only->cluster = 1;
    plan_only->tile_m = kSimtTile; plan_only->tile_n = kSimtTile; plan_only->tile_k = kSimtK; plan_only->stages = 1;
    plan_only->workspace_bytes = need;
    return GK_OK;
  }
  if (!workspace || workspace_bytes < need)
    return set_error(GK_ERR_INVALID_ARGUMENT, "this contraction runs on the gather path and needs %lld bytes of workspace (got %lld)",
                     (long long)need, (long long)workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 7) return set_error(GK_ERR_INVALID_ARGUMENT, "workspace must be 8-byte aligned");
  return launch_gather(*desc, g, a, b, (desc->beta != 0.0) ? c : nullptr, dd, static_cast<int64_t*>(workspace), stream);
}

// Offsets (in elements) of every combination of the batch modes' index values, in A, B, C and D.
struct BatchOffsets { int64_t a, b, c, d; };
static constexpr int64_t kMaxBatch = 65536;

static gk_status batch_offsets(const Groups& g, std::vector<BatchOffsets>* out) {
  if (g.Bt > kMaxBatch)
    return set_error(GK_ERR_INVALID_CONFIG, "batch modes span %lld contractions; at most %lld are launched from one call",
                     (long long)g.Bt, (long long)kMaxBatch);
  out->assign(static_cast<size_t>(g.Bt), BatchOffsets{0, 0, 0, 0});
  for (int64_t i = 0; i < g.Bt; ++i) {
    int64_t rem = i;
    BatchOffsets o{0, 0, 0, 0};
    for (const ModeInfo& m : g.b) {
      const int64_t x = rem % m.extent;
      rem /= m.extent;
      o.a += x * m.sa; o.b += x * m.sb; o.c += x * m.sc; o.d += x * m.sd;
    }
    (*out)[static_cast<size_t>(i)] = o;
  }
  return GK_OK;
}

// Batch modes (labels in A, B and C) make the call a set of independent contractions, one per
// combination of their index values: each is planned and launched on its own, on the same stream.
static gk_status contract_impl(gk_handle h, const gk_contract_desc* desc, const void* a, const void* b, const void* c,
                               void* dd, void* workspace, int64_t workspace_bytes, cudaStream_t stream,
                               gk_gemm_plan* plan_only) {
  if (!h) return set_error(GK_ERR_INVALID_ARGUMENT, "handle is NULL");
  if (!desc || desc->struct_size != sizeof(gk_contract_desc))
    return set_error(GK_ERR_INVALID_ARGUMENT, "gk_contract_desc.struct_size does not match this library (%zu)", sizeof(gk_contract_desc));
  Groups g;
  gk_status s = classify(*desc, &g);
  if (s != GK_OK) return s;
  if (g.b.empty() || plan_only) return contract_one(h, desc, g, a, b, c, dd, workspace, workspace_bytes, stream, plan_only);
  std::vector<BatchOffsets> offs;
  if ((s = batch_offsets(g, &offs)) != GK_OK) return s;
  const size_t ea = dtype_size(desc->dtype_a), eb = dtype_size(desc->dtype_b), ec = dtype_size(desc->dtype_c),
               ed = dtype_size(desc->dtype_d);
  for (const BatchOffsets& o : offs) {
    s = contract_one(h, desc, g, static_cast<const char*>(a) + o.a * ea, static_cast<const char*>(b) + o.b * eb,
                     c ? static_cast<const char*>(c) + o.c * ec : nullptr, static_cast<char*>(dd) + o.d * ed, workspace,
                     workspace_bytes, stream, nullptr);
    if (s != GK_OK) return s;
  }
  return GK_OK;
}

// ------------------------------------------------------------------------------------------------
// gather path without any allocation: the offset tables live in this fixed device array
// ------------------------------------------------------------------------------------------------
// GK_STATIC_TABLE_ENTRIES 64-bit offsets (256 KiB).  Every GPU that loads the library holds this
// array from load until the process exits.  All calls of gk_contract_static on a device share it.
static __device__ __align__(256) long long g_static_tables[GK_STATIC_TABLE_ENTRIES];

// In host code the name `g_static_tables` is only a stand-in for the symbol, not a device address:
// the address each device uses is asked for once, with that device current, and cached here.
static constexpr int kMaxDevices = 64;
static std::mutex g_static_mu;
static int64_t* g_static_ptr[kMaxDevices] = {};

static gk_status static_tables_for_current_device(int64_t** out) {
  int dev = -1;
  GK_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return set_error(GK_ERR_CUDA, "device ordinal %d is outside the supported range 0..%d", dev, kMaxDevices - 1);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_tables);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error(GK_ERR_CUDA, "cudaGetSymbolAddress(g_static_tables) failed on device %d: %s", dev,
                       cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<int64_t*>(ptr);
  }
  *out = g_static_ptr[dev];
  return GK_OK;
}

}  // namespace gk

using namespace gk;

extern "C" {

gk_status gk_contract_query(gk_handle h, const gk_contract_desc* desc, gk_gemm_plan* plan) {
  clear_error();
  if (!plan) return set_error(GK_ERR_INVALID_ARGUMENT, "plan is NULL");
  return contract_impl(h, desc, nullptr, nullptr, nullptr, nullptr, nullptr, 0, nullptr, plan);
}

gk_status gk_contract(gk_handle h, const gk_contract_desc* desc, const void* a, const void* b, const void* c,
                      void* d, void* workspace, int64_t workspace_bytes, gk_stream stream) {
  clear_error();
  if (!a || !b || !d) return set_error(GK_ERR_INVALID_ARGUMENT, "A, B or D is NULL");
  if (desc && desc->beta != 0.0 && !c)
    return set_error(GK_ERR_INVALID_ARGUMENT, "beta = %g but C is NULL (pass C, or beta = 0)", desc->beta);
  return contract_impl(h, desc, a, b, c, d, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), nullptr);
}

gk_status gk_contract_static(const gk_contract_desc* desc, const void* a, const void* b, const void* c,
                             void* d, gk_stream stream) {
  clear_error();
  if (!a || !b || !d) return set_error(GK_ERR_INVALID_ARGUMENT, "A, B or D is NULL");
  if (!desc || desc->struct_size != sizeof(gk_contract_desc))
    return set_error(GK_ERR_INVALID_ARGUMENT, "gk_contract_desc.struct_size does not match this library (%zu)",
                     sizeof(gk_contract_desc));
  if (desc->beta != 0.0 && !c)
    return set_error(GK_ERR_INVALID_ARGUMENT, "beta = %g but C is NULL (pass C, or beta = 0)", desc->beta);
  if (desc->compute == GK_TF32)
    return set_error(GK_ERR_INVALID_CONFIG, "gk_contract_static runs the gather kernel only; TF32 needs the tensor cores");
  Groups g;
  gk_status s = classify(*desc, &g);
  if (s != GK_OK) return s;
  const int64_t entries = 3 * g.M + 3 * g.N + 2 * g.K;
  if (entries > GK_STATIC_TABLE_ENTRIES)
    return set_error(GK_ERR_INVALID_CONFIG,
                     "contraction too large for gk_contract_static: 3*M + 3*N + 2*K = %lld offset-table entries, "
                     "the fixed table holds %d (M = %lld, N = %lld, K = %lld); use gk_contract with a workspace",
                     (long long)entries, GK_STATIC_TABLE_ENTRIES, (long long)g.M, (long long)g.N, (long long)g.K);
  int64_t* tables = nullptr;
  s = static_tables_for_current_device(&tables);   // first call on a device: symbol address look-up
  if (s != GK_OK) return s;
  // The tables are rewritten in full for this contraction before the gather kernel reads them
  // (same stream), so nothing has to start at zero.  Batch modes: one launch per index combination.
  std::vector<BatchOffsets> offs;
  if ((s = batch_offsets(g, &offs)) != GK_OK) return s;
  const size_t ea = dtype_size(desc->dtype_a), eb = dtype_size(desc->dtype_b), ec = dtype_size(desc->dtype_c),
               ed = dtype_size(desc->dtype_d);
  for (const BatchOffsets& o : offs) {
    s = launch_gather(*desc, g, static_cast<const char*>(a) + o.a * ea, static_cast<const char*>(b) + o.b * eb,
                      (desc->beta != 0.0) ? static_cast<const char*>(c) + o.c * ec : nullptr, static_cast<char*>(d) + o.d * ed,
                      tables, static_cast<cudaStream_t>(stream));
    if (s != GK_OK) return s;
  }
  return GK_OK;
}

}  // extern "C"
