// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D = act( alpha * sum_terms(+/- A_plane * B_plane) + beta * C + bias )
//
// One kernel covers the real product (one term), the planar complex product (four terms, two
// accumulator planes) and the dual-number product (three terms).  Operands reach shared memory by
// TMA with the 128-byte swizzle and are consumed by tcgen05.mma straight from there; accumulators
// live in tensor memory, double-buffered so the epilogue of one tile overlaps the main loop of the
// next (single-buffered for the widest tiles, which fill all 512 columns: n_sub == 2 makes one tile
// of two column blocks that reuse the same A stage, halving A's share of the shared-memory feed).
// With CG == 2 two CTAs of a cluster form one 256-row tile: each loads its own 128 rows of A and its
// own half of B's columns (no multicast), and the pair leader issues the MMAs for both.  With
// k_split > 1 a work unit is one run of k-blocks of a tile and writes partial sums to a workspace.
//
// Warp roles: warp 0 = TMA producer for A, warp 1 = MMA issuer, warp 2 = TMEM allocator, warp 3 =
// TMA producer for B, warps 4.. = epilogue (warp w reads TMEM lanes 32*(w%4)..+31; the one-plane
// kernels run eight epilogue warps, 384 threads, two per lane quarter taking alternate 32-column
// chunks; the two-plane kernels four, 256 threads).
//
// Every barrier wait is bounded (ptx.cuh: mbar_wait).  When a wait gives up, the CTA raises a
// shared abort flag, all roles leave their loops, in-flight copies and MMAs are drained with
// bounded waits, TMEM is released, and an error code is left in *status for the host.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace gk {

// 4 role warps + the epilogue warps: 8 of them for the one-plane kernels (two per TMEM lane quarter,
// taking alternate 32-column chunks), 4 for the two-plane kernels, whose epilogue needs more
// registers per thread than a 384-thread CTA leaves.
__host__ __device__ constexpr int tc_epilogue_warps(int planes) { return planes == 1 ? 8 : 4; }
__host__ __device__ constexpr int tc_threads(int planes) { return 128 + 32 * tc_epilogue_warps(planes); }
constexpr int kTcTileM = 128;              // rows per CTA (TMEM lanes)
constexpr int kTcKBytes = 128;             // bytes of K per k-block row (= swizzle span)
constexpr int kTcMmaPerKBlock = 4;         // each MMA consumes 32 bytes of K
constexpr uint64_t kTcWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait

enum TcDtype : int32_t { TC_F16 = 0, TC_BF16 = 1, TC_F32 = 2 };
enum TcAct : int32_t { TC_ACT_NONE = 0, TC_ACT_RELU = 1, TC_ACT_GELU = 2 };
enum TcBias : int32_t { TC_BIAS_NONE = 0, TC_BIAS_ROW = 1, TC_BIAS_COL = 2 };

// status word values (0 = ok)
enum TcStatus : int32_t {
  TC_ST_OK = 0,
  TC_ST_TIMEOUT_PRODUCER = 101,
  TC_ST_TIMEOUT_MMA = 102,
  TC_ST_TIMEOUT_EPILOGUE = 103,
  TC_ST_TIMEOUT_DRAIN = 104,
};

struct TcTerm {
  uint8_t a_plane, b_plane, acc_plane, negate_a;
  uint8_t first;  // first term that writes its accumulator plane: overwrites at k == 0
  uint8_t pad[3];
};

struct TcParams {
  CUtensorMap tm_a;  // dims {contiguous, strided, plane}
  CUtensorMap tm_b;
  int32_t M, N, K;
  int32_t tiles_m, tiles_n;  // cluster tiles: (128*CG) x (n_sub*bn)
  int32_t k_blocks;
  // Split-K (few tiles, long K): the k-blocks are dealt out in k_split contiguous runs of kb_per_split,
  // work unit t = tile * k_split + run; every run writes its raw FP32 partial sums to plane `run` of a
  // workspace (split_stride elements apart) and a second kernel adds the planes and applies the epilogue.
  int32_t k_split, kb_per_split;
  int64_t split_stride;
  // Strided-batched real products: work units run over (product, tile, k-run); an operand whose tensor
  // map lists the batch as its third mode has x_batched = 1 (0: shared by all products).
  int32_t batch, a_batched, b_batched;
  int64_t c_batch, d_batch;  // elements between the C / D of consecutive products
  int32_t raster_group;      // cluster tiles along M (N for the horizontal raster) walked before stepping on
  int32_t raster_kind;       // 0 = bands down M, 1 = bands along N, 2 = Z-order (power-of-two tile grids)
  int32_t z_bits;            // Z-order: low bits interleaved per dimension (min of the two log2 extents)
  int32_t bn;                // columns per MMA (multiple of 32; per-CTA B rows = bn/CG)
  int32_t n_sub;             // a cluster tile is n_sub (1 or 2) such column blocks that share A
  int32_t acc_stages;        // accumulator stages in TMEM: 2, or 1 when one tile fills all 512 columns
  int32_t skew;              // 1: a 512-column tile's two column blocks finish (and start) half a ring apart, each
                             // with its own full / empty barrier, so the epilogue of block 0 overlaps the last
                             // MMAs of block 1 and the first MMAs of the next tile overlap the epilogue of block 1
  int32_t bk;                // K elements per k-block (128 bytes)
  int32_t kps;               // k-blocks per pipeline stage (1 or 2): one full/empty barrier round trip and one
                             // tcgen05.commit serve kps k-blocks, which halves the fixed cost per k-block
  int32_t stages;
  int32_t a_mn_major, b_mn_major;
  int32_t a_boxes, b_boxes;  // TMA boxes per plane per CTA per k-block
  int32_t a_box_mn, b_box_mn;  // M/N elements per box of an MN-major operand (one swizzle span)
  int32_t a_box_bytes, b_box_bytes;
  int32_t a_plane_bytes, b_plane_bytes;  // shared memory per plane per stage per CTA
  int32_t a_planes, b_planes;
  int32_t n_terms;
  TcTerm terms[4];
  uint32_t idesc, idesc_neg;  // instruction descriptors (second one negates A)
  uint32_t a_lbo, a_sbo, a_kadv, b_lbo, b_sbo, b_kadv;  // bytes
  uint32_t a_swz, b_swz;      // descriptor swizzle field per operand (ptx.cuh: smem_desc_hi)
  uint32_t tmem_cols;         // power of two >= acc_stages * n_sub * acc_planes * bn
  // GENERIC kernels (operands that TMA cannot address: a base or leading dimension that is not a
  // multiple of 16 bytes): the producer warps read A and B with bounds-checked loads and write the same
  // swizzled stage layout themselves.  16-bit element types, one plane, one CTA per tile.
  const void* ga; const void* gb;
  int64_t g_lda, g_ldb;          // elements between consecutive values of the strided index
  int64_t g_a_batch, g_b_batch;  // elements between the operands of consecutive products of a batch
  // Tensor contractions split an index of the product in two modes: index = in + div * out.
  // For a plain matrix the divisor is INT32_MAX (out == 0).  RANK5 kernels use these in the
  // producers (5-D tensor maps: {in, out} of the contiguous index, {in, out} of the other, plane).
  int32_t a_mn_div, a_k_div, b_mn_div, b_k_div;
  // RANK5 only.  A tensor map lists its modes in order of increasing stride (what the TMA unit
  // expects), so each box is one contiguous run times ONE other mode; a k-block (or a tile's rows)
  // that spans two modes is fetched as `sub` boxes.  perm packs, 3 bits each, the tensor-map
  // position of the coordinates (mn_in, mn_out, k_in, k_out).
  int32_t a_sub, a_sub_step, a_sub_bytes, a_perm;
  int32_t b_sub, b_sub_step, b_sub_bytes, b_perm;
  // epilogue: element (m, n) of D is at d_sm0*(m % m_div) + d_sm1*(m / m_div)
  //                                   + d_sn0*(n % n_div) + d_sn1*(n / n_div); same for C.
  const void* C;
  void* D;
  int32_t m_div, n_div;       // n_div is a multiple of 32 or >= N
  int64_t c_sm0, c_sm1, c_sn0, c_sn1;
  int64_t d_sm0, d_sm1, d_sn0, d_sn1;
  int64_t c_plane, d_plane;   // elements between planes; 0 = interleaved (re, im) pairs
  int32_t dtype_c, dtype_d;
  float alpha, beta;
  const float* bias;
  int32_t bias_axis, act;
  int32_t* status;
  int32_t debug;  // measurement/test aids, 0 in production: 1 = no TMA (barriers only),
                  // 2 = no MMA, 4 = producers issue nothing (lets the bounded waits run out),
                  // 8 = per-role cycle counters written to dbg_out[blockIdx.x * 16 + i],
                  // 16 = CTA 0 leaves progress marks in the host-visible diagnostic words
  long long* dbg_out;
};

// The status word may live in host-mapped memory: plain stores, first error wins.
__device__ __forceinline__ void tc_report(int32_t* status, int32_t code) {
  volatile int32_t* s = status;
  if (s != nullptr && *s == TC_ST_OK) {
    *s = code;
    __threadfence_system();
  }
}

// Progress mark (debug bit 16): word `slot` (1..15) of the host-visible diagnostic area.
__device__ __forceinline__ void tc_mark(const int32_t* status, int debug, int slot, int32_t value) {
  if ((debug & 16) && status != nullptr && blockIdx.x == 0) {
    volatile int32_t* s = const_cast<int32_t*>(status);
    s[slot] = value;
    __threadfence_system();
  }
}

__device__ __forceinline__ float tc_load_elem(const void* p, int64_t idx, int32_t dt) {
  if (dt == TC_F32) return static_cast<const float*>(p)[idx];
  if (dt == TC_F16) return __half2float(static_cast<const __half*>(p)[idx]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

__device__ __forceinline__ void tc_store_elem(void* p, int64_t idx, int32_t dt, float v) {
  if (dt == TC_F32)
    static_cast<float*>(p)[idx] = v;
  else if (dt == TC_F16)
    static_cast<__half*>(p)[idx] = __float2half_rn(v);
  else
    static_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float tc_activation(float v, int32_t act) {
  if (act == TC_ACT_RELU) return fmaxf(v, 0.0f);
  if (act == TC_ACT_GELU) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
  return v;
}

// Epilogue of one full 32-column chunk with the element types fixed at compile time (DTC < 0: no C
// operand).  All loads of C are issued before the first use, so their latencies overlap; the
// arithmetic is the same expression, in the same order, as the element-wise path for ragged chunks.
template <int DT> struct TcElem { using type = float; };
template <> struct TcElem<TC_F16> { using type = __half; };
template <> struct TcElem<TC_BF16> { using type = __nv_bfloat16; };
__device__ __forceinline__ float tc_to_float(float x) { return x; }
__device__ __forceinline__ float tc_to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float tc_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T tc_from_float(float x);
template <> __device__ __forceinline__ float tc_from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half tc_from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 tc_from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <int PLANES, int DTC, int DTD>
__device__ __forceinline__ void tc_epilogue_chunk(const TcParams& p, const uint32_t (&v)[PLANES][32], int64_t ci,
                                                  int64_t di, float bias_row, int col0) {
  // The work is arranged as passes over the 32 register values, each pass a straight run of one kind
  // of instruction with its warp-uniform decision taken once per chunk, not once per element.
  using TC = typename TcElem<(DTC >= 0 ? DTC : TC_F32)>::type;
  using TD = typename TcElem<DTD>::type;
  const bool c_pairs = PLANES == 2 && p.c_plane == 0;
  const bool d_pairs = PLANES == 2 && p.d_plane == 0;
  float x[PLANES][32];
  if constexpr (DTC >= 0) {
    TC cv[PLANES][32];
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
      const TC* cp = static_cast<const TC*>(p.C) + (c_pairs ? 2 * ci + pl : pl * p.c_plane + ci);
      const int64_t step = c_pairs ? 2 * p.c_sn0 : p.c_sn0;
#pragma unroll
      for (int j = 0; j < 32; ++j) cv[pl][j] = cp[j * step];
    }
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float t = p.alpha * __uint_as_float(v[pl][j]);
        t += p.beta * tc_to_float(cv[pl][j]);
        x[pl][j] = t;
      }
    }
  } else {
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[pl][j] = p.alpha * __uint_as_float(v[pl][j]);
    }
  }
  if (p.bias_axis == TC_BIAS_COL) {
    const float* bias_col = p.bias + col0;
#pragma unroll
    for (int j = 0; j < 32; ++j) x[0][j] += bias_col[j];
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) x[0][j] += bias_row;
  }
  if (p.act == TC_ACT_RELU) {
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[pl][j] = fmaxf(x[pl][j], 0.0f);
    }
  } else if (p.act == TC_ACT_GELU) {
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
#pragma unroll
      for (int j = 0; j < 32; ++j) x[pl][j] = tc_activation(x[pl][j], TC_ACT_GELU);
    }
  }
  if (DTD == TC_F32 && d_pairs) {
    float2* dp = reinterpret_cast<float2*>(p.D) + di;
#pragma unroll
    for (int j = 0; j < 32; ++j) dp[j * p.d_sn0] = make_float2(x[0][j], x[PLANES - 1][j]);
  } else {
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
      TD* dp = static_cast<TD*>(p.D) + (d_pairs ? 2 * di + pl : pl * p.d_plane + di);
      const int64_t step = d_pairs ? 2 * p.d_sn0 : p.d_sn0;
#pragma unroll
      for (int j = 0; j < 32; ++j) dp[j * step] = tc_from_float<TD>(x[pl][j]);
    }
  }
}

// Even-position bits of x packed together (bit 0, 2, 4, ... -> bit 0, 1, 2, ...).
__device__ __forceinline__ uint32_t tc_even_bits(uint32_t x) {
  x &= 0x55555555u;
  x = (x | (x >> 1)) & 0x33333333u;
  x = (x | (x >> 2)) & 0x0F0F0F0Fu;
  x = (x | (x >> 4)) & 0x00FF00FFu;
  x = (x | (x >> 8)) & 0x0000FFFFu;
  return x;
}

// Cluster tile index -> (tile_m, tile_n).  Default: walk `raster_group` tiles down M, then step along
// N, so that the tiles in flight at any time share A rows and B columns in L2 (the reference's
// VerticallyTiled{T} grouping); kind 1 swaps the roles of M and N (HorizontallyTiled{T}); kind 2 is
// the Z-order curve of LebesgueCurve (M takes the even bits), the excess of the longer dimension
// continuing in its high bits.
__device__ __forceinline__ void tc_tile_coords(const TcParams& p, int t, int& tm, int& tn) {
  if (p.raster_kind == 2) {
    const uint32_t low = static_cast<uint32_t>(t) & ((1u << (2 * p.z_bits)) - 1u);
    const int rest = t >> (2 * p.z_bits);
    tm = static_cast<int>(tc_even_bits(low));
    tn = static_cast<int>(tc_even_bits(low >> 1));
    if (p.tiles_m >= p.tiles_n) tm += rest << p.z_bits;
    else tn += rest << p.z_bits;
    return;
  }
  const bool along_n = p.raster_kind == 1;
  const int major = along_n ? p.tiles_n : p.tiles_m;   // the dimension the bands cut
  const int minor = along_n ? p.tiles_m : p.tiles_n;
  const int g = p.raster_group;
  const int band = g * minor;
  const int band_id = t / band;
  const int first = band_id * g;
  const int rows = min(g, major - first);
  const int r = t - band_id * band;
  const int a = first + r % rows, b = r / rows;
  tm = along_n ? b : a;
  tn = along_n ? a : b;
}

// One box of a stage written by a warp with ordinary loads: `rows` rows of 128 bytes (64 16-bit
// elements of the contiguous index u, starting at u0) for the strided index v0 .. v0 + rows - 1, in
// the layout TMA's 128-byte swizzle produces (16-byte chunk c of row r lands at chunk c ^ (r % 8);
// dst is 1024-byte aligned).  Elements outside [0, U) x [0, V) read as zero, as TMA fills them.
__device__ __forceinline__ void tc_fill_box_generic(uint8_t* dst, const uint16_t* g, int64_t ld, int u0, int v0, int U,
                                                    int V, int rows, int lane) {
  for (int idx = lane; idx < rows * 8; idx += 32) {
    const int r = idx >> 3, c = idx & 7;
    const int u = u0 + c * 8, v = v0 + r;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (v < V && u < U) {
      const uint16_t* src = g + static_cast<int64_t>(v) * ld + u;
      if (u + 8 <= U && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        val = *reinterpret_cast<const uint4*>(src);
      } else {
        uint16_t e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = (u + j < U) ? src[j] : static_cast<uint16_t>(0);
        val.x = e[0] | (static_cast<uint32_t>(e[1]) << 16); val.y = e[2] | (static_cast<uint32_t>(e[3]) << 16);
        val.z = e[4] | (static_cast<uint32_t>(e[5]) << 16); val.w = e[6] | (static_cast<uint32_t>(e[7]) << 16);
      }
    }
    *reinterpret_cast<uint4*>(dst + r * 128 + ((c ^ (r & 7)) << 4)) = val;
  }
}

// All MMAs of one k-block as straight-line code: NSUB column blocks x NTERMS terms x the K steps of a
// k-block, no branch between them (a single warp pays 10-20 cycles for every branch it resolves, taken or
// not, and eight of them per k-block were more than the MMAs of a small tile).  `lo` is the k-block's base
// in descriptor units; the tables hold the offsets of each operand slice relative to it.  NB0 is the first
// column block (the skewed schedule of 512-column tiles issues the two blocks of a k-block apart).
template <int CG, bool TF32, int KMAX, int NSUB, int NTERMS, int NB0 = 0>
__device__ __forceinline__ void tc_issue_kblock(uint32_t lo, bool first, uint32_t d_base, uint32_t hi_a, uint32_t hi_b,
                                                const uint32_t (&off_a)[KMAX][kTcMmaPerKBlock],
                                                const uint32_t (&off_b)[KMAX][2][kTcMmaPerKBlock],
                                                const uint32_t (&d_off)[KMAX][2], const uint32_t (&t_id)[KMAX],
                                                const uint32_t (&t_keep)[KMAX]) {
#pragma unroll
  for (int ks = 0; ks < kTcMmaPerKBlock; ++ks)
#pragma unroll
    for (int nb = NB0; nb < NB0 + NSUB; ++nb)
#pragma unroll
      for (int ti = 0; ti < NTERMS; ++ti) {
        const uint32_t acc = (ks == 0 && first) ? t_keep[ti] : 1u;
        umma<CG, TF32>(d_base + d_off[ti][nb], smem_desc(lo + off_a[ti][ks], hi_a), smem_desc(lo + off_b[ti][nb][ks], hi_b),
                       t_id[ti], acc);
      }
}

// DBG selects the instance that honours TcParams::debug (measurement and test aids); in the production
// instance every such branch is compiled out, which shortens the per-stage loops of the producer and
// MMA warps (their cost per pipeline stage is instruction latency, not bandwidth).
template <int CG, int PLANES, bool TF32, bool RANK5, bool GENERIC = false, bool DBG = false>
__global__ void __launch_bounds__(tc_threads(PLANES), 1) tc_gemm_kernel(const __grid_constant__ TcParams p) {
  const int dbg = DBG ? p.debug : 0;
  static_assert(!GENERIC || (CG == 1 && PLANES == 1 && !TF32 && !RANK5), "generic loads: one CTA, one plane, 16-bit types");
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms are 1024 bytes and the pattern is a function of the address.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (CG == 2) ? cluster_cta_rank() : 0u;
  const bool leader = (rank == 0);

  const uint32_t b_sub_bytes = p.b_planes * p.b_plane_bytes;   // one column block of B in a stage
  const uint32_t kblock_bytes = p.a_planes * p.a_plane_bytes + p.n_sub * b_sub_bytes;   // operands of one k-block
  const uint32_t stage_bytes = p.kps * kblock_bytes;                                     // a stage holds kps of them
  const uint32_t ctrl = smem_base + p.stages * stage_bytes;  // control block after the stages
  // control block layout (8-byte slots): full[stages], empty[stages], tmem_full[2], tmem_empty[2],
  // drain, then two 32-bit words: tmem base, abort flag.
  const uint32_t bar_full = ctrl;
  const uint32_t bar_empty = ctrl + 8u * p.stages;
  const uint32_t bar_tfull = ctrl + 16u * p.stages;
  const uint32_t bar_tempty = bar_tfull + 16u;
  const uint32_t bar_drain = bar_tempty + 16u;
  const uint32_t tmem_slot = bar_drain + 8u;
  uint8_t* ctrl_gen = smem_gen + p.stages * stage_bytes;
  volatile uint32_t* tmem_slot_gen =
      reinterpret_cast<volatile uint32_t*>(ctrl_gen + 16 * p.stages + 40);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl_gen + 16 * p.stages + 44);

  // Let the next kernel of the stream begin its own set-up as SMs free up (it waits, as this one does
  // below, before touching global memory).
  pdl_launch_dependents();
  const uint64_t t_entry = (dbg & 8) ? global_timer_ns() : 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + 8u * s, GENERIC ? 2 : 1);   // TMA: one arrival that also expects the bytes; generic: one per producer warp
      mbar_init(bar_empty + 8u * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8u * a, 1);
      mbar_init(bar_tempty + 8u * a, tc_epilogue_warps(PLANES) * CG);  // one arrival per epilogue warp per CTA
    }
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    fence_mbar_init();
    if constexpr (!GENERIC) {
      prefetch_tensormap(&p.tm_a);
      prefetch_tensormap(&p.tm_b);
    }
  }
  if (warp == 2) {
    tmem_alloc<CG>(tmem_slot, p.tmem_cols);
    tmem_relinquish<CG>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // peer barriers are initialised before any remote use
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  if (threadIdx.x == 0) tc_mark(p.status, dbg, 1, 1);   // set-up done, TMEM allocated

  const int units_per_product = p.tiles_m * p.tiles_n * p.k_split;
  const int num_tiles = units_per_product * p.batch;         // work units
  const int cluster_id = blockIdx.x / CG;
  const int num_clusters = gridDim.x / CG;
  const int bn_cta = p.bn / CG;
  const int bn_tile = p.bn * p.n_sub;       // columns per cluster tile
  const uint32_t sub_cols = PLANES * p.bn;  // TMEM columns per column block
  const uint32_t acc_cols = p.n_sub * sub_cols;  // TMEM columns per accumulator stage
  const bool two_acc = p.acc_stages == 2;
  const bool skew = !DBG && !GENERIC && PLANES == 1 && p.skew != 0;   // the diagnostic instance keeps the plain schedule

  if constexpr (GENERIC) {
    if (warp == 0 || warp == 3) {
      // -------------------------------------------------------------- producers with ordinary loads
      // Warp 0 fills A's part of each stage, warp 3 B's; a stage is full once both have arrived.
      const bool is_a = warp == 0;
      const bool mn_major = (is_a ? p.a_mn_major : p.b_mn_major) != 0;
      const int boxes = is_a ? p.a_boxes : p.b_boxes;
      const int box_mn = is_a ? p.a_box_mn : p.b_box_mn;
      const uint32_t box_bytes = is_a ? p.a_box_bytes : p.b_box_bytes;
      const uint32_t part_off = is_a ? 0u : static_cast<uint32_t>(p.a_planes * p.a_plane_bytes);
      const int64_t ld = is_a ? p.g_lda : p.g_ldb;
      const int mn_ext = is_a ? p.M : p.N;
      const int rows_k_major = is_a ? kTcTileM : p.bn;     // rows of the one box of a K-major operand
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      pdl_wait();
      for (int t = cluster_id; t < num_tiles && ok && !(dbg & 4); t += num_clusters) {
        int tm, tn;
        const int bt = t / units_per_product;
        tc_tile_coords(p, (t - bt * units_per_product) / p.k_split, tm, tn);
        const int kb0 = (t % p.k_split) * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
        const int mn0 = is_a ? tm * kTcTileM : tn * bn_tile;
        const uint16_t* g = static_cast<const uint16_t*>(is_a ? p.ga : p.gb) + bt * (is_a ? p.g_a_batch : p.g_b_batch);
        for (int kb = kb0; kb < kb1; kb += p.kps) {
          const bool got = mbar_wait(bar_empty + 8u * s, ph ^ 1u, abort_flag, kTcWaitLimitNs);
          if (!__all_sync(0xffffffffu, got)) {
            if (lane == 0) tc_report(p.status, TC_ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          for (int j = 0; j < p.kps; ++j) {
            uint8_t* stage = smem_gen + s * stage_bytes + j * kblock_bytes + part_off;
            const int k0 = (kb + j) * p.bk;
            if (mn_major) {
              for (int bx = 0; bx < boxes; ++bx)
                tc_fill_box_generic(stage + bx * box_bytes, g, ld, mn0 + bx * box_mn, k0, mn_ext, p.K, p.bk, lane);
            } else {
              tc_fill_box_generic(stage, g, ld, k0, mn0, p.K, mn_ext, rows_k_major, lane);
            }
          }
          fence_proxy_async_smem();   // the tensor cores read shared memory through the asynchronous proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full + 8u * s);
          if (++s == p.stages) { s = 0; ph ^= 1u; }
        }
      }
    }
  }
  if (!GENERIC && (warp == 0 || warp == 3)) {
    // ------------------------------------------------------------------ TMA producers
    // Both warps load both operands, for alternate pipeline stages (warp 0 the even ones, warp 3 the odd
    // ones).  Filling a stage costs its warp a few hundred cycles whatever the stage holds - the wait for
    // the slot, the vote, the divergent region that issues the copies - so two warps on alternate stages
    // have twice the time per stage that one warp per operand had (worth 1 % on 256 x 256 tiles at 8192^3,
    // whose main loop is otherwise bound by the L2 -> shared memory rate: with the MMAs switched off it
    // still takes 606 us).  One lane per TMA box, A's boxes on the first lanes and B's behind them: every
    // lane runs the same short instruction stream with its own destination and coordinates, so the cost
    // per stage does not grow with the box count.  (Measured on B200: issuing from one elected lane of a
    // converged warp with warp-uniform operands cost ~3x more cycles per copy.)
    {
      const uint32_t which = warp == 0 ? 0u : 1u;
      const int a_subs = RANK5 ? p.a_sub : 1, b_subs = RANK5 ? p.b_sub : 1;
      const int a_per_block = p.a_planes * p.a_boxes * a_subs;             // A boxes of one k-block
      const int b_per_block = p.b_planes * p.b_boxes * b_subs;             // B boxes of one column block and k-block
      const int a_pieces = a_per_block * p.kps;                            // A boxes of one stage
      const int b_pieces = p.n_sub * b_per_block * p.kps;
      const bool is_a = lane < a_pieces;
      const bool active = lane < a_pieces + b_pieces;
      const int piece = active ? (is_a ? lane : lane - a_pieces) : 0;
      const int subs = is_a ? a_subs : b_subs;
      const int per_plane = (is_a ? p.a_boxes : p.b_boxes) * subs;
      const int per_block = is_a ? a_per_block : b_per_block;
      const int n_boxes = (is_a ? 1 : p.n_sub) * per_block;    // boxes of one k-block
      const int kj = piece / n_boxes;                          // which k-block of the stage
      const int bl = piece % n_boxes;                          // which box of that k-block
      const int nb = bl / per_block;                           // which column block (B only)
      const int pl = (bl % per_block) / per_plane;
      const int bx = (bl % per_plane) / subs;                  // which swizzle-span chunk
      const int sb = (bl % per_plane) % subs;                  // which sub-box of it (RANK5)
      const bool mn_major = (is_a ? p.a_mn_major : p.b_mn_major) != 0;
      const int sub_step = RANK5 ? (is_a ? p.a_sub_step : p.b_sub_step) : 0;
      const uint32_t dst_off =
          (is_a ? pl * p.a_plane_bytes + bx * p.a_box_bytes
                : p.a_planes * p.a_plane_bytes + nb * b_sub_bytes + pl * p.b_plane_bytes + bx * p.b_box_bytes) +
          (RANK5 ? sb * (is_a ? p.a_sub_bytes : p.b_sub_bytes) : 0) + kj * kblock_bytes;
      const void* tmap = is_a ? static_cast<const void*>(&p.tm_a) : static_cast<const void*>(&p.tm_b);
      const int mn_add = (mn_major ? bx * (is_a ? p.a_box_mn : p.b_box_mn) : sb * sub_step) + nb * p.bn;
      [[maybe_unused]] const int k_add = mn_major ? sb * sub_step : 0;
      [[maybe_unused]] const int perm = is_a ? p.a_perm : p.b_perm;
      [[maybe_unused]] const int mn_div = is_a ? p.a_mn_div : p.b_mn_div;   // RANK5 only
      [[maybe_unused]] const int k_div = is_a ? p.a_k_div : p.b_k_div;
      const uint32_t full0_signal = (CG == 2) ? map_to_cta(bar_full, 0) : bar_full;
      const uint32_t tx_bytes = stage_bytes * CG;
      int s = 0;
      uint32_t ph = 0;
      uint32_t it = 0;        // pipeline stages passed so far (both warps count all of them)
      uint32_t armed = 0;     // stages this warp has armed
      uint32_t last_it = 0;   // the last of them
      bool ok = true;
      const bool prof = (dbg & 8) != 0;
      long long pw = 0, pi = 0, pt0 = 0, pt1 = 0;
      pdl_wait();           // operands may be the previous kernel's output
      for (int t = cluster_id; t < num_tiles && ok && !(dbg & 4); t += num_clusters) {
        int tm, tn;
        const int bt = t / units_per_product;                 // which product of the batch
        tc_tile_coords(p, (t - bt * units_per_product) / p.k_split, tm, tn);
        const int kb0 = (t % p.k_split) * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
        [[maybe_unused]] const int c2 = pl + bt * (is_a ? p.a_batched : p.b_batched);   // plane, or product of a batch
        const int m_cta = (tm * CG + static_cast<int>(rank)) * kTcTileM;
        const int n_cta = tn * bn_tile + static_cast<int>(rank) * bn_cta;
        const int mn = (is_a ? m_cta : n_cta) + mn_add;
        // RANK5: the two-mode split of the M/N coordinate is fixed for the tile, and that of the K
        // coordinate advances by one k-block per step: no division inside the k loop.
        [[maybe_unused]] int mn_in = 0, mn_out = 0, k_in = 0, k_out = 0;
        if constexpr (RANK5) {
          mn_in = mn % mn_div; mn_out = mn / mn_div;
          const int kk0 = (kb0 + kj) * p.bk + k_add;
          k_in = kk0 % k_div; k_out = kk0 / k_div;
        }
        for (int kb = kb0; kb < kb1; kb += p.kps, ++it) {
          if ((it & 1u) == which) {
            if (prof) pt0 = clock64();
            const bool got = mbar_wait(bar_empty + 8u * s, ph ^ 1u, abort_flag, kTcWaitLimitNs);
            if (prof) { pt1 = clock64(); pw += pt1 - pt0; }
            if (!__all_sync(0xffffffffu, got)) {
              if (lane == 0) tc_report(p.status, TC_ST_TIMEOUT_PRODUCER);
              ok = false;
              break;
            }
            if (armed == 0 && lane == 0) tc_mark(p.status, dbg, 2 + which, 1);   // about to issue first copies
            if (dbg & 1) {
              if (lane == 0 && leader) mbar_arrive(bar_full + 8u * s);
            } else if (active) {
              // Bytes may be counted on the barrier before they are expected: the phase cannot
              // complete until the arrival that announces them.
              if (lane == 0 && leader) mbar_arrive_expect_tx(bar_full + 8u * s, tx_bytes);
              const int k0 = (kb + kj) * p.bk;     // a k-block past the end of K (or of this K-run) is loaded too:
                                                   // zeros, or operands the MMA issuer does not use
              const uint32_t dst = smem_base + s * stage_bytes + dst_off;
              if constexpr (RANK5) {
                // coordinates of (mn_in, mn_out, k_in, k_out), placed where the tensor map lists them
                const int v[4] = {mn_in, mn_out, k_in, k_out};
                int c[4] = {0, 0, 0, 0};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int pos = (perm >> (3 * q)) & 7;
#pragma unroll
                  for (int d = 0; d < 4; ++d) c[d] = (pos == d) ? v[q] : c[d];
                }
                if constexpr (CG == 2) tma_load_5d_pair(dst, tmap, full0_signal + 8u * s, c[0], c[1], c[2], c[3], pl);
                else tma_load_5d(dst, tmap, full0_signal + 8u * s, c[0], c[1], c[2], c[3], pl);
              } else {
                const int c0 = mn_major ? mn : k0;
                const int c1 = mn_major ? k0 : mn;
                if constexpr (CG == 2) tma_load_3d_pair(dst, tmap, full0_signal + 8u * s, c0, c1, c2);
                else tma_load_3d(dst, tmap, full0_signal + 8u * s, c0, c1, c2);
              }
            }
            if (armed == 0 && lane == 0) tc_mark(p.status, dbg, 2 + which, 2);   // first copies issued
            ++armed; last_it = it;
            if (prof) pi += clock64() - pt1;
          }
          if constexpr (RANK5) {
            k_in += p.kps * p.bk;
            while (k_in >= k_div) { k_in -= k_div; ++k_out; }
          }
          if (++s == p.stages) { s = 0; ph ^= 1u; }
        }
      }
      if (prof && lane == 0) {
        p.dbg_out[blockIdx.x * 16 + (which == 0 ? 0 : 9)] = pw;
        p.dbg_out[blockIdx.x * 16 + (which == 0 ? 1 : 10)] = pi;
      }
      if (!ok && lane == 0) {
        if (leader) {
          // Let this CTA's copies in flight land before shared memory is given back: the full
          // barrier of every stage this warp armed completes when its bytes arrive.
          uint32_t idx = last_it;
          for (uint32_t b = 0; b < armed && 2 * b < static_cast<uint32_t>(p.stages) + 1; ++b, idx -= 2) {
            const uint32_t st = idx % p.stages;
            const uint32_t par = (idx / p.stages) & 1u;
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(bar_full + 8u * st, par)) {
              if (global_timer_ns() - t0 > 2000000ull) break;  // 2 ms per stage at most
            }
          }
        } else {
          // The peer's copies signal the leader's barriers; give them a bounded time to land.
          const uint64_t t0 = global_timer_ns();
          while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Same discipline as the producer: the warp stays converged, descriptors are computed from
    // warp-uniform values (tcgen05.mma takes them from the uniform datapath), and only the
    // instruction itself is predicated on the elected lane.
    if (leader) {
      constexpr int kMaxTerms = (PLANES == 1) ? 1 : 4;
      const bool elected = elect_one();
      const uint32_t hi_a = smem_desc_hi(p.a_sbo, p.a_swz);
      const uint32_t hi_b = smem_desc_hi(p.b_sbo, p.b_swz);
      uint32_t t_a[kMaxTerms], t_b[kMaxTerms], t_d[kMaxTerms], t_id[kMaxTerms], t_keep[kMaxTerms];
#pragma unroll
      for (int ti = 0; ti < kMaxTerms; ++ti) {
        const TcTerm tr = p.terms[ti < p.n_terms ? ti : 0];
        t_a[ti] = smem_desc_lo(tr.a_plane * p.a_plane_bytes, p.a_lbo);
        t_b[ti] = smem_desc_lo(p.a_planes * p.a_plane_bytes + tr.b_plane * p.b_plane_bytes, p.b_lbo);
        t_d[ti] = tr.acc_plane * p.bn;
        t_id[ti] = tr.negate_a ? p.idesc_neg : p.idesc;
        t_keep[ti] = tr.first ? 0u : 1u;
      }
      const uint32_t base16 = (smem_base & 0x3FFFFu) >> 4;
      const uint32_t stage16 = stage_bytes >> 4, kblock16 = kblock_bytes >> 4;
      const uint32_t a_k16 = p.a_kadv >> 4, b_k16 = p.b_kadv >> 4;
      const uint32_t b_sub16 = b_sub_bytes >> 4;
      const int n_terms = (dbg & 2) ? 0 : p.n_terms;
      // Low descriptor words relative to the k-block's base, and accumulator columns, for every MMA of a
      // k-block: the loop then adds the base and issues.
      uint32_t off_a[kMaxTerms][kTcMmaPerKBlock], off_b[kMaxTerms][2][kTcMmaPerKBlock], d_off[kMaxTerms][2];
#pragma unroll
      for (int ti = 0; ti < kMaxTerms; ++ti) {
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          d_off[ti][nb] = nb * sub_cols + t_d[ti];
#pragma unroll
          for (int ks = 0; ks < kTcMmaPerKBlock; ++ks) off_b[ti][nb][ks] = t_b[ti] + nb * b_sub16 + ks * b_k16;
        }
#pragma unroll
        for (int ks = 0; ks < kTcMmaPerKBlock; ++ks) off_a[ti][ks] = t_a[ti] + ks * a_k16;
      }
      // (Running this loop on the elected lane alone, and polling the producers' barriers from one lane, was
      // measured and is slower than the converged warps: 744 against 728 us at 8192^3, 26.6 against 25.8 us at 2048^3.)
      const bool reporter = lane == 0;
      int s = 0;
      uint32_t s16 = base16;
      uint32_t ph = 0;
      uint32_t acc_it = 0;
      bool ok = true;
      const bool prof = (dbg & 8) != 0;
      long long mw = 0, mi = 0, mt = 0, t0 = 0, t1 = 0;
      const long long k_start = clock64();
      const uint64_t g_start = global_timer_ns();
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++acc_it) {
        const uint32_t as = two_acc ? (acc_it & 1u) : 0u;
        const uint32_t aph = (two_acc ? (acc_it >> 1) : acc_it) & 1u;
        if constexpr (PLANES == 1 && !GENERIC && !DBG) {
          if (skew) {
            // 512-column tile, one accumulator stage, barrier slot h for column block h.  Head: the first F
            // k-blocks (F = the ring's depth) go into block 0 as soon as the epilogue has drained it, then -
            // once block 1 is drained too - into block 1, which is what releases their stages.  Tail: the last
            // F k-blocks go into block 0 first, its accumulator is handed to the epilogue, then into block 1.
            const int kb0 = (t % p.k_split) * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
            const int nkb = kb1 - kb0, F = p.stages;
            auto await = [&](uint32_t bar, uint32_t par) -> bool {
              const bool g = mbar_wait(bar, par, abort_flag, kTcWaitLimitNs);
              if (!__all_sync(0xffffffffu, g)) {
                if (reporter) tc_report(p.status, TC_ST_TIMEOUT_MMA);
                return false;
              }
              tc_fence_after_sync();
              return true;
            };
            auto advance = [&]() {
              ++s; s16 += stage16;
              if (s == p.stages) { s = 0; s16 = base16; ph ^= 1u; }
            };
            ok = await(bar_tempty, aph ^ 1u);
            int s_sv = s; uint32_t s16_sv = s16, ph_sv = ph;
            for (int i = 0; i < F && ok; ++i) {
              ok = await(bar_full + 8u * s, ph);
              if (ok && elected) tc_issue_kblock<CG, TF32, kMaxTerms, 1, 1, 0>(s16, i == 0, tmem_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
              advance();
            }
            if (ok) ok = await(bar_tempty + 8u, aph ^ 1u);
            if (!ok) break;
            s = s_sv; s16 = s16_sv; ph = ph_sv;
            for (int i = 0; i < F; ++i) {
              if (elected) {
                tc_issue_kblock<CG, TF32, kMaxTerms, 1, 1, 1>(s16, i == 0, tmem_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
                umma_commit<CG>(bar_empty + 8u * s);
              }
              advance();
            }
            for (int i = F; i < nkb - F && ok; ++i) {
              ok = await(bar_full + 8u * s, ph);
              if (ok && elected) {
                tc_issue_kblock<CG, TF32, kMaxTerms, 2, 1, 0>(s16, false, tmem_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
                umma_commit<CG>(bar_empty + 8u * s);
              }
              advance();
            }
            s_sv = s; s16_sv = s16; ph_sv = ph;
            for (int i = 0; i < F && ok; ++i) {
              ok = await(bar_full + 8u * s, ph);
              if (ok && elected) tc_issue_kblock<CG, TF32, kMaxTerms, 1, 1, 0>(s16, false, tmem_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
              advance();
            }
            if (!ok) break;
            if (elected) umma_commit<CG>(bar_tfull);            // column block 0 complete
            s = s_sv; s16 = s16_sv; ph = ph_sv;
            for (int i = 0; i < F; ++i) {
              if (elected) {
                tc_issue_kblock<CG, TF32, kMaxTerms, 1, 1, 1>(s16, false, tmem_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
                umma_commit<CG>(bar_empty + 8u * s);
              }
              advance();
            }
            if (elected) umma_commit<CG>(bar_tfull + 8u);       // column block 1 complete
            continue;
          }
        }
        if (prof) t0 = clock64();
        const bool tgot = mbar_wait(bar_tempty + 8u * as, aph ^ 1u, abort_flag, kTcWaitLimitNs);
        if (prof) mt += clock64() - t0;
        if (!__all_sync(0xffffffffu, tgot)) {
          if (reporter) tc_report(p.status, TC_ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_base = tmem_base + as * acc_cols;
        const int kb0 = (t % p.k_split) * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
        bool first_kb = true;   // the first k-block of a tile (or K-run) overwrites the accumulators
        for (int kb = kb0; kb < kb1; kb += p.kps) {
          if (prof) t0 = clock64();
          const bool fgot = mbar_wait(bar_full + 8u * s, ph, abort_flag, kTcWaitLimitNs);
          if (prof) { t1 = clock64(); mw += t1 - t0; }
          if (!__all_sync(0xffffffffu, fgot)) {
            if (reporter) tc_report(p.status, TC_ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (kb == kb0 && acc_it == 0 && reporter) tc_mark(p.status, dbg, 4, 1);   // first stage landed
          // One divergent region per stage: the elected lane issues every MMA of the stage and the commit.
          // (A branch around each MMA costs the warp ~40 cycles per site whether or not it issues anything,
          // which is more than a 128 x 64 MMA takes to execute.)  Descriptors are sums of warp-uniform values.
          if (elected) {
            for (int kj = 0; kj < p.kps && kb + kj < kb1; ++kj) {   // the k-blocks of this stage that belong to the run
              const uint32_t k16 = s16 + kj * kblock16;
              if constexpr (PLANES == 1) {
                if (n_terms != 0) {
                  if (p.n_sub == 2) tc_issue_kblock<CG, TF32, kMaxTerms, 2, 1>(k16, first_kb, d_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
                  else tc_issue_kblock<CG, TF32, kMaxTerms, 1, 1>(k16, first_kb, d_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
                }
              } else {
                // two planes: one column block; four terms (complex) or three (dual)
                if (n_terms == 4) tc_issue_kblock<CG, TF32, kMaxTerms, 1, 4>(k16, first_kb, d_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
                else if (n_terms == 3) tc_issue_kblock<CG, TF32, kMaxTerms, 1, 3>(k16, first_kb, d_base, hi_a, hi_b, off_a, off_b, d_off, t_id, t_keep);
              }
              first_kb = false;
            }
            umma_commit<CG>(bar_empty + 8u * s);  // stage is free once these MMAs have read it
          }
          first_kb = false;
          if (kb == kb0 && acc_it == 0 && reporter) tc_mark(p.status, dbg, 4, 2);   // first MMAs issued
          ++s; s16 += stage16;
          if (s == p.stages) { s = 0; s16 = base16; ph ^= 1u; }
          if (prof) mi += clock64() - t1;
        }
        if (ok && elected) umma_commit<CG>(bar_tfull + 8u * as);  // accumulator complete
      }
      if (prof && reporter) {
        long long* o = p.dbg_out + blockIdx.x * 16;
        o[2] = mw; o[3] = mi; o[4] = mt; o[5] = clock64() - k_start;
        o[6] = static_cast<long long>(global_timer_ns() - g_start);
        o[11] = static_cast<long long>(g_start);          // absolute times: the launch's timeline
        o[12] = static_cast<long long>(global_timer_ns());
      }
      // Drain: nothing below may free TMEM or shared memory while an MMA is still running.
      // The commit must come from the thread that issued the MMAs.
      if (elected) {
        umma_commit_local<CG>(bar_drain);
        const uint64_t d0 = global_timer_ns();
        while (!mbar_try_wait(bar_drain, 0)) {
          if (global_timer_ns() - d0 > kTcWaitLimitNs) {
            tc_report(p.status, TC_ST_TIMEOUT_DRAIN);
            break;
          }
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int chunk_step = 32 * (tc_epilogue_warps(PLANES) / 4);
    const int chunk_first = 32 * ((warp - 4) >> 2);
    const uint32_t tempty_leader = (CG == 2) ? map_to_cta(bar_tempty, 0) : bar_tempty;
    uint32_t acc_it = 0;
    bool ok = true;
    const bool fast_store = PLANES == 1 && p.dtype_d == TC_F32 && p.beta == 0.0f &&
                            p.bias_axis != TC_BIAS_COL && p.act != TC_ACT_GELU;
    const bool fast_store16 = PLANES == 1 && p.dtype_d != TC_F32 && p.beta == 0.0f && p.bias_axis != TC_BIAS_COL &&
                              p.act != TC_ACT_GELU;
    const bool has_c = p.beta != 0.0f;
    // plain matrices only (a contraction's C is addressed through two-level strides), planar or real
    pdl_wait();             // D (and C) may still be in use by the previous kernel
    const bool prefetch_c = has_c && p.m_div >= p.M && p.n_div >= p.N && p.c_sm0 == 1 && (PLANES == 1 || p.c_plane != 0);
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++acc_it) {
      int tm, tn;
      const int bt = t / units_per_product;
      tc_tile_coords(p, (t - bt * units_per_product) / p.k_split, tm, tn);
      const int64_t split_off = static_cast<int64_t>(t % p.k_split) * p.split_stride;
      const int m = (tm * CG + static_cast<int>(rank)) * kTcTileM + q * 32 + lane;
      const int n0 = tn * bn_tile;
      const uint32_t as = two_acc ? (acc_it & 1u) : 0u;
      const uint32_t aph = (two_acc ? (acc_it >> 1) : acc_it) & 1u;
      if (prefetch_c) {
        // While the main loop of this tile runs, pull the tile's part of C into L2: one request per
        // 128-byte line (this warp's 32 rows of one column), columns dealt out to the lanes.
        const int m0 = m - lane;
        if (m0 < p.M) {
          const size_t es_c = p.dtype_c == TC_F32 ? 4 : 2;
          const char* c_line = static_cast<const char*>(p.C) + (static_cast<size_t>(m0) + static_cast<size_t>(bt) * p.c_batch) * es_c;
          for (int c = lane + chunk_first; c < bn_tile && n0 + c < p.N; c += chunk_step) {
#pragma unroll
            for (int pl = 0; pl < PLANES; ++pl)
              prefetch_l2(c_line + (static_cast<size_t>(pl) * p.c_plane + static_cast<size_t>(n0 + c) * p.c_sn0) * es_c);
          }
        }
      }
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * acc_cols;
      const bool m_ok = m < p.M;
      float bias_row = 0.0f;
      if (p.bias_axis == TC_BIAS_ROW && m_ok) bias_row = p.bias[m];
      const int m_in = m % p.m_div, m_out = m / p.m_div;
      const int64_t d_row = m_in * p.d_sm0 + m_out * p.d_sm1 + bt * p.d_batch + split_off;
      const int64_t c_row = m_in * p.c_sm0 + m_out * p.c_sm1 + bt * p.c_batch;
      // One pass over the accumulator stage - or, with the skewed schedule of 512-column tiles, one pass per
      // column block, each behind its own barrier (slot = block).
      long long e0 = 0, e1 = 0;
      for (int half = 0; half < (skew ? 2 : 1); ++half) {
      const uint32_t hb = skew ? static_cast<uint32_t>(half) : as;
      // all-or-nothing per warp: the TMEM loads below are warp-collective
      e0 = (dbg & 8) ? clock64() : 0;
      const bool got = mbar_wait(bar_tfull + 8u * hb, aph, abort_flag, kTcWaitLimitNs);
      e1 = (dbg & 8) ? clock64() : 0;
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) tc_report(p.status, TC_ST_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      if (acc_it == 0 && half == 0 && warp == 4 && lane == 0) tc_mark(p.status, dbg, 5, 1);   // first accumulator complete
      const int c_lo = chunk_first + (skew ? half * p.bn : 0), c_hi = skew ? (half + 1) * p.bn : bn_tile;
      for (int c = c_lo; c < c_hi; c += chunk_step) {
        uint32_t v[PLANES][32];
        // column c of the tile is column c % bn of block c / bn (bn is a multiple of 32)
        const uint32_t t_col = t_row + (c >= p.bn ? sub_cols + (c - p.bn) : c);
#pragma unroll
        for (int pl = 0; pl < PLANES; ++pl) tmem_ld_32x32(t_col + pl * p.bn, v[pl]);
        tmem_ld_wait();
        const int ncols = p.N - (n0 + c);  // columns of this chunk inside the matrix (may be <= 0)
        if (!m_ok || ncols <= 0) continue;
        const int n_in = (n0 + c) % p.n_div, n_out = (n0 + c) / p.n_div;  // a chunk never straddles n_div
        if (fast_store) {
          // FP32 output, no C, no per-column bias: one FMA (+ max) and one coalesced store per
          // column; a warp writes 32 consecutive rows = 128 bytes of a column of D.
          float* dp = static_cast<float*>(p.D) + d_row + n_in * p.d_sn0 + n_out * p.d_sn1;
          if (ncols >= 32) {
            if (p.act == TC_ACT_RELU) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                dp[j * p.d_sn0] = fmaxf(fmaf(p.alpha, __uint_as_float(v[0][j]), bias_row), 0.0f);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                dp[j * p.d_sn0] = fmaf(p.alpha, __uint_as_float(v[0][j]), bias_row);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < ncols) {
                const float x = fmaf(p.alpha, __uint_as_float(v[0][j]), bias_row);
                dp[j * p.d_sn0] = p.act == TC_ACT_RELU ? fmaxf(x, 0.0f) : x;
              }
            }
          }
        } else if (fast_store16 && ncols >= 32) {
          // 16-bit output, no C, no per-column bias: the same two instructions per element as above
          const int64_t di = d_row + n_in * p.d_sn0 + n_out * p.d_sn1;
          if (p.dtype_d == TC_F16) {
            __half* dp = static_cast<__half*>(p.D) + di;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = fmaf(p.alpha, __uint_as_float(v[0][j]), bias_row);
              if (p.act == TC_ACT_RELU) x = fmaxf(x, 0.0f);
              dp[j * p.d_sn0] = __float2half_rn(x);
            }
          } else {
            __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.D) + di;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = fmaf(p.alpha, __uint_as_float(v[0][j]), bias_row);
              if (p.act == TC_ACT_RELU) x = fmaxf(x, 0.0f);
              dp[j * p.d_sn0] = __float2bfloat16_rn(x);
            }
          }
        } else {
          const bool c_pairs = PLANES == 2 && p.c_plane == 0;
          const bool d_pairs = PLANES == 2 && p.d_plane == 0;
          int64_t ci = c_row + n_in * p.c_sn0 + n_out * p.c_sn1;  // element (m, n) of one plane
          int64_t di = d_row + n_in * p.d_sn0 + n_out * p.d_sn1;
          if (ncols >= 32 && (!has_c || p.dtype_c == p.dtype_d)) {
            // full chunk, C (if any) of D's type: the specialised, load-batched variants
            const int col0 = n0 + c;
            if (p.dtype_d == TC_F32) {
              if (has_c) tc_epilogue_chunk<PLANES, TC_F32, TC_F32>(p, v, ci, di, bias_row, col0);
              else tc_epilogue_chunk<PLANES, -1, TC_F32>(p, v, ci, di, bias_row, col0);
            } else if (p.dtype_d == TC_F16) {
              if (has_c) tc_epilogue_chunk<PLANES, TC_F16, TC_F16>(p, v, ci, di, bias_row, col0);
              else tc_epilogue_chunk<PLANES, -1, TC_F16>(p, v, ci, di, bias_row, col0);
            } else {
              if (has_c) tc_epilogue_chunk<PLANES, TC_BF16, TC_BF16>(p, v, ci, di, bias_row, col0);
              else tc_epilogue_chunk<PLANES, -1, TC_BF16>(p, v, ci, di, bias_row, col0);
            }
            continue;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j, ci += p.c_sn0, di += p.d_sn0) {
            if (j < ncols) {
              float bias = bias_row;
              if (p.bias_axis == TC_BIAS_COL) bias = p.bias[n0 + c + j];
              float out[PLANES];
#pragma unroll
              for (int pl = 0; pl < PLANES; ++pl) {
                float x = p.alpha * __uint_as_float(v[pl][j]);
                if (p.beta != 0.0f)
                  x += p.beta * tc_load_elem(p.C, c_pairs ? 2 * ci + pl : pl * p.c_plane + ci, p.dtype_c);
                if (pl == 0) x += bias;
                out[pl] = tc_activation(x, p.act);
              }
              if (d_pairs && p.dtype_d == TC_F32) {
                reinterpret_cast<float2*>(p.D)[di] = make_float2(out[0], out[PLANES - 1]);
              } else {
#pragma unroll
                for (int pl = 0; pl < PLANES; ++pl)
                  tc_store_elem(p.D, d_pairs ? 2 * di + pl : pl * p.d_plane + di, p.dtype_d, out[pl]);
              }
            }
          }
        }
      }
      // Accumulator stage (or column block) can be overwritten once every warp of the pair has read it.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 2) mbar_arrive_cluster(tempty_leader + 8u * hb);
        else mbar_arrive(bar_tempty + 8u * hb);
      }
      }
      if (!ok) break;
      if (acc_it == 0 && warp == 4 && lane == 0) tc_mark(p.status, dbg, 5, 2);   // first tile stored
      if ((dbg & 8) && warp == 4 && lane == 0) {
        p.dbg_out[blockIdx.x * 16 + 7] += e1 - e0;
        p.dbg_out[blockIdx.x * 16 + 8] += clock64() - e1;
        p.dbg_out[blockIdx.x * 16 + 15] = static_cast<long long>(global_timer_ns());   // last tile stored
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // the peer may still read this CTA's smem / barriers
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, p.tmem_cols);
  }
  if ((dbg & 8) && threadIdx.x == 0) {   // the launch's timeline: entry and exit of this CTA
    p.dbg_out[blockIdx.x * 16 + 13] = static_cast<long long>(t_entry);
    p.dbg_out[blockIdx.x * 16 + 14] = static_cast<long long>(global_timer_ns());
  }
}

}  // namespace gk
