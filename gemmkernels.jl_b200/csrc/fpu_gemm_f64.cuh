// FP64 GEMM on the CUDA cores (FPUOperator with Float64, configs/configs.jl:496-518 of the reference).
//
//   D = act( alpha * op(A) * op(B) + beta * C + bias ),  all FP64, FMA accumulation in K order.
//
// The FP32 kernel's design (fpu_gemm.cuh) with the element twice as wide: 128 x 128 x 16 CTA tile, 256
// threads (one CTA per SM), an 8 x 8 register tile per thread.  A warp owns 64 rows x 32 columns: eight
// lanes along M (four 2-row strips each, 16 rows apart) by four lanes along N (four 2-column strips, 8
// columns apart), so every 16-byte shared load is one 128-byte (A) or 64-byte (B) wavefront that the other
// lanes receive by broadcast.  Operands reach shared memory in two hops: a cp.async staging ring (16-byte
// chunks, coalesced, kF64Stages k-tiles deep) and, during k-tile kt, a move of tile kt + 1 into the As/Bs
// buffer the FMAs read next, which scales A by alpha and transposes an operand whose contiguous index is
// K (rows staged with their chunks XOR-swizzled: conflict-free staging reads and transposing stores).
//
// Takes tile-multiple sizes and 16-byte aligned columns only; everything else goes to the generic kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fpu_gemm.cuh"   // cp.async helpers, fpu_act

namespace gk {

constexpr int kF64BM = 128, kF64BN = 128, kF64BK = 16, kF64Threads = 256, kF64Pad = 2;
constexpr int kF64Stages = 3;                                            // k-tiles in flight in the staging ring
constexpr int kF64TileBytes = 2 * kF64BK * (kF64BM + kF64Pad) * 8;       // one operand's two As/Bs buffers
constexpr int kF64StageBytes = kF64BM * kF64BK * 8;                      // one operand tile in the ring
constexpr int kF64SmemBytes = 2 * kF64TileBytes + 2 * kF64Stages * kF64StageBytes;
constexpr int kF64Chunks = kF64BM * kF64BK / 2 / kF64Threads;            // 16-byte chunks per thread per operand tile (4)
constexpr int kF64RowChunks = kF64BK / 2;                                // chunks per K-contiguous row (8)
static_assert(kF64BM == kF64BN && kF64Threads == 2 * kF64BM, "two threads move one staged row of a K-contiguous operand");

struct F64Params {
  const double* A;
  const double* B;
  const double* C;
  double* D;
  int M, N, K;
  int64_t lda, ldb, ldc, ldd;
  double alpha, beta;
  const float* bias;
  int bias_axis;  // 0 none, 1 per row, 2 per column
  int act;        // 0 none, 1 relu, 2 gelu
  int tiles_m, tiles_n;
  int raster_group;
};

__device__ __forceinline__ double f64_act(double v, int act) {
  if (act == 1) return v > 0.0 ? v : 0.0;
  if (act == 2) return 0.5 * v * (1.0 + erf(v * 0.70710678118654752));
  return v;
}

// Chunk (x, kc) of a K-contiguous tile (row x, doubles 2*kc and 2*kc + 1) is staged at this byte offset.
__device__ __forceinline__ int f64_kmajor_offset(int x, int kc) { return 16 * (x * kF64RowChunks + (kc ^ (x & 7))); }

// Start the copies of this thread's chunks of k-tile k0 into ring slot `slot` (a shared-memory address).
//   MN-contiguous (element (x, k) at base[x + k*ld]): chunk c = (k, x / 2) in memory order, staged at 16 * c
//   K-contiguous  (element (x, k) at base[k + x*ld]): chunk c = (x, kc) = (c / 8, c % 8), staged swizzled
template <bool KMAJOR>
__device__ __forceinline__ void f64_issue_tile(uint32_t slot, const double* __restrict__ base, int64_t ld, int x0, int k0) {
#pragma unroll
  for (int i = 0; i < kF64Chunks; ++i) {
    const int c = threadIdx.x + i * kF64Threads;
    if constexpr (KMAJOR) {
      const int x = c / kF64RowChunks, kc = c % kF64RowChunks;
      fpu_cp_async16(slot + f64_kmajor_offset(x, kc), base + static_cast<int64_t>(x0 + x) * ld + k0 + kc * 2);
    } else {
      fpu_cp_async16(slot + 16u * c, base + static_cast<int64_t>(k0 + c / (kF64BM / 2)) * ld + x0 + (c % (kF64BM / 2)) * 2);
    }
  }
}

// Move this thread's share of a landed tile from ring slot `slot` into s[k][x], scaled.  K-contiguous:
// thread t takes row t % 128 and the chunks (t / 128) * 4 .. + 3 of it, so a warp's transposing stores go
// to 32 consecutive x of one k.
template <bool KMAJOR>
__device__ __forceinline__ void f64_move_tile(double (*s)[kF64BM + kF64Pad], const uint8_t* slot, double scale) {
#pragma unroll
  for (int i = 0; i < kF64Chunks; ++i) {
    if constexpr (KMAJOR) {
      const int x = threadIdx.x & (kF64BM - 1), kc = (threadIdx.x >> 7) * kF64Chunks + i;
      const double2 v = *reinterpret_cast<const double2*>(slot + f64_kmajor_offset(x, kc));
      s[2 * kc][x] = v.x * scale;
      s[2 * kc + 1][x] = v.y * scale;
    } else {
      const int c = threadIdx.x + i * kF64Threads;
      const double2 v = *reinterpret_cast<const double2*>(slot + 16 * c);
      *reinterpret_cast<double2*>(&s[c / (kF64BM / 2)][(c % (kF64BM / 2)) * 2]) = make_double2(v.x * scale, v.y * scale);
    }
  }
}

template <bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(kF64Threads, 1) fpu_gemm_f64_kernel(const F64Params p) {
  extern __shared__ __align__(16) uint8_t f64_smem[];
  double (*As)[kF64BK][kF64BM + kF64Pad] = reinterpret_cast<double (*)[kF64BK][kF64BM + kF64Pad]>(f64_smem);
  double (*Bs)[kF64BK][kF64BN + kF64Pad] = reinterpret_cast<double (*)[kF64BK][kF64BN + kF64Pad]>(f64_smem + kF64TileBytes);
  const uint8_t* ring_a = f64_smem + 2 * kF64TileBytes;                    // kF64Stages slots of A, then of B
  const uint8_t* ring_b = ring_a + kF64Stages * kF64StageBytes;
  const uint32_t ring_a32 = static_cast<uint32_t>(__cvta_generic_to_shared(ring_a));
  const uint32_t ring_b32 = static_cast<uint32_t>(__cvta_generic_to_shared(ring_b));

  // tile raster: bands of `raster_group` tiles down M, then along N (same walk as the other kernels)
  int tm, tn;
  {
    const int t = blockIdx.x, g = p.raster_group;
    const int band = g * p.tiles_n, band_id = t / band, first_m = band_id * g;
    const int rows = min(g, p.tiles_m - first_m), r = t - band_id * band;
    tm = first_m + r % rows;
    tn = r / rows;
  }
  const int m0 = tm * kF64BM, n0 = tn * kF64BN;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ma = (warp & 1) * 64 + (lane & 7) * 2;     // first row of this thread's strips (+ 16 per strip)
  const int nb = (warp >> 1) * 32 + (lane >> 3) * 2;   // first column of its strips (+ 8 per strip)

  // acc[2*s + e][j]: row ma + 16*s + e, column nb + 8*(j / 2) + j % 2
  double acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0;

  const int kt_count = p.K / kF64BK;
  // Ring slot of k-tile kt: kt % kF64Stages.  One commit group per tile, empty past the end, so "all but the
  // newest kF64Stages - 2 groups have landed" always names the tile after next.
#pragma unroll
  for (int j = 0; j < kF64Stages; ++j) {
    if (j < kt_count) {
      f64_issue_tile<A_KMAJOR>(ring_a32 + j * kF64StageBytes, p.A, p.lda, m0, j * kF64BK);
      f64_issue_tile<B_KMAJOR>(ring_b32 + j * kF64StageBytes, p.B, p.ldb, n0, j * kF64BK);
    }
    fpu_cp_commit();
  }
  fpu_cp_wait<kF64Stages - 2>();   // this thread's copies of the first two tiles
  __syncthreads();                 // ... and everybody else's
  // alpha scales A on its way in, as the reference's shared_to_regs_a transform does
  f64_move_tile<A_KMAJOR>(As[0], ring_a, p.alpha);
  f64_move_tile<B_KMAJOR>(Bs[0], ring_b, 1.0);
  __syncthreads();

  int slot = 0;   // ring slot of k-tile kt
  for (int kt = 0; kt < kt_count; ++kt) {
    const int cur = kt & 1;
    // The slot of tile kt was emptied during the previous k-tile (before its barrier): refill it.
    if (kt + kF64Stages < kt_count) {
      f64_issue_tile<A_KMAJOR>(ring_a32 + slot * kF64StageBytes, p.A, p.lda, m0, (kt + kF64Stages) * kF64BK);
      f64_issue_tile<B_KMAJOR>(ring_b32 + slot * kF64StageBytes, p.B, p.ldb, n0, (kt + kF64Stages) * kF64BK);
    }
    fpu_cp_commit();
    slot = slot + 1 == kF64Stages ? 0 : slot + 1;
    if (kt + 1 < kt_count) {
      // Tile kt + 1 landed before the last barrier; buffer cur ^ 1 was last read before it too.
      f64_move_tile<A_KMAJOR>(As[cur ^ 1], ring_a + slot * kF64StageBytes, p.alpha);
      f64_move_tile<B_KMAJOR>(Bs[cur ^ 1], ring_b + slot * kF64StageBytes, 1.0);
    }
#pragma unroll
    for (int k = 0; k < kF64BK; ++k) {
      double a[8], b[8];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const double2 va = *reinterpret_cast<const double2*>(&As[cur][k][ma + 16 * s]);
        const double2 vb = *reinterpret_cast<const double2*>(&Bs[cur][k][nb + 8 * s]);
        a[2 * s] = va.x; a[2 * s + 1] = va.y;
        b[2 * s] = vb.x; b[2 * s + 1] = vb.y;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    fpu_cp_wait<kF64Stages - 2>();   // tile kt + 2 is needed from the next k-tile's start
    __syncthreads();
  }

  // epilogue: 16-byte stores of two consecutive rows
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = n0 + nb + 8 * (j >> 1) + (j & 1);
    const double bias_n = p.bias_axis == 2 ? static_cast<double>(__ldg(p.bias + n)) : 0.0;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int m = m0 + ma + 16 * s;
      double2 v = make_double2(acc[2 * s][j], acc[2 * s + 1][j]);
      if (p.beta != 0.0) {
        const double2 c = *reinterpret_cast<const double2*>(p.C + m + static_cast<int64_t>(n) * p.ldc);
        v.x = fma(p.beta, c.x, v.x); v.y = fma(p.beta, c.y, v.y);
      }
      if (p.bias_axis == 1) {
        v.x += static_cast<double>(__ldg(p.bias + m)); v.y += static_cast<double>(__ldg(p.bias + m + 1));
      } else {
        v.x += bias_n; v.y += bias_n;
      }
      v.x = f64_act(v.x, p.act); v.y = f64_act(v.y, p.act);
      *reinterpret_cast<double2*>(p.D + m + static_cast<int64_t>(n) * p.ldd) = v;
    }
  }
}

}  // namespace gk
