// FP32 GEMM on the CUDA cores (FPUOperator): results that must not go through the tensor cores.
//
//   D = act( alpha * op(A) * op(B) + beta * C + bias ),  all FP32, FP32 FMA accumulation in K order.
//
// 128 x 128 x 16 CTA tile, 128 threads (two CTAs per SM), a 16 x 8 register tile per thread.  A warp
// owns 128 rows x 32 columns: eight lanes along M (four 4-row strips each, 32 rows apart) by four lanes
// along N (two 4-column strips, 16 columns apart).  Operands are staged in shared memory as As[k][m] /
// Bs[k][n], so a k-step is six 16-byte shared loads per 128 FMAs, and each load is one 128-byte (A) or
// 64-byte (B) wavefront that the other lanes receive by broadcast: shared-memory bandwidth (128 B per
// clock per SM against 128 FMA lanes) is what an 8 x 8 register tile runs out of first.
//
// Global -> shared memory in two hops.  The threads copy the next k-tiles as they lie in memory into a
// staging ring with cp.async (16-byte chunks, coalesced, kFpuStages tiles deep, no registers held across
// the compute loop).  During k-tile kt every thread moves its share of tile kt + 1 from the ring into
// the As/Bs buffer the FMAs read next - scaling A by alpha, widening 16-bit types, and transposing an
// operand whose contiguous index is K (a transposed A, an untransposed B): those rows are staged with
// their 16-byte chunks XOR-swizzled so that both the staging reads (32 consecutive rows per warp) and
// the transposing stores are free of bank conflicts.  Two As/Bs buffers, one barrier per k-tile; the
// tile after next must have landed before that barrier, the ring slot of the tile just consumed is
// refilled right after it.
//
// A and B may be Float16 or BFloat16 (the FPU operator's Float16 -> Float32 configuration): they are
// widened to Float32 as they are loaded, the arithmetic is the same FP32 FMA chain.
//
// Takes tile-multiple sizes and 16-byte aligned rows only (the reference's UnsafeAligned* layouts,
// src/layout.jl:192-270); everything else goes to the generic kernel in simt_gemm.cuh.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gk {

constexpr int kFpuBM = 128, kFpuBN = 128, kFpuBK = 16, kFpuThreads = 128, kFpuPad = 4;
constexpr int kFpuStages = 4;                                   // k-tiles in flight in the staging ring
constexpr int kFpuTileBytes = 2 * kFpuBK * (kFpuBM + kFpuPad) * 4;   // one operand's two As/Bs buffers
constexpr int kFpuStageBytes = kFpuBM * kFpuBK * 4;             // one operand tile in the ring (Float32 size)
constexpr int kFpuSmemBytes = 2 * kFpuTileBytes + 2 * kFpuStages * kFpuStageBytes;
static_assert(kFpuThreads == kFpuBM && kFpuBM == kFpuBN, "a thread moves one staged row of a K-contiguous operand");

struct FpuParams {
  const void* A;   // Float32, or Float16 / BFloat16 widened to Float32 on the way into shared memory
  const void* B;
  const float* C;
  float* D;
  int M, N, K;
  int64_t lda, ldb, ldc, ldd;
  float alpha, beta;
  const float* bias;
  int bias_axis;  // 0 none, 1 per row, 2 per column
  int act;        // 0 none, 1 relu, 2 gelu
  int tiles_m, tiles_n;
  int raster_group;
  // Tail split.  CTAs start in block order, two per SM, so the tiles of the last, partly filled round are
  // the highest-numbered ones.  When that round would fill at most half of the slots, each of its tiles
  // (those from split_first on) is cut along K into split_q parts that run side by side: block
  // split_first + u handles part u % split_q of tile split_first + u / split_q and writes its raw
  // partial sums to ws (one 128 x 128 FP32 tile per part); fpu_tail_reduce_kernel adds the parts and
  // applies the epilogue.  split_q == 1: no split.
  int split_first, split_q, kt_per_part;
  float* ws;
};

// One operand tile is 128 (M or N index x) by 16 (k) elements = 128 * kChunks 16-byte chunks of E =
// 16 / sizeof(T) elements; every thread copies, and later moves, kChunks of them.
//   MN-contiguous (element (x, k) at base[x + k*ld]): chunk c = (k, x / E) in memory order, staged at 16 * c;
//     thread t copies and moves chunks t + 128 * i.
//   K-contiguous  (element (x, k) at base[k + x*ld]): a row x is R = 16 / E chunks; chunk (x, kc) is staged at
//     16 * (x * R + (kc ^ swz(x))), swz(x) = (x / (8 / R)) % R.  Thread t copies chunks (x, kc) = ((t + 128 * i) / R,
//     (t + 128 * i) % R) - neighbouring lanes read neighbouring memory - and moves chunks (x, kc) = (t, i): the
//     lanes of a warp then take 32 consecutive rows, so the transposing stores into As[k][x] hit 32 different
//     banks, and the swizzle spreads their 16-byte staging reads over all banks too.
template <typename T> struct FpuChunk {
  static constexpr int E = 16 / static_cast<int>(sizeof(T));
  static constexpr int kChunks = kFpuBM * kFpuBK / E / kFpuThreads;
  static constexpr int R = kFpuBK / E;   // chunks per K-contiguous row (== kChunks)
};

__device__ __forceinline__ void fpu_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void fpu_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void fpu_cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T> __device__ __forceinline__ int fpu_kmajor_offset(int x, int kc) {
  constexpr int R = FpuChunk<T>::R;
  return 16 * (x * R + (kc ^ ((x / (8 / R)) % R)));
}

// Start the copies of this thread's chunks of k-tile k0 into ring slot `slot` (a shared-memory address).
template <bool KMAJOR, typename T>
__device__ __forceinline__ void fpu_issue_tile(uint32_t slot, const T* __restrict__ base, int64_t ld, int x0, int k0) {
  constexpr int E = FpuChunk<T>::E;
#pragma unroll
  for (int i = 0; i < FpuChunk<T>::kChunks; ++i) {
    const int c = threadIdx.x + i * kFpuThreads;
    if constexpr (KMAJOR) {
      const int x = c / FpuChunk<T>::R, kc = c % FpuChunk<T>::R;
      fpu_cp_async16(slot + fpu_kmajor_offset<T>(x, kc), base + static_cast<int64_t>(x0 + x) * ld + k0 + kc * E);
    } else {
      fpu_cp_async16(slot + 16u * c, base + static_cast<int64_t>(k0 + c / (kFpuBM / E)) * ld + x0 + (c % (kFpuBM / E)) * E);
    }
  }
}

__device__ __forceinline__ void fpu_widen(const uint4& raw, float (&v)[4], const float*) {
  v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y); v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
}
__device__ __forceinline__ void fpu_widen(const uint4& raw, float (&v)[8], const __half*) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
    v[2 * q] = f.x; v[2 * q + 1] = f.y;
  }
}
__device__ __forceinline__ void fpu_widen(const uint4& raw, float (&v)[8], const __nv_bfloat16*) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[q]));
    v[2 * q] = f.x; v[2 * q + 1] = f.y;
  }
}

// Move this thread's share of a landed tile from ring slot `slot` into s[k][x], scaled.
template <bool KMAJOR, typename T>
__device__ __forceinline__ void fpu_move_tile(float (*s)[kFpuBM + kFpuPad], const uint8_t* slot, float scale) {
  constexpr int E = FpuChunk<T>::E;
#pragma unroll
  for (int i = 0; i < FpuChunk<T>::kChunks; ++i) {
    float v[E];
    if constexpr (KMAJOR) {
      const int x = threadIdx.x;
      fpu_widen(*reinterpret_cast<const uint4*>(slot + fpu_kmajor_offset<T>(x, i)), v, static_cast<const T*>(nullptr));
#pragma unroll
      for (int e = 0; e < E; ++e) s[i * E + e][x] = v[e] * scale;
    } else {
      const int c = threadIdx.x + i * kFpuThreads;
      fpu_widen(*reinterpret_cast<const uint4*>(slot + 16 * c), v, static_cast<const T*>(nullptr));
      const int k = c / (kFpuBM / E), x = (c % (kFpuBM / E)) * E;
#pragma unroll
      for (int h = 0; h < E / 4; ++h)
        *reinterpret_cast<float4*>(&s[k][x + 4 * h]) =
            make_float4(v[4 * h] * scale, v[4 * h + 1] * scale, v[4 * h + 2] * scale, v[4 * h + 3] * scale);
    }
  }
}

__device__ __forceinline__ float fpu_act(float v, int act) {
  if (act == 1) return fmaxf(v, 0.0f);
  if (act == 2) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
  return v;
}

template <bool A_KMAJOR, bool B_KMAJOR, typename TIn>
__global__ void __launch_bounds__(kFpuThreads, 2) fpu_gemm_kernel(const FpuParams p) {
  const TIn* gA = static_cast<const TIn*>(p.A);
  const TIn* gB = static_cast<const TIn*>(p.B);
  extern __shared__ __align__(16) uint8_t fpu_smem[];
  float (*As)[kFpuBK][kFpuBM + kFpuPad] = reinterpret_cast<float (*)[kFpuBK][kFpuBM + kFpuPad]>(fpu_smem);
  float (*Bs)[kFpuBK][kFpuBN + kFpuPad] = reinterpret_cast<float (*)[kFpuBK][kFpuBN + kFpuPad]>(fpu_smem + kFpuTileBytes);
  const uint8_t* ring_a = fpu_smem + 2 * kFpuTileBytes;                    // kFpuStages slots of A, then of B
  const uint8_t* ring_b = ring_a + kFpuStages * kFpuStageBytes;
  const uint32_t ring_a32 = static_cast<uint32_t>(__cvta_generic_to_shared(ring_a));
  const uint32_t ring_b32 = static_cast<uint32_t>(__cvta_generic_to_shared(ring_b));

  // which tile, and which part of its K range
  int t = blockIdx.x, part = 0;
  const bool split = p.split_q > 1 && t >= p.split_first;
  if (split) {
    const int u = t - p.split_first;
    t = p.split_first + u / p.split_q;
    part = u % p.split_q;
  }
  // tile raster: bands of `raster_group` tiles down M, then along N (same walk as the tcgen05 path)
  int tm, tn;
  {
    const int g = p.raster_group;
    const int band = g * p.tiles_n, band_id = t / band, first_m = band_id * g;
    const int rows = min(g, p.tiles_m - first_m), r = t - band_id * band;
    tm = first_m + r % rows;
    tn = r / rows;
  }
  const int m0 = tm * kFpuBM, n0 = tn * kFpuBN;
  const int lane = threadIdx.x & 31;
  const int ma = (lane & 7) * 4;                              // first row of this thread's strips (+ 32 per strip)
  const int nb = (threadIdx.x >> 5) * 32 + (lane >> 3) * 4;   // first column of its strips (+ 16 for the second)

  // Accumulators are kept as pairs of consecutive rows: Blackwell's packed FP32 FMA (fma.rn.f32x2)
  // does two IEEE fused multiply-adds per issued instruction, which halves the issue slots the
  // 128 FMAs per k-step need.  acc[2*s + h][j]: rows ma + 32*s + 2*h + {0, 1}, column j of the strips.
  float2 acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = make_float2(0.0f, 0.0f);

  const int kt_all = p.K / kFpuBK;
  const int kt_first = split ? part * p.kt_per_part : 0;
  const int kt_count = split ? min(kt_all, kt_first + p.kt_per_part) : kt_all;   // one past the last k-tile
  // Ring slot of k-tile kt: (kt - kt_first) % kFpuStages.  One commit group per tile, empty past the end, so
  // "all but the newest kFpuStages - 2 groups have landed" always names the tile after next.
#pragma unroll
  for (int j = 0; j < kFpuStages; ++j) {
    if (kt_first + j < kt_count) {
      fpu_issue_tile<A_KMAJOR>(ring_a32 + j * kFpuStageBytes, gA, p.lda, m0, (kt_first + j) * kFpuBK);
      fpu_issue_tile<B_KMAJOR>(ring_b32 + j * kFpuStageBytes, gB, p.ldb, n0, (kt_first + j) * kFpuBK);
    }
    fpu_cp_commit();
  }
  fpu_cp_wait<kFpuStages - 2>();   // this thread's copies of the first two tiles
  __syncthreads();                 // ... and everybody else's
  // alpha scales A on its way in, as the reference's shared_to_regs_a transform does
  fpu_move_tile<A_KMAJOR, TIn>(As[0], ring_a, p.alpha);
  fpu_move_tile<B_KMAJOR, TIn>(Bs[0], ring_b, 1.0f);
  __syncthreads();

  int slot = 0;   // ring slot of k-tile kt
  for (int kt = kt_first; kt < kt_count; ++kt) {
    const int cur = (kt - kt_first) & 1;
    // The slot of tile kt was emptied during the previous k-tile (before its barrier): refill it.
    if (kt + kFpuStages < kt_count) {
      fpu_issue_tile<A_KMAJOR>(ring_a32 + slot * kFpuStageBytes, gA, p.lda, m0, (kt + kFpuStages) * kFpuBK);
      fpu_issue_tile<B_KMAJOR>(ring_b32 + slot * kFpuStageBytes, gB, p.ldb, n0, (kt + kFpuStages) * kFpuBK);
    }
    fpu_cp_commit();
    slot = slot + 1 == kFpuStages ? 0 : slot + 1;
    if (kt + 1 < kt_count) {
      // Tile kt + 1 landed before the last barrier; buffer cur ^ 1 was last read before it too.  Plain loads
      // and stores: the compiler spreads them among the FMAs below.
      fpu_move_tile<A_KMAJOR, TIn>(As[cur ^ 1], ring_a + slot * kFpuStageBytes, p.alpha);
      fpu_move_tile<B_KMAJOR, TIn>(Bs[cur ^ 1], ring_b + slot * kFpuStageBytes, 1.0f);
    }
    // Fragments of k-step k + 1 are loaded before the FMAs of k-step k are issued.
    float4 fa[2][4], fb[2][2];
#pragma unroll
    for (int sm = 0; sm < 4; ++sm) fa[0][sm] = *reinterpret_cast<const float4*>(&As[cur][0][ma + 32 * sm]);
    fb[0][0] = *reinterpret_cast<const float4*>(&Bs[cur][0][nb]);
    fb[0][1] = *reinterpret_cast<const float4*>(&Bs[cur][0][nb + 16]);
#pragma unroll
    for (int k = 0; k < kFpuBK; ++k) {
      const int f = k & 1;
      if (k + 1 < kFpuBK) {
#pragma unroll
        for (int sm = 0; sm < 4; ++sm) fa[f ^ 1][sm] = *reinterpret_cast<const float4*>(&As[cur][k + 1][ma + 32 * sm]);
        fb[f ^ 1][0] = *reinterpret_cast<const float4*>(&Bs[cur][k + 1][nb]);
        fb[f ^ 1][1] = *reinterpret_cast<const float4*>(&Bs[cur][k + 1][nb + 16]);
      }
      float2 a[8];
#pragma unroll
      for (int sm = 0; sm < 4; ++sm) {
        a[2 * sm] = make_float2(fa[f][sm].x, fa[f][sm].y);
        a[2 * sm + 1] = make_float2(fa[f][sm].z, fa[f][sm].w);
      }
      const float b[8] = {fb[f][0].x, fb[f][0].y, fb[f][0].z, fb[f][0].w, fb[f][1].x, fb[f][1].y, fb[f][1].z, fb[f][1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 bb = make_float2(b[j], b[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i][j] = __ffma2_rn(a[i], bb, acc[i][j]);
      }
    }
    fpu_cp_wait<kFpuStages - 2>();   // tile kt + 2 is needed from the next k-tile's start
    __syncthreads();
  }

  // epilogue: each thread owns rows m0 + ma + 32*s + {0..3} and columns n0 + nb + 16*(j / 4) + j % 4
  if (split) {
    // raw partial sums (alpha is in them already: it scaled A on its way into shared memory)
    float* w = p.ws + (static_cast<size_t>(t - p.split_first) * p.split_q + part) * (kFpuBM * kFpuBN);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nl = nb + (j >> 2) * 16 + (j & 3);
#pragma unroll
      for (int sm = 0; sm < 4; ++sm) {
        const int ml = ma + 32 * sm;
        *reinterpret_cast<float4*>(w + ml + nl * kFpuBM) =
            make_float4(acc[sm * 2][j].x, acc[sm * 2][j].y, acc[sm * 2 + 1][j].x, acc[sm * 2 + 1][j].y);
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = n0 + nb + (j >> 2) * 16 + (j & 3);
    const float bias_n = p.bias_axis == 2 ? __ldg(p.bias + n) : 0.0f;
#pragma unroll
    for (int sm = 0; sm < 4; ++sm) {
      const int m = m0 + ma + 32 * sm;
      float4 v = make_float4(acc[sm * 2][j].x, acc[sm * 2][j].y, acc[sm * 2 + 1][j].x, acc[sm * 2 + 1][j].y);
      if (p.beta != 0.0f) {
        const float4 c = *reinterpret_cast<const float4*>(p.C + m + static_cast<int64_t>(n) * p.ldc);
        v.x = fmaf(p.beta, c.x, v.x); v.y = fmaf(p.beta, c.y, v.y);
        v.z = fmaf(p.beta, c.z, v.z); v.w = fmaf(p.beta, c.w, v.w);
      }
      if (p.bias_axis == 1) {
        const float4 bm = __ldg(reinterpret_cast<const float4*>(p.bias + m));
        v.x += bm.x; v.y += bm.y; v.z += bm.z; v.w += bm.w;
      } else {
        v.x += bias_n; v.y += bias_n; v.z += bias_n; v.w += bias_n;
      }
      v.x = fpu_act(v.x, p.act); v.y = fpu_act(v.y, p.act);
      v.z = fpu_act(v.z, p.act); v.w = fpu_act(v.w, p.act);
      *reinterpret_cast<float4*>(p.D + m + static_cast<int64_t>(n) * p.ldd) = v;
    }
  }
}

// Second pass of the tail split: one block per split tile adds its parts and applies the epilogue.
__global__ void __launch_bounds__(256) fpu_tail_reduce_kernel(const FpuParams p) {
  const int t = p.split_first + blockIdx.x;
  int tm, tn;
  {
    const int g = p.raster_group;
    const int band = g * p.tiles_n, band_id = t / band, first_m = band_id * g;
    const int rows = min(g, p.tiles_m - first_m), r = t - band_id * band;
    tm = first_m + r % rows;
    tn = r / rows;
  }
  const int m0 = tm * kFpuBM, n0 = tn * kFpuBN;
  const float* w = p.ws + static_cast<size_t>(blockIdx.x) * p.split_q * (kFpuBM * kFpuBN);
  for (int e = threadIdx.x; e < kFpuBM * kFpuBN / 4; e += blockDim.x) {
    const int ml = (e % (kFpuBM / 4)) * 4, nl = e / (kFpuBM / 4);
    float4 v = *reinterpret_cast<const float4*>(w + ml + nl * kFpuBM);
    for (int q = 1; q < p.split_q; ++q) {
      const float4 u = *reinterpret_cast<const float4*>(w + static_cast<size_t>(q) * (kFpuBM * kFpuBN) + ml + nl * kFpuBM);
      v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
    }
    const int m = m0 + ml, n = n0 + nl;
    if (p.beta != 0.0f) {
      const float4 c = *reinterpret_cast<const float4*>(p.C + m + static_cast<int64_t>(n) * p.ldc);
      v.x = fmaf(p.beta, c.x, v.x); v.y = fmaf(p.beta, c.y, v.y); v.z = fmaf(p.beta, c.z, v.z); v.w = fmaf(p.beta, c.w, v.w);
    }
    if (p.bias_axis == 1) {
      const float4 bm = __ldg(reinterpret_cast<const float4*>(p.bias + m));
      v.x += bm.x; v.y += bm.y; v.z += bm.z; v.w += bm.w;
    } else if (p.bias_axis == 2) {
      const float bn = __ldg(p.bias + n);
      v.x += bn; v.y += bn; v.z += bn; v.w += bn;
    }
    v.x = fpu_act(v.x, p.act); v.y = fpu_act(v.y, p.act); v.z = fpu_act(v.z, p.act); v.w = fpu_act(v.w, p.act);
    *reinterpret_cast<float4*>(p.D + m + static_cast<int64_t>(n) * p.ldd) = v;
  }
}

}  // namespace gk
