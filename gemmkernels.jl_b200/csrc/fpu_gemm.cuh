// FP32 GEMM on the CUDA cores (FPUOperator): results that must not go through the tensor cores.
//
//   D = act( alpha * op(A) * op(B) + beta * C + bias ),  all FP32, FP32 FMA accumulation in K order.
//
// 128 x 128 x 16 CTA tile, 256 threads, an 8 x 8 register tile per thread (two 4-wide strips along
// M and along N), operands staged in shared memory as As[k][m] / Bs[k][n] so the inner loop is four
// 16-byte shared loads per 64 FMAs.  Global loads are 16-byte vectors prefetched into registers one
// k-tile ahead; an operand whose contiguous index is K (a transposed A, an untransposed B) is
// transposed on its way into shared memory.  Two shared-memory buffers, one barrier per k-tile.
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

constexpr int kFpuBM = 128, kFpuBN = 128, kFpuBK = 16, kFpuThreads = 256, kFpuPad = 4;

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

// Global -> registers for one operand tile: 2 float4 per thread.
//   MN-contiguous: element (x, k) at base[x + k*ld]  (x = m or n): rows of 128 floats per k
//   K-contiguous : element (x, k) at base[k + x*ld]               : rows of 16 floats per x
// Four consecutive elements as Float32.
__device__ __forceinline__ float4 fpu_load4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 fpu_load4(const __half* p) {
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 fpu_load4(const __nv_bfloat16* p) {
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <bool KMAJOR, typename TIn>
__device__ __forceinline__ void fpu_load_tile(const TIn* __restrict__ base, int64_t ld, int x0, int k0,
                                              float4 (&r)[2]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = threadIdx.x + i * kFpuThreads;
    if constexpr (KMAJOR) {
      const int x = idx >> 2, k4 = idx & 3;
      r[i] = fpu_load4(base + static_cast<int64_t>(x0 + x) * ld + k0 + k4 * 4);
    } else {
      const int k = idx >> 5, x4 = idx & 31;
      r[i] = fpu_load4(base + static_cast<int64_t>(k0 + k) * ld + x0 + x4 * 4);
    }
  }
}

template <bool KMAJOR>
__device__ __forceinline__ void fpu_store_tile(float (*s)[kFpuBM + kFpuPad], const float4 (&r)[2], float scale) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = threadIdx.x + i * kFpuThreads;
    float4 v = r[i];
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    if constexpr (KMAJOR) {
      const int x = idx >> 2, k4 = idx & 3;
      s[k4 * 4 + 0][x] = v.x; s[k4 * 4 + 1][x] = v.y; s[k4 * 4 + 2][x] = v.z; s[k4 * 4 + 3][x] = v.w;
    } else {
      const int k = idx >> 5, x4 = idx & 31;
      *reinterpret_cast<float4*>(&s[k][x4 * 4]) = v;
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
  __shared__ __align__(16) float As[2][kFpuBK][kFpuBM + kFpuPad];
  __shared__ __align__(16) float Bs[2][kFpuBK][kFpuBN + kFpuPad];

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
  const int tx = threadIdx.x & 15;  // strip along M
  const int ty = threadIdx.x >> 4;  // strip along N

  // Accumulators are kept as pairs of consecutive rows: Blackwell's packed FP32 FMA (fma.rn.f32x2)
  // does two IEEE fused multiply-adds per issued instruction, which halves the issue slots the
  // 64 FMAs per k-step need and leaves room for the shared-memory loads.
  float2 acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = make_float2(0.0f, 0.0f);

  float4 ra[2], rb[2];
  const int kt_all = p.K / kFpuBK;
  const int kt_first = split ? part * p.kt_per_part : 0;
  const int kt_count = split ? min(kt_all, kt_first + p.kt_per_part) : kt_all;   // one past the last k-tile
  fpu_load_tile<A_KMAJOR>(gA, p.lda, m0, kt_first * kFpuBK, ra);
  fpu_load_tile<B_KMAJOR>(gB, p.ldb, n0, kt_first * kFpuBK, rb);
  // alpha scales A on its way in, as the reference's shared_to_regs_a transform does
  fpu_store_tile<A_KMAJOR>(As[0], ra, p.alpha);
  fpu_store_tile<B_KMAJOR>(Bs[0], rb, 1.0f);
  __syncthreads();

  for (int kt = kt_first; kt < kt_count; ++kt) {
    const int cur = (kt - kt_first) & 1;
    const bool more = kt + 1 < kt_count;
    if (more) {
      fpu_load_tile<A_KMAJOR>(gA, p.lda, m0, (kt + 1) * kFpuBK, ra);
      fpu_load_tile<B_KMAJOR>(gB, p.ldb, n0, (kt + 1) * kFpuBK, rb);
    }
#pragma unroll
    for (int k = 0; k < kFpuBK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][tx * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + tx * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][ty * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + ty * 4]);
      const float2 a[4] = {make_float2(a0.x, a0.y), make_float2(a0.z, a0.w), make_float2(a1.x, a1.y),
                           make_float2(a1.z, a1.w)};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 bb = make_float2(b[j], b[j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][j] = __ffma2_rn(a[i], bb, acc[i][j]);
      }
    }
    if (more) {
      fpu_store_tile<A_KMAJOR>(As[cur ^ 1], ra, p.alpha);
      fpu_store_tile<B_KMAJOR>(Bs[cur ^ 1], rb, 1.0f);
    }
    __syncthreads();
  }

  // epilogue: each thread owns rows m0 + {tx*4..+3, 64 + tx*4..+3} and columns n0 + {ty*4..+3, 64 + ..}
  if (split) {
    // raw partial sums (alpha is in them already: it scaled A on its way into shared memory)
    float* w = p.ws + (static_cast<size_t>(t - p.split_first) * p.split_q + part) * (kFpuBM * kFpuBN);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nl = (j >> 2) * 64 + ty * 4 + (j & 3);
#pragma unroll
      for (int ih = 0; ih < 2; ++ih) {
        const int ml = ih * 64 + tx * 4;
        *reinterpret_cast<float4*>(w + ml + nl * kFpuBM) =
            make_float4(acc[ih * 2][j].x, acc[ih * 2][j].y, acc[ih * 2 + 1][j].x, acc[ih * 2 + 1][j].y);
      }
    }
    return;
  }
#pragma unroll
  for (int jh = 0; jh < 2; ++jh)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = jh * 4 + jj;
      const int n = n0 + jh * 64 + ty * 4 + jj;
      const float bias_n = p.bias_axis == 2 ? __ldg(p.bias + n) : 0.0f;
#pragma unroll
      for (int ih = 0; ih < 2; ++ih) {
        const int m = m0 + ih * 64 + tx * 4;
        float4 v = make_float4(acc[ih * 2][j].x, acc[ih * 2][j].y, acc[ih * 2 + 1][j].x, acc[ih * 2 + 1][j].y);
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
