// Generic SIMT GEMM: any size, any leading dimension, any transpose, every element-type triple of
// the reference's FPU operator (src/operator.jl:35-153, configs/configs.jl:496-518) and the
// max-plus (tropical) variant.  Loads are predicated (out-of-range reads give the additive
// identity, out-of-range stores are dropped), which is the contract of the reference's
// bounds-checked ColMajor/RowMajor layouts (src/layout.jl:117-144).
//
// This is the correctness backstop for shapes the fast kernels do not take (unaligned leading
// dimensions, integer and FP64 types).  The FP32 fast path is fpu_gemm.cuh.
#pragma once
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gk {

struct SimtParams {
  const void* A;
  const void* B;
  const void* C;
  void* D;
  int64_t M, N, K;
  int64_t a_sm, a_sk;  // element strides of A along m and k
  int64_t b_sk, b_sn;  // element strides of B along k and n
  int64_t ldc, ldd;
  double alpha, beta;
  const float* bias;
  int32_t bias_axis;   // 0 none, 1 per row, 2 per column
  int32_t act;         // 0 none, 1 relu, 2 gelu
  int32_t has_c;       // 0: C is not read (beta == 0 or Layout.Zero)
  int32_t a_zero;      // 1: A*B contributes nothing (alpha == 0 or Layout.Zero operands)
};

template <typename T> __device__ __forceinline__ T simt_neg_inf();
template <> __device__ __forceinline__ float simt_neg_inf<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double simt_neg_inf<double>() { return -INFINITY; }
template <> __device__ __forceinline__ int16_t simt_neg_inf<int16_t>() { return INT16_MIN; }
template <> __device__ __forceinline__ int32_t simt_neg_inf<int32_t>() { return INT32_MIN; }
template <> __device__ __forceinline__ int64_t simt_neg_inf<int64_t>() { return INT64_MIN; }

template <typename TAcc, typename TIn>
__device__ __forceinline__ TAcc simt_cvt_in(TIn v) { return static_cast<TAcc>(v); }
template <> __device__ __forceinline__ float simt_cvt_in<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float simt_cvt_in<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename TOut, typename TAcc>
__device__ __forceinline__ TOut simt_cvt_out(TAcc v) { return static_cast<TOut>(v); }
template <> __device__ __forceinline__ __half simt_cvt_out<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 simt_cvt_out<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

template <typename TAcc>
__device__ __forceinline__ TAcc simt_fma(TAcc a, TAcc b, TAcc c) { return a * b + c; }
template <> __device__ __forceinline__ float simt_fma<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double simt_fma<double>(double a, double b, double c) { return fma(a, b, c); }

template <typename TAcc>
__device__ __forceinline__ TAcc simt_act(TAcc v, int act) {
  if (act == 1) return v > TAcc(0) ? v : TAcc(0);
  if (act == 2) {
    const double x = static_cast<double>(v);
    return static_cast<TAcc>(0.5 * x * (1.0 + erf(x * 0.70710678118654752)));
  }
  return v;
}

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;
constexpr int kSimtThreads = 256;

// TM x TM outputs per thread, a (16 TM) x (16 TM) tile per CTA: TM = 4 (64 x 64 tiles) for small problems and
// 8-byte accumulators, TM = 8 (128 x 128 tiles, twice the FMAs per shared-memory load) for large ones.
template <typename TIn, typename TOut, typename TAcc, bool TROPICAL, int TM>
__global__ void __launch_bounds__(kSimtThreads) simt_gemm_kernel(const SimtParams p) {
  constexpr int TILE = 16 * TM;
  __shared__ TAcc As[kSimtK][TILE + 1];
  __shared__ TAcc Bs[kSimtK][TILE + 1];

  const TIn* A = static_cast<const TIn*>(p.A);
  const TIn* B = static_cast<const TIn*>(p.B);
  const TOut* C = static_cast<const TOut*>(p.C);
  TOut* D = static_cast<TOut*>(p.D);

  const int64_t m0 = static_cast<int64_t>(blockIdx.x) * TILE;
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * TILE;
  const int tx = threadIdx.x & 15;  // TM rows each, 16 apart
  const int ty = threadIdx.x >> 4;  // TM columns each, 16 apart

  const TAcc alpha = static_cast<TAcc>(p.alpha);
  const TAcc beta = static_cast<TAcc>(p.beta);
  const TAcc ident = TROPICAL ? simt_neg_inf<TAcc>() : TAcc(0);

  TAcc acc[TM][TM];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TM; ++j) {
      const int64_t m = m0 + tx + 16 * i, n = n0 + ty + 16 * j;
      TAcc c = ident;
      if (TROPICAL && p.has_c && m < p.M && n < p.N)
        c = beta * simt_cvt_in<TAcc, TOut>(C[m + n * p.ldc]);
      acc[i][j] = c;
    }

  if (!p.a_zero) {
    for (int64_t k0 = 0; k0 < p.K; k0 += kSimtK) {
      // TILE x 16 elements per operand, TM per thread
#pragma unroll
      for (int r = 0; r < TM; ++r) {
        const int e = threadIdx.x + r * kSimtThreads;
        {
          // A: walk the contiguous index fastest
          const int mm = (p.a_sm == 1) ? (e % TILE) : (e >> 4);
          const int kk = (p.a_sm == 1) ? (e / TILE) : (e & 15);
          const int64_t m = m0 + mm, k = k0 + kk;
          TAcc v = ident;
          if (m < p.M && k < p.K) {
            v = simt_cvt_in<TAcc, TIn>(A[m * p.a_sm + k * p.a_sk]);
            v = v * alpha;  // alpha scales A, as the reference's shared_to_regs_a transform does
          }
          As[kk][mm] = v;
        }
        {
          const int nn = (p.b_sn == 1) ? (e % TILE) : (e >> 4);
          const int kk = (p.b_sn == 1) ? (e / TILE) : (e & 15);
          const int64_t n = n0 + nn, k = k0 + kk;
          TAcc v = ident;
          if (n < p.N && k < p.K) v = simt_cvt_in<TAcc, TIn>(B[k * p.b_sk + n * p.b_sn]);
          Bs[kk][nn] = v;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kSimtK; ++kk) {
        TAcc a[TM], b[TM];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = As[kk][tx + 16 * i];
#pragma unroll
        for (int j = 0; j < TM; ++j) b[j] = Bs[kk][ty + 16 * j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TM; ++j) {
            if (TROPICAL) {
              // max-plus: padding holds -inf (floats) or INT_MIN; keep integer sums from wrapping
              TAcc s;
              if constexpr (std::is_floating_point<TAcc>::value) s = a[i] + b[j];   // -inf + x stays -inf
              else s = (a[i] == ident || b[j] == ident) ? ident : a[i] + b[j];
              acc[i][j] = s > acc[i][j] ? s : acc[i][j];
            } else {
              acc[i][j] = simt_fma<TAcc>(a[i], b[j], acc[i][j]);
            }
          }
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TM; ++j) {
      const int64_t m = m0 + tx + 16 * i, n = n0 + ty + 16 * j;
      if (m < p.M && n < p.N) {
        TAcc v = acc[i][j];
        if (!TROPICAL && p.has_c) v = v + beta * simt_cvt_in<TAcc, TOut>(C[m + n * p.ldc]);
        if (p.bias_axis == 1) v = v + static_cast<TAcc>(p.bias[m]);
        if (p.bias_axis == 2) v = v + static_cast<TAcc>(p.bias[n]);
        v = simt_act<TAcc>(v, p.act);
        D[m + n * p.ldd] = simt_cvt_out<TOut, TAcc>(v);
      }
    }
}

}  // namespace gk
