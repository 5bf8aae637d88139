// Second pass of a split-K product: D = act( alpha * sum_s partial[s] + beta * C + bias ).
//
// The partial sums are `splits` sets of `planes` column-major M x N FP32 planes (leading dimension M,
// planes M*N elements apart, sets `stride` elements apart).  D and C are addressed as the tcgen05
// epilogue addresses them: two-level strides per index (plain matrices: one level) and, for
// two-plane (complex / dual) results, planar or interleaved pairs.  Pure streaming: each thread
// handles four consecutive rows of one column when the result is a plain one-plane matrix and M and
// the pointers allow 16-byte accesses to the planes, one element otherwise.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gk {

struct SplitKReduceParams {
  const float* partial;
  int splits, planes;
  int64_t stride;
  int M, N;
  float alpha, beta;
  const void* C; int dtype_c;   // dtype: 0 F16, 1 BF16, 2 F32 (TcDtype)
  void* D; int dtype_d;
  // element (m, n) of plane pl is at sm0*(m % m_div) + sm1*(m / m_div) + sn0*(n % n_div) + sn1*(n / n_div),
  // then pl * plane (planar) or 2 * index + pl (plane == 0: interleaved pairs)
  int m_div, n_div;
  int64_t c_sm0, c_sm1, c_sn0, c_sn1, c_plane;
  int64_t d_sm0, d_sm1, d_sn0, d_sn1, d_plane;
  const float* bias; int bias_axis;          // 0 none, 1 per row, 2 per column
  int act;                                   // 0 none, 1 ReLU, 2 GELU
};

__device__ __forceinline__ float splitk_load(const void* p, int64_t i, int dt) {
  if (dt == 2) return static_cast<const float*>(p)[i];
  if (dt == 0) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void splitk_store(void* p, int64_t i, int dt, float v) {
  if (dt == 2) static_cast<float*>(p)[i] = v;
  else if (dt == 0) static_cast<__half*>(p)[i] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float splitk_finish(const SplitKReduceParams& p, float sum, int m, int n, int pl, int64_t ci) {
  float x = p.alpha * sum;
  if (p.beta != 0.0f) x += p.beta * splitk_load(p.C, p.planes == 2 && p.c_plane == 0 ? 2 * ci + pl : pl * p.c_plane + ci, p.dtype_c);
  if (pl == 0) {
    if (p.bias_axis == 1) x += p.bias[m];
    else if (p.bias_axis == 2) x += p.bias[n];
  }
  if (p.act == 1) x = fmaxf(x, 0.0f);
  else if (p.act == 2) x = 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
  return x;
}

template <bool VEC4>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const SplitKReduceParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // the partial sums come from the kernel before this one
  const int rows = VEC4 ? p.M / 4 : p.M;          // units along M
  const int64_t units = static_cast<int64_t>(rows) * p.N;
  const int64_t plane_elems = static_cast<int64_t>(p.M) * p.N;
  for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < units;
       u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(u / rows);
    const int r = static_cast<int>(u - static_cast<int64_t>(n) * rows);
    if constexpr (VEC4) {
      // plain one-plane matrix, unit row stride
      const int m = 4 * r;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const float* src = p.partial + m + static_cast<int64_t>(n) * p.M;
      for (int s = 0; s < p.splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + s * p.stride);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const float out[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
        splitk_store(p.D, m + i + static_cast<int64_t>(n) * p.d_sn0, p.dtype_d,
                     splitk_finish(p, out[i], m + i, n, 0, m + i + static_cast<int64_t>(n) * p.c_sn0));
    } else {
      const int m_in = r % p.m_div, m_out = r / p.m_div, n_in = n % p.n_div, n_out = n / p.n_div;
      const int64_t di = m_in * p.d_sm0 + m_out * p.d_sm1 + n_in * p.d_sn0 + n_out * p.d_sn1;
      const int64_t ci = m_in * p.c_sm0 + m_out * p.c_sm1 + n_in * p.c_sn0 + n_out * p.c_sn1;
      for (int pl = 0; pl < p.planes; ++pl) {
        float acc = 0.0f;
        const float* src = p.partial + pl * plane_elems + r + static_cast<int64_t>(n) * p.M;
        for (int s = 0; s < p.splits; ++s) acc += src[s * p.stride];
        splitk_store(p.D, p.planes == 2 && p.d_plane == 0 ? 2 * di + pl : pl * p.d_plane + di, p.dtype_d,
                     splitk_finish(p, acc, r, n, pl, ci));
      }
    }
  }
}

}  // namespace gk
