// GEMM with a diagonal A (Layout.Diagonal, src/layout.jl:225-236):  D = act(alpha * diag(v) * op(B)
// + beta * C + bias), M == K.  A product with a diagonal matrix is a row scaling: each output
// element needs one element of B, so this is an HBM-bound streaming kernel (no tensor cores, no
// shared memory): B, C read once, D written once, v stays in L2.  Algorithmic bytes per element of
// D: sizeof(B) + sizeof(C) (when read) + sizeof(D).
//
// Column-major B and D with 16-byte aligned columns take the vector path: a thread owns 8
// consecutive rows of one column (16 bytes of a 16-bit B, 32 bytes of an FP32 D), a warp covers 256
// rows, so every access is a full coalesced line.  Anything else takes the scalar path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gk {

struct DiagParams {
  const void* v;      // the diagonal: first M elements
  const void* B;
  const void* C;
  void* D;
  int64_t M, N;
  int64_t b_sm, b_sn; // element strides of op(B) along m and n
  int64_t ldc, ldd;
  int dtype_ab, dtype_c, dtype_d;   // 0 f16, 1 bf16, 2 f32
  float alpha, beta;
  const float* bias;
  int bias_axis, act;
  int has_c;
};

__device__ __forceinline__ float diag_load(const void* p, int64_t i, int dt) {
  if (dt == 2) return static_cast<const float*>(p)[i];
  if (dt == 0) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void diag_store(void* p, int64_t i, int dt, float x) {
  if (dt == 2) static_cast<float*>(p)[i] = x;
  else if (dt == 0) static_cast<__half*>(p)[i] = __float2half_rn(x);
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
}

__device__ __forceinline__ float diag_act(float x, int act) {
  if (act == 1) return fmaxf(x, 0.0f);
  if (act == 2) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
  return x;
}

// Scalar path: any strides, any of the three element types.
__global__ void __launch_bounds__(256) diag_gemm_scalar_kernel(const DiagParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // launched with stream serialisation: see launch_dependent
  const int64_t total = p.M * p.N;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = i % p.M, n = i / p.M;
    float x = p.alpha * diag_load(p.v, m, p.dtype_ab) * diag_load(p.B, m * p.b_sm + n * p.b_sn, p.dtype_ab);
    if (p.has_c) x += p.beta * diag_load(p.C, m + n * p.ldc, p.dtype_c);
    if (p.bias_axis == 1) x += p.bias[m];
    if (p.bias_axis == 2) x += p.bias[n];
    diag_store(p.D, m + n * p.ldd, p.dtype_d, diag_act(x, p.act));
  }
}

// Vector path: 16-bit v and B (column-major), FP32 C and D, M a multiple of 8, aligned columns.
template <typename T16>
__global__ void __launch_bounds__(256) diag_gemm_vec_kernel(const DiagParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t m8 = p.M / 8;
  const int64_t total = m8 * p.N;
  const T16* v = static_cast<const T16*>(p.v);
  const T16* B = static_cast<const T16*>(p.B);
  const float* C = static_cast<const float*>(p.C);
  float* D = static_cast<float*>(p.D);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = (i % m8) * 8, n = i / m8;
    const uint4 bv = __ldcs(reinterpret_cast<const uint4*>(B + m + n * p.b_sn));   // streamed once
    const uint4 vv = __ldg(reinterpret_cast<const uint4*>(v + m));                 // reused by every column
    const T16* bh = reinterpret_cast<const T16*>(&bv);
    const T16* vh = reinterpret_cast<const T16*>(&vv);
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = p.alpha * static_cast<float>(vh[j]) * static_cast<float>(bh[j]);
    if (p.has_c) {
      const float4 c0 = __ldcs(reinterpret_cast<const float4*>(C + m + n * p.ldc));
      const float4 c1 = __ldcs(reinterpret_cast<const float4*>(C + m + 4 + n * p.ldc));
      x[0] += p.beta * c0.x; x[1] += p.beta * c0.y; x[2] += p.beta * c0.z; x[3] += p.beta * c0.w;
      x[4] += p.beta * c1.x; x[5] += p.beta * c1.y; x[6] += p.beta * c1.z; x[7] += p.beta * c1.w;
    }
    if (p.bias_axis == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] += p.bias[m + j];
    } else if (p.bias_axis == 2) {
      const float bn = p.bias[n];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] += bn;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = diag_act(x[j], p.act);
    __stcs(reinterpret_cast<float4*>(D + m + n * p.ldd), make_float4(x[0], x[1], x[2], x[3]));
    __stcs(reinterpret_cast<float4*>(D + m + 4 + n * p.ldd), make_float4(x[4], x[5], x[6], x[7]));
  }
}

}  // namespace gk
