/*
 * Plain C restatement of the reference's definition of the GEMM math — TEST INFRASTRUCTURE ONLY
 * (used by tests/ to cross-check the numpy oracle; never linked into or called from the product
 * library).
 *
 * PARITY UNPINNED: GemmKernels.jl ships no golden vectors for this path and cannot run here;
 * this file and gemm_oracle.py pin each other on the fixtures in tests/golden/.
 *
 * Follows configs/configs.jl:49-74 of the GemmKernels.jl repository (get_custom_mul!):
 *     res = beta * C[i,j];  for k: res = alpha * update(A[i,k], B[k,j], res);  C[i,j] = res
 * For the ordinary product alpha is applied once to the finished sum (alpha*sum + beta*C), which
 * is what LinearAlgebra.mul!(C, A, B, alpha, beta) computes.  All matrices are column-major with
 * explicit leading dimensions; ta/tb != 0 means the operand is stored transposed.
 */
#include <math.h>
#include <stdint.h>

#define A_AT(i, k) (ta ? A[(k) + (int64_t)(i) * lda] : A[(i) + (int64_t)(k) * lda])
#define B_AT(k, j) (tb ? B[(j) + (int64_t)(k) * ldb] : B[(k) + (int64_t)(j) * ldb])

#define DEFINE_GEMM(NAME, TIN, TOUT, TACC)                                                         \
  void NAME(int64_t M, int64_t N, int64_t K, int ta, int tb, double alpha, const TIN* A,           \
            int64_t lda, const TIN* B, int64_t ldb, double beta, const TOUT* C, int64_t ldc,       \
            TOUT* D, int64_t ldd) {                                                                \
    for (int64_t j = 0; j < N; ++j)                                                                \
      for (int64_t i = 0; i < M; ++i) {                                                            \
        TACC acc = 0;                                                                              \
        for (int64_t k = 0; k < K; ++k) acc += (TACC)A_AT(i, k) * (TACC)B_AT(k, j);                \
        TACC r = (TACC)alpha * acc;                                                                \
        if (C && beta != 0.0) r += (TACC)beta * (TACC)C[i + j * ldc];                              \
        D[i + j * ldd] = (TOUT)r;                                                                  \
      }                                                                                            \
  }

DEFINE_GEMM(oracle_gemm_f32, float, float, float)
DEFINE_GEMM(oracle_gemm_f32_f64acc, float, float, double)
DEFINE_GEMM(oracle_gemm_f64, double, double, double)
DEFINE_GEMM(oracle_gemm_i16, int16_t, int16_t, int16_t)
DEFINE_GEMM(oracle_gemm_i32, int32_t, int32_t, int32_t)
DEFINE_GEMM(oracle_gemm_i64, int64_t, int64_t, int64_t)

/* max-plus: D[i,j] = max(beta*C[i,j], max_k(alpha*A[i,k] + B[k,j])) with alpha = beta = 1 in the
 * reference's configurations (configs/configs.jl:230-231, src/operator.jl:134-137). */
void oracle_tropical_f32(int64_t M, int64_t N, int64_t K, int ta, int tb, const float* A,
                         int64_t lda, const float* B, int64_t ldb, const float* C, int64_t ldc,
                         float* D, int64_t ldd) {
  for (int64_t j = 0; j < N; ++j)
    for (int64_t i = 0; i < M; ++i) {
      float r = C ? C[i + j * ldc] : -INFINITY;
      for (int64_t k = 0; k < K; ++k) {
        const float s = A_AT(i, k) + B_AT(k, j);
        r = s > r ? s : r;
      }
      D[i + j * ldd] = r;
    }
}
