// De-interleaving pre-pass for complex / dual operands stored as (re, im) pairs (the reference's
// Interleaved* global layouts, src/layout.jl:276-334): writes the two planes the tcgen05 kernel
// reads through TMA into a caller-provided workspace.  HBM-bound copy: every pair is read once
// (one 4- or 8-byte load per thread, a full line per warp) and each plane written once.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gk {

// in: pairs, element (r, c) at in[2 * (r + c * ld_in)]; out: plane p at out[p * plane + r + c * ld_out]
template <typename TPair, typename TElem>
__global__ void __launch_bounds__(256) split_planes_kernel(const TPair* __restrict__ in, TElem* __restrict__ out,
                                                            int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                                                            int64_t plane) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i % rows, c = i / rows;
    const TPair v = in[r + c * ld_in];
    out[r + c * ld_out] = v.x;
    out[plane + r + c * ld_out] = v.y;
  }
}

}  // namespace gk
