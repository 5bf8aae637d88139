// Host-side shared declarations of the library: handle, error reporting, small helpers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>
#include <string>
#include <vector>

#include "../../include/gemmkernels_b200.h"

namespace gk {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

gk_status set_error(gk_status s, const char* fmt, ...);
void clear_error();

inline int dtype_size(int32_t dt) {
  switch (dt) {
    case GK_F16: case GK_BF16: case GK_I16: return 2;
    case GK_F32: case GK_I32: case GK_TF32: return 4;
    case GK_F64: case GK_I64: return 8;
    default: return 0;
  }
}

inline const char* dtype_name(int32_t dt) {
  switch (dt) {
    case GK_F16: return "Float16";
    case GK_BF16: return "BFloat16";
    case GK_F32: return "Float32";
    case GK_F64: return "Float64";
    case GK_I16: return "Int16";
    case GK_I32: return "Int32";
    case GK_I64: return "Int64";
    case GK_TF32: return "TF32";
    default: return "?";
  }
}

#define GK_CUDA_CHECK(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return gk::set_error(GK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                  \
                           cudaGetErrorString(_e), __FILE__, __LINE__);                  \
  } while (0)

// Launch with programmatic stream serialisation: the kernel may begin while its predecessor in the
// stream drains; it must execute griddepcontrol.wait before its first global access (ptx.cuh: pdl_wait).
template <typename P>
inline cudaError_t launch_dependent(void (*kernel)(const P), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    const P& params) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at{};
  at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, params);
}

struct MgpuState;   // mgpu.cu: communicator, communication stream and events of the sharded path

}  // namespace gk

struct gk_handle_s {
  int device = 0;
  int sm_count = 0;
  int max_smem_optin = 0;
  int cc_major = 0, cc_minor = 0;
  int32_t* status_host = nullptr;  // pinned, mapped: device-side waits report here
  int32_t* status_dev = nullptr;   // the same word as the device sees it
  gk::EncodeTiledFn encode_tiled = nullptr;
  std::mutex mu;                   // guards the caches below
  std::mutex host_mu;              // serialises gk_gemm_host calls (shared staging buffers)
  int max_clusters[2][4] = {};     // tc kernel [planes-1][tf32 + 2*rank5] -> co-resident CTA pairs
  bool attr_set[2][2][2][4] = {};  // tc kernel [debug instance][cg-1][planes-1][tf32 + 2*rank5]: smem attribute set
  bool attr_set_generic[2] = {};   // the same for the generic-load instances
  bool fpu_attr_set[12] = {};      // FFMA kernel instances (3 operand types x 4 transposes): shared-memory limit raised
  bool f64_attr_set[4] = {};       // FP64 kernel instances (4 transposes): shared-memory limit raised
  // staging buffers of gk_gemm_host (grown on demand, freed by gk_destroy)
  void* stage_dev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};  // A, B, C, D, bias
  size_t stage_bytes[5] = {0, 0, 0, 0, 0};
  // copy streams and events of the pipelined gk_gemm_host (created on first use)
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  std::vector<cudaEvent_t> events;
  std::vector<gk_tuning_entry> tuning;   // loaded by gk_load_tuning (guarded by mu)
  gk::MgpuState* mgpu = nullptr;   // set by gk_mgpu_init, released by gk_mgpu_destroy / gk_destroy
};

namespace gk {
// api.cu: grows staging buffer `slot` of the handle to at least `bytes` (never shrinks)
gk_status stage_reserve(gk_handle h, int slot, size_t bytes);
// api.cu: creates the two copy streams and at least `n_events` untimed events of the handle
gk_status host_streams_reserve(gk_handle h, size_t n_events);
// mgpu.cu: releases the communicator (called by gk_destroy)
void mgpu_release(gk_handle h);
}  // namespace gk
