// Column-sharded GEMM over the GPUs of one box: D[:, J_r] = A * B[:, J_r], one rank per GPU.
//
// The blocks are independent; the only exchange is A.  Two forms:
//   * operands on the device: A is resident on every rank, or it is broadcast from one rank in
//     K-panels over NCCL on a communication stream while the panels that have arrived are
//     multiplied on the caller's stream (stream events order the two; no kernel waits on a flag);
//   * operands in host memory: every rank uploads 1/world of A over its own PCIe link, NCCL
//     all-gathers assemble A in each GPU's memory over NVLink chunk by chunk, and each row chunk of
//     D is multiplied and downloaded as soon as its chunk of A is whole.
// Kernels read this GPU's memory only.  NCCL is found with dlopen at gk_mgpu_init, so the library
// itself has no link-time dependency on it.
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>

#include "common.h"

namespace gk {

// The few NCCL declarations used here (its public C ABI; see nccl.h).
typedef struct ncclComm* NcclComm;
struct NcclUniqueId { char internal[GK_MGPU_UNIQUE_ID_BYTES]; };
typedef int NcclResult;           // 0 = ncclSuccess
constexpr int kNcclUint8 = 1;     // ncclUint8

struct NcclApi {
  void* lib = nullptr;
  NcclResult (*GetUniqueId)(NcclUniqueId*) = nullptr;
  NcclResult (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  NcclResult (*CommDestroy)(NcclComm) = nullptr;
  NcclResult (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
  NcclResult (*Broadcast)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(NcclResult) = nullptr;
  std::string origin;
};

static std::mutex g_nccl_mu;
static NcclApi g_nccl;

static gk_status nccl_load(NcclApi** out) {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (!g_nccl.lib) {
    void* lib = nullptr;
    std::string origin;
    if (const char* env = std::getenv("GK_NCCL_LIB")) {
      lib = dlopen(env, RTLD_NOW | RTLD_LOCAL);
      origin = env;
      if (!lib) return set_error(GK_ERR_UNSUPPORTED, "GK_NCCL_LIB = %s cannot be loaded: %s", env, dlerror());
    }
    // a copy the process holds already (PyTorch's, NCCL_jll's) comes first: one NCCL per process
    if (!lib) { lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_LOCAL); origin = "libnccl.so.2 (already loaded)"; }
    if (!lib) { lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL); origin = "libnccl.so.2"; }
    if (!lib) { lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL); origin = "libnccl.so"; }
    if (!lib)
      return set_error(GK_ERR_UNSUPPORTED, "NCCL not found (set GK_NCCL_LIB to the path of libnccl.so.2): %s", dlerror());
    NcclApi api;
    api.lib = lib; api.origin = origin;
    bool ok = true;
    auto sym = [&](const char* name) { void* p = dlsym(lib, name); if (!p) ok = false; return p; };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    if (!ok) return set_error(GK_ERR_UNSUPPORTED, "%s lacks an NCCL entry point this library needs", origin.c_str());
    g_nccl = api;
  }
  *out = &g_nccl;
  return GK_OK;
}

#define GK_NCCL_CHECK(api, expr)                                                                          \
  do {                                                                                                    \
    gk::NcclResult _r = (expr);                                                                           \
    if (_r != 0)                                                                                          \
      return gk::set_error(GK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, (api)->GetErrorString(_r), __FILE__, __LINE__); \
  } while (0)

struct MgpuState {
  NcclApi* api = nullptr;
  NcclComm comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t comm_stream = nullptr;
  std::vector<cudaEvent_t> events;   // untimed, for ordering between streams
  std::vector<cudaEvent_t> timed;    // for gk_mgpu_times
};

void mgpu_release(gk_handle h) {
  if (!h || !h->mgpu) return;
  MgpuState* m = h->mgpu;
  if (m->comm_stream) cudaStreamSynchronize(m->comm_stream);
  if (m->comm && m->api) m->api->CommDestroy(m->comm);
  for (cudaEvent_t e : m->events) cudaEventDestroy(e);
  for (cudaEvent_t e : m->timed) cudaEventDestroy(e);
  if (m->comm_stream) cudaStreamDestroy(m->comm_stream);
  delete m;
  h->mgpu = nullptr;
}

static gk_status reserve_events(std::vector<cudaEvent_t>* v, size_t n, unsigned flags) {
  while (v->size() < n) {
    cudaEvent_t e;
    GK_CUDA_CHECK(cudaEventCreateWithFlags(&e, flags));
    v->push_back(e);
  }
  return GK_OK;
}

// Row chunks of A for the host path: about 32 MiB of A per chunk, eight at most, rows per chunk a
// multiple of 256 (whole tiles) and, for a transposed A whose chunks are cut among the ranks by
// rows, of the world size.
static gk_status host_plan(const gk_gemm_desc& d, int world, int* chunks, int64_t* rows) {
  if (world < 1) return set_error(GK_ERR_INVALID_ARGUMENT, "world = %d", world);
  if (d.number != GK_REAL || d.layout_a != GK_LAYOUT_DENSE || d.layout_b != GK_LAYOUT_DENSE || d.batch > 1)
    return set_error(GK_ERR_INVALID_CONFIG, "the sharded host path takes single real products of dense operands");
  if (d.m < 1 || d.n < 0 || d.k < 1) return set_error(GK_ERR_DIMENSION_MISMATCH, "Dimensions do not match: empty product");
  const int64_t cut = d.trans_a ? d.m : d.k;    // the index each chunk is dealt out by among the ranks
  if (cut % world)
    return set_error(GK_ERR_INVALID_CONFIG, "%s = %lld is not divisible by the %d ranks that each upload a share of A",
                     d.trans_a ? "M" : "K", (long long)cut, world);
  int64_t unit = 256;
  if (d.trans_a) while (unit % world) unit += 256;
  const size_t a_bytes = static_cast<size_t>(d.m) * d.k * dtype_size(d.dtype_a);
  int n = static_cast<int>((a_bytes + (16u << 20)) / (32u << 20));
  n = std::max(1, std::min(n, 8));
  int64_t mr = (d.m + n - 1) / n;
  mr = (mr + unit - 1) / unit * unit;
  if (mr >= d.m) mr = d.m;
  *rows = mr;
  *chunks = static_cast<int>((d.m + mr - 1) / mr);
  return GK_OK;
}

}  // namespace gk

using namespace gk;

extern "C" {

gk_status gk_mgpu_unique_id(void* id_out) {
  clear_error();
  if (!id_out) return set_error(GK_ERR_INVALID_ARGUMENT, "id_out is NULL");
  NcclApi* api = nullptr;
  gk_status s = nccl_load(&api);
  if (s != GK_OK) return s;
  NcclUniqueId id;
  GK_NCCL_CHECK(api, api->GetUniqueId(&id));
  std::memcpy(id_out, id.internal, GK_MGPU_UNIQUE_ID_BYTES);
  return GK_OK;
}

gk_status gk_mgpu_init(gk_handle h, int32_t rank, int32_t world, const void* unique_id) {
  clear_error();
  if (!h || !unique_id) return set_error(GK_ERR_INVALID_ARGUMENT, "handle or unique_id is NULL");
  if (world < 1 || rank < 0 || rank >= world)
    return set_error(GK_ERR_INVALID_ARGUMENT, "rank %d outside a world of %d", rank, world);
  if (h->mgpu) return set_error(GK_ERR_INVALID_ARGUMENT, "this handle has joined a communicator already");
  NcclApi* api = nullptr;
  gk_status s = nccl_load(&api);
  if (s != GK_OK) return s;
  int dev = -1;
  GK_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev != h->device)
    return set_error(GK_ERR_INVALID_ARGUMENT, "device %d is current but the handle belongs to device %d", dev, h->device);
  MgpuState* m = new (std::nothrow) MgpuState();
  if (!m) return set_error(GK_ERR_CUDA, "out of host memory");
  m->api = api; m->rank = rank; m->world = world;
  NcclUniqueId id;
  std::memcpy(id.internal, unique_id, GK_MGPU_UNIQUE_ID_BYTES);
  NcclResult r = api->CommInitRank(&m->comm, world, id, rank);
  if (r != 0) {
    delete m;
    return set_error(GK_ERR_CUDA, "ncclCommInitRank failed: %s", api->GetErrorString(r));
  }
  cudaError_t e = cudaStreamCreateWithFlags(&m->comm_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    api->CommDestroy(m->comm);
    delete m;
    return set_error(GK_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(e));
  }
  h->mgpu = m;
  return GK_OK;
}

gk_status gk_mgpu_destroy(gk_handle h) {
  clear_error();
  mgpu_release(h);
  return GK_OK;
}

gk_status gk_mgpu_host_plan(const gk_gemm_desc* desc, int32_t world, int32_t* chunks, int64_t* rows_per_chunk) {
  clear_error();
  if (!desc || !chunks || !rows_per_chunk) return set_error(GK_ERR_INVALID_ARGUMENT, "descriptor or output is NULL");
  if (desc->struct_size != sizeof(gk_gemm_desc))
    return set_error(GK_ERR_INVALID_ARGUMENT, "gk_gemm_desc.struct_size is %u, this library expects %zu",
                     desc->struct_size, sizeof(gk_gemm_desc));
  int n = 0;
  int64_t rows = 0;
  gk_status s = host_plan(*desc, world, &n, &rows);
  if (s != GK_OK) return s;
  *chunks = n; *rows_per_chunk = rows;
  return GK_OK;
}

gk_status gk_mgpu_broadcast(gk_handle h, void* buf, int64_t bytes, int32_t root, gk_stream stream) {
  clear_error();
  if (!h || !buf || bytes < 0) return set_error(GK_ERR_INVALID_ARGUMENT, "handle or buffer is NULL, or a negative size");
  if (!h->mgpu) return set_error(GK_ERR_INVALID_ARGUMENT, "gk_mgpu_init has not been called on this handle");
  MgpuState* m = h->mgpu;
  if (root < 0 || root >= m->world) return set_error(GK_ERR_INVALID_ARGUMENT, "root %d outside a world of %d", root, m->world);
  if (bytes == 0 || m->world == 1) return GK_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  gk_status s = reserve_events(&m->events, 2, cudaEventDisableTiming);
  if (s != GK_OK) return s;
  GK_CUDA_CHECK(cudaEventRecord(m->events[0], st));
  GK_CUDA_CHECK(cudaStreamWaitEvent(m->comm_stream, m->events[0], 0));
  GK_NCCL_CHECK(m->api, m->api->Broadcast(buf, buf, static_cast<size_t>(bytes), kNcclUint8, root, m->comm, m->comm_stream));
  GK_CUDA_CHECK(cudaEventRecord(m->events[1], m->comm_stream));
  GK_CUDA_CHECK(cudaStreamWaitEvent(st, m->events[1], 0));
  return GK_OK;
}

gk_status gk_mgpu_gemm_colshard(gk_handle h, const gk_gemm_desc* desc, void* a, int32_t a_mode, int32_t root,
                                int32_t k_panels, const void* b, const void* c, void* d, const gk_epilogue_desc* epi,
                                void* workspace, int64_t workspace_bytes, gk_stream stream) {
  clear_error();
  if (!h || !desc) return set_error(GK_ERR_INVALID_ARGUMENT, "handle or descriptor is NULL");
  if (a_mode == GK_MGPU_A_RESIDENT || !h->mgpu || h->mgpu->world == 1)
    return gk_gemm(h, desc, a, b, c, d, epi, workspace, workspace_bytes, stream);
  if (a_mode != GK_MGPU_A_BROADCAST) return set_error(GK_ERR_INVALID_ARGUMENT, "unknown a_mode %d", a_mode);
  MgpuState* m = h->mgpu;
  if (root < 0 || root >= m->world) return set_error(GK_ERR_INVALID_ARGUMENT, "root %d outside a world of %d", root, m->world);
  if (desc->struct_size != sizeof(gk_gemm_desc)) return set_error(GK_ERR_INVALID_ARGUMENT, "gk_gemm_desc.struct_size mismatch");
  if (desc->number != GK_REAL || desc->layout_a != GK_LAYOUT_DENSE || desc->batch > 1 || !a)
    return set_error(GK_ERR_INVALID_CONFIG, "the broadcast form takes single real products with a dense A");
  const gk_gemm_desc& dd = *desc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es_a = dtype_size(dd.dtype_a), es_b = dtype_size(dd.dtype_b);
  const size_t es_c = dtype_size(dd.dtype_c), es_d = dtype_size(dd.dtype_d);
  // Panels.  A column-major A (M x K) is contiguous in runs of whole columns, i.e. in panels of K: the
  // product of panel p adds to D (beta = 1 from the second panel on; bias and activation with the
  // last), which costs one more read and write of the D block per extra panel.  A transposed A
  // (stored K x M) is contiguous in panels of M: each is an independent block of rows of D, nothing
  // accumulates.  Panel boundaries are multiples of 256, so every panel starts 16-byte aligned.
  const bool by_m = dd.trans_a != 0;
  const int64_t cut = by_m ? dd.m : dd.k;
  int panels = k_panels;
  if (panels <= 0) {
    if (by_m) {
      panels = cut >= 8192 ? 4 : cut >= 2048 ? 2 : 1;
    } else {
      // rough times in seconds: broadcast at NVLink rate, product at the tensor-core rate, D traffic at HBM rate
      const double bcast = static_cast<double>(dd.m) * dd.k * es_a / 600e9;
      const double extra = 2.0 * dd.m * dd.n * es_d / 6.0e12;          // per extra panel
      double best = 1e30;
      for (int p : {1, 2, 4}) {
        if (cut < 2048 * p && p > 1) continue;
        const double t = bcast / p + (p - 1) * extra;                    // what the product cannot hide
        if (t < best) { best = t; panels = p; }
      }
    }
  }
  int64_t step = (cut + panels - 1) / panels;
  step = (step + 255) / 256 * 256;
  panels = static_cast<int>((cut + step - 1) / step);
  gk_status s = reserve_events(&m->events, static_cast<size_t>(panels) + 1, cudaEventDisableTiming);
  if (s != GK_OK) return s;
  // the transfers start after whatever the caller queued on `stream` (A may still be in use there)
  GK_CUDA_CHECK(cudaEventRecord(m->events[0], st));
  GK_CUDA_CHECK(cudaStreamWaitEvent(m->comm_stream, m->events[0], 0));
  const int64_t a_rows = by_m ? dd.k : dd.m;      // rows of the stored A
  gk_epilogue_desc epi_p;
  if (epi) epi_p = *epi;
  for (int p = 0; p < panels; ++p) {
    const int64_t x0 = p * step, xn = std::min<int64_t>(step, cut - x0);   // stored columns x0 .. x0 + xn
    char* a_p = static_cast<char*>(a) + static_cast<size_t>(x0) * dd.lda * es_a;
    // the last column of a panel is sent without the padding behind it
    const size_t bytes = (static_cast<size_t>(xn - 1) * dd.lda + a_rows) * es_a;
    GK_NCCL_CHECK(m->api, m->api->Broadcast(a_p, a_p, bytes, kNcclUint8, root, m->comm, m->comm_stream));
    GK_CUDA_CHECK(cudaEventRecord(m->events[p + 1], m->comm_stream));
    GK_CUDA_CHECK(cudaStreamWaitEvent(st, m->events[p + 1], 0));
    gk_gemm_desc blk = dd;
    if (blk.max_ctas == 0 && panels > 1) blk.max_ctas = std::max(2, (h->sm_count - 16) & ~1);   // leave SMs to NCCL
    const void* b_p = b;
    const void* c_p = c;
    void* d_p = d;
    const gk_epilogue_desc* e_p = epi;
    if (by_m) {
      blk.m = xn;
      if (c) c_p = static_cast<const char*>(c) + static_cast<size_t>(x0) * es_c;
      d_p = static_cast<char*>(d) + static_cast<size_t>(x0) * es_d;
      if (epi && epi->bias_axis == GK_BIAS_ROW && epi->bias) { epi_p.bias = epi->bias + x0; e_p = &epi_p; }
    } else {
      blk.k = xn;
      b_p = static_cast<const char*>(b) + (dd.trans_b ? static_cast<size_t>(x0) * dd.ldb : static_cast<size_t>(x0)) * es_b;
      if (p > 0) { blk.beta = 1.0; blk.layout_c = GK_LAYOUT_DENSE; blk.dtype_c = dd.dtype_d; blk.ldc = dd.ldd; c_p = d; }
      if (p != panels - 1) e_p = nullptr;
    }
    s = gk_gemm(h, &blk, a_p, b_p, c_p, d_p, e_p, workspace, workspace_bytes, stream);
    if (s != GK_OK) {
      cudaStreamSynchronize(m->comm_stream);
      return s;
    }
  }
  return GK_OK;
}

gk_status gk_mgpu_gemm_colshard_host(gk_handle h, const gk_gemm_desc* desc, const void* a_host, const void* b_host,
                                     const void* c_host, void* d_host, const gk_epilogue_desc* epi, gk_stream stream,
                                     gk_mgpu_times* times) {
  clear_error();
  if (!h || !desc) return set_error(GK_ERR_INVALID_ARGUMENT, "handle or descriptor is NULL");
  if (!h->mgpu || h->mgpu->world == 1) {
    const gk_status s1 = gk_gemm_host(h, desc, a_host, b_host, c_host, d_host, epi, stream);
    if (times) std::memset(times, 0, sizeof(*times));
    return s1;
  }
  MgpuState* m = h->mgpu;
  const gk_gemm_desc& d = *desc;
  if (d.struct_size != sizeof(gk_gemm_desc)) return set_error(GK_ERR_INVALID_ARGUMENT, "gk_gemm_desc.struct_size mismatch");
  int R = 0;
  int64_t mr = 0;
  gk_status s = host_plan(d, m->world, &R, &mr);
  if (s != GK_OK) return s;
  if (!a_host || !b_host || !d_host) return set_error(GK_ERR_INVALID_ARGUMENT, "A, B or D is NULL");
  const bool read_c = d.layout_c == GK_LAYOUT_DENSE && d.beta != 0.0;
  if (read_c && !c_host) return set_error(GK_ERR_INVALID_ARGUMENT, "beta = %g but C is NULL", d.beta);
  const bool has_bias = epi && epi->bias_axis != GK_BIAS_NONE;
  if (has_bias && !epi->bias) return set_error(GK_ERR_INVALID_ARGUMENT, "bias axis set but bias pointer is NULL");
  if (d.n == 0) return GK_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int W = m->world, rank = m->rank;
  const size_t es_a = dtype_size(d.dtype_a), es_b = dtype_size(d.dtype_b), es_c = dtype_size(d.dtype_c),
               es_d = dtype_size(d.dtype_d);
  const size_t a_bytes = static_cast<size_t>(d.m) * d.k * es_a;                       // chunk-major, no padding
  const size_t b_bytes = static_cast<size_t>(d.ldb) * (d.trans_b ? d.k : d.n) * es_b;
  const size_t c_bytes = read_c ? static_cast<size_t>(d.ldc) * d.n * es_c : 0;
  const size_t d_bytes = static_cast<size_t>(d.ldd) * d.n * es_d;
  const size_t bias_bytes = has_bias ? sizeof(float) * static_cast<size_t>(epi->bias_axis == GK_BIAS_ROW ? d.m : d.n) : 0;
  std::lock_guard<std::mutex> lock(h->host_mu);
  const size_t need[5] = {a_bytes, b_bytes, c_bytes, d_bytes, bias_bytes};
  for (int i = 0; i < 5; ++i)
    if (need[i] && (s = stage_reserve(h, i, need[i])) != GK_OK) return s;
  if ((s = host_streams_reserve(h, 2)) != GK_OK) return s;
  if ((s = reserve_events(&m->events, 4 * static_cast<size_t>(R) + 4, cudaEventDisableTiming)) != GK_OK) return s;
  const bool timing = times != nullptr;
  if (timing && (s = reserve_events(&m->timed, 4 * static_cast<size_t>(R) + 4, cudaEventDefault)) != GK_OK) return s;
  char* a_dev = static_cast<char*>(h->stage_dev[0]);
  char* b_dev = static_cast<char*>(h->stage_dev[1]);
  char* c_dev = static_cast<char*>(h->stage_dev[2]);
  char* d_dev = static_cast<char*>(h->stage_dev[3]);
  size_t ev = 0, tv = 0;
  auto fail = [&](gk_status code) {
    cudaStreamSynchronize(h->copy_in); cudaStreamSynchronize(m->comm_stream); cudaStreamSynchronize(st);
    cudaStreamSynchronize(h->copy_out);
    return code;
  };
  // everything starts after what the caller queued on `stream`
  GK_CUDA_CHECK(cudaEventRecord(m->events[ev], st));
  GK_CUDA_CHECK(cudaStreamWaitEvent(h->copy_in, m->events[ev], 0));
  GK_CUDA_CHECK(cudaStreamWaitEvent(m->comm_stream, m->events[ev], 0));
  GK_CUDA_CHECK(cudaStreamWaitEvent(h->copy_out, m->events[ev], 0));
  ++ev;
  cudaEvent_t t_up0 = nullptr, t_up1 = nullptr, t_dn0 = nullptr, t_dn1 = nullptr;
  if (timing) {
    t_up0 = m->timed[tv++]; t_up1 = m->timed[tv++]; t_dn0 = m->timed[tv++]; t_dn1 = m->timed[tv++];
    GK_CUDA_CHECK(cudaEventRecord(t_up0, h->copy_in));
  }
  int64_t h2d = 0, d2h = 0;
  if (has_bias) {
    GK_CUDA_CHECK(cudaMemcpyAsync(h->stage_dev[4], epi->bias, bias_bytes, cudaMemcpyHostToDevice, h->copy_in));
    h2d += static_cast<int64_t>(bias_bytes);
  }
  // This rank's share of chunk i: 1/W of the chunk's columns (a chunk is a column-major matrix of its
  // own on the device, mr_i x K for a column-major A, K x mr_i for a transposed one), which is one
  // contiguous piece at offset rank * piece: the layout an in-place all-gather assembles.
  auto upload_piece = [&](int i) -> cudaError_t {
    const int64_t i0 = i * mr, mi = std::min<int64_t>(mr, d.m - i0);
    char* chunk = a_dev + static_cast<size_t>(i0) * d.k * es_a;
    if (!d.trans_a) {
      const int64_t kc = d.k / W, k0 = rank * kc;
      h2d += mi * kc * static_cast<int64_t>(es_a);
      return cudaMemcpy2DAsync(chunk + static_cast<size_t>(k0) * mi * es_a, mi * es_a,
                               static_cast<const char*>(a_host) + (static_cast<size_t>(k0) * d.lda + i0) * es_a, d.lda * es_a,
                               mi * es_a, kc, cudaMemcpyHostToDevice, h->copy_in);
    }
    const int64_t mc = mi / W, c0 = i0 + rank * mc;
    h2d += mc * d.k * static_cast<int64_t>(es_a);
    return cudaMemcpy2DAsync(chunk + static_cast<size_t>(rank) * mc * d.k * es_a, d.k * es_a,
                             static_cast<const char*>(a_host) + static_cast<size_t>(c0) * d.lda * es_a, d.lda * es_a,
                             d.k * es_a, mc, cudaMemcpyHostToDevice, h->copy_in);
  };
  gk_epilogue_desc epi_blk;
  if (epi) epi_blk = *epi;
  size_t ev_b = 0;
  std::vector<cudaEvent_t> t_coll, t_comp;
  for (int i = 0; i < R; ++i) {
    const int64_t i0 = i * mr, mi = std::min<int64_t>(mr, d.m - i0);
    if (mi % W && d.trans_a) return fail(set_error(GK_ERR_INVALID_CONFIG, "chunk of %lld rows is not divisible by %d ranks", (long long)mi, W));
    GK_CUDA_CHECK(upload_piece(i));
    GK_CUDA_CHECK(cudaEventRecord(m->events[ev], h->copy_in));
    GK_CUDA_CHECK(cudaStreamWaitEvent(m->comm_stream, m->events[ev], 0));
    ++ev;
    // assemble the chunk on every rank
    char* chunk = a_dev + static_cast<size_t>(i0) * d.k * es_a;
    const size_t piece = static_cast<size_t>(mi) * d.k * es_a / W;
    if (timing) { t_coll.push_back(m->timed[tv++]); GK_CUDA_CHECK(cudaEventRecord(t_coll.back(), m->comm_stream)); }
    {
      const NcclResult r = m->api->AllGather(chunk + rank * piece, chunk, piece, kNcclUint8, m->comm, m->comm_stream);
      if (r != 0) return fail(set_error(GK_ERR_CUDA, "ncclAllGather failed: %s", m->api->GetErrorString(r)));
    }
    if (timing) { t_coll.push_back(m->timed[tv++]); GK_CUDA_CHECK(cudaEventRecord(t_coll.back(), m->comm_stream)); }
    GK_CUDA_CHECK(cudaEventRecord(m->events[ev], m->comm_stream));
    GK_CUDA_CHECK(cudaStreamWaitEvent(st, m->events[ev], 0));
    ++ev;
    if (i == 0) {
      // this rank's block of B goes up behind its first piece of A, while that chunk is gathered
      GK_CUDA_CHECK(cudaMemcpyAsync(b_dev, b_host, b_bytes, cudaMemcpyHostToDevice, h->copy_in));
      h2d += static_cast<int64_t>(b_bytes);
      ev_b = ev;
      GK_CUDA_CHECK(cudaEventRecord(m->events[ev], h->copy_in));
      ++ev;
    }
    if (read_c) {
      GK_CUDA_CHECK(cudaMemcpy2DAsync(c_dev + static_cast<size_t>(i0) * es_c, d.ldc * es_c,
                                      static_cast<const char*>(c_host) + static_cast<size_t>(i0) * es_c, d.ldc * es_c,
                                      mi * es_c, d.n, cudaMemcpyHostToDevice, h->copy_in));
      h2d += mi * d.n * static_cast<int64_t>(es_c);
      GK_CUDA_CHECK(cudaEventRecord(m->events[ev], h->copy_in));
      GK_CUDA_CHECK(cudaStreamWaitEvent(st, m->events[ev], 0));
      ++ev;
    }
    if (i == 0) GK_CUDA_CHECK(cudaStreamWaitEvent(st, m->events[ev_b], 0));
    if (i == R - 1 && timing) GK_CUDA_CHECK(cudaEventRecord(t_up1, h->copy_in));
    gk_gemm_desc blk = d;
    blk.m = mi;
    blk.lda = d.trans_a ? d.k : mi;
    if (has_bias)
      epi_blk.bias = static_cast<const float*>(h->stage_dev[4]) + (epi->bias_axis == GK_BIAS_ROW ? i0 : 0);
    if (timing) { t_comp.push_back(m->timed[tv++]); GK_CUDA_CHECK(cudaEventRecord(t_comp.back(), st)); }
    s = gk_gemm(h, &blk, chunk, b_dev, read_c ? c_dev + static_cast<size_t>(i0) * es_c : nullptr,
                d_dev + static_cast<size_t>(i0) * es_d, epi ? &epi_blk : nullptr, nullptr, 0, stream);
    if (s != GK_OK) return fail(s);
    if (timing) { t_comp.push_back(m->timed[tv++]); GK_CUDA_CHECK(cudaEventRecord(t_comp.back(), st)); }
    GK_CUDA_CHECK(cudaEventRecord(m->events[ev], st));
    GK_CUDA_CHECK(cudaStreamWaitEvent(h->copy_out, m->events[ev], 0));
    ++ev;
    if (i == 0 && timing) GK_CUDA_CHECK(cudaEventRecord(t_dn0, h->copy_out));
    GK_CUDA_CHECK(cudaMemcpy2DAsync(static_cast<char*>(d_host) + static_cast<size_t>(i0) * es_d, d.ldd * es_d,
                                    d_dev + static_cast<size_t>(i0) * es_d, d.ldd * es_d, mi * es_d, d.n,
                                    cudaMemcpyDeviceToHost, h->copy_out));
    d2h += mi * d.n * static_cast<int64_t>(es_d);
  }
  if (timing) GK_CUDA_CHECK(cudaEventRecord(t_dn1, h->copy_out));
  GK_CUDA_CHECK(cudaEventRecord(m->events[ev], h->copy_out));
  GK_CUDA_CHECK(cudaStreamWaitEvent(st, m->events[ev], 0));
  GK_CUDA_CHECK(cudaStreamSynchronize(st));
  GK_CUDA_CHECK(cudaStreamSynchronize(m->comm_stream));
  if (timing) {
    std::memset(times, 0, sizeof(*times));
    auto span = [](cudaEvent_t a0, cudaEvent_t a1) { float ms = 0.0f; return cudaEventElapsedTime(&ms, a0, a1) == cudaSuccess ? ms : 0.0f; };
    times->upload_ms = span(t_up0, t_up1);
    times->download_ms = span(t_dn0, t_dn1);
    times->total_ms = span(t_up0, t_dn1);
    for (size_t i = 0; i + 1 < t_coll.size(); i += 2) times->collective_ms += span(t_coll[i], t_coll[i + 1]);
    for (size_t i = 0; i + 1 < t_comp.size(); i += 2) times->compute_ms += span(t_comp[i], t_comp[i + 1]);
    times->chunks = R;
    times->h2d_bytes = h2d; times->d2h_bytes = d2h;
    (void)cudaGetLastError();
  }
  int32_t code = 0;
  return gk_poll_status(h, &code);
}

}  // extern "C"
