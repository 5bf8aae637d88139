/*
 * gemmkernels_b200 — C ABI of the Blackwell (sm_100a) GEMM engine that sits behind the
 * GemmKernels.jl API.  Plain pointers and sizes only; every pointer named "device" is a CUDA
 * device pointer owned by the caller (never freed or retained past the call).  Work is enqueued
 * asynchronously on the caller's stream in the caller's current context; no call synchronises
 * unless its comment says so.  All functions return a gk_status; gk_last_error_message() gives
 * the text of the last failure on the calling thread.
 *
 * Reference interface replaced (paths inside the GemmKernels.jl repository):
 *   gk_gemm            the kernel launch in GemmKernels.matmul, src/matmul.jl:38-43, together with
 *                      the device code it launches (src/kernel.jl:10-574, src/operator.jl,
 *                      src/layout.jl, src/epilogue.jl:14-73, src/transform.jl:19-30)
 *   gk_gemm_query      the launch-geometry and limit checks of src/matmul.jl:24-41
 *   gk_create/destroy  no counterpart (CUDA.jl keeps the context); holds per-device caches
 */
#ifndef GEMMKERNELS_B200_H
#define GEMMKERNELS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GK_API __attribute__((visibility("default")))
#else
#define GK_API
#endif

#define GK_VERSION_MAJOR 0
#define GK_VERSION_MINOR 2

typedef struct gk_handle_s* gk_handle;
typedef void* gk_stream; /* a CUstream / cudaStream_t; NULL = the legacy default stream */

typedef enum gk_status {
  GK_OK = 0,
  GK_ERR_INVALID_CONFIG = 1,     /* maps to GemmKernels.ConfigError (src/config.jl:78-82)        */
  GK_ERR_UNSUPPORTED = 2,        /* a Transform/Epilogue/dtype outside the enumerated set         */
  GK_ERR_DIMENSION_MISMATCH = 3, /* maps to DimensionMismatch (src/matmul.jl:75-77)               */
  GK_ERR_CUDA = 4,               /* a CUDA runtime / driver call failed                           */
  GK_ERR_TIMEOUT = 5,            /* a bounded device-side wait gave up; the context stays usable  */
  GK_ERR_INVALID_ARGUMENT = 6
} gk_status;

typedef enum gk_dtype {
  GK_F16 = 0,
  GK_BF16 = 1,
  GK_F32 = 2,
  GK_F64 = 3,
  GK_I16 = 4,
  GK_I32 = 5,
  GK_I64 = 6,
  GK_TF32 = 7 /* compute type only: FP32 storage read by the tensor cores as TF32 */
} gk_dtype;

/* Operator.* of src/operator.jl.  TCGEN05 replaces the WMMA operators (operator.jl:163-372);
 * FPU is FPUOp (operator.jl:35-153), FPU_TROPICAL is TropicalFPUOp (max-plus). */
typedef enum gk_operator {
  GK_OP_AUTO = 0,
  GK_OP_TCGEN05 = 1,
  GK_OP_FPU = 2,
  GK_OP_FPU_TROPICAL = 3
} gk_operator;

/* Number system of the product: real, complex (WMMAComplexOp, operator.jl:251-314) or dual
 * numbers (WMMADualOp, operator.jl:320-372).  Complex and dual operands have two planes. */
typedef enum gk_number { GK_REAL = 0, GK_COMPLEX = 1, GK_DUAL = 2 } gk_number;

/* Per-operand layout kind.  DENSE covers ColMajor/RowMajor/UnsafeAligned* (layout.jl:111-270);
 * ZERO is Layout.Zero (layout.jl:82-89): the operand is not read; DIAGONAL is Layout.Diagonal
 * (layout.jl:225-236): A is a length-M vector holding the diagonal of a square matrix. */
typedef enum gk_layout_kind { GK_LAYOUT_DENSE = 0, GK_LAYOUT_ZERO = 1, GK_LAYOUT_DIAGONAL = 2 } gk_layout_kind;

typedef enum gk_activation { GK_ACT_NONE = 0, GK_ACT_RELU = 1, GK_ACT_GELU = 2 } gk_activation;

/* Bias axis.  COL is the reference's Epilogue.Bias (epilogue.jl:44-52: one value per column of D,
 * length N); ROW is one value per row of D (length M). */
typedef enum gk_bias_axis { GK_BIAS_NONE = 0, GK_BIAS_ROW = 1, GK_BIAS_COL = 2 } gk_bias_axis;

/* CTASwizzle.* of src/cta-swizzle.jl:26-160, reinterpreted as raster orders of the persistent
 * tile scheduler. */
typedef enum gk_raster {
  GK_RASTER_AUTO = 0,
  GK_RASTER_IDENTITY = 1,      /* column-major walk over tiles                       */
  GK_RASTER_HORIZONTAL = 2,    /* HorizontallyTiled{T}: bands of T tiles along N     */
  GK_RASTER_VERTICAL = 3,      /* VerticallyTiled{T}: bands of T tiles along M       */
  GK_RASTER_LEBESGUE = 4       /* LebesgueCurve: Z-order                             */
} gk_raster;

/*
 * D = act( alpha * op(A) * op(B) + beta * C + bias ),  op(X) = X or X^T.
 * All matrices are column-major (Julia order): element (i, j) of a stored matrix X is at
 * X[i + j * ldx].  trans_a = 0: A is stored M x K; trans_a = 1: A is stored K x M (the reference's
 * RowMajor global layout).  Likewise trans_b with K x N / N x K.  C and D are M x N and may alias.
 * For GK_COMPLEX / GK_DUAL, plane_x is the element distance between the two planes of operand x
 * (real/imaginary, or value/derivative); plane_x = 0 means interleaved pairs, in which case ldx
 * counts pairs.
 */
typedef struct gk_gemm_desc {
  uint32_t struct_size; /* sizeof(gk_gemm_desc), for ABI evolution */
  int32_t number;       /* gk_number */
  int64_t m, n, k;
  int32_t trans_a, trans_b;
  int32_t dtype_a, dtype_b, dtype_c, dtype_d; /* gk_dtype of the stored elements */
  int32_t compute;      /* gk_dtype the multiply runs in: F16/BF16/TF32 (TCGEN05), others (FPU) */
  int32_t op;           /* gk_operator */
  int64_t lda, ldb, ldc, ldd;
  int64_t plane_a, plane_b, plane_c, plane_d;
  int32_t layout_a, layout_b, layout_c; /* gk_layout_kind */
  int32_t raster;       /* gk_raster */
  double alpha, beta;
  /* Tuning overrides; 0 = use the built-in table. */
  int32_t tile_n;       /* 32..256, multiple of 32 (per CTA pair when cta_group = 2); 512 = two 256-column
                           accumulators that share each A stage, single accumulator stage (real products) */
  int32_t cta_group;    /* 1 or 2 */
  int32_t stages;       /* shared-memory pipeline depth */
  int32_t raster_group; /* T of the tiled rasters */
  int32_t max_ctas;     /* cap on the persistent grid */
  int32_t debug;        /* diagnostic bits, 0 in production: 1 no TMA, 2 no MMA, 4 idle producers (lets the
                           bounded waits run out), 8 per-role cycle counters into the workspace, 16 progress
                           marks for gk_debug_marks */
  int32_t host_chunk_mib; /* gk_gemm_host only: size of the upload / download chunks in MiB (0 = 32) */
  int32_t a_resident;   /* gk_gemm_host only: 1 = `a_host` is a DEVICE pointer (A is already resident, e.g.
                           after a broadcast from another rank) and is used in place, not uploaded */
  /* Strided-batched products: `batch` independent GEMMs of the same shape, operand x of product i at
   * x + i * batch_stride_x elements (batch_stride_a / _b = 0 shares that operand between the products).
   * batch <= 1 is the single product.  Real number system only.  On the tensor-core path the whole
   * batch is one launch (batch strides that are not multiples of 16 bytes, like such leading
   * dimensions, make its producers use ordinary loads instead of TMA); the SIMT families launch once
   * per product.  The reference has no batched entry point. */
  int32_t batch;
  int32_t k_blocks_per_stage; /* tuning override: 128-byte k-blocks per pipeline stage, 1 or 2 (0 = choose) */
  int64_t batch_stride_a, batch_stride_b, batch_stride_c, batch_stride_d;
} gk_gemm_desc;

typedef struct gk_epilogue_desc {
  uint32_t struct_size;
  int32_t bias_axis;   /* gk_bias_axis */
  const float* bias;   /* device, FP32, length M (ROW) or N (COL) */
  int32_t activation;  /* gk_activation, applied last (the reference's shared_to_global_d hook) */
  int32_t reserved[3];
} gk_epilogue_desc;

typedef struct gk_gemm_plan {
  int32_t kernel;       /* 1 = tcgen05, 2 = FPU (SIMT FFMA), 3 = generic SIMT, 4 = diagonal scale,
                           5 = contraction gather kernel */
  int32_t grid, block, cluster;
  int32_t smem_bytes, tmem_columns;
  int32_t tile_m, tile_n, tile_k, stages; /* tile_k: K elements per pipeline stage */
  int64_t workspace_bytes;
} gk_gemm_plan;

/* Version of the loaded library: major * 1000 + minor. */
GK_API int32_t gk_version(void);

/* Text of the last error raised on the calling thread ("" if none). Never NULL. */
GK_API const char* gk_last_error_message(void);

/* Creates the per-device state (SM count, driver entry points, a host-visible status word that
 * device-side waits report into).  Uses the current device.  Allocates; call once, not per GEMM. */
GK_API gk_status gk_create(gk_handle* out);
GK_API gk_status gk_destroy(gk_handle h);

/* Reads and clears the device-side status word without synchronising: GK_OK, or GK_ERR_TIMEOUT if
 * a kernel launched through this handle abandoned a wait since the last call. */
GK_API gk_status gk_poll_status(gk_handle h, int32_t* raw_code);

/* Copies the 16 host-visible diagnostic words of the handle: word 0 is the status word above; words
 * 1..15 are progress marks that tcgen05 kernels launched with the debug-marks bit leave behind
 * (how far each role got).  Reads host memory only: usable even after the context has failed. */
GK_API gk_status gk_debug_marks(gk_handle h, int32_t* out16);

/* Measures what the FP32 FMA pipe of this GPU sustains: a register-only kernel of independent packed
 * FMA chains on every SM, timed with CUDA events on `stream` (synchronises it).  *tflops gets
 * 2 flop per FMA / time.  The denominator for rooflines of the FPU operator, for which no library
 * GEMM figure exists.  No counterpart in the reference. */
GK_API gk_status gk_measure_fp32_fma(gk_handle h, double* tflops, gk_stream stream);

/* Fills *plan with what gk_gemm would launch for this descriptor; launches nothing. */
GK_API gk_status gk_gemm_query(gk_handle h, const gk_gemm_desc* desc, const gk_epilogue_desc* epi,
                        gk_gemm_plan* plan);

/*
 * Measured tile choices.  The reference ships what its tuning sweep found as the package's defaults
 * (tuning/tune.jl, tuning/wmma.jl:34-47); here the sweep (python -m gemmkernels_b200.tuning) writes
 * one entry per problem it measured, a generated table of them is compiled into the library, and a
 * caller may load its own on top.  When a descriptor leaves tile_n and cta_group at 0, the planner
 * takes the entry of the same element type, transposes and C use whose (m, n, k) matches exactly,
 * else the nearest one whose extents are all within a factor 1.5; without one it falls back to its
 * built-in cost model.  Entries apply to single real tensor-core products.
 */
typedef struct gk_tuning_entry {
  int32_t dtype;        /* gk_dtype of A and B (GK_F32 stands for the TF32 path) */
  int32_t trans_a, trans_b;
  int32_t has_c;        /* measured with beta != 0 (the epilogue reads C) */
  int64_t m, n, k;
  int32_t tile_n, cta_group, stages, raster_group;   /* as in gk_gemm_desc; 0 = leave to the planner */
  int32_t k_blocks_per_stage, reserved;
} gk_tuning_entry;

/* Replaces the handle's table with `count` entries (copied); count = 0 clears it.  The compiled-in
 * table stays underneath: a loaded entry wins over a compiled-in one at equal distance. */
GK_API gk_status gk_load_tuning(gk_handle h, const gk_tuning_entry* entries, int32_t count);

/* Enqueues one GEMM on `stream`.  a, b, c, d are device pointers (c may be NULL when beta == 0 or
 * layout_c is ZERO; c == d is allowed).  epi may be NULL.  workspace is a 256-byte aligned device
 * buffer of workspace_bytes bytes (NULL / 0 when there is none); gk_gemm_query reports in
 * plan.workspace_bytes how much the descriptor can use.  It is REQUIRED when complex / dual A or B
 * are interleaved (plane_a / plane_b == 0): they are split into planes there first, on the same
 * stream; a buffer that is too small is refused with GK_ERR_INVALID_ARGUMENT.  It is OPTIONAL for
 * tensor-core products with few output tiles and a long K: given enough room, K is cut into runs over
 * the otherwise idle SMs (split-K: FP32 partial sums in the workspace, one reduction pass that
 * applies alpha, beta, bias and activation); with NULL, or with a buffer smaller than the partial
 * sums need, the same product runs unsplit.  The FP32 FFMA kernel uses a workspace the same way for the
 * tiles of a last round that would fill at most half of the GPU.  Nothing is ever written beyond
 * workspace_bytes. */
GK_API gk_status gk_gemm(gk_handle h, const gk_gemm_desc* desc, const void* a, const void* b,
                  const void* c, void* d, const gk_epilogue_desc* epi, void* workspace,
                  int64_t workspace_bytes, gk_stream stream);

/*
 * Tensor contraction (GETT): D[modes_c] = alpha * sum over contracted modes of A[modes_a] * B[modes_b]
 * + beta * C[modes_c].  The reference has no such function in src/; this replaces the driver of
 * benchmarks/tensor-contractions/run.jl:88-131 (custom layouts that map one contraction onto the
 * GEMM kernels) with an entry point, e.g. GemmKernels.contract!(D, "abcd", A, "aebf", B, "dfce").
 * A mode label is any integer (characters, usually).  A label in A and C is a free mode of A, in B
 * and C a free mode of B, in A and B a contracted mode; a label in all three is a batch mode: the
 * call is one independent contraction per value of that index (launched one by one on the stream;
 * at most 65536).  Strides
 * are in elements and arbitrary (column-major tensors have strides 1, e0, e0*e1, ...); C and D share
 * modes_c / extents_c and have their own strides.  Tensors are read in place: when every index
 * splits into at most two modes that tile into TMA boxes the tensor cores run it through 5-D tensor
 * maps; otherwise a gather kernel runs it and needs a workspace (gk_contract_query reports
 * plan.kernel == 5 and plan.workspace_bytes).  On the tensor-core path a reported workspace is
 * optional, as for gk_gemm: given one (256-byte aligned), few output tiles with a long contracted
 * index are cut along K over the idle SMs.
 */
#define GK_MAX_MODES 8

typedef struct gk_contract_desc {
  uint32_t struct_size;
  int32_t rank_a, rank_b, rank_c;
  int32_t modes_a[GK_MAX_MODES], modes_b[GK_MAX_MODES], modes_c[GK_MAX_MODES];
  int64_t extents_a[GK_MAX_MODES], extents_b[GK_MAX_MODES], extents_c[GK_MAX_MODES];
  int64_t strides_a[GK_MAX_MODES], strides_b[GK_MAX_MODES], strides_c[GK_MAX_MODES],
      strides_d[GK_MAX_MODES];
  int32_t dtype_a, dtype_b, dtype_c, dtype_d; /* gk_dtype */
  int32_t compute;      /* F16 / BF16 / TF32: tensor cores when possible; F32: gather kernel */
  int32_t force_gather; /* 1 = always use the gather kernel (testing) */
  double alpha, beta;
  int32_t tile_n, cta_group, stages; /* tuning overrides, 0 = choose */
  int32_t debug;        /* diagnostic bits as in gk_gemm_desc.debug, 0 in production */
  int32_t reserved[2];
} gk_contract_desc;

GK_API gk_status gk_contract_query(gk_handle h, const gk_contract_desc* desc, gk_gemm_plan* plan);

/* Enqueues the contraction on `stream`.  c may be NULL when beta == 0; c == d is allowed.
 * workspace / workspace_bytes: device scratch — the gather path's offset tables (required there,
 * 8-byte aligned) or the partial sums of a split along K (optional); may be NULL / 0 when the query
 * reports workspace_bytes == 0. */
GK_API gk_status gk_contract(gk_handle h, const gk_contract_desc* desc, const void* a, const void* b,
                             const void* c, void* d, void* workspace, int64_t workspace_bytes,
                             gk_stream stream);

/*
 * gk_contract_static — the gather-path contraction for callers that must not allocate.
 * (No counterpart in the reference.)
 *
 * Who this is for: code that runs where device memory cannot be asked for at all — a host
 * application whose memory pool has already claimed the whole GPU (CUDA.jl's and PyTorch's caching
 * allocators do this under pressure, so a plain cudaMalloc from a library fails), a plug-in
 * callback whose contract forbids allocation, or a latency-bound loop that cannot afford the
 * device-wide synchronisation an allocation may imply.  Such callers have no handle either
 * (gk_create allocates), so this entry point takes none.
 *
 * What it does: the same arithmetic as gk_contract on its gather path (plan.kernel == 5): inputs
 * and outputs are the caller's; the per-index offset tables, which gk_contract puts in the caller's
 * workspace, go into a fixed array inside the library instead.  It calls no cudaMalloc, cudaFree or
 * any other allocating routine.
 *
 * Limits and rules:
 *  - The array holds GK_STATIC_TABLE_ENTRIES 64-bit offsets (256 KiB, held by every GPU that loads
 *    the library until the process exits).  A contraction needs 3*M + 3*N + 2*K entries (M, N, K =
 *    products of the free modes of A, of B, and of the contracted modes); anything larger is
 *    rejected with GK_ERR_INVALID_CONFIG and a message giving the numbers.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
 *    caches it; make that first call outside any stream capture.
 *  - All calls on one device share the one array and it keeps the last call's tables.  Each call
 *    rewrites every entry it reads before reading it, so stale contents are harmless, but two calls
 *    whose kernels can overlap on the GPU (different streams, no dependency) race on the tables:
 *    keep calls on one stream or order them with events.
 *  - Same element types as the gather path: A/B Float16, BFloat16 or Float32 (one type), C/D
 *    Float32 (or Float16 with Float16 inputs); FP32 accumulation; compute = GK_TF32 is rejected.
 */
#define GK_STATIC_TABLE_ENTRIES 32768

GK_API gk_status gk_contract_static(const gk_contract_desc* desc, const void* a, const void* b,
                                    const void* c, void* d, gk_stream stream);

/* The same GEMM for callers whose matrices live in host memory (Julia `Array`s rather than
 * `CuArray`s; the reference has no such method — CUDA.jl users would `CuArray(A)` first, which is
 * what this call does internally): copies a, b (and c, and the bias named by epi) to device
 * staging buffers kept in the handle, runs gk_gemm, copies D back to d_host and returns once
 * d_host is complete (it synchronises `stream`).  Large real products are cut into blocks (row chunks
 * of A by column chunks of B) whose uploads, kernels and downloads overlap on two copy streams owned by
 * the handle; small ones run copy, compute, copy on `stream`.  Pinned host memory makes the copies
 * faster (and is what lets them overlap) but is not required.  Calls on one handle are serialised. */
GK_API gk_status gk_gemm_host(gk_handle h, const gk_gemm_desc* desc, const void* a_host,
                              const void* b_host, const void* c_host, void* d_host,
                              const gk_epilogue_desc* epi, gk_stream stream);


/*
 * Column-sharded GEMM over the GPUs of one box: D[:, J_r] = A * B[:, J_r], rank r owns the column
 * block J_r of B, C and D; the only exchange is A.  The reference has no multi-GPU code; these
 * entry points have no counterpart there.  One rank per GPU — a process per GPU (torchrun,
 * Julia's Distributed, MPI) or a thread per GPU — each with its own handle.  The library finds NCCL
 * at gk_mgpu_init with dlopen (the environment variable GK_NCCL_LIB, else a libnccl.so.2 that the
 * process has loaded already, else the system's), so it still loads on machines without NCCL.
 * Kernels only ever read this GPU's own memory: A arrives through NCCL into local buffers first.
 */
#define GK_MGPU_UNIQUE_ID_BYTES 128

/* Fills id_out (GK_MGPU_UNIQUE_ID_BYTES bytes) on ONE rank; hand the bytes to every rank by any
 * means (a file, a socket, torch.distributed, MPI) and pass them to gk_mgpu_init. */
GK_API gk_status gk_mgpu_unique_id(void* id_out);

/* Joins the communicator of `world` ranks as `rank` with the handle's device (collective: every
 * rank calls it; blocks until all have).  Creates the handle's communication stream. */
GK_API gk_status gk_mgpu_init(gk_handle h, int32_t rank, int32_t world, const void* unique_id);
GK_API gk_status gk_mgpu_destroy(gk_handle h);

typedef enum gk_mgpu_a_mode {
  GK_MGPU_A_RESIDENT = 0,  /* every rank already holds A at `a`: nothing is exchanged              */
  GK_MGPU_A_BROADCAST = 1  /* rank `root` holds A at `a`; it is sent into every rank's `a` first   */
} gk_mgpu_a_mode;

/* This rank's block of the sharded product, device operands (collective when a_mode is BROADCAST:
 * every rank calls it with the same m, k, a_mode, root and k_panels).  desc describes the local block
 * (n = this rank's column count; may differ between ranks).  a: device buffer of the whole A on every
 * rank.  With GK_MGPU_A_BROADCAST, A travels in `k_panels` panels (0 = choose) over NCCL on the
 * handle's communication stream while the product of the panels that have arrived runs on `stream`,
 * so the transfer overlaps the arithmetic.  A column-major A is cut into panels of K (D accumulates
 * panel by panel, bias and activation are applied with the last panel; each extra panel re-reads
 * and re-writes the D block, which the automatic choice weighs against the transfer it hides); a
 * transposed A (trans_a = 1) is cut into panels of M, independent row blocks of D.  Enqueues only;
 * the result is complete when `stream` is. */
GK_API gk_status gk_mgpu_gemm_colshard(gk_handle h, const gk_gemm_desc* desc, void* a, int32_t a_mode,
                                       int32_t root, int32_t k_panels, const void* b, const void* c, void* d,
                                       const gk_epilogue_desc* epi, void* workspace, int64_t workspace_bytes,
                                       gk_stream stream);

/* Sends `bytes` bytes at `buf` from rank `root` into every rank's `buf` (collective), on the handle's
 * communication stream, ordered after what `stream` holds so far; `stream` then waits for it.  What
 * "A broadcast once" means for callers that keep A resident over many products. */
GK_API gk_status gk_mgpu_broadcast(gk_handle h, void* buf, int64_t bytes, int32_t root, gk_stream stream);

/* Times of the phases of one gk_mgpu_gemm_colshard_host call, in milliseconds (device clocks). */
typedef struct gk_mgpu_times {
  float upload_ms;      /* first to last host-to-device copy of this rank (its pieces of A, its B)  */
  float collective_ms;  /* sum of the all-gathers that assemble A                                   */
  float compute_ms;     /* sum of the GEMM kernels of this rank                                     */
  float download_ms;    /* first to last device-to-host copy of this rank's D                       */
  float total_ms;       /* first upload to last download                                            */
  int32_t chunks;       /* row chunks A was cut into                                                */
  int32_t reserved;
  int64_t h2d_bytes, d2h_bytes; /* bytes this rank moved over PCIe                                  */
} gk_mgpu_times;

/* The same with operands and result in HOST memory (collective).  a_host points at the whole A in
 * this rank's host memory, but each rank reads — and sends over its own PCIe link — only 1/world of
 * it; NCCL all-gathers assemble A in every GPU's memory over NVLink, chunk by chunk, while this
 * rank's block of B goes up, and each row chunk of D is multiplied and sent back as soon as its
 * chunk of A is complete.  b_host, c_host, d_host are this rank's column blocks.  Needs K (or, for a
 * transposed A, M) divisible by world; real products only.  Returns when d_host is complete.
 * times may be NULL. */
GK_API gk_status gk_mgpu_gemm_colshard_host(gk_handle h, const gk_gemm_desc* desc, const void* a_host,
                                            const void* b_host, const void* c_host, void* d_host,
                                            const gk_epilogue_desc* epi, gk_stream stream, gk_mgpu_times* times);

/* How gk_mgpu_gemm_colshard_host would cut A for this descriptor and world size: number of row chunks
 * and rows per chunk (the last may be shorter).  Host arithmetic only; needs no GPU and no handle. */
GK_API gk_status gk_mgpu_host_plan(const gk_gemm_desc* desc, int32_t world, int32_t* chunks, int64_t* rows_per_chunk);

#ifdef __cplusplus
}
#endif
#endif /* GEMMKERNELS_B200_H */
