/*
 * libxtc_cuda -- C ABI of the B200 (sm_100a) execution backend for XTC graphs.
 *
 * Every entry point has C linkage, takes plain pointers and sizes, returns an
 * int status (XTC_CUDA_OK == 0) and records a message readable through
 * xtc_cuda_last_error().  There is no CPU fallback: on a machine without a
 * CUDA device the compute entry points return XTC_CUDA_ERR_RUNTIME.
 *
 * Each declaration cites the piece of the reference (xtc-tools/xtc, paths
 * relative to that project) whose role it takes over.
 */
#ifndef XTC_CUDA_H_
#define XTC_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XTC_CUDA_ABI_VERSION 1

enum {
  XTC_CUDA_OK = 0,
  XTC_CUDA_ERR_INVALID = 1,        /* bad argument (shape, alignment, NULL, unknown step) */
  XTC_CUDA_ERR_RUNTIME = 2,        /* a CUDA runtime/driver call failed                     */
  XTC_CUDA_ERR_UNSUPPORTED = 3,    /* legal request the kernels do not cover                */
  XTC_CUDA_ERR_DEVICE_TIMEOUT = 4, /* a bounded in-kernel wait gave up (see device_status)  */
  XTC_CUDA_ERR_NOMEM = 5
};

/* ------------------------------------------------------------------------
 * Device, memory, streams.
 * Replaces src/xtc/runtimes/accelerator/gpu/GPUDevice.py:131-215 (mgpuMemAlloc,
 * mgpuMemFree, mgpuMemcpy, mgpuStreamCreate, mgpuStreamSynchronize) and the
 * aligned allocator src/xtc/csrcs/runtimes/host/alloc.c:9-38 (256-byte default
 * alignment, src/xtc/csrcs/runtimes/host/cndarray.c:16).
 * ---------------------------------------------------------------------- */
int xtc_cuda_abi_version(void);
int xtc_cuda_device_count(int* count);
int xtc_cuda_set_device(int device);
int xtc_cuda_get_device(int* device);
int xtc_cuda_device_name(int device, char* buf, size_t buf_len);
int xtc_cuda_malloc(void** ptr, size_t bytes);
int xtc_cuda_free(void* ptr);
int xtc_cuda_host_alloc(void** ptr, size_t bytes); /* pinned host memory */
int xtc_cuda_host_free(void* ptr);
int xtc_cuda_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
int xtc_cuda_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
int xtc_cuda_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int xtc_cuda_memset(void* dst, int byte_value, size_t bytes, void* stream);
int xtc_cuda_stream_create(void** stream);
int xtc_cuda_stream_destroy(void* stream);
int xtc_cuda_stream_synchronize(void* stream);
int xtc_cuda_device_synchronize(void);
/* Events order work between streams (record on one, wait on another) and let the
 * host wait for a point of a stream: what a host loop needs to overlap the copies
 * of neighbouring steps with their kernels.  The reference's device interface
 * stops at streams (mgpuStreamCreate / mgpuStreamSynchronize, same file). */
int xtc_cuda_event_create(void** event);
int xtc_cuda_event_destroy(void* event);
int xtc_cuda_event_record(void* event, void* stream);
int xtc_cuda_event_synchronize(void* event);
int xtc_cuda_stream_wait_event(void* stream, void* event);
/* Free and total device memory of the current device (cudaMemGetInfo).  The
 * reference's device interface has no such query
 * (src/xtc/runtimes/accelerator/gpu/GPUDevice.py:131-215); tests use it to show
 * that an entry point allocates nothing. */
int xtc_cuda_mem_info(size_t* free_bytes, size_t* total_bytes);
/* Synchronises the device, then reads and clears the status words that kernels
 * set when one of their bounded waits gives up (0 = none): the per-device word
 * of the regular entry points and the word of xtc_cuda_gemm_f32_3xtf32_noalloc.
 * Allocates nothing once the device has been used.  Error reporting in the
 * reference is the (results, code, message) tuple of
 * src/xtc/utils/evaluation.py:129-145. */
int xtc_cuda_device_status(int* status);
/* Self-test of the bounded waits: launches one CTA whose single waiting thread
 * waits on a barrier that nothing completes, gives up after limit_ms
 * (1..1000) exactly as the compute kernels do after their 2 s, records the
 * give-up code in the device status word and returns normally.  The next
 * xtc_cuda_device_status therefore reads a non-zero status and clears it.  No
 * counterpart in the reference (its kernels have no in-kernel waits). */
int xtc_cuda_selftest_bounded_wait(int limit_ms, void* stream);
const char* xtc_cuda_last_error(void);

/* ------------------------------------------------------------------------
 * Kernels.  All pointers are device pointers; tensors are float32, dense,
 * C-contiguous unless a leading dimension says otherwise.
 * ---------------------------------------------------------------------- */

enum {
  XTC_CUDA_GEMM_A_TRANSPOSED = 1, /* A is stored [K, M] row-major (a fused O.transpose) */
  XTC_CUDA_GEMM_B_TRANSPOSED = 2, /* B is stored [N, K] row-major (layout=[1,0])        */
  XTC_CUDA_FUSE_RELU = 4          /* out = max(out, relu_threshold) in the epilogue     */
};

enum {
  XTC_CUDA_PRECISION_TF32 = 0,   /* one TF32 tensor-core product, fp32 accumulate        */
  XTC_CUDA_PRECISION_3XTF32 = 1, /* hi/lo split, three products: ~fp32 accuracy          */
  XTC_CUDA_PRECISION_FP32_SIMT = 2 /* CUDA-core fp32 FMA (no tensor cores)               */
};

/* Kernel parameters a schedule maps onto (0 = let the library choose).  These
 * are what the Scheduler's tile / unroll / parallelize directives turn into:
 * the reference records the same directives in
 * src/xtc/backends/mlir/MlirNodeScheduler.py:84-170. */
typedef struct xtc_cuda_gemm_config {
  int32_t tile_m;    /* CTA tile rows     : 128, or 256 = one tile per CTA pair    */
  int32_t tile_n;    /* CTA tile columns  : 64, 128 or 256                        */
  int32_t tile_k;    /* K per pipeline stage: 32 or 64                            */
  int32_t stages;    /* shared-memory ring depth (0 = as many as fit)             */
  int32_t precision; /* XTC_CUDA_PRECISION_*                                      */
  int32_t epilogue;  /* 0 = default; 1 = direct global stores; 2 = TMA stores     */
  int32_t variant;   /* conv2d: 0 = auto; 1 = im2col fetch per filter tap;
                        2 = resident weights + halo tiles (stride 1 only);
                        3 = the same with two filter taps per MMA (at most 64
                        filters, filter rows of two taps or more);
                        4 = resident weights with a sliding input window: a run of
                        consecutive tiles per CTA, the input through a ring of
                        128-position chunks (stride 1, at most 128 filters, a halo
                        run of at most 256 positions);
                        5 = streamed weights beside halo tiles, for filter banks that
                        do not fit in shared memory: CTA pairs, 128 filters per work
                        item, a pipeline stage = one 32-channel halo slab + the
                        weights of every tap (stride 1, C and F multiples of 4, 2 to
                        32 taps, two such stages in shared memory; `stages` applies,
                        tile_k = 16 halves the slabs).
                        With nothing named the library takes it where the whole bank
                        does not fit one CTA and the layer has work for most pairs.
                        With the workspace xtc_cuda_conv2d_workspace_bytes asks for
                        (zeroed before its first use; the kernel leaves its flags zero)
                        large layers are dealt out to the CTA pairs in (work item,
                        channel slab) units instead of whole work items.
                        GEMM with tile_m = 256: 2 = store C without the L2
                        evict-first hint (the default hints it)                   */
  int32_t split_k;   /* GEMM: CTAs sharing one output tile along K; 0 or 1 = off unless
                        the whole config is zero, when the library decides.  2 to 8
                        pieces of a tile at most 128 columns wide, N a multiple of 4, C
                        16-byte aligned, all clusters resident at once: the pieces are
                        the CTAs of one thread-block cluster and are summed through
                        distributed shared memory, no workspace (variant = 1 opts out).
                        Any other split needs the workspace of
                        xtc_cuda_gemm_workspace_bytes, zeroed before its
                        first use (the kernel leaves its counters zero again).
                        conv2d (im2col kernels, tile_m = 128): 2 to 8 = the cluster
                        form under the same conditions, else the layer runs unsplit.
                        With tile_m = 256: 0 = when the last round of tiles would leave
                        CTA pairs idle, share the K blocks of the last tiles out evenly
                        (same workspace rule; without a workspace the tiles simply go
                        round-robin); 1 = never                                      */
} xtc_cuda_gemm_config;

/* C[M,N] = A[M,K] * B[K,N]  (+ optional relu).  Replaces the loop nest the
 * reference generates for O.matmul: linalg.fill(0) + linalg.matmul,
 * src/xtc/backends/mlir/MlirOps.py:189-270; semantics
 * src/xtc/graphs/xtc/operators.py:159-221 (np.dot) and, for the fused relu,
 * operators.py:224-249.  `workspace` is scratch for the 3xTF32 operand split
 * (size from xtc_cuda_gemm_workspace_bytes); it may be NULL for TF32. */
int xtc_cuda_gemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, int flags, float relu_threshold,
                      const xtc_cuda_gemm_config* cfg, void* workspace, size_t workspace_bytes,
                      void* stream);
int xtc_cuda_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int flags,
                                  const xtc_cuda_gemm_config* cfg, size_t* bytes);
/* The tile, K stage and split the library picks for a TF32 product of this shape when the
 * caller names nothing (16-byte aligned operands assumed; products of at most 8 rows run on the
 * matrix-vector kernel instead, which has no such parameters): a starting point for a search
 * over xtc_cuda_gemm_config, as the reference's strategies start from default_schedule
 * (src/xtc/search/strategies.py:95-98).  Host arithmetic plus cached device queries. */
int xtc_cuda_gemm_default_config(int64_t M, int64_t N, int64_t K, xtc_cuda_gemm_config* out);

/* xtc_cuda_gemm_f32 whose epilogue also writes every output tile to the same
 * position of n_extra (<= 7) further buffers with the pitch ldc: the copies of C
 * held by the other GPUs of the box, mapped into this process with
 * xtc_cuda_ipc_import.  This fuses the all-gather of a row-sharded matmul into
 * the GEMM: rank r passes C = its own full-size buffer + r's row offset and the
 * peers' buffers + the same offset.  Stores to peers are plain 128-bit stores
 * over NVLink, issued (CTA-pair kernel, cfg.variant != 1) by four copier warps
 * per CTA that read finished tiles back from the local C, so the tensor pipeline
 * never waits for the link, or (cfg.variant = 1, and the one-CTA kernel) by the
 * epilogue warps themselves; the caller orders them against readers on the other GPUs (a
 * stream-ordered collective or barrier after the call).  The reference has no
 * multi-GPU execution (its GPU runtime is pinned to device 0,
 * src/xtc/runtimes/accelerator/gpu/GPUDevice.py:95-97); this implements the
 * partitioning the benchmark configuration asks for. */
int xtc_cuda_gemm_f32_bcast(const float* A, const float* B, float* C, float* const* extra_dst,
                            int n_extra, int64_t M, int64_t N, int64_t K, int64_t lda,
                            int64_t ldb, int64_t ldc, int flags, float relu_threshold,
                            const xtc_cuda_gemm_config* cfg, void* workspace,
                            size_t workspace_bytes, void* stream);
/* The same fused all-gather through an NVLink multicast object (NVLS): every
 * rank's full-size C is bound to one multicast object, mcast_C is this rank's row
 * block seen through the multicast mapping (C is the same block through the
 * rank's own unicast mapping), and the copier warps issue ONE multimem.st per
 * 128-bit vector, which the NVSwitch writes into every bound GPU's memory (this
 * GPU's too), instead of one store per peer.  CTA-pair kernel only (tile_m = 256 or
 * 0), TF32 only.  Creating and binding the multicast object is the caller's job
 * (xtc_b200.dist uses torch's symmetric-memory allocator); every rank must unbind
 * before any rank exits.  Ordering against readers as for xtc_cuda_gemm_f32_bcast.
 * No reference counterpart (same remark). */
int xtc_cuda_gemm_f32_mcast(const float* A, const float* B, float* C, float* mcast_C, int64_t M,
                            int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int flags,
                            float relu_threshold, const xtc_cuda_gemm_config* cfg, void* workspace,
                            size_t workspace_bytes, void* stream);
/* Share a device allocation (from xtc_cuda_malloc) with the other processes of
 * the box: export fills a 64-byte handle to send them; import maps the peer's
 * allocation here; release unmaps it.  Same remark: no reference counterpart. */
int xtc_cuda_ipc_export(void* device_ptr, void* handle64);
int xtc_cuda_ipc_import(const void* handle64, void** device_ptr);
int xtc_cuda_ipc_release(void* device_ptr);

/* The library all-gather of a row-sharded matmul, for hosts that keep the GEMM
 * and the exchange apart instead of using xtc_cuda_gemm_f32_bcast: NCCL, one
 * process per GPU.  Rank 0 fills a 128-byte identifier with
 * xtc_cuda_comm_unique_id and hands it to the other ranks by the host's own
 * channel; every rank then calls xtc_cuda_comm_init (collective; the calling
 * thread's current device is the rank's GPU).  xtc_cuda_allgather_rows works in
 * place on a buffer of world x rows_per_rank rows of row_bytes bytes that every
 * rank holds: rank r owns rows [r * rows_per_rank, (r + 1) * rows_per_rank), and
 * the call delivers rows [row_lo, row_hi) OF EVERY RANK'S BLOCK (block-relative
 * numbers) to all ranks, stream-ordered.  The whole block (0, rows_per_rank) is
 * one ncclAllGather; a sub-range, which lets the host overlap the exchange of
 * finished row chunks with the GEMM of the next, is one grouped broadcast per
 * owner.  NCCL is loaded with dlopen at the first call (libnccl.so.2; the copy
 * already in the process, if any): without it these calls return
 * XTC_CUDA_ERR_UNSUPPORTED and nothing else in the library is affected.
 * The reference has no multi-GPU execution (GPUDevice.py:95-97, as above). */
typedef struct xtc_cuda_comm xtc_cuda_comm;
int xtc_cuda_comm_unique_id(void* id128);
int xtc_cuda_comm_init(xtc_cuda_comm** comm, int world, int rank, const void* id128);
int xtc_cuda_allgather_rows(xtc_cuda_comm* comm, void* c, int64_t rows_per_rank,
                            int64_t row_bytes, int64_t row_lo, int64_t row_hi, void* stream);
int xtc_cuda_comm_destroy(xtc_cuda_comm* comm);

/* A stream-ordered barrier between up to 8 GPUs of a box (one process each) that costs one
 * warp: every rank holds an array of 8 ints (from xtc_cuda_malloc, zeroed once) and maps the
 * peers' arrays with xtc_cuda_ipc_import.  The call stores `epoch` (increasing by one per
 * barrier) into slot my_rank of every peer's array, after everything `stream` did before,
 * peer-to-peer copies included, and makes `stream` wait until the local slots of all
 * peer_ranks have reached it (a bounded wait, about 2 s: on giving up the kernel records
 * XTC_CUDA_ERR_DEVICE_TIMEOUT's status and returns).  What follows on `stream` may read what the
 * peers wrote into this GPU's memory before their barrier.  No reference counterpart (same
 * remark as the other multi-GPU calls). */
int xtc_cuda_peer_barrier(int* local_flags, int* const* peer_flags, const int* peer_ranks,
                          int n_peers, int my_rank, int epoch, void* stream);

/* The 3xTF32 GEMM for callers that must not allocate device memory.  This entry
 * point has no counterpart in the reference.
 *
 * Who needs it: code that runs after the application has handed the whole GPU
 * to its own memory pool (a cudaMalloc made now would fail, or carve memory out
 * from under that pool), and code on a latency-critical path where the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  Such
 * a caller cannot provide the workspace xtc_cuda_gemm_f32 wants for the operand
 * split either, so here the split lives in a fixed 32 MiB array that is part of
 * the library image: every GPU that loads the library holds those 32 MiB until
 * the process exits.
 *
 * C[M,N] = A * B (+ relu), A, B and C dense (lda = K or M, ldb = N or K, ldc = N),
 * 16-byte aligned, row lengths multiples of 4 (all three are checked); flags as
 * for xtc_cuda_gemm_f32.
 * Limit: 2 * (round256(4*M*K) + round256(4*K*N)) <= 32 MiB, i.e. about
 * M*K + K*N <= 4 Mi elements; larger problems are refused with
 * XTC_CUDA_ERR_INVALID and a message that states both sizes (the element
 * counts are bounded before any byte count is formed, so no extent up to 2^31
 * can wrap past the check).
 *
 * The call makes no cudaMalloc / cudaFree and calls no allocating library
 * routine.  The first call on each device looks up the device address of the
 * built-in array (cudaGetSymbolAddress, with that device current); make that
 * first call before starting any stream capture.  All calls share the one
 * array: two calls whose kernels can overlap on the GPU (different streams, no
 * ordering between them) race on it; calls on one stream are safe.  The array
 * keeps the previous call's contents, which is harmless: every byte the GEMM
 * reads is rewritten by the split kernels of the same call first.  A bounded
 * wait that gives up inside this variant is recorded in a second word of the
 * library image; xtc_cuda_device_status reads and clears it together with the
 * regular status word (with two cudaMemcpy calls on the cached address, no
 * allocation). */
int xtc_cuda_gemm_f32_3xtf32_noalloc(const float* A, const float* B, float* C, int64_t M,
                                     int64_t N, int64_t K, int flags, float relu_threshold,
                                     void* stream);

/* Y[B,OH,OW,F] = conv2d(pad(X[B,H,W,C]), Wt[R,S,C,F]) (+ optional relu), NHWC x
 * HWIO, stride (stride_h, stride_w).  pad_* is a zero padding of H and W fused
 * into the operand fetch (the reference needs a separate O.pad node for it).
 * Replaces the 7-D linalg.generic of src/xtc/backends/mlir/MlirOps.py:331-420;
 * semantics src/xtc/graphs/xtc/operators.py:252-347 and, for the fused pad,
 * operators.py:350-433 with constant_value == 0.
 * `workspace` (size from xtc_cuda_conv2d_workspace_bytes for the same shape and
 * cfg; zeroed before its first use, may be reused by later calls) serves
 * three things: the partial sums of a split of K the library chose, the
 * partial sums and flags of the streamed-weights kernel's balanced form
 * (cfg.variant 5, or the library's own choice of it), and, for thin
 * inputs (C not a multiple of 4, or at most 8 channels where the
 * resident-weights kernel does not apply, with nothing named in cfg), the
 * packed form of the layer: the S*C values a filter row needs per output
 * position are contiguous in NHWC, so they are gathered into
 * P[B, H, OW, ceil4(S*C)] and the layer runs as an R x 1 convolution on the
 * tensor cores (K = 7 x 32 for a 7x7 filter on 3 channels, where one K block
 * per tap would be 49 x 32).  Without the workspace the call still succeeds:
 * unsplit, and thin inputs with C % 4 != 0 on a CUDA-core kernel. */
int xtc_cuda_conv2d_nhwc_f32(const float* X, const float* Wt, float* Y, int64_t B, int64_t H,
                             int64_t W, int64_t C, int64_t R, int64_t S, int64_t F, int stride_h,
                             int stride_w, int pad_top, int pad_bottom, int pad_left,
                             int pad_right, int flags, float relu_threshold,
                             const xtc_cuda_gemm_config* cfg, void* workspace,
                             size_t workspace_bytes, void* stream);
int xtc_cuda_conv2d_workspace_bytes(int64_t B, int64_t H, int64_t W, int64_t C, int64_t R,
                                    int64_t S, int64_t F, int stride_h, int stride_w, int pad_top,
                                    int pad_bottom, int pad_left, int pad_right,
                                    const xtc_cuda_gemm_config* cfg, size_t* bytes);

#define XTC_CUDA_MAX_DIMS 6

/* Y = transpose(X, axes) for ndim <= XTC_CUDA_MAX_DIMS; bit-exact.  Replaces
 * src/xtc/graphs/xtc/operators.py:757-787 (np.transpose); the only compiled
 * lowering in the reference is TVM's, src/xtc/backends/tvm/TVMOps.py:688-778. */
int xtc_cuda_transpose_f32(const float* X, float* Y, int ndim, const int64_t* shape,
                           const int32_t* axes, void* stream);

/* Y = pad(X) with per-axis (lo, hi) widths and a constant; negative widths crop
 * (O.unpad).  Bit-exact.  Replaces linalg.fill + linalg.copy into a subview,
 * src/xtc/backends/mlir/MlirOps.py:718-735 (pad), :778-887 (pad2d / unpad);
 * semantics src/xtc/graphs/xtc/operators.py:413-433 (np.pad, mode="constant"). */
int xtc_cuda_pad_f32(const float* X, float* Y, int ndim, const int64_t* shape, const int64_t* lo,
                     const int64_t* hi, float value, void* stream);

/* Y = max(X, threshold) elementwise.  Replaces src/xtc/backends/mlir/MlirOps.py:
 * 459-557; semantics src/xtc/graphs/xtc/operators.py:224-249. */
int xtc_cuda_relu_f32(const float* X, float* Y, int64_t n, float threshold, void* stream);

/* hi = round_to_tf32(X), lo = X - hi: the operand split of the 3xTF32 mode. */
int xtc_cuda_split_tf32(const float* X, float* hi, float* lo, int64_t n, void* stream);

/* ------------------------------------------------------------------------
 * Plans: a lowered graph = a list of steps over numbered buffer slots.
 * Slots [0, n_inputs) are the graph inputs, [n_inputs, n_inputs + n_outputs)
 * the graph outputs, in the order of the reference's payload signature
 * `void <graph.name>(void* in0.., void* out0..)` produced by
 * src/xtc/backends/mlir/MlirGraphBackend.py:144-148; the remaining slots are
 * intermediates the plan owns (the reference puts them in memref.alloca,
 * MlirGraphBackend.py:96-103).
 * ---------------------------------------------------------------------- */
enum {
  XTC_CUDA_STEP_GEMM = 1,
  XTC_CUDA_STEP_CONV2D = 2,
  XTC_CUDA_STEP_TRANSPOSE = 3,
  XTC_CUDA_STEP_PAD = 4,
  XTC_CUDA_STEP_RELU = 5,
  XTC_CUDA_STEP_COPY = 6
};

typedef struct xtc_cuda_step {
  int32_t kind;
  int32_t in0, in1, out; /* buffer slots; in1 = -1 when unused */
  int32_t flags;         /* XTC_CUDA_GEMM_* | XTC_CUDA_FUSE_RELU */
  int32_t ndim;          /* transpose / pad: rank of the input                      */
  float relu_threshold;
  float pad_value;
  /* GEMM: {M, N, K, lda, ldb, ldc}; CONV2D: {B, H, W, C, R, S}; TRANSPOSE / PAD:
   * input shape; RELU / COPY: {numel}. */
  int64_t dims[XTC_CUDA_MAX_DIMS];
  /* CONV2D: {F, stride_h, stride_w}; TRANSPOSE: axes; PAD: lo widths. */
  int64_t aux0[XTC_CUDA_MAX_DIMS];
  /* CONV2D: {pad_top, pad_bottom, pad_left, pad_right}; PAD: hi widths. */
  int64_t aux1[XTC_CUDA_MAX_DIMS];
  xtc_cuda_gemm_config cfg;
} xtc_cuda_step;

typedef struct xtc_cuda_plan xtc_cuda_plan;

/* Workspace of one step as xtc_cuda_plan_create allocates it: its size and how
 * many leading bytes the plan clears once (split-K tile counters, one int per
 * output tile whatever their number, and split-tail flags must read zero at the
 * first launch; the kernels leave them zero again).  A caller that drives
 * xtc_cuda_gemm_f32 / xtc_cuda_conv2d_nhwc_f32 directly clears the same bytes
 * of the workspace it passes.  Needs no device.  The reference keeps no such
 * scratch (its split reductions are sequential loops,
 * src/xtc/backends/mlir/MlirNodeScheduler.py:139-160). */
int xtc_cuda_step_workspace_bytes(const struct xtc_cuda_step* step, size_t* total_bytes,
                                  size_t* zeroed_bytes);

/* slot_bytes[n_slots] gives every slot's size.  The plan allocates the
 * intermediates and any kernel workspace on the current device.  Plays the role
 * of Compiler.compile -> Module, src/xtc/backends/mlir/MlirCompiler.py:67-110. */
int xtc_cuda_plan_create(xtc_cuda_plan** plan, const xtc_cuda_step* steps, int n_steps,
                         int n_inputs, int n_outputs, int n_slots, const size_t* slot_bytes);
int xtc_cuda_plan_destroy(xtc_cuda_plan* plan);
/* io[n_inputs + n_outputs]: device pointers.  Asynchronous on `stream`.  The
 * launches of a run are captured into a CUDA graph the first time a given set of
 * io pointers is seen and replayed with one graph launch afterwards (the
 * reference pays a host call per node instead, evaluate_perf.c:99-103). */
int xtc_cuda_plan_run(xtc_cuda_plan* plan, void* const* io, void* stream);
/* `count` runs back to back on `stream`, issued from one host call: run j uses the
 * pointer set io_sets[((first + j) % n_sets) * (n_inputs + n_outputs) ...].  For a
 * caller whose step is shorter than a host call from its own language (a few
 * microseconds from Python): the reference's timing loop issues its `number` calls
 * from C for the same reason (src/xtc/csrcs/runtimes/host/evaluate_perf.c:99-103).
 * Several sets let the caller rotate buffers so that no run finds its inputs in L2. */
int xtc_cuda_plan_run_sets(xtc_cuda_plan* plan, void* const* io_sets, int n_sets, int first,
                           int count, void* stream);
/* enabled = 0 turns graph replay off (every run issues its launches directly);
 * 1 turns it on.  Default: on for plans of two or more launches, off for a plan
 * that is a single kernel (its runs then overlap back to back through programmatic
 * dependent launch, which graph launches do not). */
int xtc_cuda_plan_set_graph_mode(xtc_cuda_plan* plan, int enabled);
/* io: HOST pointers.  Copies inputs to the device, runs, copies outputs back,
 * synchronises: the call the per-module payload makes, equivalent to calling
 * the reference payload with host memory (src/xtc/utils/cfunc.py:89-110). */
int xtc_cuda_plan_run_host(xtc_cuda_plan* plan, void* const* io);

/* Pipelined form of xtc_cuda_plan_run_host for a caller that runs the module on
 * a sequence of host batches (the evaluator's repeat loop,
 * src/xtc/runtimes/host/evaluator.py:109-141, with host arrays): up to `depth`
 * runs are in flight, the input copy of run i+1 and the output copy of run i-1
 * overlapping the kernels of run i on three streams.  Host buffers should be
 * page-locked (xtc_cuda_host_alloc) for the copies to overlap.
 * submit() returns once the run is queued; it blocks only while `depth` earlier
 * runs are still undelivered.  The output buffers of a run are valid after a
 * later submit() reused its slot or after wait(), which also reports a device
 * status error.  depth in [1, 8]; the pipeline owns depth sets of device io
 * buffers.  The plan must outlive the pipeline. */
typedef struct xtc_cuda_pipeline xtc_cuda_pipeline;
int xtc_cuda_pipeline_create(xtc_cuda_pipeline** pipe, xtc_cuda_plan* plan, int depth);
int xtc_cuda_pipeline_submit(xtc_cuda_pipeline* pipe, void* const* io);
int xtc_cuda_pipeline_wait(xtc_cuda_pipeline* pipe);
int xtc_cuda_pipeline_destroy(xtc_cuda_pipeline* pipe);

/* CUDA-event twin of evaluate_perf, src/xtc/csrcs/runtimes/host/
 * evaluate_perf.c:63-125: one untimed warm-up call when number > 0, then
 * `repeat` measurements of `number` back-to-back runs, doubling the count until
 * a measurement lasts min_repeat_ms; results[r] = seconds per run. */
int xtc_cuda_evaluate(xtc_cuda_plan* plan, void* const* io, int repeat, int number,
                      int min_repeat_ms, double* results);
/* Number of steps (kernel-level operations) of a plan. */
int xtc_cuda_plan_step_count(const xtc_cuda_plan* plan, int* n_steps);

/* Peak fused-multiply-add rate of the tensor pipe for "float32" (TF32 inputs),
 * in FMA/s: same unit as evaluate_flops, src/xtc/csrcs/runtimes/host/
 * evaluate_flops.c:461-495, so ops_count / peak keeps its meaning. */
int xtc_cuda_peak_fma(const char* dtype, double* fma_per_second);
/* The same probe for one MMA instruction shape (rows 64 or 128, columns 64, 128 or
 * 256, K = 8, operands resident in shared memory): the rate the tensor pipe and the
 * shared-memory operand reads sustain for that shape, in FMA/s.  What a search
 * space is pruned with: a 64-row instruction occupies the pipe as long as a
 * 128-row one, so a 64-row tile halves the rate.  evaluate_flops in the reference
 * probes one shape per dtype only. */
int xtc_cuda_mma_rate(int tile_m, int tile_n, double* fma_per_second);

#ifdef __cplusplus
}
#endif
#endif /* XTC_CUDA_H_ */
