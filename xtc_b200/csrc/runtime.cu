// Device runtime behind the C ABI: error strings, device/memory/stream calls,
// tensor-map encoding, plans (lowered graphs), the CUDA-event evaluation loop
// and the tensor-pipe peak probe.
#include <stdarg.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace xtc {

// ---------------------------------------------------------------------------
// error string (thread local)
// ---------------------------------------------------------------------------
static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_error; }

// ---------------------------------------------------------------------------
// per-device state
// ---------------------------------------------------------------------------
static constexpr int MAX_DEVICES = 64;
static std::mutex g_mutex;
static int* g_status[MAX_DEVICES] = {};
static int g_sms[MAX_DEVICES] = {};

int* device_status_word(int dev) {
  if (dev < 0 || dev >= MAX_DEVICES) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, 256) != cudaSuccess) return nullptr;
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count(int dev) {
  if (dev < 0 || dev >= MAX_DEVICES) return 1;
  if (g_sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 1;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

static void* driver_entry(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
  if (q != cudaDriverEntryPointSuccess) return nullptr;
  return fn;
}
encode_tiled_fn get_encode_tiled() {
  static encode_tiled_fn fn = reinterpret_cast<encode_tiled_fn>(driver_entry("cuTensorMapEncodeTiled"));
  return fn;
}
encode_im2col_fn get_encode_im2col() {
  static encode_im2col_fn fn = reinterpret_cast<encode_im2col_fn>(driver_entry("cuTensorMapEncodeIm2col"));
  return fn;
}

bool make_tmap_4d_plain(CUtensorMap* map, const void* base, const uint64_t dims[4],
                        const uint64_t strides[3], const uint32_t box[4]) {
  encode_tiled_fn enc = get_encode_tiled();
  if (!enc) return false;
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t st[3] = {strides[0] * sizeof(float), strides[1] * sizeof(float), strides[2] * sizeof(float)};
  cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), d, st, b, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  encode_tiled_fn enc = get_encode_tiled();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return XTC_CUDA_ERR_RUNTIME;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * sizeof(float)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d): base=%p rows=%llu cols=%llu ld=%llu box=%ux%u",
              static_cast<int>(r), base, (unsigned long long)rows, (unsigned long long)cols,
              (unsigned long long)ld, box_cols, box_rows);
    return XTC_CUDA_ERR_INVALID;
  }
  return XTC_CUDA_OK;
}

}  // namespace xtc

using namespace xtc;

// ---------------------------------------------------------------------------
// device / memory / streams
// ---------------------------------------------------------------------------
extern "C" int xtc_cuda_abi_version(void) { return XTC_CUDA_ABI_VERSION; }
extern "C" const char* xtc_cuda_last_error(void) { return get_error(); }

extern "C" int xtc_cuda_device_count(int* count) {
  XTC_REQUIRE(count != nullptr, "device_count: NULL");
  *count = 0;
  XTC_CUDA_CHECK(cudaGetDeviceCount(count));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_set_device(int device) {
  XTC_CUDA_CHECK(cudaSetDevice(device));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_get_device(int* device) {
  XTC_REQUIRE(device != nullptr, "get_device: NULL");
  XTC_CUDA_CHECK(cudaGetDevice(device));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_device_name(int device, char* buf, size_t buf_len) {
  XTC_REQUIRE(buf && buf_len > 0, "device_name: NULL buffer");
  cudaDeviceProp prop;
  XTC_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
  snprintf(buf, buf_len, "%s", prop.name);
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_malloc(void** ptr, size_t bytes) {
  XTC_REQUIRE(ptr != nullptr, "malloc: NULL");
  *ptr = nullptr;
  if (bytes == 0) bytes = 256;
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    set_error("malloc: out of device memory (%zu bytes)", bytes);
    return XTC_CUDA_ERR_NOMEM;
  }
  XTC_CUDA_CHECK(e);
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_free(void* ptr) {
  if (ptr) XTC_CUDA_CHECK(cudaFree(ptr));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_host_alloc(void** ptr, size_t bytes) {
  XTC_REQUIRE(ptr != nullptr, "host_alloc: NULL");
  *ptr = nullptr;
  if (bytes == 0) bytes = 256;
  XTC_CUDA_CHECK(cudaMallocHost(ptr, bytes));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_host_free(void* ptr) {
  if (ptr) XTC_CUDA_CHECK(cudaFreeHost(ptr));
  return XTC_CUDA_OK;
}
static int copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, void* stream) {
  if (bytes == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(dst && src, "memcpy: NULL pointer");
  XTC_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, kind, static_cast<cudaStream_t>(stream)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
  return copy(dst, src, bytes, cudaMemcpyHostToDevice, stream);
}
extern "C" int xtc_cuda_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
  return copy(dst, src, bytes, cudaMemcpyDeviceToHost, stream);
}
extern "C" int xtc_cuda_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
  return copy(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
}
extern "C" int xtc_cuda_memset(void* dst, int byte_value, size_t bytes, void* stream) {
  if (bytes == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(dst != nullptr, "memset: NULL pointer");
  XTC_CUDA_CHECK(cudaMemsetAsync(dst, byte_value, bytes, static_cast<cudaStream_t>(stream)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_stream_create(void** stream) {
  XTC_REQUIRE(stream != nullptr, "stream_create: NULL");
  cudaStream_t s;
  XTC_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_stream_destroy(void* stream) {
  if (stream) XTC_CUDA_CHECK(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_stream_synchronize(void* stream) {
  XTC_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_event_create(void** event) {
  XTC_REQUIRE(event != nullptr, "event_create: NULL");
  cudaEvent_t e;
  XTC_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  *event = e;
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_event_destroy(void* event) {
  if (event) XTC_CUDA_CHECK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_event_record(void* event, void* stream) {
  XTC_REQUIRE(event != nullptr, "event_record: NULL event");
  XTC_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_event_synchronize(void* event) {
  XTC_REQUIRE(event != nullptr, "event_synchronize: NULL event");
  XTC_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_stream_wait_event(void* stream, void* event) {
  XTC_REQUIRE(event != nullptr, "stream_wait_event: NULL event");
  XTC_CUDA_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_device_synchronize(void) {
  XTC_CUDA_CHECK(cudaDeviceSynchronize());
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_device_status(int* status) {
  XTC_REQUIRE(status != nullptr, "device_status: NULL");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  int* word = device_status_word(dev);
  XTC_REQUIRE(word != nullptr, "device_status: status word unavailable");
  XTC_CUDA_CHECK(cudaDeviceSynchronize());
  XTC_CUDA_CHECK(cudaMemcpy(status, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) XTC_CUDA_CHECK(cudaMemset(word, 0, sizeof(int)));
  // the allocation-free GEMM reports into a word of its own (it may not use the
  // allocated one): read and clear that too
  int noalloc = 0;
  int rc = noalloc_status_fetch_and_clear(dev, &noalloc);
  if (rc != XTC_CUDA_OK) return rc;
  if (*status == 0) *status = noalloc;
  if (*status != 0) set_error("a kernel's bounded wait gave up (device status %d)", *status);
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_mem_info(size_t* free_bytes, size_t* total_bytes) {
  XTC_REQUIRE(free_bytes && total_bytes, "mem_info: NULL");
  XTC_CUDA_CHECK(cudaMemGetInfo(free_bytes, total_bytes));
  return XTC_CUDA_OK;
}

// ---------------------------------------------------------------------------
// self-test of the bounded wait
// ---------------------------------------------------------------------------
namespace xtc {
// One thread waits, for at most limit_ns, on a barrier phase that nothing completes,
// records the give-up code exactly as the compute kernels do and returns.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    dev::mbar_init(&bar, 1);
    dev::fence_barrier_init();
    if (!dev::mbar_wait_limit(&bar, 0, limit_ns)) atomicCAS(status, 0, dev::STATUS_WAIT_TIMEOUT_LOAD);
  }
}
}  // namespace xtc

extern "C" int xtc_cuda_selftest_bounded_wait(int limit_ms, void* stream) {
  XTC_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, "selftest_bounded_wait: limit %d ms not in [1, 1000]", limit_ms);
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  int* word = device_status_word(dev);
  XTC_REQUIRE(word != nullptr, "selftest_bounded_wait: status word unavailable");
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint64_t>(limit_ms) * 1000000ull, word);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}

// ---------------------------------------------------------------------------
// plans
// ---------------------------------------------------------------------------
struct xtc_cuda_plan {
  std::vector<xtc_cuda_step> steps;
  int n_inputs = 0, n_outputs = 0;
  std::vector<size_t> slot_bytes;
  std::vector<void*> owned;       // intermediates, index = slot - n_io (nullptr for io slots)
  std::vector<void*> workspace;   // per step
  std::vector<size_t> workspace_bytes;
  std::vector<void*> staging;     // device copies of io slots for run_host (lazy)
  int device = 0;
  // CUDA-graph replay: the launches of one run, captured once per distinct set of
  // io pointers and replayed with a single cudaGraphLaunch afterwards.
  struct Replay {
    std::vector<void*> io;
    cudaGraphExec_t exec;
  };
  std::vector<Replay> replays;
  int graph_mode = 1;
  cudaStream_t capture_stream = nullptr;
};

static int step_workspace(const xtc_cuda_step& s, size_t* bytes) {
  *bytes = 0;
  if (s.kind == XTC_CUDA_STEP_GEMM)
    return xtc_cuda_gemm_workspace_bytes(s.dims[0], s.dims[1], s.dims[2], s.flags, &s.cfg, bytes);
  if (s.kind == XTC_CUDA_STEP_CONV2D)
    return xtc_cuda_conv2d_workspace_bytes(s.dims[0], s.dims[1], s.dims[2], s.dims[3], s.dims[4],
                                           s.dims[5], s.aux0[0], (int)s.aux0[1], (int)s.aux0[2],
                                           (int)s.aux1[0], (int)s.aux1[1], (int)s.aux1[2],
                                           (int)s.aux1[3], &s.cfg, bytes);
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_step_workspace_bytes(const xtc_cuda_step* step, size_t* total_bytes,
                                             size_t* zeroed_bytes) {
  XTC_REQUIRE(step && total_bytes && zeroed_bytes, "step_workspace_bytes: NULL argument");
  *zeroed_bytes = 0;
  int rc = step_workspace(*step, total_bytes);
  if (rc != XTC_CUDA_OK) return rc;
  // The split-K tile counters (one int per output tile, however many tiles there are) and
  // the split-tail flags sit at the start of the workspace and must read zero at the first
  // launch; the partial tiles behind them are written before they are read.  The whole
  // workspace is cleared: it is done once per plan.  The 3xTF32 operand split is rewritten
  // by every run before it is read and needs no clearing.
  const bool split3 = step->kind == XTC_CUDA_STEP_GEMM && step->cfg.precision == XTC_CUDA_PRECISION_3XTF32;
  *zeroed_bytes = split3 ? 0 : *total_bytes;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_create(xtc_cuda_plan** plan, const xtc_cuda_step* steps, int n_steps,
                                    int n_inputs, int n_outputs, int n_slots,
                                    const size_t* slot_bytes) {
  XTC_REQUIRE(plan != nullptr, "plan_create: NULL plan");
  *plan = nullptr;
  XTC_REQUIRE(steps && n_steps > 0, "plan_create: no steps");
  XTC_REQUIRE(n_inputs >= 0 && n_outputs > 0 && n_slots >= n_inputs + n_outputs && slot_bytes,
              "plan_create: bad slot counts (%d inputs, %d outputs, %d slots)", n_inputs,
              n_outputs, n_slots);
  for (int i = 0; i < n_steps; ++i) {
    const xtc_cuda_step& s = steps[i];
    XTC_REQUIRE(s.kind >= XTC_CUDA_STEP_GEMM && s.kind <= XTC_CUDA_STEP_COPY,
                "plan_create: step %d has unknown kind %d", i, s.kind);
    XTC_REQUIRE(s.in0 >= 0 && s.in0 < n_slots && s.out >= 0 && s.out < n_slots &&
                    s.in1 >= -1 && s.in1 < n_slots,
                "plan_create: step %d references a slot out of range", i);
    XTC_REQUIRE(s.out >= n_inputs, "plan_create: step %d writes a graph input", i);
  }
  xtc_cuda_plan* p = new xtc_cuda_plan();
  p->steps.assign(steps, steps + n_steps);
  p->n_inputs = n_inputs;
  p->n_outputs = n_outputs;
  p->slot_bytes.assign(slot_bytes, slot_bytes + n_slots);
  p->owned.assign(n_slots, nullptr);
  p->workspace.assign(n_steps, nullptr);
  p->workspace_bytes.assign(n_steps, 0);
  p->staging.assign(n_inputs + n_outputs, nullptr);
  // Graph replay pays for plans of several launches.  A plan that is one kernel is
  // launched directly: back-to-back runs then overlap through programmatic dependent
  // launch (measured: 512x1024x256 matmul 12.5 -> 10.3 us per run, 4096^3 190 -> 187 us).
  int launches = 0;
  for (int i = 0; i < n_steps; ++i)
    launches += (steps[i].kind == XTC_CUDA_STEP_GEMM && steps[i].cfg.precision == XTC_CUDA_PRECISION_3XTF32) ? 3 : 1;
  p->graph_mode = launches >= 2 ? 1 : 0;
  int rc = XTC_CUDA_OK;
  if (cudaGetDevice(&p->device) != cudaSuccess) rc = XTC_CUDA_ERR_RUNTIME;
  for (int s = n_inputs + n_outputs; s < n_slots && rc == XTC_CUDA_OK; ++s)
    rc = xtc_cuda_malloc(&p->owned[s], p->slot_bytes[s]);
  for (int i = 0; i < n_steps && rc == XTC_CUDA_OK; ++i) {
    size_t need = 0, zeroed = 0;
    rc = xtc_cuda_step_workspace_bytes(&p->steps[i], &need, &zeroed);
    if (rc == XTC_CUDA_OK && need > 0) {
      rc = xtc_cuda_malloc(&p->workspace[i], need);
      p->workspace_bytes[i] = need;
      if (rc == XTC_CUDA_OK && zeroed > 0 && cudaMemset(p->workspace[i], 0, zeroed) != cudaSuccess)
        rc = XTC_CUDA_ERR_RUNTIME;
    }
  }
  if (rc != XTC_CUDA_OK) {
    xtc_cuda_plan_destroy(p);
    return rc;
  }
  *plan = p;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_destroy(xtc_cuda_plan* plan) {
  if (!plan) return XTC_CUDA_OK;
  for (void* q : plan->owned) if (q) cudaFree(q);
  for (void* q : plan->workspace) if (q) cudaFree(q);
  for (void* q : plan->staging) if (q) cudaFree(q);
  for (auto& r : plan->replays) cudaGraphExecDestroy(r.exec);
  if (plan->capture_stream) cudaStreamDestroy(plan->capture_stream);
  delete plan;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_step_count(const xtc_cuda_plan* plan, int* n_steps) {
  XTC_REQUIRE(plan && n_steps, "plan_step_count: NULL");
  *n_steps = static_cast<int>(plan->steps.size());
  return XTC_CUDA_OK;
}

static int plan_launch(xtc_cuda_plan* plan, void* const* io, void* stream) {
  const int n_io = plan->n_inputs + plan->n_outputs;
  auto slot = [&](int s) -> void* { return s < n_io ? io[s] : plan->owned[s]; };
  for (size_t i = 0; i < plan->steps.size(); ++i) {
    const xtc_cuda_step& s = plan->steps[i];
    const float* in0 = static_cast<const float*>(slot(s.in0));
    const float* in1 = s.in1 >= 0 ? static_cast<const float*>(slot(s.in1)) : nullptr;
    float* out = static_cast<float*>(slot(s.out));
    int rc = XTC_CUDA_OK;
    switch (s.kind) {
      case XTC_CUDA_STEP_GEMM:
        rc = xtc_cuda_gemm_f32(in0, in1, out, s.dims[0], s.dims[1], s.dims[2], s.dims[3],
                               s.dims[4], s.dims[5], s.flags, s.relu_threshold, &s.cfg,
                               plan->workspace[i], plan->workspace_bytes[i], stream);
        break;
      case XTC_CUDA_STEP_CONV2D:
        rc = xtc_cuda_conv2d_nhwc_f32(in0, in1, out, s.dims[0], s.dims[1], s.dims[2], s.dims[3],
                                      s.dims[4], s.dims[5], s.aux0[0], (int)s.aux0[1],
                                      (int)s.aux0[2], (int)s.aux1[0], (int)s.aux1[1],
                                      (int)s.aux1[2], (int)s.aux1[3], s.flags, s.relu_threshold,
                                      &s.cfg, plan->workspace[i], plan->workspace_bytes[i], stream);
        break;
      case XTC_CUDA_STEP_TRANSPOSE: {
        int32_t axes[XTC_CUDA_MAX_DIMS];
        for (int d = 0; d < s.ndim; ++d) axes[d] = static_cast<int32_t>(s.aux0[d]);
        rc = xtc_cuda_transpose_f32(in0, out, s.ndim, s.dims, axes, stream);
        break;
      }
      case XTC_CUDA_STEP_PAD:
        rc = xtc_cuda_pad_f32(in0, out, s.ndim, s.dims, s.aux0, s.aux1, s.pad_value, stream);
        break;
      case XTC_CUDA_STEP_RELU:
        rc = xtc_cuda_relu_f32(in0, out, s.dims[0], s.relu_threshold, stream);
        break;
      case XTC_CUDA_STEP_COPY:
        rc = xtc_cuda_memcpy_d2d(out, in0, static_cast<size_t>(s.dims[0]) * 4, stream);
        break;
      default:
        set_error("plan_run: unknown step kind %d", s.kind);
        rc = XTC_CUDA_ERR_INVALID;
    }
    if (rc != XTC_CUDA_OK) return rc;
  }
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_set_graph_mode(xtc_cuda_plan* plan, int enabled) {
  XTC_REQUIRE(plan != nullptr, "plan_set_graph_mode: NULL plan");
  plan->graph_mode = enabled ? 1 : 0;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_run(xtc_cuda_plan* plan, void* const* io, void* stream) {
  XTC_REQUIRE(plan && io, "plan_run: NULL plan or io");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!plan->graph_mode) return plan_launch(plan, io, stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return plan_launch(plan, io, stream);  // the caller is capturing: just record the launches
  }
  const size_t n_io = static_cast<size_t>(plan->n_inputs + plan->n_outputs);
  for (auto& r : plan->replays) {
    if (memcmp(r.io.data(), io, n_io * sizeof(void*)) == 0) {
      XTC_CUDA_CHECK(cudaGraphLaunch(r.exec, s));
      return XTC_CUDA_OK;
    }
  }
  // First run on these buffers: capture the launches on a private stream.
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  device_status_word(dev);  // allocate outside the capture
  if (!plan->capture_stream)
    XTC_CUDA_CHECK(cudaStreamCreateWithFlags(&plan->capture_stream, cudaStreamNonBlocking));
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  bool ok = cudaStreamBeginCapture(plan->capture_stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
  int rc = XTC_CUDA_OK;
  if (ok) {
    rc = plan_launch(plan, io, plan->capture_stream);
    ok = cudaStreamEndCapture(plan->capture_stream, &graph) == cudaSuccess && graph != nullptr;
  }
  if (rc != XTC_CUDA_OK) {  // a real argument error: report it, not a capture problem
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    return rc;
  }
  if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
  if (graph) cudaGraphDestroy(graph);
  if (!ok) {
    cudaGetLastError();
    plan->graph_mode = 0;  // replay unavailable here: keep launching directly
    return plan_launch(plan, io, stream);
  }
  if (plan->replays.size() >= 256) {
    cudaGraphExecDestroy(plan->replays.front().exec);
    plan->replays.erase(plan->replays.begin());
  }
  plan->replays.push_back({std::vector<void*>(io, io + n_io), exec});
  XTC_CUDA_CHECK(cudaGraphLaunch(exec, s));
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_run_sets(xtc_cuda_plan* plan, void* const* io_sets, int n_sets, int first,
                                      int count, void* stream) {
  XTC_REQUIRE(plan && io_sets, "plan_run_sets: NULL plan or io_sets");
  XTC_REQUIRE(n_sets >= 1 && first >= 0 && count >= 0,
              "plan_run_sets: %d sets, first %d, count %d", n_sets, first, count);
  const size_t n_io = static_cast<size_t>(plan->n_inputs + plan->n_outputs);
  for (int j = 0; j < count; ++j) {
    const size_t set = (static_cast<size_t>(first) + static_cast<size_t>(j)) % static_cast<size_t>(n_sets);
    if (int rc = xtc_cuda_plan_run(plan, io_sets + set * n_io, stream)) return rc;
  }
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_plan_run_host(xtc_cuda_plan* plan, void* const* io) {
  XTC_REQUIRE(plan && io, "plan_run_host: NULL plan or io");
  const int n_io = plan->n_inputs + plan->n_outputs;
  int rc;
  for (int s = 0; s < n_io; ++s) {
    XTC_REQUIRE(io[s] != nullptr, "plan_run_host: io[%d] is NULL", s);
    if (!plan->staging[s] && (rc = xtc_cuda_malloc(&plan->staging[s], plan->slot_bytes[s])))
      return rc;
  }
  for (int s = 0; s < plan->n_inputs; ++s)
    if ((rc = xtc_cuda_memcpy_h2d(plan->staging[s], io[s], plan->slot_bytes[s], nullptr))) return rc;
  if ((rc = xtc_cuda_plan_run(plan, plan->staging.data(), nullptr))) return rc;
  for (int s = plan->n_inputs; s < n_io; ++s)
    if ((rc = xtc_cuda_memcpy_d2h(io[s], plan->staging[s], plan->slot_bytes[s], nullptr))) return rc;
  XTC_CUDA_CHECK(cudaStreamSynchronize(nullptr));
  int status = 0;
  if ((rc = xtc_cuda_device_status(&status))) return rc;
  return status == 0 ? XTC_CUDA_OK : XTC_CUDA_ERR_DEVICE_TIMEOUT;
}

// ---------------------------------------------------------------------------
// host pipeline: overlapped H2D copy / run / D2H copy of successive runs
// ---------------------------------------------------------------------------
struct xtc_cuda_pipeline {
  xtc_cuda_plan* plan = nullptr;
  int depth = 0;
  long submitted = 0;
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
  std::vector<std::vector<void*>> staging;  // [depth][n_io] device buffers
  std::vector<cudaEvent_t> in_done, run_done, out_done;
};

extern "C" int xtc_cuda_pipeline_destroy(xtc_cuda_pipeline* pipe) {
  if (!pipe) return XTC_CUDA_OK;
  if (pipe->s_out) cudaStreamSynchronize(pipe->s_out);
  for (auto& set : pipe->staging)
    for (void* q : set)
      if (q) cudaFree(q);
  for (auto e : pipe->in_done) cudaEventDestroy(e);
  for (auto e : pipe->run_done) cudaEventDestroy(e);
  for (auto e : pipe->out_done) cudaEventDestroy(e);
  if (pipe->s_in) cudaStreamDestroy(pipe->s_in);
  if (pipe->s_run) cudaStreamDestroy(pipe->s_run);
  if (pipe->s_out) cudaStreamDestroy(pipe->s_out);
  delete pipe;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_pipeline_create(xtc_cuda_pipeline** pipe, xtc_cuda_plan* plan, int depth) {
  XTC_REQUIRE(pipe && plan, "pipeline_create: NULL argument");
  XTC_REQUIRE(depth >= 1 && depth <= 8, "pipeline_create: depth %d not in [1, 8]", depth);
  *pipe = nullptr;
  xtc_cuda_pipeline* p = new xtc_cuda_pipeline();
  p->plan = plan;
  p->depth = depth;
  const int n_io = plan->n_inputs + plan->n_outputs;
  int rc = XTC_CUDA_OK;
  auto ok = [&](cudaError_t e) {
    if (e != cudaSuccess && rc == XTC_CUDA_OK) {
      set_error("pipeline_create: %s", cudaGetErrorString(e));
      rc = XTC_CUDA_ERR_RUNTIME;
    }
  };
  ok(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking));
  ok(cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking));
  ok(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
  p->staging.assign(depth, std::vector<void*>(n_io, nullptr));
  for (int d = 0; d < depth && rc == XTC_CUDA_OK; ++d) {
    for (int s = 0; s < n_io && rc == XTC_CUDA_OK; ++s)
      rc = xtc_cuda_malloc(&p->staging[d][s], plan->slot_bytes[s]);
    cudaEvent_t e;
    ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); p->in_done.push_back(e);
    ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); p->run_done.push_back(e);
    ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); p->out_done.push_back(e);
  }
  if (rc != XTC_CUDA_OK) {
    xtc_cuda_pipeline_destroy(p);
    return rc;
  }
  *pipe = p;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_pipeline_submit(xtc_cuda_pipeline* pipe, void* const* io) {
  XTC_REQUIRE(pipe && io, "pipeline_submit: NULL argument");
  xtc_cuda_plan* plan = pipe->plan;
  const int n_io = plan->n_inputs + plan->n_outputs;
  const int slot = static_cast<int>(pipe->submitted % pipe->depth);
  // the run that used this slot `depth` submissions ago must have delivered its outputs
  if (pipe->submitted >= pipe->depth) XTC_CUDA_CHECK(cudaEventSynchronize(pipe->out_done[slot]));
  std::vector<void*>& dev = pipe->staging[slot];
  for (int s = 0; s < plan->n_inputs; ++s) {
    XTC_REQUIRE(io[s] != nullptr, "pipeline_submit: io[%d] is NULL", s);
    XTC_CUDA_CHECK(cudaMemcpyAsync(dev[s], io[s], plan->slot_bytes[s], cudaMemcpyHostToDevice, pipe->s_in));
  }
  XTC_CUDA_CHECK(cudaEventRecord(pipe->in_done[slot], pipe->s_in));
  XTC_CUDA_CHECK(cudaStreamWaitEvent(pipe->s_run, pipe->in_done[slot], 0));
  int rc = xtc_cuda_plan_run(plan, dev.data(), pipe->s_run);
  if (rc != XTC_CUDA_OK) return rc;
  XTC_CUDA_CHECK(cudaEventRecord(pipe->run_done[slot], pipe->s_run));
  XTC_CUDA_CHECK(cudaStreamWaitEvent(pipe->s_out, pipe->run_done[slot], 0));
  for (int s = plan->n_inputs; s < n_io; ++s) {
    XTC_REQUIRE(io[s] != nullptr, "pipeline_submit: io[%d] is NULL", s);
    XTC_CUDA_CHECK(cudaMemcpyAsync(io[s], dev[s], plan->slot_bytes[s], cudaMemcpyDeviceToHost, pipe->s_out));
  }
  XTC_CUDA_CHECK(cudaEventRecord(pipe->out_done[slot], pipe->s_out));
  ++pipe->submitted;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_pipeline_wait(xtc_cuda_pipeline* pipe) {
  XTC_REQUIRE(pipe != nullptr, "pipeline_wait: NULL argument");
  XTC_CUDA_CHECK(cudaStreamSynchronize(pipe->s_out));
  int status = 0;
  int rc = xtc_cuda_device_status(&status);
  if (rc != XTC_CUDA_OK) return rc;
  return status == 0 ? XTC_CUDA_OK : XTC_CUDA_ERR_DEVICE_TIMEOUT;
}

extern "C" int xtc_cuda_evaluate(xtc_cuda_plan* plan, void* const* io, int repeat, int number,
                                 int min_repeat_ms, double* results) {
  XTC_REQUIRE(plan && io && results, "evaluate: NULL argument");
  XTC_REQUIRE(repeat > 0 && number >= 0 && min_repeat_ms >= 0, "evaluate: bad repeat/number/min_repeat_ms");
  cudaStream_t s;
  XTC_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  cudaEvent_t e0, e1;
  XTC_CUDA_CHECK(cudaEventCreate(&e0));
  XTC_CUDA_CHECK(cudaEventCreate(&e1));
  int rc = XTC_CUDA_OK;
  if (number > 0) {
    rc = xtc_cuda_plan_run(plan, io, s);  // warm-up, untimed
    if (rc == XTC_CUDA_OK && cudaStreamSynchronize(s) != cudaSuccess) rc = XTC_CUDA_ERR_RUNTIME;
  } else {
    number = 1;
  }
  for (int r = 0; r < repeat && rc == XTC_CUDA_OK; ++r) {
    long attempts = number;
    for (;;) {
      cudaEventRecord(e0, s);
      for (long a = 0; a < attempts && rc == XTC_CUDA_OK; ++a) rc = xtc_cuda_plan_run(plan, io, s);
      cudaEventRecord(e1, s);
      if (rc != XTC_CUDA_OK) break;
      cudaError_t e = cudaEventSynchronize(e1);
      if (e != cudaSuccess) {
        set_error("evaluate: %s", cudaGetErrorString(e));
        rc = XTC_CUDA_ERR_RUNTIME;
        break;
      }
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      if (ms >= static_cast<float>(min_repeat_ms) || attempts > (1l << 24)) {
        results[r] = static_cast<double>(ms) * 1e-3 / static_cast<double>(attempts);
        break;
      }
      attempts *= 2;
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamDestroy(s);
  if (rc != XTC_CUDA_OK) return rc;
  int status = 0;
  if ((rc = xtc_cuda_device_status(&status))) return rc;
  return status == 0 ? XTC_CUDA_OK : XTC_CUDA_ERR_DEVICE_TIMEOUT;
}
