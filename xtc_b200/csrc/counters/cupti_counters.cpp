// GPU hardware counters through the CUPTI range profiler.  Everything launched between
// start and stop is ONE user-defined range, so a counter's value is the hardware's sum
// over all kernels of the measured runs; metrics that need several passes are collected by
// the caller repeating the same launches (user replay) until stop says it has them all.
// (Automatic per-kernel ranges with kernel replay are the other mode of this API; on the
// B200 / driver 580 / CUPTI 12.9 combination this was written on that mode accepted every
// call and recorded no range, so it is not used.)
// Built into its own library so that the kernel library has no CUPTI dependency.
#include <cuda.h>
#include <cupti_profiler_host.h>
#include <cupti_profiler_target.h>
#include <cupti_range_profiler.h>
#include <cupti_target.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../../include/xtc_cuda_counters.h"

namespace {

thread_local char g_error[1024] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

const char* cupti_text(CUptiResult r) {
  const char* s = nullptr;
  if (cuptiGetResultString(r, &s) != CUPTI_SUCCESS || s == nullptr) return "unknown CUPTI error";
  return s;
}

#define CUPTI_TRY(call, code)                                                         \
  do {                                                                                \
    CUptiResult _r = (call);                                                          \
    if (_r != CUPTI_SUCCESS) return fail((code), "%s: %s (%d)", #call, cupti_text(_r), (int)_r); \
  } while (0)

// The current CUDA context, without linking the driver library.
CUcontext current_context() {
  typedef CUresult (*get_fn)(CUcontext*);
  static get_fn get = nullptr;
  if (!get) {
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return nullptr;
    get = reinterpret_cast<get_fn>(dlsym(lib, "cuCtxGetCurrent"));
    if (!get) return nullptr;
  }
  CUcontext ctx = nullptr;
  if (get(&ctx) != CUDA_SUCCESS) return nullptr;
  return ctx;
}

int current_device() {
  typedef CUresult (*get_fn)(CUdevice*);
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return 0;
  get_fn get = reinterpret_cast<get_fn>(dlsym(lib, "cuCtxGetDevice"));
  CUdevice dev = 0;
  if (!get || get(&dev) != CUDA_SUCCESS) return 0;
  return static_cast<int>(dev);
}

bool g_profiler_initialised = false;

}  // namespace

struct xtc_cuda_counters {
  std::vector<std::string> names;       // what the profiler is asked for
  std::vector<const char*> name_ptrs;
  CUpti_Profiler_Host_Object* host = nullptr;
  CUpti_RangeProfiler_Object* range = nullptr;
  std::vector<uint8_t> config, data;
  size_t max_ranges = 1;
  int passes = 0;
  bool started = false;   // between start and stop
  bool collecting = false;  // passes of one measurement still outstanding
};

extern "C" const char* xtc_cuda_counters_last_error(void) { return g_error; }

extern "C" int xtc_cuda_counters_close(xtc_cuda_counters* s) {
  if (!s) return XTC_CUDA_COUNTERS_OK;
  if (s->range) {
    CUpti_RangeProfiler_Disable_Params p = {CUpti_RangeProfiler_Disable_Params_STRUCT_SIZE};
    p.pRangeProfilerObject = s->range;
    cuptiRangeProfilerDisable(&p);
  }
  if (s->host) {
    CUpti_Profiler_Host_Deinitialize_Params p = {CUpti_Profiler_Host_Deinitialize_Params_STRUCT_SIZE};
    p.pHostObject = s->host;
    cuptiProfilerHostDeinitialize(&p);
  }
  delete s;
  return XTC_CUDA_COUNTERS_OK;
}

static int open_impl(xtc_cuda_counters* s, CUcontext ctx) {
  if (!g_profiler_initialised) {
    CUpti_Profiler_Initialize_Params init = {CUpti_Profiler_Initialize_Params_STRUCT_SIZE};
    CUPTI_TRY(cuptiProfilerInitialize(&init), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
    g_profiler_initialised = true;
  }
  CUpti_Device_GetChipName_Params chip = {CUpti_Device_GetChipName_Params_STRUCT_SIZE};
  chip.deviceIndex = static_cast<size_t>(current_device());
  CUPTI_TRY(cuptiDeviceGetChipName(&chip), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);

  // which raw counters this context may read (fails while another profiling session is active)
  std::vector<uint8_t> avail;
  CUpti_Profiler_GetCounterAvailability_Params ca = {CUpti_Profiler_GetCounterAvailability_Params_STRUCT_SIZE};
  ca.ctx = ctx;
  CUPTI_TRY(cuptiProfilerGetCounterAvailability(&ca), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  avail.resize(ca.counterAvailabilityImageSize);
  ca.pCounterAvailabilityImage = avail.data();
  CUPTI_TRY(cuptiProfilerGetCounterAvailability(&ca), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);

  CUpti_Profiler_Host_Initialize_Params hi = {CUpti_Profiler_Host_Initialize_Params_STRUCT_SIZE};
  hi.profilerType = CUPTI_PROFILER_TYPE_RANGE_PROFILER;
  hi.pChipName = chip.pChipName;
  hi.pCounterAvailabilityImage = avail.data();
  CUPTI_TRY(cuptiProfilerHostInitialize(&hi), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  s->host = hi.pHostObject;

  CUpti_Profiler_Host_ConfigAddMetrics_Params add = {CUpti_Profiler_Host_ConfigAddMetrics_Params_STRUCT_SIZE};
  add.pHostObject = s->host;
  add.ppMetricNames = s->name_ptrs.data();
  add.numMetrics = s->name_ptrs.size();
  CUPTI_TRY(cuptiProfilerHostConfigAddMetrics(&add), XTC_CUDA_COUNTERS_ERR_METRIC);
  CUpti_Profiler_Host_GetConfigImageSize_Params cs = {CUpti_Profiler_Host_GetConfigImageSize_Params_STRUCT_SIZE};
  cs.pHostObject = s->host;
  CUPTI_TRY(cuptiProfilerHostGetConfigImageSize(&cs), XTC_CUDA_COUNTERS_ERR_METRIC);
  s->config.resize(cs.configImageSize);
  CUpti_Profiler_Host_GetConfigImage_Params ci = {CUpti_Profiler_Host_GetConfigImage_Params_STRUCT_SIZE};
  ci.pHostObject = s->host;
  ci.configImageSize = s->config.size();
  ci.pConfigImage = s->config.data();
  CUPTI_TRY(cuptiProfilerHostGetConfigImage(&ci), XTC_CUDA_COUNTERS_ERR_METRIC);
  CUpti_Profiler_Host_GetNumOfPasses_Params np = {CUpti_Profiler_Host_GetNumOfPasses_Params_STRUCT_SIZE};
  np.configImageSize = s->config.size();
  np.pConfigImage = s->config.data();
  CUPTI_TRY(cuptiProfilerHostGetNumOfPasses(&np), XTC_CUDA_COUNTERS_ERR_METRIC);
  s->passes = static_cast<int>(np.numOfPasses);

  CUpti_RangeProfiler_Enable_Params en = {CUpti_RangeProfiler_Enable_Params_STRUCT_SIZE};
  en.ctx = ctx;
  CUPTI_TRY(cuptiRangeProfilerEnable(&en), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  s->range = en.pRangeProfilerObject;

  CUpti_RangeProfiler_GetCounterDataSize_Params ds = {CUpti_RangeProfiler_GetCounterDataSize_Params_STRUCT_SIZE};
  ds.pRangeProfilerObject = s->range;
  ds.pMetricNames = s->name_ptrs.data();
  ds.numMetrics = s->name_ptrs.size();
  ds.maxNumOfRanges = s->max_ranges;
  ds.maxNumRangeTreeNodes = static_cast<uint32_t>(s->max_ranges);
  CUPTI_TRY(cuptiRangeProfilerGetCounterDataSize(&ds), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  s->data.assign(ds.counterDataSize, 0);
  return XTC_CUDA_COUNTERS_OK;
}

// A fresh counter data image and the session configuration: before every start.
static int arm(xtc_cuda_counters* s) {
  CUpti_RangeProfiler_CounterDataImage_Initialize_Params di = {
      CUpti_RangeProfiler_CounterDataImage_Initialize_Params_STRUCT_SIZE};
  di.pRangeProfilerObject = s->range;
  di.counterDataSize = s->data.size();
  di.pCounterData = s->data.data();
  CUPTI_TRY(cuptiRangeProfilerCounterDataImageInitialize(&di), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  CUpti_RangeProfiler_SetConfig_Params sc = {CUpti_RangeProfiler_SetConfig_Params_STRUCT_SIZE};
  sc.pRangeProfilerObject = s->range;
  sc.configSize = s->config.size();
  sc.pConfig = s->config.data();
  sc.counterDataImageSize = s->data.size();
  sc.pCounterDataImage = s->data.data();
  sc.range = CUPTI_UserRange;
  sc.replayMode = CUPTI_UserReplay;
  sc.maxRangesPerPass = s->max_ranges;
  sc.numNestingLevels = 1;
  sc.minNestingLevel = 1;
  sc.passIndex = 0;
  sc.targetNestingLevel = 0;
  CUPTI_TRY(cuptiRangeProfilerSetConfig(&sc), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  return XTC_CUDA_COUNTERS_OK;
}

extern "C" int xtc_cuda_counters_open(xtc_cuda_counters** session, const char* const* names, int n) {
  if (!session) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_open: NULL session");
  *session = nullptr;
  if (!names || n <= 0 || n > 64)
    return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_open: between 1 and 64 metric names are needed");
  CUcontext ctx = current_context();
  if (!ctx)
    return fail(XTC_CUDA_COUNTERS_ERR_UNAVAILABLE,
                "counters_open: no current CUDA context (no driver, or the device was not initialised)");
  xtc_cuda_counters* s = new xtc_cuda_counters();
  for (int i = 0; i < n; ++i) {
    if (!names[i] || !names[i][0]) {
      delete s;
      return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_open: empty metric name at %d", i);
    }
    if (strcmp(names[i], "cycles") == 0) s->names.push_back("gpu__cycles_elapsed.sum");
    else if (strcmp(names[i], "clocks") == 0) s->names.push_back("gpu__time_duration.sum");
    else s->names.push_back(names[i]);
  }
  for (auto& nm : s->names) s->name_ptrs.push_back(nm.c_str());
  int rc = open_impl(s, ctx);
  if (rc != XTC_CUDA_COUNTERS_OK) {
    char keep[sizeof(g_error)];
    memcpy(keep, g_error, sizeof(keep));
    xtc_cuda_counters_close(s);
    memcpy(g_error, keep, sizeof(keep));
    return rc;
  }
  *session = s;
  return XTC_CUDA_COUNTERS_OK;
}

extern "C" int xtc_cuda_counters_passes(const xtc_cuda_counters* s, int* passes) {
  if (!s || !passes) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_passes: NULL argument");
  *passes = s->passes;
  return XTC_CUDA_COUNTERS_OK;
}

extern "C" int xtc_cuda_counters_start(xtc_cuda_counters* s) {
  if (!s) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_start: NULL session");
  if (s->started) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_start: already started");
  if (!s->collecting) {  // first pass of a measurement: fresh counter data, pass 0
    int rc = arm(s);
    if (rc != XTC_CUDA_COUNTERS_OK) return rc;
    s->collecting = true;
  }
  CUpti_RangeProfiler_Start_Params p = {CUpti_RangeProfiler_Start_Params_STRUCT_SIZE};
  p.pRangeProfilerObject = s->range;
  CUPTI_TRY(cuptiRangeProfilerStart(&p), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  CUpti_RangeProfiler_PushRange_Params push = {CUpti_RangeProfiler_PushRange_Params_STRUCT_SIZE};
  push.pRangeProfilerObject = s->range;
  push.pRangeName = "run";
  CUptiResult r = cuptiRangeProfilerPushRange(&push);
  if (r != CUPTI_SUCCESS) {
    CUpti_RangeProfiler_Stop_Params stop = {CUpti_RangeProfiler_Stop_Params_STRUCT_SIZE};
    stop.pRangeProfilerObject = s->range;
    cuptiRangeProfilerStop(&stop);
    s->collecting = false;
    return fail(XTC_CUDA_COUNTERS_ERR_UNAVAILABLE, "cuptiRangeProfilerPushRange: %s (%d)", cupti_text(r), (int)r);
  }
  s->started = true;
  return XTC_CUDA_COUNTERS_OK;
}

extern "C" int xtc_cuda_counters_stop(xtc_cuda_counters* s, int* again) {
  if (!s || !again) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_stop: NULL argument");
  if (!s->started) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_stop: not started");
  *again = 0;
  s->started = false;
  CUpti_RangeProfiler_PopRange_Params pop = {CUpti_RangeProfiler_PopRange_Params_STRUCT_SIZE};
  pop.pRangeProfilerObject = s->range;
  CUptiResult popped = cuptiRangeProfilerPopRange(&pop);
  CUpti_RangeProfiler_Stop_Params p = {CUpti_RangeProfiler_Stop_Params_STRUCT_SIZE};
  p.pRangeProfilerObject = s->range;
  CUptiResult stopped = cuptiRangeProfilerStop(&p);
  if (popped != CUPTI_SUCCESS || stopped != CUPTI_SUCCESS) {
    s->collecting = false;
    const CUptiResult bad = popped != CUPTI_SUCCESS ? popped : stopped;
    return fail(XTC_CUDA_COUNTERS_ERR_UNAVAILABLE, "counters_stop: %s (%d)", cupti_text(bad), (int)bad);
  }
  if (!p.isAllPassSubmitted) {  // the metrics need another pass over the same launches
    *again = 1;
    return XTC_CUDA_COUNTERS_OK;
  }
  s->collecting = false;
  CUpti_RangeProfiler_DecodeData_Params d = {CUpti_RangeProfiler_DecodeData_Params_STRUCT_SIZE};
  d.pRangeProfilerObject = s->range;
  CUPTI_TRY(cuptiRangeProfilerDecodeData(&d), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  if (d.numOfRangeDropped > 0)
    return fail(XTC_CUDA_COUNTERS_ERR_UNAVAILABLE, "counters_stop: the profiler dropped %zu range(s)",
                d.numOfRangeDropped);
  return XTC_CUDA_COUNTERS_OK;
}

extern "C" int xtc_cuda_counters_read(xtc_cuda_counters* s, double* values) {
  if (!s || !values) return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_read: NULL argument");
  if (s->started || s->collecting)
    return fail(XTC_CUDA_COUNTERS_ERR_INVALID, "counters_read: the measurement is not complete");
  CUpti_RangeProfiler_GetCounterDataInfo_Params info = {CUpti_RangeProfiler_GetCounterDataInfo_Params_STRUCT_SIZE};
  info.pCounterDataImage = s->data.data();
  info.counterDataImageSize = s->data.size();
  CUPTI_TRY(cuptiRangeProfilerGetCounterDataInfo(&info), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
  const size_t n = s->names.size();
  for (size_t i = 0; i < n; ++i) values[i] = 0.0;
  std::vector<double> one(n);
  for (size_t r = 0; r < info.numTotalRanges; ++r) {
    CUpti_Profiler_Host_EvaluateToGpuValues_Params ev = {CUpti_Profiler_Host_EvaluateToGpuValues_Params_STRUCT_SIZE};
    ev.pHostObject = s->host;
    ev.pCounterDataImage = s->data.data();
    ev.counterDataImageSize = s->data.size();
    ev.rangeIndex = r;
    ev.ppMetricNames = s->name_ptrs.data();
    ev.numMetrics = n;
    ev.pMetricValues = one.data();
    CUPTI_TRY(cuptiProfilerHostEvaluateToGpuValues(&ev), XTC_CUDA_COUNTERS_ERR_UNAVAILABLE);
    for (size_t i = 0; i < n; ++i) values[i] += one[i];
  }
  if (info.numTotalRanges == 0)
    return fail(XTC_CUDA_COUNTERS_ERR_UNAVAILABLE, "counters_read: the profiler recorded no range");
  return XTC_CUDA_COUNTERS_OK;
}
