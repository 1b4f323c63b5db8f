/*
 * libxtc_cuda_counters -- GPU hardware counters for the evaluator of the CUDA
 * backend, read in-process with the CUPTI range profiler.
 *
 * Takes the place of the reference's GPU perf-event module,
 * src/xtc/csrcs/runtimes/accelerator/gpu/perf_event_gpu.cpp:56-233, which its
 * timing loop drives through open / start / stop (src/xtc/csrcs/runtimes/host/
 * evaluate_perf.c:83-116) for every `pmu_counters=["gpu.<metric>"]` entry.  Same
 * naming: "cycles" is gpu__cycles_elapsed.sum, "clocks" is gpu__time_duration.sum,
 * any other name is passed to the profiler as it is (perf_event_gpu.cpp:221-233).
 * Same accumulation: a counter's value is its SUM over every kernel launched
 * between start and stop (perf_event_gpu.cpp:193-203 adds up its per-kernel
 * ranges), as a double.  Here the launches between start and stop form one
 * user-defined range, so the hardware does the adding; gpu__time_duration.sum
 * of a range is the time from its first launch to its last completion, which
 * includes the gaps between launches and a few microseconds of range overhead
 * (measure several runs per range for short kernels).  A set of metrics the
 * hardware cannot count in one go takes several passes: stop() then asks for the
 * same launches `again`.
 *
 * A library of its own, so that libxtc_cuda.so does not depend on CUPTI.  Plain C
 * ABI, int status returns (0 = ok), message from xtc_cuda_counters_last_error().
 * One session per process at a time; the CUDA context of the calling thread must
 * exist (any earlier call into libxtc_cuda.so on that device creates it).
 */
#ifndef XTC_CUDA_COUNTERS_H_
#define XTC_CUDA_COUNTERS_H_

#ifdef __cplusplus
extern "C" {
#endif

enum {
  XTC_CUDA_COUNTERS_OK = 0,
  XTC_CUDA_COUNTERS_ERR_INVALID = 1,     /* bad argument or call order                    */
  XTC_CUDA_COUNTERS_ERR_UNAVAILABLE = 2, /* CUPTI or the driver refuses (privileges, busy) */
  XTC_CUDA_COUNTERS_ERR_METRIC = 3       /* a metric name the chip does not know          */
};

typedef struct xtc_cuda_counters xtc_cuda_counters;

/* Opens a session for `n` metrics (names without the "gpu." prefix) on the
 * current context.  Replaces open_perf_events__gpu. */
int xtc_cuda_counters_open(xtc_cuda_counters** session, const char* const* names, int n);
/* Passes over the measured launches these metrics take. */
int xtc_cuda_counters_passes(const xtc_cuda_counters* session, int* passes);
/* Every kernel launched by this context from start to stop is counted; the
 * caller synchronises the device before stop.  *again = 1: launch the same work
 * once more between another start / stop (next pass); 0: the measurement is
 * complete.  Replaces start_perf_events__gpu / stop_perf_events__gpu. */
int xtc_cuda_counters_start(xtc_cuda_counters* session);
int xtc_cuda_counters_stop(xtc_cuda_counters* session, int* again);
/* values[n]: each metric over the launches of the last completed measurement.
 * Replaces read_perf_events__gpu. */
int xtc_cuda_counters_read(xtc_cuda_counters* session, double* values);
/* Replaces close_perf_events__gpu. */
int xtc_cuda_counters_close(xtc_cuda_counters* session);
const char* xtc_cuda_counters_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* XTC_CUDA_COUNTERS_H_ */
