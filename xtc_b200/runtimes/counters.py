"""GPU hardware counters for the evaluator (``pmu_counters=["gpu.<metric>", ...]``).

ctypes binding of ``libxtc_cuda_counters.so`` (``include/xtc_cuda_counters.h``), the CUPTI
range-profiler module that takes the place of the reference's
``csrcs/runtimes/accelerator/gpu/perf_event_gpu.cpp``.  The reference's timing loop opens the
events, brackets ``number`` calls of the payload with start / stop and stores ``value / number``
per repeat (``csrcs/runtimes/host/evaluate_perf.c:83-116``); ``GpuCounters.measure`` is that
loop for a plan.

Names: ``gpu.cycles`` = ``gpu__cycles_elapsed.sum``, ``gpu.clocks`` = ``gpu__time_duration.sum``
(nanoseconds), anything else after ``gpu.`` is a profiler metric name as ``ncu --metrics``
takes it.  Counters without the ``gpu.`` prefix are host CPU events (libpfm in the reference):
they do not exist for a GPU run and read -1.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_void_p
from pathlib import Path
from typing import Any, Callable

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libxtc_cuda_counters.so"

OK, ERR_INVALID, ERR_UNAVAILABLE, ERR_METRIC = 0, 1, 2, 3

SIGNATURES: dict[str, tuple] = {
    "xtc_cuda_counters_open": (c_int, [POINTER(c_void_p), POINTER(c_char_p), c_int]),
    "xtc_cuda_counters_passes": (c_int, [c_void_p, POINTER(c_int)]),
    "xtc_cuda_counters_start": (c_int, [c_void_p]),
    "xtc_cuda_counters_stop": (c_int, [c_void_p, POINTER(c_int)]),
    "xtc_cuda_counters_read": (c_int, [c_void_p, POINTER(c_double)]),
    "xtc_cuda_counters_close": (c_int, [c_void_p]),
    "xtc_cuda_counters_last_error": (c_char_p, []),
}


class CountersError(RuntimeError):
    def __init__(self, code: int, message: str) -> None:
        super().__init__(f"GPU counters unavailable ({code}): {message}")
        self.code, self.message = code, message


_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise CountersError(ERR_UNAVAILABLE, f"{LIB_PATH} is missing (python -m xtc_b200.build)")
        try:
            lib = ctypes.CDLL(str(LIB_PATH))
        except OSError as e:  # CUPTI itself could not be loaded
            raise CountersError(ERR_UNAVAILABLE, str(e)) from None
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


def split_counter_names(pmu_counters: list[str]) -> tuple[list[int], list[str]]:
    """(positions, metric names) of the ``gpu.`` entries of a pmu_counters list."""
    pos = [i for i, c in enumerate(pmu_counters) if c.startswith("gpu.")]
    return pos, [pmu_counters[i][4:] for i in pos]


class GpuCounters:
    """One profiling session on the calling thread's CUDA context."""

    def __init__(self, metrics: list[str]) -> None:
        self.lib = load()
        self.metrics = list(metrics)
        self.handle = c_void_p()
        names = (c_char_p * len(metrics))(*[m.encode() for m in metrics])
        self._check(self.lib.xtc_cuda_counters_open(byref(self.handle), names, len(metrics)))

    def _check(self, code: int) -> None:
        if code != OK:
            msg = self.lib.xtc_cuda_counters_last_error()
            raise CountersError(code, msg.decode(errors="replace") if msg else "")

    @property
    def passes(self) -> int:
        n = c_int(0)
        self._check(self.lib.xtc_cuda_counters_passes(self.handle, byref(n)))
        return n.value

    def measure(self, run: Callable[[], Any], synchronize: Callable[[], Any]) -> list[float]:
        """Each counter over every kernel `run()` launches.  `run` is called once per pass
        the metrics need (it must launch the same work every time)."""
        for _ in range(64):
            self._check(self.lib.xtc_cuda_counters_start(self.handle))
            again = c_int(0)
            try:
                run()
                synchronize()
            finally:
                code = self.lib.xtc_cuda_counters_stop(self.handle, byref(again))
            self._check(code)
            if not again.value:
                break
        else:
            raise CountersError(ERR_UNAVAILABLE, "the profiler kept asking for more passes")
        values = (c_double * len(self.metrics))()
        self._check(self.lib.xtc_cuda_counters_read(self.handle, values))
        return [float(v) for v in values]

    def close(self) -> None:
        if self.handle is not None and self.handle.value:
            self.lib.xtc_cuda_counters_close(self.handle)
            self.handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
