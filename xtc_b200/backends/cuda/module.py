"""Module, Evaluator and Executor of the CUDA backend.

Same contracts as the reference's host and GPU targets
(``targets/host/HostModule.py:26-135``, ``HostEvaluator.py:28-120``,
``targets/accelerator/gpu/GPUEvaluator.py:47-112``): ``evaluate()`` returns
``(results, code, message)`` with ``repeat`` floats of seconds per call,
``validate=True`` first compares one run against the graph's NumPy evaluation
with ``np.allclose``, caller-provided output arrays are written in place.

Differences, all deliberate: inputs live in device memory during timing (the
reference maps host memory into the GPU, ``GPUEvaluator.py:67-78``), time is
CUDA-event time of the launches (``xtc_cuda_evaluate``), and ``rtol`` / ``atol``
are configurable because TF32 results on non-integer data do not satisfy
NumPy's default tolerances.
"""

from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Any, Callable

import numpy as np

from ... import capi
from ...capi import byref, c_void_p
from ...runtimes.cuda import CudaDevice, NDArray
from ...utils.numpy import np_init
from .lowering import Plan


class PlanHandle:
    """Owns one ``xtc_cuda_plan`` on one device."""

    def __init__(self, plan: Plan, device: CudaDevice) -> None:
        self.plan = plan
        self.device = device
        self.lib = device.lib
        self._io_cache: dict[tuple, ctypes.Array] = {}
        device.activate()
        n = len(plan.steps)
        steps = (capi.Step * n)(*[s.to_c() for s in plan.steps])
        sizes = (ctypes.c_size_t * len(plan.slot_bytes))(*plan.slot_bytes)
        self.handle = c_void_p()
        capi.check(self.lib.xtc_cuda_plan_create(byref(self.handle), steps, n, plan.n_inputs,
                                                 plan.n_outputs, len(plan.slot_bytes), sizes))

    def _io(self, pointers: list[int]) -> ctypes.Array:
        key = tuple(pointers)
        arr = self._io_cache.get(key)
        if arr is None:
            assert len(pointers) == self.plan.n_inputs + self.plan.n_outputs
            if len(self._io_cache) > 1024:
                self._io_cache.clear()
            arr = self._io_cache[key] = (c_void_p * len(pointers))(*pointers)
        return arr

    def set_graph_mode(self, enabled: bool) -> None:
        capi.check(self.lib.xtc_cuda_plan_set_graph_mode(self.handle, int(enabled)))

    def run(self, pointers: list[int], stream: int | None = None) -> None:
        """Launch on device pointers (asynchronous on ``stream``).  The device of
        the plan must be the calling thread's current device (``device.activate()``)."""
        rc = self.lib.xtc_cuda_plan_run(self.handle, self._io(pointers), stream)
        if rc:
            capi.check(rc)

    def pointer_sets(self, sets: list[list[int]]) -> ctypes.Array:
        """The flat pointer table ``run_sets`` takes: one row of device pointers per set."""
        n_io = self.plan.n_inputs + self.plan.n_outputs
        assert sets and all(len(s) == n_io for s in sets)
        return (c_void_p * (n_io * len(sets)))(*[p for s in sets for p in s])

    def run_sets(self, table: ctypes.Array, first: int, count: int,
                 stream: int | None = None) -> None:
        """``count`` runs back to back from one call (``xtc_cuda_plan_run_sets``): run j on
        row ``(first + j) % n_sets`` of ``table`` (see ``pointer_sets``)."""
        n_sets = len(table) // (self.plan.n_inputs + self.plan.n_outputs)
        rc = self.lib.xtc_cuda_plan_run_sets(self.handle, table, n_sets, first, count, stream)
        if rc:
            capi.check(rc)

    def run_host(self, arrays: list[np.ndarray]) -> None:
        """Host arrays in, host arrays out (copies inside), synchronous."""
        self.device.activate()
        ptrs = [a.ctypes.data for a in arrays]
        capi.check(self.lib.xtc_cuda_plan_run_host(self.handle, self._io(ptrs)))

    def pipeline(self, depth: int = 3) -> "HostPipeline":
        """Overlapped host-array executor over this plan (``xtc_cuda_pipeline_*``)."""
        return HostPipeline(self, depth)

    def evaluate(self, pointers: list[int], repeat: int, number: int,
                 min_repeat_ms: int) -> list[float]:
        self.device.activate()
        results = (ctypes.c_double * repeat)()
        capi.check(self.lib.xtc_cuda_evaluate(self.handle, self._io(pointers), repeat, number,
                                              min_repeat_ms, results))
        return [float(x) for x in results]

    def close(self) -> None:
        if self.handle is not None and self.handle.value:
            self.device.activate()
            self.lib.xtc_cuda_plan_destroy(self.handle)
            self.handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class HostPipeline:
    """Runs a plan on a sequence of host batches with the input copy, the kernels
    and the output copy of neighbouring batches overlapped.

    ``submit(arrays)`` queues one run on host arrays (inputs then outputs, the
    payload's argument order); an output array holds its result once ``wait()``
    has returned, or once ``depth`` later submits have been accepted.  Page-locked
    arrays (``CudaDevice.host_alloc`` / ``xtc_cuda_host_alloc``) are needed for
    the copies to actually overlap."""

    def __init__(self, plan_handle: PlanHandle, depth: int = 3) -> None:
        self._owner = plan_handle
        self.lib = plan_handle.lib
        self.handle: c_void_p | None = c_void_p()
        plan_handle.device.activate()
        capi.check(self.lib.xtc_cuda_pipeline_create(byref(self.handle), plan_handle.handle, depth))

    def submit(self, arrays: list[np.ndarray]) -> None:
        ptrs = [a.ctypes.data for a in arrays]
        rc = self.lib.xtc_cuda_pipeline_submit(self.handle, self._owner._io(ptrs))
        if rc:
            capi.check(rc)

    def wait(self) -> None:
        capi.check(self.lib.xtc_cuda_pipeline_wait(self.handle))

    def close(self) -> None:
        if self.handle is not None and self.handle.value:
            self._owner.device.activate()
            self.lib.xtc_cuda_pipeline_destroy(self.handle)
            self.handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class CudaModule:
    def __init__(self, name: str, payload_name: str, file_name: str, file_type: str,
                 plan: Plan, graph: Any = None, backend: Any = None, **kwargs: Any) -> None:
        self._name = name
        self._payload_name = payload_name
        self._file_name = file_name
        self._file_type = file_type
        self._plan = plan
        self._graph = graph
        self._backend = backend
        self._bare_ptr = True
        self._np_inputs_spec = backend.np_inputs_spec if backend is not None else None
        self._np_outputs_spec = backend.np_outputs_spec if backend is not None else None
        self._reference_impl = backend.reference_impl if backend is not None else None

    name = property(lambda self: self._name)
    payload_name = property(lambda self: self._payload_name)
    file_name = property(lambda self: self._file_name)
    file_type = property(lambda self: self._file_type)
    plan = property(lambda self: self._plan)
    graph = property(lambda self: self._graph)

    def export(self) -> None:
        """Nothing to do, as in the reference's host module (``targets/host/HostModule.py:98-99``):
        the payload library already sits at ``file_name``."""

    def get_evaluator(self, **kwargs: Any) -> "CudaEvaluator":
        return CudaEvaluator(self, **kwargs)

    def get_executor(self, **kwargs: Any) -> "CudaExecutor":
        return CudaExecutor(self, **kwargs)


class CudaEvaluator:
    def __init__(self, module: CudaModule, **kwargs: Any) -> None:
        self._module = module
        self._repeat = kwargs.get("repeat", 1)
        self._min_repeat_ms = kwargs.get("min_repeat_ms", 100)
        self._number = kwargs.get("number", 1)
        self._validate = kwargs.get("validate", False)
        self._parameters = kwargs.get("parameters")
        self._init_zero = kwargs.get("init_zero", False)
        self._np_inputs_spec = kwargs.get("np_inputs_spec", module._np_inputs_spec)
        self._np_outputs_spec = kwargs.get("np_outputs_spec", module._np_outputs_spec)
        self._reference_impl = kwargs.get("reference_impl", module._reference_impl)
        self._pmu_counters = kwargs.get("pmu_counters", [])
        # None = derived from the plan's arithmetic when validating (see _tolerances)
        self._rtol = kwargs.get("rtol")
        self._atol = kwargs.get("atol")
        device = kwargs.get("device", kwargs.get("runtime"))
        if device is None:
            device = self._graph_device(module.graph)
        self._device = device if isinstance(device, CudaDevice) else CudaDevice(int(device or 0))

    @staticmethod
    def _graph_device(graph: Any) -> CudaDevice | None:
        """The device a graph's tensors were declared on with ``O.tensor(..., device=gpu)`` /
        ``O.matmul(..., device=gpu)`` (the reference's offload tensors,
        ``tests/filecheck/backends/target_gpu/test_matmul_mlir_offload_tensor.py:8-19``): every
        tensor lives in device memory here anyway, so the declaration only picks the GPU."""
        if graph is None:
            return None
        types = list(getattr(graph, "inputs_types", None) or []) + list(
            getattr(graph, "outputs_types", None) or [])
        for t in types:
            dev = getattr(t, "device", None)
            if isinstance(dev, CudaDevice):
                return dev
        return None

    @property
    def module(self) -> CudaModule:
        return self._module

    def _tolerances(self, ref: np.ndarray) -> tuple[float, float]:
        """(rtol, atol) of the ``validate=True`` comparison.  The reference compares with
        NumPy's defaults (``utils/evaluation.py:129-145``), which fp32 arithmetic meets; a
        plan whose contractions run as single-pass TF32 is correct to about 1e-3 of the
        largest output, so its default bound is the tolerance of the parity tests: 1e-2
        relative to max|ref| (integer-valued data, the default ``np_init`` inputs, are exact
        in every mode and pass either bound)."""
        if self._rtol is not None or self._atol is not None:
            return (1e-5 if self._rtol is None else self._rtol,
                    1e-8 if self._atol is None else self._atol)
        tf32 = any(s.kind in ("gemm", "conv2d")
                   and s.config.get("precision", capi.PRECISION_TF32) == capi.PRECISION_TF32
                   for s in self._module.plan.steps)
        if not tf32:
            return 1e-5, 1e-5 * float(np.max(np.abs(ref))) if ref.size else 0.0
        return 1e-2, 1e-2 * float(np.max(np.abs(ref))) if ref.size else 0.0

    def _read_counters(self, handle: "PlanHandle", pointers: list[int]) -> tuple[list[float], str]:
        """``repeat x len(pmu_counters)`` values, each a counter summed over the kernels of
        ``number`` runs and divided by ``number`` (the layout and the division of
        ``csrcs/runtimes/host/evaluate_perf.c:104-116``).  Entries that cannot be read are -1
        and the returned message says why: names without the ``gpu.`` prefix are host CPU
        events, which a GPU run does not have; ``gpu.`` names go to the CUPTI range profiler."""
        from ...runtimes import counters as gc

        dev = self._device
        names = list(self._pmu_counters)
        number = max(int(self._number), 1)
        width = len(names)
        results = [-1.0] * (self._repeat * width)
        positions, metrics = gc.split_counter_names(names)
        notes = []
        host_only = [n for i, n in enumerate(names) if i not in positions]
        if host_only:
            notes.append(f"host CPU counters are not collected for a GPU run: {host_only}")
        handle.run(pointers)  # untimed warm-up, as the timing loop does
        dev.synchronize()
        if metrics:
            handle.set_graph_mode(False)  # plain launches inside the profiled range
            session = None
            try:
                session = gc.GpuCounters(metrics)
                for r in range(self._repeat):
                    values = session.measure(
                        lambda: [handle.run(pointers) for _ in range(number)], dev.synchronize)
                    for pos, value in zip(positions, values):
                        results[r * width + pos] = value / number
            except gc.CountersError as e:
                notes.append(str(e))
            finally:
                if session is not None:
                    session.close()
        if dev.status() != 0:
            raise capi.XtcCudaError(capi.ERR_DEVICE_TIMEOUT, "a kernel's bounded wait gave up")
        return results, "; ".join(notes)

    def _host_parameters(self) -> tuple[list[Any], list[Any]]:
        """(inputs, outputs) as NumPy arrays or device-resident NDArrays."""
        if self._parameters is None:
            assert self._np_inputs_spec is not None and self._np_outputs_spec is not None
            init = np.zeros if self._init_zero else np.empty
            ins = [np_init(spec["shape"], spec["dtype"]) for spec in self._np_inputs_spec()]
            outs = [init(shape=spec["shape"], dtype=spec["dtype"]) for spec in self._np_outputs_spec()]
            return ins, outs
        ins, outs = self._parameters
        return list(ins), list(outs)

    def evaluate(self) -> tuple[list[float], int, str]:
        plan = self._module.plan
        dev = self._device
        try:
            if not dev.detect_accelerator():
                return ([], 1, f"no CUDA device {dev.ordinal} available")
            handle = PlanHandle(plan, dev)
        except (capi.XtcCudaError, RuntimeError) as e:
            return ([], 1, f"Error creating the plan: {e}")
        owned: list[c_void_p] = []
        try:
            ins, outs = self._host_parameters()
            pointers: list[int] = []
            for arr, nbytes in zip(ins + outs, plan.slot_bytes):
                if isinstance(arr, NDArray) and arr.is_on_device():
                    assert arr.nbytes == nbytes, "parameter size does not match the graph"
                    pointers.append(arr.data)
                    continue
                host = arr.numpy() if isinstance(arr, NDArray) else arr
                assert isinstance(host, np.ndarray) and host.nbytes == nbytes, (
                    "parameter size does not match the graph")
                ptr = dev.memory_allocate(nbytes)
                owned.append(ptr)
                pointers.append(int(ptr.value))
            n_in = plan.n_inputs
            for arr, ptr, layout in zip(ins, pointers[:n_in], plan.input_layouts):
                if not (isinstance(arr, NDArray) and arr.is_on_device()):
                    host = arr.numpy() if isinstance(arr, NDArray) else arr
                    if layout is not None and list(layout) == [1, 0]:
                        host = host.T  # the graph declares this input as stored transposed
                    host = np.ascontiguousarray(host)
                    dev.memory_copy_to(c_void_p(ptr), host, host.nbytes)
            if self._init_zero:
                for ptr, nbytes in zip(pointers[n_in:], plan.slot_bytes[n_in:]):
                    dev.memory_fill_zero(c_void_p(ptr), nbytes)

            def read_outputs() -> list[np.ndarray]:
                result = []
                for i, (arr, ptr) in enumerate(zip(outs, pointers[n_in:])):
                    shape = plan.slot_shapes[n_in + i]
                    host = np.empty(shape, dtype=np.float32)
                    dev.memory_copy_from(c_void_p(ptr), host, host.nbytes)
                    result.append(host)
                return result

            if self._validate:
                assert self._reference_impl is not None
                ref_ins = [a.numpy() if isinstance(a, NDArray) else np.asarray(a) for a in ins]
                ref_outs = [np.empty(plan.slot_shapes[n_in + i], dtype=np.float32)
                            for i in range(plan.n_outputs)]
                self._reference_impl(*ref_ins, *ref_outs)
                handle.run(pointers)
                dev.synchronize()
                if dev.status() != 0:
                    return ([], 1, "Error in execution: a kernel's bounded wait gave up")
                for ref, got in zip(ref_outs, read_outputs()):
                    rtol, atol = self._tolerances(ref)
                    if not np.allclose(ref, got, rtol=rtol, atol=atol):
                        return ([], 1, "Error in validation: outputs differ")

            message = ""
            if self._pmu_counters:
                results, message = self._read_counters(handle, pointers)
            else:
                results = handle.evaluate(pointers, self._repeat, self._number, self._min_repeat_ms)

            if self._parameters is not None:
                for arr, got in zip(outs, read_outputs()):
                    if isinstance(arr, np.ndarray):
                        np.copyto(arr, got.reshape(arr.shape))
            return (results, 0, message)
        except capi.XtcCudaError as e:
            return ([], 1, f"Error in execution: {e}")
        finally:
            for ptr in owned:
                try:
                    dev.memory_free(ptr)
                except capi.XtcCudaError:
                    pass
            handle.close()


class CudaExecutor:
    def __init__(self, module: CudaModule, **kwargs: Any) -> None:
        self._evaluator = CudaEvaluator(module, repeat=1, min_repeat_ms=0, number=1, **kwargs)

    def execute(self) -> int:
        _, code, _ = self._evaluator.evaluate()
        return code

    @property
    def module(self) -> CudaModule:
        return self._evaluator.module
