"""Device runtime and device-resident arrays over the C ABI.

``CudaDevice`` takes the role of the reference's ``GPUDevice``
(``runtimes/accelerator/gpu/GPUDevice.py:33-353``): one object per GPU ordinal
with the ``memory_*`` calls of ``itf/runtime/accelerator.py:69-135`` -- but it
talks to ``libxtc_cuda.so`` instead of MLIR's CUDA runtime wrappers, and it
knows about more than device 0.  ``NDArray`` mirrors
``runtimes/types/ndarray.py:27-237``: built from a NumPy array, optionally
placed on a device, read back with ``.numpy()``.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Any

import numpy as np

from .. import capi
from ..capi import byref, c_void_p


class CudaDevice:
    """One B200 as seen through ``libxtc_cuda.so``."""

    _instances: dict[int, "CudaDevice"] = {}
    _lock = threading.Lock()

    def __new__(cls, ordinal: int = 0) -> "CudaDevice":
        with cls._lock:
            inst = cls._instances.get(ordinal)
            if inst is None:
                inst = super().__new__(cls)
                inst._init(ordinal)
                cls._instances[ordinal] = inst
        return inst

    def _init(self, ordinal: int) -> None:
        self.lib = capi.load()
        self.ordinal = ordinal
        self._name: str | None = None

    # -- identification ------------------------------------------------------
    @staticmethod
    def count() -> int:
        n = ctypes.c_int(0)
        capi.check(capi.load().xtc_cuda_device_count(byref(n)))
        return n.value

    def detect_accelerator(self) -> bool:
        try:
            return self.count() > self.ordinal
        except capi.XtcCudaError:
            return False

    def init_device(self) -> None:
        self.activate()

    def deinit_device(self) -> None:
        pass

    def activate(self) -> None:
        capi.check(self.lib.xtc_cuda_set_device(self.ordinal))

    def target_name(self) -> str:
        return "cuda"

    def device_name(self) -> str:
        if self._name is None:
            buf = ctypes.create_string_buffer(256)
            capi.check(self.lib.xtc_cuda_device_name(self.ordinal, buf, 256))
            self._name = buf.value.decode()
        return self._name

    def device_arch(self) -> str:
        return "sm_100a"

    def device_id(self) -> int:
        return self.ordinal

    # -- memory --------------------------------------------------------------
    def memory_allocate(self, size_bytes: int) -> c_void_p:
        self.activate()
        ptr = c_void_p()
        capi.check(self.lib.xtc_cuda_malloc(byref(ptr), int(size_bytes)))
        return ptr

    def memory_free(self, handle: c_void_p) -> None:
        if handle is not None and handle.value:
            self.activate()
            capi.check(self.lib.xtc_cuda_free(handle))

    def memory_copy_to(self, acc_handle: c_void_p, src: Any, size_bytes: int) -> None:
        self.activate()
        capi.check(self.lib.xtc_cuda_memcpy_h2d(acc_handle, _as_void_p(src), int(size_bytes), None))
        capi.check(self.lib.xtc_cuda_stream_synchronize(None))

    def memory_copy_from(self, acc_handle: c_void_p, dst: Any, size_bytes: int) -> None:
        self.activate()
        capi.check(self.lib.xtc_cuda_memcpy_d2h(_as_void_p(dst), acc_handle, int(size_bytes), None))
        capi.check(self.lib.xtc_cuda_stream_synchronize(None))

    def memory_fill_zero(self, acc_handle: c_void_p, size_bytes: int) -> None:
        self.activate()
        capi.check(self.lib.xtc_cuda_memset(acc_handle, 0, int(size_bytes), None))

    def memory_data_pointer(self, acc_handle: c_void_p) -> c_void_p:
        return acc_handle

    def synchronize(self) -> None:
        self.activate()
        capi.check(self.lib.xtc_cuda_device_synchronize())

    def status(self) -> int:
        """Reads and clears the word kernels set when a bounded wait gives up."""
        self.activate()
        s = ctypes.c_int(0)
        capi.check(self.lib.xtc_cuda_device_status(byref(s)))
        return s.value

    def evaluate_flops(self, dtype_name: str | bytes) -> float:
        """Tensor-pipe peak in FMA/s (the unit of the reference's evaluate_flops)."""
        self.activate()
        name = dtype_name if isinstance(dtype_name, bytes) else dtype_name.encode()
        out = ctypes.c_double(0.0)
        capi.check(self.lib.xtc_cuda_peak_fma(name, byref(out)))
        return out.value


def _as_void_p(obj: Any) -> c_void_p:
    if isinstance(obj, np.ndarray):
        return obj.ctypes.data_as(c_void_p)
    if isinstance(obj, c_void_p):
        return obj
    return c_void_p(int(obj))


class NDArray:
    """A host array with an optional device mirror."""

    def __init__(self, array: Any, runtime: CudaDevice | None = None,
                 layout: list[int] | None = None) -> None:
        if isinstance(array, NDArray):
            raise RuntimeError("copy from NDArray not supported")
        assert isinstance(array, np.ndarray)
        self.layout = layout
        self.runtime = runtime
        if self.is_transposed():
            array = np.ascontiguousarray(array.T)
        self._host = np.ascontiguousarray(array)
        self.device_handle: c_void_p | None = None
        if isinstance(runtime, CudaDevice):
            self._to_device()

    def is_transposed(self) -> bool:
        if self.layout is None:
            return False
        assert len(self.layout) == 2, "Only 2D layouts are implemented"
        return list(self.layout) == [1, 0]

    def is_on_device(self) -> bool:
        return self.device_handle is not None

    def _to_device(self) -> None:
        assert isinstance(self.runtime, CudaDevice)
        self.device_handle = self.runtime.memory_allocate(self._host.nbytes)
        self.runtime.memory_copy_to(self.device_handle, self._host, self._host.nbytes)

    def numpy(self, out: np.ndarray | None = None) -> np.ndarray:
        if self.is_on_device():
            self.runtime.memory_copy_from(self.device_handle, self._host, self._host.nbytes)
        result = self._host.T.copy() if self.is_transposed() else self._host
        if out is None:
            return np.array(result)
        assert out.flags["C_CONTIGUOUS"] and out.dtype == result.dtype and out.size == result.size
        np.copyto(out, result.reshape(out.shape))
        return out

    @property
    def data(self) -> int:
        """Address of the payload: the device pointer when on a device."""
        if self.is_on_device():
            return int(self.device_handle.value)
        return int(self._host.ctypes.data)

    dtype = property(lambda self: self._host.dtype)
    dtype_str = property(lambda self: str(self._host.dtype))
    shape = property(lambda self: tuple(self._host.shape))
    ndim = property(lambda self: self._host.ndim)
    size = property(lambda self: self._host.size)
    nbytes = property(lambda self: self._host.nbytes)

    def __del__(self) -> None:
        handle, self.device_handle = getattr(self, "device_handle", None), None
        if handle is not None:
            try:
                self.runtime.memory_free(handle)
            except Exception:
                pass
