"""ctypes binding of libxtc_cuda.so (include/xtc_cuda.h).

Loading fails loudly when the library has not been built: there is no CPU or
PyTorch fallback behind these calls.
"""

from __future__ import annotations

import ctypes
from ctypes import (
    POINTER,
    Structure,
    byref,
    c_char_p,
    c_double,
    c_float,
    c_int,
    c_int32,
    c_int64,
    c_size_t,
    c_void_p,
)
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libxtc_cuda.so"

MAX_DIMS = 6

OK = 0
ERR_INVALID = 1
ERR_RUNTIME = 2
ERR_UNSUPPORTED = 3
ERR_DEVICE_TIMEOUT = 4
ERR_NOMEM = 5

GEMM_A_TRANSPOSED = 1
GEMM_B_TRANSPOSED = 2
FUSE_RELU = 4

PRECISION_TF32 = 0
PRECISION_3XTF32 = 1
PRECISION_FP32_SIMT = 2

STEP_GEMM = 1
STEP_CONV2D = 2
STEP_TRANSPOSE = 3
STEP_PAD = 4
STEP_RELU = 5
STEP_COPY = 6


class GemmConfig(Structure):
    _fields_ = [
        ("tile_m", c_int32),
        ("tile_n", c_int32),
        ("tile_k", c_int32),
        ("stages", c_int32),
        ("precision", c_int32),
        ("epilogue", c_int32),
        ("variant", c_int32),
        ("split_k", c_int32),
    ]


class Step(Structure):
    _fields_ = [
        ("kind", c_int32),
        ("in0", c_int32),
        ("in1", c_int32),
        ("out", c_int32),
        ("flags", c_int32),
        ("ndim", c_int32),
        ("relu_threshold", c_float),
        ("pad_value", c_float),
        ("dims", c_int64 * MAX_DIMS),
        ("aux0", c_int64 * MAX_DIMS),
        ("aux1", c_int64 * MAX_DIMS),
        ("cfg", GemmConfig),
    ]


class XtcCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libxtc_cuda error {code}: {message}")
        self.code = code
        self.message = message


# name -> (restype, argtypes); every symbol include/xtc_cuda.h declares.
SIGNATURES: dict[str, tuple] = {
    "xtc_cuda_abi_version": (c_int, []),
    "xtc_cuda_device_count": (c_int, [POINTER(c_int)]),
    "xtc_cuda_set_device": (c_int, [c_int]),
    "xtc_cuda_get_device": (c_int, [POINTER(c_int)]),
    "xtc_cuda_device_name": (c_int, [c_int, c_char_p, c_size_t]),
    "xtc_cuda_malloc": (c_int, [POINTER(c_void_p), c_size_t]),
    "xtc_cuda_free": (c_int, [c_void_p]),
    "xtc_cuda_host_alloc": (c_int, [POINTER(c_void_p), c_size_t]),
    "xtc_cuda_host_free": (c_int, [c_void_p]),
    "xtc_cuda_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "xtc_cuda_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "xtc_cuda_memcpy_d2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "xtc_cuda_memset": (c_int, [c_void_p, c_int, c_size_t, c_void_p]),
    "xtc_cuda_stream_create": (c_int, [POINTER(c_void_p)]),
    "xtc_cuda_stream_destroy": (c_int, [c_void_p]),
    "xtc_cuda_stream_synchronize": (c_int, [c_void_p]),
    "xtc_cuda_device_synchronize": (c_int, []),
    "xtc_cuda_event_create": (c_int, [POINTER(c_void_p)]),
    "xtc_cuda_event_destroy": (c_int, [c_void_p]),
    "xtc_cuda_event_record": (c_int, [c_void_p, c_void_p]),
    "xtc_cuda_event_synchronize": (c_int, [c_void_p]),
    "xtc_cuda_stream_wait_event": (c_int, [c_void_p, c_void_p]),
    "xtc_cuda_device_status": (c_int, [POINTER(c_int)]),
    "xtc_cuda_mem_info": (c_int, [POINTER(c_size_t), POINTER(c_size_t)]),
    "xtc_cuda_selftest_bounded_wait": (c_int, [c_int, c_void_p]),
    "xtc_cuda_step_workspace_bytes": (c_int, [POINTER(Step), POINTER(c_size_t), POINTER(c_size_t)]),
    "xtc_cuda_last_error": (c_char_p, []),
    "xtc_cuda_gemm_f32": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
         c_int, c_float, POINTER(GemmConfig), c_void_p, c_size_t, c_void_p],
    ),
    "xtc_cuda_gemm_f32_bcast": (
        c_int,
        [c_void_p, c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int64, c_int64, c_int64,
         c_int64, c_int64, c_int64, c_int, c_float, POINTER(GemmConfig), c_void_p, c_size_t,
         c_void_p],
    ),
    "xtc_cuda_gemm_f32_mcast": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
         c_int64, c_int, c_float, POINTER(GemmConfig), c_void_p, c_size_t, c_void_p],
    ),
    "xtc_cuda_ipc_export": (c_int, [c_void_p, c_void_p]),
    "xtc_cuda_ipc_import": (c_int, [c_void_p, POINTER(c_void_p)]),
    "xtc_cuda_ipc_release": (c_int, [c_void_p]),
    "xtc_cuda_comm_unique_id": (c_int, [c_void_p]),
    "xtc_cuda_comm_init": (c_int, [POINTER(c_void_p), c_int, c_int, c_void_p]),
    "xtc_cuda_allgather_rows": (
        c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p],
    ),
    "xtc_cuda_comm_destroy": (c_int, [c_void_p]),
    "xtc_cuda_peer_barrier": (
        c_int, [c_void_p, POINTER(c_void_p), POINTER(c_int), c_int, c_int, c_int, c_void_p],
    ),
    "xtc_cuda_gemm_f32_3xtf32_noalloc": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_float, c_void_p],
    ),
    "xtc_cuda_gemm_default_config": (c_int, [c_int64, c_int64, c_int64, POINTER(GemmConfig)]),
    "xtc_cuda_gemm_workspace_bytes": (
        c_int, [c_int64, c_int64, c_int64, c_int, POINTER(GemmConfig), POINTER(c_size_t)],
    ),
    "xtc_cuda_conv2d_nhwc_f32": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
         POINTER(GemmConfig), c_void_p, c_size_t, c_void_p],
    ),
    "xtc_cuda_conv2d_workspace_bytes": (
        c_int,
        [c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int,
         c_int, c_int, c_int, POINTER(GemmConfig), POINTER(c_size_t)],
    ),
    "xtc_cuda_transpose_f32": (
        c_int, [c_void_p, c_void_p, c_int, POINTER(c_int64), POINTER(c_int32), c_void_p],
    ),
    "xtc_cuda_pad_f32": (
        c_int,
        [c_void_p, c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
         c_float, c_void_p],
    ),
    "xtc_cuda_relu_f32": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "xtc_cuda_split_tf32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "xtc_cuda_plan_create": (
        c_int,
        [POINTER(c_void_p), POINTER(Step), c_int, c_int, c_int, c_int, POINTER(c_size_t)],
    ),
    "xtc_cuda_plan_destroy": (c_int, [c_void_p]),
    "xtc_cuda_plan_run": (c_int, [c_void_p, POINTER(c_void_p), c_void_p]),
    "xtc_cuda_plan_run_sets": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_void_p]),
    "xtc_cuda_plan_set_graph_mode": (c_int, [c_void_p, c_int]),
    "xtc_cuda_plan_run_host": (c_int, [c_void_p, POINTER(c_void_p)]),
    "xtc_cuda_pipeline_create": (c_int, [POINTER(c_void_p), c_void_p, c_int]),
    "xtc_cuda_pipeline_submit": (c_int, [c_void_p, POINTER(c_void_p)]),
    "xtc_cuda_pipeline_wait": (c_int, [c_void_p]),
    "xtc_cuda_pipeline_destroy": (c_int, [c_void_p]),
    "xtc_cuda_evaluate": (
        c_int, [c_void_p, POINTER(c_void_p), c_int, c_int, c_int, POINTER(c_double)],
    ),
    "xtc_cuda_plan_step_count": (c_int, [c_void_p, POINTER(c_int)]),
    "xtc_cuda_peak_fma": (c_int, [c_char_p, POINTER(c_double)]),
    "xtc_cuda_mma_rate": (c_int, [c_int, c_int, POINTER(c_double)]),
}

_lib: ctypes.CDLL | None = None


def load(path: str | Path | None = None) -> ctypes.CDLL:
    """dlopen the library and bind every signature.  Raises if it is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path is not None else LIB_PATH
    if not p.exists():
        raise RuntimeError(
            f"{p} is missing: build it with `python -m xtc_b200.build` "
            "(nvcc, sm_100a). There is no fallback implementation."
        )
    lib = ctypes.CDLL(str(p))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.xtc_cuda_abi_version() != 1:
        raise RuntimeError("libxtc_cuda.so ABI version mismatch")
    if path is None:
        _lib = lib
    return lib


def last_error() -> str:
    msg = load().xtc_cuda_last_error()
    return msg.decode(errors="replace") if msg else ""


def check(code: int) -> None:
    if code != OK:
        raise XtcCudaError(code, last_error())


def i64_array(values) -> ctypes.Array:
    vals = list(values)
    return (c_int64 * len(vals))(*vals)


def i32_array(values) -> ctypes.Array:
    vals = list(values)
    return (c_int32 * len(vals))(*vals)


__all__ = [
    "load", "check", "last_error", "XtcCudaError", "GemmConfig", "Step", "SIGNATURES",
    "byref", "i64_array", "i32_array",
]
