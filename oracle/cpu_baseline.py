"""Loader and timing helpers of the CPU loop-nest restatement (oracle/cpu_loopnest.c).

TEST / BASELINE INFRASTRUCTURE: imported only by tests/, __graft_entry__.py and
the cpu_baseline / reference legs of bench.py.
"""

from __future__ import annotations

import ctypes
import subprocess
import time
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libxtc_cpu_ref.so"


def build(force: bool = False) -> Path:
    src = HERE / "cpu_loopnest.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "libxtc_cpu_ref.so"], check=True,
                       capture_output=True)
    return LIB


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(build()))
        lib.xtc_ref_max_threads.restype = c_int
        lib.xtc_ref_matmul.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                       c_int64, c_int64, c_int64, c_int]
        lib.xtc_ref_conv2d.argtypes = [c_void_p, c_void_p, c_void_p] + [c_int64] * 9 + [c_int]
        lib.xtc_ref_relu.argtypes = [c_void_p, c_void_p, c_int64, c_float]
        lib.xtc_ref_pad_hw.argtypes = [c_void_p, c_void_p] + [c_int64] * 8 + [c_float]
        lib.xtc_ref_transpose2d.argtypes = [c_void_p, c_void_p, c_int64, c_int64]
        lib.xtc_ref_matmul_blocked.argtypes = [c_void_p] * 3 + [c_int64] * 6 + [c_int, c_int]
        lib.xtc_ref_matmul_blocked.restype = c_int
        lib.xtc_ref_conv2d_blocked.argtypes = [c_void_p] * 3 + [c_int64] * 9 + [c_int, c_int]
        lib.xtc_ref_conv2d_blocked.restype = c_int
        lib.xtc_ref_micro_shape.argtypes = [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
        lib.xtc_ref_conv_micro_shape.argtypes = [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
        lib.xtc_ref_peak_fma.restype = ctypes.c_double
        _lib = lib
    return _lib


def _p(a: np.ndarray) -> c_void_p:
    return a.ctypes.data_as(c_void_p)


def threads() -> int:
    return int(load().xtc_ref_max_threads())


def matmul(a: np.ndarray, b: np.ndarray, relu: bool = False, tiles=(64, 0, 64)) -> np.ndarray:
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    load().xtc_ref_matmul(_p(a), _p(b), _p(c), m, n, k, tiles[0], tiles[1], tiles[2], int(relu))
    return c


def conv2d(x: np.ndarray, w: np.ndarray, stride=(1, 1), relu: bool = False) -> np.ndarray:
    b, h, wd, c = x.shape
    r, s, _, f = w.shape
    oh, ow = (h - r) // stride[0] + 1, (wd - s) // stride[1] + 1
    y = np.empty((b, oh, ow, f), np.float32)
    load().xtc_ref_conv2d(_p(x), _p(w), _p(y), b, h, wd, c, r, s, f, stride[0], stride[1], int(relu))
    return y


def micro_shapes() -> list[tuple[int, int]]:
    """(rows, columns) of the register tile of every matmul micro-kernel, by index."""
    lib, out = load(), []
    for i in range(lib.xtc_ref_micro_count()):
        r, c = c_int(), c_int()
        lib.xtc_ref_micro_shape(i, ctypes.byref(r), ctypes.byref(c))
        out.append((r.value, c.value))
    return out


def conv_micro_shapes() -> list[tuple[int, int]]:
    """(pixels, filters) of the register tile of every conv2d micro-kernel, by index."""
    lib, out = load(), []
    for i in range(lib.xtc_ref_conv_micro_count()):
        r, c = c_int(), c_int()
        lib.xtc_ref_conv_micro_shape(i, ctypes.byref(r), ctypes.byref(c))
        out.append((r.value, c.value))
    return out


def peak_fma() -> float:
    """FMA/s of the host cores (register-resident vector FMA chains on every thread)."""
    return float(load().xtc_ref_peak_fma())


def matmul_blocked(a: np.ndarray, b: np.ndarray, sample=(128, 512, 256, 7), relu: bool = False,
                   out: np.ndarray | None = None) -> np.ndarray:
    """The two-level tiled, packed, register-blocked nest; sample = (mc, nc, kc, micro)."""
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32) if out is None else out
    rc = load().xtc_ref_matmul_blocked(_p(a), _p(b), _p(c), m, n, k, int(sample[0]), int(sample[1]),
                                       int(sample[2]), int(sample[3]), int(relu))
    if rc:
        raise ValueError(f"illegal matmul sample {tuple(sample)}")
    return c


def conv2d_blocked(x: np.ndarray, w: np.ndarray, stride=(1, 1), micro: int = 2, relu: bool = False,
                   out: np.ndarray | None = None) -> np.ndarray:
    b, h, wd, c = x.shape
    r, s, _, f = w.shape
    oh, ow = (h - r) // stride[0] + 1, (wd - s) // stride[1] + 1
    y = np.empty((b, oh, ow, f), np.float32) if out is None else out
    rc = load().xtc_ref_conv2d_blocked(_p(x), _p(w), _p(y), b, h, wd, c, r, s, f, stride[0], stride[1],
                                       int(micro), int(relu))
    if rc:
        raise ValueError(f"illegal conv2d micro-kernel {micro}")
    return y


def relu(x: np.ndarray, threshold: float = 0.0) -> np.ndarray:
    y = np.empty_like(x)
    load().xtc_ref_relu(_p(x), _p(y), x.size, threshold)
    return y


def pad_hw(x: np.ndarray, pt: int, pb: int, pl: int, pr: int, value: float = 0.0) -> np.ndarray:
    b, h, w, c = x.shape
    y = np.empty((b, h + pt + pb, w + pl + pr, c), np.float32)
    load().xtc_ref_pad_hw(_p(x), _p(y), b, h, w, c, pt, pb, pl, pr, value)
    return y


def transpose2d(x: np.ndarray) -> np.ndarray:
    r, c = x.shape
    y = np.empty((c, r), np.float32)
    load().xtc_ref_transpose2d(_p(x), _p(y), r, c)
    return y


def run_config(name: str, inputs, sample=None) -> np.ndarray:
    """The benchmark graphs on the CPU loop nests.  `sample` selects the register-blocked
    nests with that tuned sample ((mc, nc, kc, micro) for the matmul graphs, (micro,) for
    c3); None runs the one-level nests with their fixed default tiles."""
    if name == "c4a":
        return transpose2d(inputs[0])
    a, b = inputs
    if sample is not None:
        if name == "c3":
            return conv2d_blocked(pad_hw(a, 1, 1, 1, 1, 0.0), b, (1, 1), micro=sample[0], relu=True)
        lhs = transpose2d(a) if name == "c4" else a
        return matmul_blocked(lhs, b, sample, relu=name == "c2")
    if name == "c1":
        return matmul(a, b)
    if name == "c2":
        return matmul(a, b, relu=True)
    if name == "c3":
        return conv2d(pad_hw(a, 1, 1, 1, 1, 0.0), b, (1, 1), relu=True)
    if name == "c4":
        return matmul(transpose2d(a), b)
    if name == "c5":
        return matmul(a, b)
    raise KeyError(name)
