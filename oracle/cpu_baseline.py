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


def run_config(name: str, inputs) -> np.ndarray:
    """The benchmark graphs on the CPU loop nests."""
    if name == "c4a":
        return transpose2d(inputs[0])
    a, b = inputs
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


MATMUL_TILE_CANDIDATES = [(64, 0, 64), (32, 256, 128), (64, 512, 64), (128, 256, 32), (16, 1024, 256)]


def tune_matmul(m: int, n: int, k: int, budget_s: float = 5.0):
    """Pick the fastest of a few (ti, tj, tk) tilings on a row block: a small
    stand-in for the reference's loop-explore search over tile factors."""
    rows = min(m, 512)
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (rows, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    best, best_t = MATMUL_TILE_CANDIDATES[0], float("inf")
    t_start = time.perf_counter()
    for cand in MATMUL_TILE_CANDIDATES:
        t0 = time.perf_counter()
        matmul(a, b, tiles=cand)
        t = time.perf_counter() - t0
        if t < best_t:
            best, best_t = cand, t
        if time.perf_counter() - t_start > budget_s:
            break
    return best
