"""Randomised parity of the C-ABI entry points with the oracle, on a real GPU.

Seeded random shapes (ragged, tiny, unaligned), operand layouts, fused relu
thresholds and kernel configurations (automatic and explicit tiles, every
precision, split-K with and without a workspace) go through
``xtc_cuda_gemm_f32``, ``xtc_cuda_conv2d_nhwc_f32``, ``xtc_cuda_transpose_f32``
and ``xtc_cuda_pad_f32`` and are compared with oracle/xtc_oracle.py evaluated in
float64.  A configuration the library does not implement must be refused with a
message (never run wrongly); every accepted call must be within tolerance, leave
the device status word at 0 and leave the guard bands around its output
untouched.  Calls that were given a workspace run twice on it: the kernels must
leave it reusable.

Tolerances as in test_cuda_parity.py: TF32 1e-2, 3xTF32 / fp32 2e-5 of
max|y64|; transpose and pad bit-exact.
"""

import ctypes
import random

import numpy as np
import pytest

from oracle import xtc_oracle as xo
from xtc_b200.capi import GemmConfig, byref, c_void_p
from xtc_b200.runtimes.cuda import CudaDevice

pytestmark = pytest.mark.gpu

GUARD = 1024  # floats on each side of an output
SENTINEL = np.float32(7777.0)
A_T, B_T, RELU = 1, 2, 4


@pytest.fixture(scope="module")
def dev(cuda_lib):
    d = CudaDevice(0)
    assert d.detect_accelerator(), "no CUDA device: the gpu tests need one"
    d.activate()
    return d


class DeviceArray:
    """A device copy of a host array, optionally between two guard bands."""

    def __init__(self, dev, host: np.ndarray, guard: int = 0):
        self.dev, self.guard, self.n = dev, guard, host.size
        full = np.full(host.size + 2 * guard, SENTINEL, np.float32)
        full[guard:guard + host.size] = host.reshape(-1)
        self.base = dev.memory_allocate(max(full.nbytes, 4))
        dev.memory_copy_to(self.base, full, full.nbytes)
        self.ptr = c_void_p(self.base.value + 4 * guard)

    def read(self) -> tuple[np.ndarray, bool]:
        full = np.empty(self.n + 2 * self.guard, np.float32)
        self.dev.memory_copy_from(self.base, full, full.nbytes)
        g = self.guard
        intact = bool((full[:g] == SENTINEL).all() and (full[g + self.n:] == SENTINEL).all())
        return full[g:g + self.n], intact

    def free(self):
        self.dev.memory_free(self.base)


def workspace(dev, nbytes: int):
    return DeviceArray(dev, np.zeros(nbytes // 4 + 16, np.float32))


def last_error(dev) -> str:
    return (dev.lib.xtc_cuda_last_error() or b"").decode()


def pick_dim(rng: random.Random, top: int) -> int:
    k = rng.random()
    if k < 0.3:
        return rng.choice([1, 2, 3, 4, 7, 8, 16, 31, 32, 33, 64, 100, 127, 128, 129])
    if k < 0.7:
        return 4 * rng.randint(1, top // 4)
    return rng.randint(1, top)


def random_config(rng: random.Random, conv: bool) -> GemmConfig:
    cfg = GemmConfig()
    if rng.random() > 0.4:
        cfg.tile_m = rng.choice([0, 128, 256])
        cfg.tile_n = rng.choice([0, 64, 128, 256])
        cfg.tile_k = rng.choice([0, 32, 64])
        cfg.stages = rng.choice([0, 0, 2, 3, 4])
        cfg.epilogue = rng.choice([0, 1, 2])
        cfg.split_k = rng.choice([0, 0, 1, 2, 3, 4, 5, 6, 7, 8])
        if conv:
            cfg.variant = rng.choice([0, 1, 2, 3, 4, 5])
    cfg.precision = rng.choice([0, 0, 0, 2] if conv else [0, 0, 0, 1, 2])
    return cfg


def describe(cfg: GemmConfig) -> list[int]:
    return [cfg.tile_m, cfg.tile_n, cfg.tile_k, cfg.stages, cfg.precision, cfg.epilogue,
            cfg.variant, cfg.split_k]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_gemm_calls(dev, seed):
    rng = random.Random(1000 + seed)
    nprng = np.random.default_rng(1000 + seed)
    lib = dev.lib
    accepted = 0
    for _ in range(40):
        M, N, K = pick_dim(rng, 1200), pick_dim(rng, 1200), pick_dim(rng, 1500)
        flags = rng.choice([0, 0, 0, A_T, B_T, A_T | B_T]) | rng.choice([0, RELU])
        thr = rng.choice([0.0, 0.0, 0.1])
        cfg = random_config(rng, conv=False)
        a = nprng.uniform(-0.5, 0.5, (K, M) if flags & A_T else (M, K)).astype(np.float32)
        b = nprng.uniform(-0.5, 0.5, (N, K) if flags & B_T else (K, N)).astype(np.float32)
        case = f"gemm M={M} N={N} K={K} flags={flags} thr={thr} cfg={describe(cfg)}"
        nbytes = ctypes.c_size_t(0)
        rc = lib.xtc_cuda_gemm_workspace_bytes(M, N, K, flags, byref(cfg), byref(nbytes))
        ws = None
        if rc == 0 and nbytes.value and (cfg.precision == 1 or rng.random() < 0.7):
            ws = workspace(dev, nbytes.value)
        da, db = DeviceArray(dev, a), DeviceArray(dev, b)
        dc = DeviceArray(dev, np.full(M * N, np.nan, np.float32), GUARD)
        y64 = xo.matmul((a.T if flags & A_T else a).astype(np.float64),
                        (b.T if flags & B_T else b).astype(np.float64))
        if flags & RELU:
            y64 = xo.relu(y64, thr)
        tol = 1e-2 if cfg.precision == 0 else 2e-5
        for run in range(2 if ws is not None else 1):
            rc = lib.xtc_cuda_gemm_f32(da.ptr, db.ptr, dc.ptr, M, N, K, a.shape[1], b.shape[1], N,
                                       flags, thr, byref(cfg), ws.ptr if ws else None,
                                       4 * ws.n if ws else 0, None)
            if rc != 0:
                assert last_error(dev).startswith("gemm:"), f"{case}: refused without a message"
                break
            dev.synchronize()
            y, intact = dc.read()
            assert dev.status() == 0, case
            assert intact, f"{case}: wrote outside C"
            err = np.abs(y.reshape(M, N) - y64).max() / max(np.abs(y64).max(), 1e-6)
            assert err <= tol, f"{case} run {run}: error {err}"
            accepted += run == 0
        for d in (da, db, dc, ws):
            if d is not None:
                d.free()
    assert accepted >= 25  # most of the random space is implemented


@pytest.mark.parametrize("seed", [0, 1])
def test_random_conv2d_calls(dev, seed):
    rng = random.Random(2000 + seed)
    nprng = np.random.default_rng(2000 + seed)
    lib = dev.lib
    accepted = 0
    for _ in range(40):
        B, H, W = rng.randint(1, 3), rng.randint(3, 30), rng.randint(3, 30)
        C = rng.choice([1, 3, 4, 8, 16, 32, 64, 128, 20])
        F = rng.choice([1, 5, 8, 16, 24, 64, 128, 256])
        R, S = rng.randint(1, 5), rng.randint(1, 5)
        sh, sw = rng.choice([1, 1, 2, 3]), rng.choice([1, 1, 2])
        pt, pb, pl, pr = (rng.choice([0, 0, 1, 2]) for _ in range(4))
        if H + pt + pb < R or W + pl + pr < S:
            continue
        flags, thr = rng.choice([0, RELU]), rng.choice([0.0, 0.05])
        cfg = random_config(rng, conv=True)
        case = (f"conv B={B} H={H} W={W} C={C} R={R} S={S} F={F} stride={sh, sw} "
                f"pad={pt, pb, pl, pr} flags={flags} thr={thr} cfg={describe(cfg)}")
        x = nprng.uniform(0, 1, (B, H, W, C)).astype(np.float32)
        w = (0.2 * nprng.standard_normal((R, S, C, F))).astype(np.float32)
        xp = xo.pad(x.astype(np.float64), {1: (pt, pb), 2: (pl, pr)}, 0.0)
        y64 = xo.conv2d(xp, w.astype(np.float64), (sh, sw))
        if flags & RELU:
            y64 = xo.relu(y64, thr)
        nbytes = ctypes.c_size_t(0)
        rc = lib.xtc_cuda_conv2d_workspace_bytes(B, H, W, C, R, S, F, sh, sw, pt, pb, pl, pr,
                                                 byref(cfg), byref(nbytes))
        ws = workspace(dev, nbytes.value) if rc == 0 and nbytes.value and rng.random() < 0.8 else None
        dx, dw = DeviceArray(dev, x), DeviceArray(dev, w)
        dy = DeviceArray(dev, np.full(y64.size, np.nan, np.float32), GUARD)
        tol = 1e-2 if cfg.precision == 0 else 2e-5
        for run in range(2 if ws is not None else 1):
            rc = lib.xtc_cuda_conv2d_nhwc_f32(dx.ptr, dw.ptr, dy.ptr, B, H, W, C, R, S, F, sh, sw,
                                              pt, pb, pl, pr, flags, thr, byref(cfg),
                                              ws.ptr if ws else None, 4 * ws.n if ws else 0, None)
            if rc != 0:
                assert last_error(dev).startswith(("conv2d:", "gemm:")), f"{case}: refused without a message"
                break
            dev.synchronize()
            y, intact = dy.read()
            assert dev.status() == 0, case
            assert intact, f"{case}: wrote outside Y"
            err = np.abs(y.reshape(y64.shape) - y64).max() / max(np.abs(y64).max(), 1e-6)
            assert err <= tol, f"{case} run {run}: error {err}"
            accepted += run == 0
        for d in (dx, dw, dy, ws):
            if d is not None:
                d.free()
    assert accepted >= 20


def random_shape(rng: random.Random, ndim: int, budget: int) -> list[int]:
    while True:
        if ndim == 2 and rng.random() < 0.5:
            shape = [rng.choice([63, 64, 65, 128, 192, 257, 1000, 1024, 2048]),
                     rng.choice([4, 64, 100, 128, 320, 1024, 2048])]
        else:
            shape = [rng.choice([1, 2, 3, 4, 5, 7, 8, 16, 31, 32, 64, 65, 128, 200]) for _ in range(ndim)]
        if int(np.prod(shape)) <= budget:
            return shape


def test_random_transposes_are_bit_exact(dev):
    rng = random.Random(3000)
    nprng = np.random.default_rng(3000)
    for _ in range(80):
        ndim = rng.randint(1, 6)
        shape = random_shape(rng, ndim, 1 << 21)
        axes = list(range(ndim))
        rng.shuffle(axes)
        if rng.random() < 0.3:
            axes.reverse()
        x = nprng.standard_normal(shape).astype(np.float32)
        want = np.ascontiguousarray(xo.transpose(x, axes))
        dx = DeviceArray(dev, x)
        dy = DeviceArray(dev, np.full(x.size, np.nan, np.float32), GUARD)
        rc = dev.lib.xtc_cuda_transpose_f32(dx.ptr, dy.ptr, ndim, (ctypes.c_int64 * ndim)(*shape),
                                            (ctypes.c_int32 * ndim)(*axes), None)
        assert rc == 0, f"transpose {shape} {axes}: {last_error(dev)}"
        dev.synchronize()
        y, intact = dy.read()
        assert dev.status() == 0 and intact, f"transpose {shape} {axes}"
        assert np.array_equal(y.view(np.int32), want.reshape(-1).view(np.int32)), f"transpose {shape} {axes}"
        dx.free()
        dy.free()


def test_random_pads_and_crops_are_bit_exact(dev):
    rng = random.Random(4000)
    nprng = np.random.default_rng(4000)
    done = 0
    for _ in range(100):
        ndim = rng.randint(1, 5)
        shape = random_shape(rng, ndim, 1 << 19)
        lo = [rng.choice([0, 0, 1, 2, 3, -1]) for _ in range(ndim)]
        hi = [rng.choice([0, 0, 1, 2, 5, -1]) for _ in range(ndim)]
        if min(s + l + h for s, l, h in zip(shape, lo, hi)) < 1:
            continue
        value = rng.choice([0.0, 0.0, -1.5, float("inf")])
        x = nprng.standard_normal(shape).astype(np.float32)
        # negative widths crop (O.unpad), positive ones pad with the constant
        crop = [(max(-l, 0), max(-h, 0)) for l, h in zip(lo, hi)]
        grow = [(max(l, 0), max(h, 0)) for l, h in zip(lo, hi)]
        want = np.ascontiguousarray(xo.pad(xo.unpad(x, tuple(crop)), tuple(grow), value))
        dx = DeviceArray(dev, x)
        dy = DeviceArray(dev, np.full(want.size, np.nan, np.float32), GUARD)
        rc = dev.lib.xtc_cuda_pad_f32(dx.ptr, dy.ptr, ndim, (ctypes.c_int64 * ndim)(*shape),
                                      (ctypes.c_int64 * ndim)(*lo), (ctypes.c_int64 * ndim)(*hi),
                                      ctypes.c_float(value), None)
        assert rc == 0, f"pad {shape} {lo} {hi}: {last_error(dev)}"
        dev.synchronize()
        y, intact = dy.read()
        assert dev.status() == 0 and intact, f"pad {shape} {lo} {hi}"
        assert np.array_equal(y.view(np.int32), want.reshape(-1).view(np.int32)), f"pad {shape} {lo} {hi} {value}"
        dx.free()
        dy.free()
        done += 1
    assert done >= 60
