"""The allocation-free 3xTF32 GEMM entry point, through the C ABI.

`xtc_cuda_gemm_f32_3xtf32_noalloc` serves callers that may not touch the device
allocator: a process whose own memory pool already owns the whole GPU, or a
latency-critical loop that cannot afford the device-wide synchronisation of
cudaMalloc / cudaFree.  Its operand-split scratch is a fixed 32 MiB array inside
the library instead of a caller workspace.  It must give the results of the
regular entry point (`xtc_cuda_gemm_f32`, precision 3xTF32, caller workspace),
call after call, although all calls share that one array.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.  It also passes when run alone in a fresh
process (the first call on a device does the one-time address look-up).
"""

import ctypes

import numpy as np
import pytest

from xtc_b200 import capi
from xtc_b200.capi import GemmConfig, byref, c_void_p
from xtc_b200.runtimes.cuda import CudaDevice

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5  # max|y - y64| / max|y64|, the tolerance of the 3xTF32 mode in the other GPU tests


def _rel_err(y, y64):
    return float(np.max(np.abs(y.astype(np.float64) - y64)) / np.max(np.abs(y64)))


def _put(dev, arr):
    arr = np.ascontiguousarray(arr)
    p = dev.memory_allocate(arr.nbytes)
    dev.memory_copy_to(p, arr, arr.nbytes)
    return p


def _get(dev, p, shape):
    out = np.empty(shape, np.float32)
    dev.memory_copy_from(p, out, out.nbytes)
    return out


def _both_entry_points(dev, A, B, flags, thr):
    """(result of the regular 3xTF32 entry point, result of the no-alloc one)."""
    lib = dev.lib
    a_t, b_t = bool(flags & capi.GEMM_A_TRANSPOSED), bool(flags & capi.GEMM_B_TRANSPOSED)
    M, K = A.shape
    N = B.shape[1]
    As = np.ascontiguousarray(A.T) if a_t else A
    Bs = np.ascontiguousarray(B.T) if b_t else B
    dA, dB = _put(dev, As), _put(dev, Bs)
    dC1, dC2 = dev.memory_allocate(M * N * 4), dev.memory_allocate(M * N * 4)
    for d in (dC1, dC2):
        capi.check(lib.xtc_cuda_memset(d, 0xFF, M * N * 4, None))
    cfg = GemmConfig(precision=capi.PRECISION_3XTF32, tile_n=64 if N <= 64 else 128, tile_k=32,
                     epilogue=1)
    ws = ctypes.c_size_t(0)
    capi.check(lib.xtc_cuda_gemm_workspace_bytes(M, N, K, flags, byref(cfg), byref(ws)))
    dW = dev.memory_allocate(ws.value)
    capi.check(lib.xtc_cuda_gemm_f32(dA, dB, dC1, M, N, K, As.shape[1], Bs.shape[1], N, flags, thr,
                                     byref(cfg), dW, ws.value, None))
    capi.check(lib.xtc_cuda_gemm_f32_3xtf32_noalloc(dA, dB, dC2, M, N, K, flags, thr, None))
    dev.synchronize()
    regular, noalloc = _get(dev, dC1, (M, N)), _get(dev, dC2, (M, N))
    for d in (dA, dB, dC1, dC2, dW):
        dev.memory_free(d)
    return regular, noalloc


def test_noalloc_gemm_matches_the_regular_entry_point_twice_in_a_row(cuda_lib):
    dev = CudaDevice(0)
    assert dev.detect_accelerator(), "this test needs a CUDA device"
    dev.activate()
    rng = np.random.default_rng(2026)
    # two calls in a row with different shapes and data: the second must not see the first's scratch
    cases = [((512, 1024, 256), 0, 0.0),
             ((384, 640, 200), capi.FUSE_RELU | capi.GEMM_A_TRANSPOSED, 0.125)]
    for (M, K, N), flags, thr in cases:
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        B = rng.normal(0, 0.05, (K, N)).astype(np.float32)
        y64 = A.astype(np.float64) @ B.astype(np.float64)
        if flags & capi.FUSE_RELU:
            y64 = np.maximum(y64, thr)
        regular, noalloc = _both_entry_points(dev, A, B, flags, thr)
        assert _rel_err(regular, y64) <= FP32_TOL
        assert _rel_err(noalloc, y64) <= FP32_TOL
        assert _rel_err(noalloc, regular.astype(np.float64)) <= FP32_TOL
        # same kernels, same arithmetic, same order: the bits agree as well
        assert np.array_equal(noalloc, regular)
    # reads (and would clear) the status word of this entry point as well as the regular one
    assert dev.status() == 0


def _free_bytes(dev):
    free, total = ctypes.c_size_t(0), ctypes.c_size_t(0)
    capi.check(dev.lib.xtc_cuda_mem_info(byref(free), byref(total)))
    return free.value


def test_noalloc_gemm_leaves_free_device_memory_unchanged(cuda_lib):
    """What the entry point is for: after the first call on the device (which resolves the
    address of the built-in array), a call takes nothing from the device allocator."""
    dev = CudaDevice(0)
    assert dev.detect_accelerator(), "this test needs a CUDA device"
    dev.activate()
    M, K, N = 256, 512, 128
    rng = np.random.default_rng(7)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    dA, dB, dC = _put(dev, A), _put(dev, B), dev.memory_allocate(M * N * 4)
    lib = dev.lib
    capi.check(lib.xtc_cuda_gemm_f32_3xtf32_noalloc(dA, dB, dC, M, N, K, 0, 0.0, None))  # warm-up
    assert dev.status() == 0
    before = _free_bytes(dev)
    for _ in range(3):
        capi.check(lib.xtc_cuda_gemm_f32_3xtf32_noalloc(dA, dB, dC, M, N, K, 0, 0.0, None))
    assert dev.status() == 0  # synchronises, reads both status words: no allocation either
    assert _free_bytes(dev) == before
    y64 = A.astype(np.float64) @ B.astype(np.float64)
    assert _rel_err(_get(dev, dC, (M, N)), y64) <= FP32_TOL
    for d in (dA, dB, dC):
        dev.memory_free(d)


def test_noalloc_gemm_refuses_what_does_not_fit(cuda_lib):
    dev = CudaDevice(0)
    assert dev.detect_accelerator(), "this test needs a CUDA device"
    dev.activate()
    p = dev.memory_allocate(1024)
    rc = dev.lib.xtc_cuda_gemm_f32_3xtf32_noalloc(p, p, p, 4096, 4096, 4096, 0, 0.0, None)
    assert rc == capi.ERR_INVALID
    msg = capi.last_error()
    assert "scratch" in msg and str(32 << 20) in msg
    # just over the limit: 1024 x 2048 + 2048 x 1024 elements fill the 32 MiB exactly, one
    # more row of A does not fit
    big = dev.memory_allocate(4 * 1028 * 2048)
    rc = dev.lib.xtc_cuda_gemm_f32_3xtf32_noalloc(big, big, big, 1028, 1024, 2048, 0, 0.0, None)
    assert rc == capi.ERR_INVALID and "scratch" in capi.last_error()
    # extents whose byte counts would wrap a 64-bit product must be refused, not wrapped
    huge = (1 << 31) - 4
    rc = dev.lib.xtc_cuda_gemm_f32_3xtf32_noalloc(big, big, big, huge, huge, huge, 0, 0.0, None)
    assert rc == capi.ERR_INVALID and "scratch" in capi.last_error()
    # a misaligned C is refused like a misaligned operand
    rc = dev.lib.xtc_cuda_gemm_f32_3xtf32_noalloc(big, big, c_void_p(big.value + 4), 64, 64, 64, 0,
                                                  0.0, None)
    assert rc == capi.ERR_INVALID and "aligned" in capi.last_error()
    rc = dev.lib.xtc_cuda_gemm_f32_3xtf32_noalloc(None, p, p, 8, 8, 8, 0, 0.0, None)
    assert rc == capi.ERR_INVALID
    dev.memory_free(big)
    dev.memory_free(p)
