"""The five benchmark graphs of this backend, built with the graph DSL.

Each configuration gives the graph, its seeded synthetic inputs, the
algorithmic work used for throughput numbers (FLOPs = 2 x FMAs of the
contraction nodes; bytes = every graph input read once + every graph output
written once, plus read+write of any intermediate a kernel materialises) and
the schedule this backend runs it with by default.

  c1  matmul            A[512,1024] @ B[1024,256]                 seed 0
  c2  matmul -> relu    A[4096,4096] @ B[4096,4096]               seed 1
  c3  pad -> conv2d 3x3 -> relu, NHWC [32,56,56,64], 64 filters   seed 2
  c4  transpose -> matmul  X[8192,8192]^T @ W[8192,1024]          seed 3
  c5  matmul            A[65536,8192] @ B[8192,8192] (row-sharded) seed 4
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import numpy as np

from .graphs.xtc import op as O

NAMES = ("c1", "c2", "c3", "c4", "c4a", "c5")
# the standalone elementwise kernels on 512 MiB tensors (bandwidth measurements only)
MOVEMENT_NAMES = ("relu512", "pad512")


@dataclass
class Config:
    name: str
    graph: Any
    contraction: str            # name of the node the schedule applies to
    input_shapes: list[tuple[int, ...]]
    output_shape: tuple[int, ...]
    flops: int
    bytes: int
    bound: str                  # "tensor" or "hbm"
    shards: str                 # "rows" (c5), "batch" (c3) or "" (single GPU)
    schedule: Callable[[Any], None]


def _scaled(n: int, scale: int) -> int:
    return max(n // scale, 1)


def inputs(name: str, scale: int = 1, batch: int | None = None) -> list[np.ndarray]:
    """Seeded inputs in graph-input order (one generator per configuration)."""
    s = scale
    if name == "c1":
        rng = np.random.default_rng(0)
        return [rng.uniform(-1, 1, (_scaled(512, s), _scaled(1024, s))).astype(np.float32),
                rng.uniform(-1, 1, (_scaled(1024, s), _scaled(256, s))).astype(np.float32)]
    if name == "c2":
        rng = np.random.default_rng(1)
        n = _scaled(4096, s)
        return [rng.uniform(-1, 1, (n, n)).astype(np.float32),
                rng.uniform(-1, 1, (n, n)).astype(np.float32)]
    if name == "c3":
        rng = np.random.default_rng(2)
        b = batch if batch is not None else _scaled(32, s)
        return [rng.uniform(0, 1, (b, 56, 56, 64)).astype(np.float32),
                rng.normal(0, np.sqrt(2 / 576), (3, 3, 64, 64)).astype(np.float32)]
    if name == "c4":
        rng = np.random.default_rng(3)
        n = _scaled(8192, s)
        return [rng.uniform(-1, 1, (n, n)).astype(np.float32),
                rng.normal(0, 0.02, (n, _scaled(1024, s))).astype(np.float32)]
    if name == "c4a":
        return inputs("c4", s)[:1]
    if name == "c5":
        rng = np.random.default_rng(4)
        k = _scaled(8192, s)
        return [rng.uniform(-1, 1, (_scaled(65536, s), k)).astype(np.float32),
                rng.normal(0, 1 / np.sqrt(8192), (k, k)).astype(np.float32)]
    if name == "relu512":
        rng = np.random.default_rng(5)
        return [rng.uniform(-1, 1, (_scaled(32768, s), 4096)).astype(np.float32)]
    if name == "pad512":
        rng = np.random.default_rng(6)
        return [rng.uniform(-1, 1, (_scaled(16, s), 256, 512, 64)).astype(np.float32)]
    raise KeyError(name)


def input_rows(name: str, lo: int, hi: int) -> list[np.ndarray]:
    """Rows [lo, hi) of the first input of a row-sharded configuration (c5) plus its
    replicated second input, bit-identical to slicing ``inputs(name)`` but without drawing
    the other rows: the generator is advanced past them (one draw per uniform element)."""
    if name != "c5":
        raise KeyError(f"{name} is not row-sharded")
    k, m = 8192, 65536
    assert 0 <= lo <= hi <= m
    rng = np.random.default_rng(4)
    rng.bit_generator.advance(lo * k)
    a = rng.uniform(-1, 1, (hi - lo, k)).astype(np.float32)
    rng = np.random.default_rng(4)
    rng.bit_generator.advance(m * k)
    b = rng.normal(0, 1 / np.sqrt(8192), (k, k)).astype(np.float32)
    return [a, b]


def _gemm_schedule(tile_n: int, tile_k: int, stages: int = 0, tma_store: bool = True,
                   tile_m: int = 128, fuse_a: bool = False, split: tuple[int, int] | None = None):
    def apply(sch: Any) -> None:
        if split is not None:
            # (pieces, K): the reduction cut into equal segments that run concurrently, one
            # CTA of a thread-block cluster each; on c1, 7.6 us against 10.0 us unsplit
            pieces, k_extent = split
            sch.split("k", {f"k_s{i}": i * (k_extent // pieces) for i in range(pieces)})
        if fuse_a:
            # read the transposed operand in place (column-major A tiles) instead of
            # materialising the transpose: on c4, 193 us against 293 us
            sch.fuse_producer_at("i", 0)
        sch.tile("i", {"i1": tile_m})  # 256 rows = the CTA-pair kernel
        sch.tile("j", {"j1": tile_n})
        sch.tile("k", {"k1": tile_k})
        if stages:
            sch.unroll({"k1": stages})
        sch.parallelize(["i", "j"])
        if tma_store:
            sch.vectorize(["j1"])
    return apply


def _conv_schedule(tile_n: int, tile_k: int, tma_store: bool = False, resident: bool = True):
    def apply(sch: Any) -> None:
        if resident:
            # filter bank packed in shared memory for the whole kernel, input fetched as
            # halo tiles: no per-tap tile parameters to choose
            sch.pack_at("b", 1)
            sch.parallelize(["b", "h", "w"])
            return
        sch.tile("f", {"f1": tile_n})
        sch.tile("c", {"c1": tile_k})
        sch.parallelize(["b", "h", "w"])
        if tma_store:
            sch.vectorize(["f1"])
    return apply


def build(name: str, scale: int = 1, batch: int | None = None, rows: int | None = None) -> Config:
    """Build configuration `name`.  `scale` divides the large extents (for tests);
    `batch` / `rows` override c3's batch and c5's row count (per-GPU shards)."""
    s = scale
    if name == "c1":
        m, k, n = _scaled(512, s), _scaled(1024, s), _scaled(256, s)
        a = O.tensor((m, k), "float32", name="A")
        b = O.tensor((k, n), "float32", name="B")
        with O.graph(name="c1_matmul") as gb:
            O.matmul(a, b, name="C")
        return Config(name, gb.graph, "C", [(m, k), (k, n)], (m, n), 2 * m * n * k,
                      4 * (m * k + k * n + m * n), "tensor", "",
                      _gemm_schedule(64, 64, split=(4, k) if k % 256 == 0 else None))
    if name == "c2":
        n = _scaled(4096, s)
        a = O.tensor((n, n), "float32", name="A")
        b = O.tensor((n, n), "float32", name="B")
        with O.graph(name="c2_matmul_relu") as gb:
            m_ = O.matmul(a, b, name="mm")
            O.relu(m_, name="relu")
        return Config(name, gb.graph, "mm", [(n, n), (n, n)], (n, n), 2 * n ** 3, 12 * n * n,
                      "tensor", "", _gemm_schedule(256, 64, tile_m=256))
    if name == "c3":
        bsz = batch if batch is not None else _scaled(32, s)
        x = O.tensor((bsz, 56, 56, 64), "float32", name="X")
        w = O.tensor((3, 3, 64, 64), "float32", name="W")
        with O.graph(name="c3_pad_conv_relu") as gb:
            p = O.pad(x, padding={1: (1, 1), 2: (1, 1)}, constant_value=0.0, name="pad")
            c = O.conv2d(p, w, stride=(1, 1), name="conv")
            O.relu(c, name="relu")
        out = bsz * 56 * 56 * 64
        return Config(name, gb.graph, "conv", [(bsz, 56, 56, 64), (3, 3, 64, 64)], (bsz, 56, 56, 64),
                      2 * out * 576, 4 * (out + 36864 + out), "tensor", "batch",
                      _conv_schedule(64, 64))
    if name == "c4":
        n, j = _scaled(8192, s), _scaled(1024, s)
        x = O.tensor((n, n), "float32", name="X")
        w = O.tensor((n, j), "float32", name="W")
        with O.graph(name="c4_transpose_matmul") as gb:
            t = O.transpose(x, axes=(1, 0), name="xt")
            O.matmul(t, w, name="mm")
        return Config(name, gb.graph, "mm", [(n, n), (n, j)], (n, j), 2 * n * n * j,
                      4 * (n * n + n * j + n * j) + 8 * n * n, "tensor", "",
                      _gemm_schedule(256, 64, tile_m=256, fuse_a=True))
    if name == "c4a":  # the transpose of c4 alone: a pure data-movement graph
        n = _scaled(8192, s)
        x = O.tensor((n, n), "float32", name="X")
        with O.graph(name="c4a_transpose") as gb:
            O.transpose(x, axes=(1, 0), name="xt")
        return Config(name, gb.graph, "xt", [(n, n)], (n, n), 0, 8 * n * n, "hbm", "",
                      lambda sch: None)
    if name == "relu512":  # a relu with no producer to fuse into: the standalone kernel
        shape = (_scaled(32768, s), 4096)
        x = O.tensor(shape, "float32", name="X")
        with O.graph(name="relu512") as gb:
            O.relu(x, name="relu")
        n = shape[0] * shape[1]
        return Config(name, gb.graph, "relu", [shape], shape, 0, 8 * n, "hbm", "", lambda sch: None)
    if name == "pad512":  # a pad with no convolution to fuse into: the standalone kernel
        shape = (_scaled(16, s), 256, 512, 64)
        x = O.tensor(shape, "float32", name="X")
        with O.graph(name="pad512") as gb:
            O.pad(x, padding={1: (1, 1), 2: (1, 1)}, constant_value=0.0, name="pad")
        out = (shape[0], 258, 514, 64)
        return Config(name, gb.graph, "pad", [shape], out, 0,
                      4 * (shape[0] * 256 * 512 * 64 + out[0] * 258 * 514 * 64), "hbm", "",
                      lambda sch: None)
    if name == "c5":
        k = _scaled(8192, s)
        m = rows if rows is not None else _scaled(65536, s)
        a = O.tensor((m, k), "float32", name="A")
        b = O.tensor((k, k), "float32", name="B")
        with O.graph(name="c5_matmul") as gb:
            O.matmul(a, b, name="C")
        return Config(name, gb.graph, "C", [(m, k), (k, k)], (m, k), 2 * m * k * k,
                      4 * (2 * m * k + k * k), "tensor", "rows",
                      _gemm_schedule(256, 32, tile_m=256))
    raise KeyError(name)


def compile_config(cfg: Config, precision: str = "tf32", fuse_transpose: bool | None = None,
                   dump_file: str | None = None, shared_lib: bool = False):
    """Backend -> default schedule -> compiled module."""
    from .backends.cuda import Backend

    impl = Backend(cfg.graph)
    sch = impl.get_scheduler(default_node=cfg.contraction)
    cfg.schedule(sch)
    comp = impl.get_compiler(shared_lib=shared_lib, dump_file=dump_file, precision=precision,
                             fuse_transpose=fuse_transpose)
    return comp.compile(sch.schedule())
