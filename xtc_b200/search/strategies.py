"""Search strategies over the kernels' real parameter space.

A strategy turns a sample (a flat list of ints, the reference's convention,
``search/strategies.py:22-164`` of the reference's ``itf/search/strategy.py``)
into ordinary scheduler calls -- ``tile / unroll / vectorize / parallelize`` --
on the contraction node of a graph, so the same sample works through any
front end that drives the ``Scheduler`` interface.  The reference's strategies
enumerate divisors of the loop extents and prune with CPU notions (vector
width, register count, L1/L2 footprint; ``search/strategies.py:150-171,
555-620``); here the space is what the CUDA kernels implement and the filter
is the shared-memory budget of the pipeline.

Sample layout of ``cuda_gemm`` (also used for conv2d):
    [tile_m, tile_n, tile_k, stages, tma_store, split_k]
``split_k`` (1 to 8) cuts a matmul's reduction into segments that run
concurrently, one CTA of a thread-block cluster each (``scheduler.split``).
"""

from __future__ import annotations

import itertools
import random
from typing import Any, Callable

SMEM_BUDGET = 232448 - 1024 - 1024  # dynamic shared memory minus alignment slack and barriers
EPILOGUE_STAGING = 4 * 2 * 32 * 32 * 4


def contraction_node(graph: Any) -> Any:
    nodes = [n for n in graph.nodes.values() if n.operation.name in ("matmul", "conv2d")]
    if not nodes:
        raise ValueError("the graph has no matmul or conv2d node to schedule")
    return nodes[-1]


class StrategyCudaGemm:
    """Exhaustive / random search over CTA tile, K per stage, pipeline depth, epilogue."""

    name = "cuda_gemm"
    sample_names = ["tile_m", "tile_n", "tile_k", "stages", "tma_store", "split_k"]

    # Rows: 128 (one CTA per tile) or 256 (a CTA pair).  No 64-row tile: a 64 x N x 8 MMA
    # occupies the tensor pipe exactly as long as a 128 x N x 8 one (xtc_cuda_mma_rate on a
    # B200: 57 / 67 / 133 clocks for N = 64 / 128 / 256 with either row count), so it can only
    # halve the rate; small problems get more CTAs by splitting K inside a cluster instead.
    TILE_M = (128, 256)
    TILE_N = (64, 128, 256)
    TILE_K = (32, 64)
    STAGES = (0, 2, 3, 4, 6)  # 0 = as deep as shared memory allows
    SPLITS = (1, 2, 3, 4, 5, 6, 7, 8)  # pieces of the reduction (one CTA per tile, tile_n <= 128)

    def __init__(self, graph: Any, tile_m: tuple[int, ...] | None = None,
                 tile_n: tuple[int, ...] | None = None, tile_k: tuple[int, ...] | None = None,
                 stages: tuple[int, ...] | None = None, splits: tuple[int, ...] | None = None,
                 **_ignored: Any) -> None:
        self._graph = graph
        self._node = contraction_node(graph)
        self._op = self._node.operation
        self._is_conv = self._op.name == "conv2d"
        self.tile_m = tuple(tile_m or self.TILE_M)
        self.tile_n = tuple(tile_n or self.TILE_N)
        self.tile_k = tuple(tile_k or self.TILE_K)
        self.stages = tuple(stages or self.STAGES)
        self.splits = tuple(splits or self.SPLITS) if not self._is_conv else (1,)
        self._k_extent = 0 if self._is_conv else int(list(self._op.dims.values())[2])

    @property
    def graph(self) -> Any:
        return self._graph

    @property
    def node_name(self) -> str:
        return self._node.name

    # -- the space ----------------------------------------------------------------
    @staticmethod
    def stage_bytes(tile_m: int, tile_n: int, tile_k: int) -> int:
        """Shared memory one pipeline stage takes in one CTA."""
        if tile_m == 256:  # CTA pair: each CTA holds 128 rows of A and half of the B tile
            return (128 + tile_n // 2) * tile_k * 4
        return (128 + tile_n) * tile_k * 4

    def is_legal(self, sample: list[int]) -> bool:
        tm, tn, tk, st, tma = sample[:5]
        split = sample[5] if len(sample) > 5 else 1
        if tm not in self.TILE_M or tn not in self.TILE_N or tk not in self.TILE_K:
            return False
        if split not in self.SPLITS:
            return False
        if split > 1 and (self._is_conv or tm != 128 or tn > 128 or self._k_extent % (split * tk)):
            return False
        if tma not in (0, 1) or not (st == 0 or 2 <= st <= 8):
            return False
        budget = SMEM_BUDGET - (EPILOGUE_STAGING if (tma or tm == 256) else 0)
        depth = max(st, 2)
        return depth * self.stage_bytes(tm, tn, tk) <= budget

    def exhaustive(self):
        for s in itertools.product(self.tile_m, self.tile_n, self.tile_k, self.stages, (0, 1),
                                   self.splits):
            s = list(s)
            if self.is_legal(s):
                yield s

    def sample(self, num: int, seed: int | None = 0) -> list[list[int]]:
        space = list(self.exhaustive())
        rng = random.Random(seed)
        rng.shuffle(space)
        return space[: max(num, 0)]

    def default_schedule(self, opt_level: int = 2) -> list[int]:
        """O0: smallest tiles, shallow pipeline; O2: a wide tile, deepest pipeline; O3: what the
        library itself would pick for this product (xtc_cuda_gemm_default_config), where that is
        a point of this space."""
        if opt_level <= 0:
            return [128, 64, 32, 2, 0, 1]
        if opt_level == 1:
            return [128, 128, 32, 0, 0, 1]
        if opt_level == 2 or self._is_conv:
            return [128, 256 if not self._is_conv else 64, 32 if not self._is_conv else 64, 0, 1, 1]
        return self.library_default() or [256, 256, 32, 0, 1, 1]

    def library_default(self) -> list[int] | None:
        """The library's own choice for this matmul as a sample, or None (no library built, a
        convolution, or a choice outside this space)."""
        if self._is_conv:
            return None
        try:
            import ctypes

            from .. import capi

            m, n, k = (int(v) for v in self._op.dims.values())
            cfg = capi.GemmConfig()
            if capi.load().xtc_cuda_gemm_default_config(m, n, k, ctypes.byref(cfg)) != capi.OK:
                return None
        except Exception:  # the search must not depend on the kernel library being present
            return None
        sample = [cfg.tile_m, cfg.tile_n, cfg.tile_k, 0, 1, max(cfg.split_k, 1)]
        return sample if self.is_legal(sample) else None

    # -- sample -> scheduler calls ---------------------------------------------------
    def generate(self, scheduler: Any, sample: list[int]) -> None:
        tm, tn, tk, st, tma = [int(v) for v in sample[:5]]
        split = int(sample[5]) if len(sample) > 5 else 1
        dims = list(self._op.dims)
        target = scheduler.node(self.node_name) if hasattr(scheduler, "node") else scheduler
        if self._is_conv:
            row, col, red = dims[2], dims[3], dims[6]
            target.tile(row, {f"{row}1": tm})  # pixels per CTA (128) or CTA pair (256)
            target.tile(col, {f"{col}1": tn})
            target.tile(red, {f"{red}1": tk})
            target.parallelize(dims[:3])
        else:
            row, col, red = dims
            if split > 1:
                piece = self._k_extent // split
                target.split(red, {f"{red}_s{i}": i * piece for i in range(split)})
            target.tile(row, {f"{row}1": tm})
            target.tile(col, {f"{col}1": tn})
            target.tile(red, {f"{red}1": tk})
            target.parallelize([row, col])
        if st:
            target.unroll({f"{red}1": st})
        if tma:
            target.vectorize([f"{col}1"])


class StrategyCudaConv:
    """The convolution kernels' whole space: which kernel, then that kernel's parameters.

    Sample ``[variant, tile_m, tile_n, tile_k, stages, tma_store, split_k]``:
      variant 2  resident weights + halo tiles (stride 1, filter bank fits in shared memory):
                 tile_m = output positions per tile (128 = one CTA, 256 = a CTA pair with
                 half a filter bank each), tile_k = channels per pipeline stage (16 or 32,
                 32 only for pairs), stages; tile_n, tma_store and split_k do not apply
      variant 3  the same with two neighbouring filter taps per MMA (at most 64 filters, filter
                 rows of two taps or more, one CTA per tile)
      variant 4  resident weights with a sliding input window: a run of consecutive tiles per
                 CTA, the input through a ring of 128-position chunks (at most 128 filters, a
                 halo run of at most 256 positions); no other parameter applies
      variant 5  streamed weights beside halo tiles, for filter banks that do not fit in shared
                 memory: CTA pairs, 128 filters per tile, a stage = one 32-channel halo slab + every
                 tap's weights (2 to 32 taps, two such stages must fit); ``tile_k`` = 16 halves the
                 slabs, ``stages`` sets the depth
      variant 1  implicit GEMM, one im2col fetch per filter tap: the GEMM kernels' tile_m /
                 tile_n / tile_k / stages / epilogue, and split_k = 2 to 8 pieces of the
                 reduction in one thread-block cluster (one CTA per tile, tile_n <= 128)
    """

    name = "cuda_conv"
    sample_names = ["variant", "tile_m", "tile_n", "tile_k", "stages", "tma_store", "split_k"]

    def __init__(self, graph: Any, **_ignored: Any) -> None:
        self._graph = graph
        self._node = contraction_node(graph)
        self._op = self._node.operation
        if self._op.name != "conv2d":
            raise ValueError("cuda_conv schedules a conv2d node")
        d = {k: int(v) for k, v in self._op.dims.items()}
        self._b, self._h, self._w, self._f, self._r, self._s, self._c = d.values()
        stride = self._op.attrs.get("stride", (1, 1))
        stride = (stride, stride) if isinstance(stride, int) else tuple(stride)
        self._stride = (int(stride[0]), int(stride[-1]))
        self._in_w = (self._w - 1) * self._stride[1] + self._s  # width of the (padded) input
        self._gemm = StrategyCudaGemm(graph)

    graph = property(lambda self: self._graph)
    node_name = property(lambda self: self._node.name)

    def resident_stages(self, tile_m: int, slab: int, taps: bool = False) -> int:
        """Halo stages that fit next to the filter bank (0 = this layer cannot run resident)."""
        if self._stride != (1, 1) or self._f > 256 or (tile_m == 256 and slab != 32):
            return 0
        if taps and (tile_m != 128 or self._f > 64 or self._s < 2):
            return 0
        bn = 64 if self._f <= 64 else 128 if self._f <= 128 else 256
        run = 128 + (self._r - 1) * self._in_w + self._s - 1  # halo pixels of a 128-position tile
        if run > 1024:
            return 0
        stage = -(-run * slab * 4 // 1024) * 1024
        bank = self._r * self._s * -(-self._c // 32) * (bn // 2 if tile_m == 256 else bn) * 128
        room = SMEM_BUDGET - bank - (1024 if taps else 0)  # the two-tap kernel exchanges rows
        return max(min(room // stage, 8), 0) if room >= 2 * stage else 0

    def sliding_window_fits(self) -> bool:
        """Whether the sliding-window kernel takes this layer (conv2d_halo_slide.cuh)."""
        if self._stride != (1, 1) or self._f > 128 or self._r * self._s < 2 or self._c % 4 or self._f % 4:
            return False
        run = 128 + (self._r - 1) * self._in_w + self._s - 1
        bank = self._r * self._s * -(-self._c // 32) * (64 if self._f <= 64 else 128) * 128
        return run <= 256 and bank + 5 * 16384 + 2048 <= SMEM_BUDGET + 2048

    def streamed_stages(self, slab: int = 32) -> int:
        """Stages of the streamed-weights kernel that fit with slabs of ``slab`` channels (0 = it
        does not take this layer)."""
        taps = self._r * self._s
        if self._stride != (1, 1) or self._c % 4 or self._f % 4 or not 2 <= taps <= 32:
            return 0
        run = 128 + (self._r - 1) * self._in_w + self._s - 1
        if run > 1024:
            return 0
        stage = -(-run * slab * 4 // 1024) * 1024 + taps * 64 * slab * 4
        fit = SMEM_BUDGET // stage
        return min(fit, 6) if fit >= 2 else 0

    def library_streams(self) -> bool:
        """Whether the library, with nothing named, runs this layer on the streamed-weights kernel
        (the rule of ``xtc_cuda_conv2d_nhwc_f32``: no room for the whole filter bank beside one
        CTA's stages, work for most CTA pairs or at most two channel slabs, and most positions of
        the padded grid are outputs)."""
        if self.streamed_stages() < 2 or self.resident_stages(128, 32) or self.resident_stages(128, 16):
            return False
        grid = ((self._h - 1) * self._stride[0] + self._r) * self._in_w
        items = -(-self._b * grid // 256) * -(-self._f // 128)
        return (items >= 40 or -(-self._c // 32) <= 2) and self._h * self._w * 10 >= grid * 7

    def is_legal(self, sample: list[int]) -> bool:
        variant, tm, tn, tk, st, tma, split = sample
        if variant == 5:
            fit = self.streamed_stages(tk) if tk in (16, 32) else 0
            return (fit >= 2 and tm == 256 and tn == 128 and tma == 0 and split == 1
                    and (st == 0 or 2 <= st <= fit))
        if variant == 4:
            return (self.sliding_window_fits() and tm == 128 and tk == 32 and st == 0 and tma == 0
                    and split == 1 and tn == (64 if self._f <= 64 else 128))
        if variant in (2, 3):
            fit = self.resident_stages(tm, tk, variant == 3) if tm in (128, 256) and tk in (16, 32) else 0
            return (fit >= 2 and (st == 0 or 2 <= st <= fit) and tma == 0 and split == 1
                    and tn == (64 if self._f <= 64 else 128 if self._f <= 128 else 256))
        if variant != 1 or self._c % 4 or self._f % 4:
            return False
        if not self._gemm.is_legal([tm, tn, tk, st, tma, 1]) or split not in StrategyCudaGemm.SPLITS:
            return False
        k_blocks = self._r * self._s * -(-self._c // tk)
        return split == 1 or (tm == 128 and tn <= 128 and split <= k_blocks)

    def exhaustive(self):
        g = self._gemm
        tn_res = 64 if self._f <= 64 else 128 if self._f <= 128 else 256
        for variant, tm, slab, st in itertools.product((2, 3), (128, 256), (16, 32), (0, 2, 3, 4)):
            s = [variant, tm, tn_res, slab, st, 0, 1]
            if self.is_legal(s):
                yield s
        if self.is_legal([4, 128, min(tn_res, 128), 32, 0, 0, 1]):
            yield [4, 128, min(tn_res, 128), 32, 0, 0, 1]
        for slab, st in itertools.product((32, 16), (0, 2, 3, 4)):
            if self.is_legal([5, 256, 128, slab, st, 0, 1]):
                yield [5, 256, 128, slab, st, 0, 1]
        for tm, tn, tk, st, tma, split in itertools.product(g.tile_m, g.tile_n, g.tile_k, g.stages,
                                                            (0, 1), StrategyCudaGemm.SPLITS):
            s = [1, tm, tn, tk, st, tma, split]
            if self.is_legal(s):
                yield s

    def sample(self, num: int, seed: int | None = 0) -> list[list[int]]:
        space = list(self.exhaustive())
        random.Random(seed).shuffle(space)
        return space[: max(num, 0)]

    def default_schedule(self, opt_level: int = 2) -> list[int]:
        resident = [2, 128, 64 if self._f <= 64 else 128 if self._f <= 128 else 256, 32, 0, 0, 1]
        if opt_level >= 2 and self.is_legal(resident):
            return resident
        if opt_level >= 3 and self.library_streams():
            return [5, 256, 128, 32, 0, 0, 1]  # what the library picks itself for such a layer
        return [1, 128, 64 if self._f <= 64 else 128, 32, 2 if opt_level <= 0 else 0, 1, 1]

    def generate(self, scheduler: Any, sample: list[int]) -> None:
        variant, tm, tn, tk, st, tma, split = (int(v) for v in sample)
        b, h, w, f, r, s, c = list(self._op.dims)
        target = scheduler.node(self.node_name) if hasattr(scheduler, "node") else scheduler
        if variant == 5:
            target.pack_at(w, 0)  # the input window packed once per slab; the weights stream
        if variant in (2, 3, 4):
            target.pack_at(b, 1)  # the filter bank stays packed on chip
            if variant == 3:
                target.tile(s, {f"{s}1": 2})  # two neighbouring taps per MMA
            if variant == 4:
                target.pack_at(w, 0)  # and the input window, from one tile to the next
        elif split > 1:
            piece = -(-self._c // split)
            target.split(c, {f"{c}_s{i}": i * piece for i in range(split)})
        target.tile(w, {f"{w}1": tm})
        if variant == 1:
            target.tile(f, {f"{f}1": tn})
        target.tile(c, {f"{c}1": tk})
        target.parallelize([b, h, w])
        if st:
            target.unroll({f"{c}1": st})
        if tma:
            target.vectorize([f"{f}1"])


class Strategies:
    """Name -> strategy registry (cf. ``search/strategies.py:1190-1283``)."""

    _registry: dict[str, Callable[..., Any]] = {"cuda_gemm": StrategyCudaGemm,
                                                 "cuda_conv": StrategyCudaConv}

    @classmethod
    def register(cls, name: str, factory: Callable[..., Any]) -> None:
        cls._registry[name] = factory

    @classmethod
    def names(cls) -> list[str]:
        return sorted(cls._registry)

    @classmethod
    def create(cls, name: str, graph: Any, **options: Any) -> Any:
        if name not in cls._registry:
            raise KeyError(f"unknown strategy {name!r}; known: {cls.names()}")
        return cls._registry[name](graph, **options)
