"""Scheduler of the CUDA backend: records the reference's scheduling directives
per node and maps them onto the parameters of the hand-written kernels.

The recording side keeps the field names and ``./``-rooted loop names of the
reference's ``MlirNodeScheduler`` (``backends/mlir/MlirNodeScheduler.py:17-232``,
``MlirLoopNames.py:10-19``) so that ``str(schedule)`` reads the same.  The
mapping side is new: for a contraction node (matmul / conv2d)

  tile(i, {i1: TM, ...})   first tile level of the row dim   -> CTA tile rows
  tile(j, {j1: TN, ...})   first tile level of the column dim -> CTA tile columns
  tile(k, {k1: TK, ...})   first tile level of the reduction  -> K per pipeline stage
  unroll({k1: U})          unroll of that reduction tile      -> pipeline depth (stages)
  vectorize([j<inner>])    vectorised innermost column tile   -> 128-byte TMA-store epilogue
  parallelize([...])       outer parallel axes                -> recorded; the grid is always
                                                                 persistent over output tiles
  fuse_producer_at(_, idx)                                    -> fold the transpose producing
                                                                 operand idx into the GEMM
  split(k, {n segments})   matmul reduction cut into segments -> split-K over n CTAs per tile
                           (conv2d: split(c, ...), the im2col kernels)
  pack_at(_, 0)            conv2d input window packed on chip, alone -> streamed weights + halo tiles
  pack_at(_, 1)            conv2d filter bank packed on chip  -> resident weights + halo tiles;
                           the first tile of c is then the channel slab of a stage (16 or 32),
                           tile(s, {s1: 2}) puts two neighbouring filter taps into one MMA;
                           pack_at(_, 0) as well keeps the input window on chip across
                           consecutive tiles (a run of tiles per CTA, the input through a ring)
  tile rows 256                                               -> CTA pairs (two SMs per MMA)

Values the kernels do not implement are snapped to the nearest legal value
(``strict=False``, the default, so that any schedule written for another
backend still runs) or rejected with ``ScheduleError`` (``strict=True``, what
an autotuner wants so illegal points are never measured).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

DEFAULT_ROOT = "."

LEGAL_TILE_M = (128, 256)
LEGAL_TILE_N = (64, 128, 256)
LEGAL_TILE_K = (32, 64)
LEGAL_SLAB = (16, 32)  # channels per stage of the resident-weights convolution
MAX_STAGES = 8


class ScheduleError(ValueError):
    """A directive has no legal mapping onto the kernels (strict mode)."""


def make_loop_name(root: str, name: str) -> str:
    return f"{root}/{name}"


def basename(loop_name: str) -> str:
    return loop_name.split("/")[-1]


@dataclass(frozen=True)
class CudaNodeSchedule:
    node_name: str
    node_ident: str
    dims: list[str]
    splits: dict[str, dict[str, int]]
    tiles: dict[str, dict[str, int]]
    permutation: dict[str, list[str]]
    vectorization: list[str]
    parallelization: list[str]
    unrolling: dict[str, int]
    packed_buffers: dict[str, list[int]]
    write_buffers: list[str]
    fused: list[tuple[str, int]]
    kernel: dict[str, int] = field(default_factory=dict)


@dataclass
class LoopNestNode:
    """Loop-nest view of one scheduled node (cf. ``schedules/loop_nest.py:79-118``)."""

    root: str
    tiles: dict[str, dict[str, int]]
    splits: dict[str, dict[str, int]] = field(default_factory=dict)
    interchange: list[str] = field(default_factory=list)
    vectorize: list[str] = field(default_factory=list)
    parallelize: list[str] = field(default_factory=list)
    unroll: dict[str, int] = field(default_factory=dict)
    buffer_at: dict[str, str | None] = field(default_factory=dict)
    pack_at: dict[str, tuple[int, str | None, bool]] = field(default_factory=dict)
    children: list["LoopNestNode"] = field(default_factory=list)

    def pretty_print(self, indent: int = 0) -> str:
        lines = []
        sizes = {t: s for tiles in self.tiles.values() for t, s in tiles.items()}
        owner = {t: d for d, tiles in self.tiles.items() for t in tiles}
        for depth, loop in enumerate(self.interchange):
            text = f"tile({owner[loop]}, {sizes[loop]})" if loop in sizes else f"loop {loop}"
            notes = []
            if loop in self.parallelize:
                notes.append("parallelized")
            if loop in self.vectorize:
                notes.append("vectorized")
            if loop in self.unroll:
                notes.append(f"unroll({self.unroll[loop]})")
            lines.append(" " * (indent + 2 * depth) + text + (f"  // {', '.join(notes)}" if notes else ""))
        lines.append(" " * (indent + 2 * len(self.interchange)) + "...")
        return "\n".join(lines)


@dataclass
class LoopNest:
    abstract_dims: list[str]
    root_node: LoopNestNode | None = None

    def pretty_print(self) -> str:
        return "" if self.root_node is None else self.root_node.pretty_print()


class CudaNodeScheduler:
    """Directive recorder for one node."""

    def __init__(self, node_name: str, node_ident: str, op_name: str, dims: dict[str, int]):
        self.node_name = node_name
        self.node_ident = node_ident
        self.op_name = op_name
        self.dim_sizes = dict(dims)
        self.dims = list(dims)
        self.splits: dict[str, dict[str, int]] = {}
        self.tiles: dict[str, dict[str, int]] = {d: {} for d in self.dims}
        self.permutation: dict[str, list[str]] = {}
        self.vectorization: list[str] = []
        self.parallelization: list[str] = []
        self.unrolling: dict[str, int] = {}
        self.packed_buffers: dict[str, list[int]] = {}
        self.write_buffers: list[str] = []
        self.fused: list[tuple[str, int]] = []

    # -- recording (same semantics as MlirNodeScheduler.py:139-232) ---------
    def set_dims(self, dims: list[str]) -> None:
        assert len(dims) == len(self.dims)
        self.dim_sizes = dict(zip(dims, self.dim_sizes.values()))
        self.dims = list(dims)
        self.tiles = {d: {} for d in self.dims}

    def split(self, dim: str, segments: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        named = {make_loop_name(root, k): v for k, v in segments.items()}
        self.splits[dim] = named
        for s in named:
            self.tiles[s] = {}

    def tile(self, dim: str, tiles: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        assert dim in self.tiles, f"unknown dimension {dim!r} (have {list(self.tiles)})"
        for name, size in tiles.items():
            assert int(size) >= 1, f"tile size must be >= 1: {name}={size}"
            self.tiles[dim][make_loop_name(root, name)] = int(size)

    def interchange(self, permutation: list[str], root: str = DEFAULT_ROOT) -> None:
        self.permutation[root] = [make_loop_name(root, a) for a in permutation]

    def vectorize(self, axes: list[str], root: str = DEFAULT_ROOT) -> None:
        self.vectorization += [make_loop_name(root, a) for a in axes]

    def parallelize(self, axes: list[str], root: str = DEFAULT_ROOT) -> None:
        self.parallelization = [make_loop_name(root, a) for a in axes]

    def unroll(self, unrolls: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        for name, factor in unrolls.items():
            assert int(factor) >= 1, f"unroll factor must be >= 1: {name}={factor}"
            self.unrolling[make_loop_name(root, name)] = int(factor)

    def buffer_at(self, axis: str, mtype: str | None = None, root: str = DEFAULT_ROOT) -> None:
        # The accumulator of a contraction always lives in tensor memory; recorded only.
        self.write_buffers.append(make_loop_name(root, axis))

    def pack_at(self, axis: str, input_idx: int, mtype: str | None = None, pad: bool = False,
                root: str = DEFAULT_ROOT) -> None:
        # Operands are always staged in shared memory by TMA; recorded only.
        self.packed_buffers.setdefault(make_loop_name(root, axis), []).append(input_idx)

    def fuse_producer_at(self, axis: str, input_idx: int, root: str = DEFAULT_ROOT) -> None:
        self.fused.append((make_loop_name(root, axis), input_idx))

    def default_interchange(self, root: str) -> list[str]:
        order = [make_loop_name(root, d) for d in self.dims]
        depth = max((len(v) for v in self.tiles.values()), default=0)
        for level in range(depth):
            for tiles in self.tiles.values():
                if level < len(tiles):
                    order.append(list(tiles)[level])
        return order

    # -- mapping onto kernel parameters ---------------------------------------
    def _role_dims(self) -> tuple[str | None, str | None, str | None]:
        """(row, column, reduction) dimension names of a contraction node."""
        if self.op_name == "matmul" and len(self.dims) == 3:
            return self.dims[0], self.dims[1], self.dims[2]
        if self.op_name == "conv2d" and len(self.dims) == 7:
            # rows are the fused b*h*w output pixels: the first tile of w sets how many
            # consecutive pixels a CTA (128) or a CTA pair (256) takes; columns f; reduction c
            return self.dims[2], self.dims[3], self.dims[6]
        return None, None, None

    def kernel_config(self, strict: bool) -> dict[str, int]:
        row, col, red = self._role_dims()
        if col is None:
            return {}
        cfg: dict[str, int] = {}

        def first_tile(dim: str | None) -> tuple[str | None, int | None]:
            if dim is None or not self.tiles.get(dim):
                return None, None
            name = next(iter(self.tiles[dim]))
            return name, self.tiles[dim][name]

        def snap(value: int, legal: tuple[int, ...], what: str) -> int:
            if value in legal:
                return value
            if strict:
                raise ScheduleError(f"{self.node_name}: {what}={value} is not one of {legal}")
            return min(legal, key=lambda v: (abs(v - value), -v))

        # pack_at(_, 1) on a conv2d: keep operand 1 (the filter bank) packed in shared memory
        # for the whole kernel -> the resident-weights / halo-tile convolution, whose
        # pipeline stage is a slab of 16 or 32 channels
        resident = self.op_name == "conv2d" and any(1 in idx for idx in self.packed_buffers.values())
        # pack_at(_, 0) alone: the streamed-weights kernel, whose stage is a channel slab too
        streamed = (self.op_name == "conv2d" and not resident
                    and any(0 in idx for idx in self.packed_buffers.values()))
        _, tm = first_tile(row)
        _, tn = first_tile(col)
        kname, tk = first_tile(red)
        if tm is not None:
            cfg["tile_m"] = snap(tm, LEGAL_TILE_M, "CTA tile rows")
        if tn is not None:
            cfg["tile_n"] = snap(tn, LEGAL_TILE_N, "CTA tile columns")
        if tk is not None:
            cfg["tile_k"] = (snap(tk, LEGAL_SLAB, "channels per stage") if resident or streamed
                             else snap(tk, LEGAL_TILE_K, "K per stage"))
        if kname is not None and kname in self.unrolling:
            u = self.unrolling[kname]
            if 2 <= u <= MAX_STAGES:
                cfg["stages"] = u
            elif strict:
                raise ScheduleError(f"{self.node_name}: pipeline depth {u} not in [2, {MAX_STAGES}]")
        col_tiles = list(self.tiles.get(col, {}))
        inner_col = col_tiles[-1] if col_tiles else make_loop_name(DEFAULT_ROOT, col)
        if inner_col in self.vectorization:
            cfg["epilogue"] = 2
        if self.op_name == "matmul" and red in self.splits and len(self.splits[red]) > 1:
            # split(k, {...}): the reduction cut into segments that run concurrently
            cfg["split_k"] = len(self.splits[red])
        if self.op_name == "conv2d" and red in self.splits and len(self.splits[red]) > 1:
            # split(c, {...}) on a conv2d: the reduction (taps x channels) shared by that many
            # CTAs of a thread-block cluster
            cfg["split_k"] = len(self.splits[red])
        if resident:
            cfg["variant"] = 2
            # tile(s, {s1: 2}): two neighbouring taps of a filter row per MMA
            s_dim = self.dims[5]
            s_tiles = list(self.tiles.get(s_dim, {}).values())
            if s_tiles and s_tiles[0] == 2:
                cfg["variant"] = 3
            elif s_tiles and strict and s_tiles[0] != 1:
                raise ScheduleError(f"{self.node_name}: taps per MMA = {s_tiles[0]} is not 1 or 2")
            elif any(0 in idx for idx in self.packed_buffers.values()):
                # pack_at(_, 0) too: the input window stays on chip from one tile to the next
                cfg["variant"] = 4
        elif streamed:
            # a tile's input window is packed on chip once per channel slab and read by every
            # filter tap, the weights stream beside it (CTA pairs, 128 filters per work item)
            slab = cfg.get("tile_k")
            cfg = {k: v for k, v in cfg.items() if k not in ("tile_m", "tile_n", "tile_k", "split_k", "epilogue")}
            cfg["variant"] = 5
            if slab == 16:
                cfg["tile_k"] = 16  # 16-channel slabs: twice as many, half as large stages
        return cfg

    def node_schedule(self, strict: bool = False) -> CudaNodeSchedule:
        if not self.permutation:
            self.permutation[DEFAULT_ROOT] = self.default_interchange(DEFAULT_ROOT)
        return CudaNodeSchedule(
            node_name=self.node_name, node_ident=self.node_ident, dims=list(self.dims),
            splits=self.splits, tiles=self.tiles, permutation=self.permutation,
            vectorization=self.vectorization, parallelization=self.parallelization,
            unrolling=self.unrolling, packed_buffers=self.packed_buffers,
            write_buffers=self.write_buffers, fused=self.fused,
            kernel=self.kernel_config(strict))

    def loop_nest(self) -> LoopNest:
        perm = self.permutation.get(DEFAULT_ROOT) or self.default_interchange(DEFAULT_ROOT)
        keep = set(perm)
        node = LoopNestNode(
            root=self.node_name,
            tiles={d: {basename(t): s for t, s in tiles.items()}
                   for d, tiles in self.tiles.items() if d in self.dims},
            interchange=[basename(p) for p in perm],
            vectorize=[basename(v) for v in self.vectorization if v in keep],
            parallelize=[basename(p) for p in self.parallelization if p in keep],
            unroll={basename(k): v for k, v in self.unrolling.items() if k in keep},
        )
        return LoopNest(abstract_dims=list(self.dims), root_node=node)


class CudaSchedule:
    """The frozen result of scheduling: one record per graph node."""

    def __init__(self, scheduler: "CudaScheduler", nodes_schedules: list[CudaNodeSchedule]):
        self._scheduler = scheduler
        self._nodes_schedules = nodes_schedules

    @property
    def scheduler(self) -> "CudaScheduler":
        return self._scheduler

    @property
    def schedule_impl(self) -> list[CudaNodeSchedule]:
        return self._nodes_schedules

    def node_configs(self) -> dict[str, dict[str, int]]:
        return {s.node_name: dict(s.kernel) for s in self._nodes_schedules if s.kernel}

    def fused_transposes(self) -> dict[str, set[int]]:
        out: dict[str, set[int]] = {}
        for s in self._nodes_schedules:
            for _, idx in s.fused:
                out.setdefault(s.node_name, set()).add(idx)
        return out

    def __str__(self) -> str:
        return str(self._nodes_schedules)


class CudaScheduler:
    """``Backend.get_scheduler(nodes=None, default_node=None, strict=False)``.

    Directives apply to the default node.  The reference takes the *last* node
    (``backends/mlir/MlirScheduler.py:48-62``), which for ``matmul -> relu``
    graphs is the relu; here the default is the last contraction node when the
    graph has one, because that is the node whose kernel has parameters.
    """

    node_scheduler = CudaNodeScheduler  # the per-node recorder (a subclass may map differently)

    def __init__(self, backend: Any, nodes: list[str] | None = None,
                 default_node: str | None = None, strict: bool = False) -> None:
        self._backend = backend
        self._strict = strict
        graph = backend.graph
        self._node_schedulers: list[CudaNodeScheduler] = []
        for node in graph.nodes.values():
            if nodes is not None and node.name not in nodes:
                continue
            op = node.operation
            self._node_schedulers.append(
                self.node_scheduler(node.name, f"__xtc_id_{node.name}_", op.name,
                                    {k: int(v) for k, v in op.dims.items()}))
        if default_node is not None:
            cands = [s for s in self._node_schedulers if s.node_name == default_node]
            assert cands, f"default_node {default_node!r} is not a node of the graph"
        else:
            cands = ([s for s in self._node_schedulers if s.op_name in ("matmul", "conv2d")]
                     or self._node_schedulers)
        self._current = cands[-1] if cands else None

    @property
    def backend(self) -> Any:
        return self._backend

    @property
    def _cur(self) -> CudaNodeScheduler:
        assert self._current is not None, "graph has no node to schedule"
        return self._current

    def node(self, name: str) -> CudaNodeScheduler:
        """The recorder of a specific node, for schedules that touch several nodes."""
        for s in self._node_schedulers:
            if s.node_name == name:
                return s
        raise KeyError(name)

    def schedule(self) -> CudaSchedule:
        return CudaSchedule(self, [s.node_schedule(self._strict) for s in self._node_schedulers])

    def set_dims(self, dims: list[str]) -> None:
        self._cur.set_dims(dims)

    def split(self, dim: str, segments: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        self._cur.split(dim, segments, root=root)

    def strip_mine(self, dim: str, tiles: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        self.tile(dim, tiles, root=root)

    def tile(self, dim: str, tiles: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        self._cur.tile(dim, tiles, root=root)

    def interchange(self, permutation: list[str], root: str = DEFAULT_ROOT) -> None:
        self._cur.interchange(permutation, root=root)

    def vectorize(self, axes: list[str], root: str = DEFAULT_ROOT) -> None:
        self._cur.vectorize(axes, root=root)

    def parallelize(self, axes: list[str], root: str = DEFAULT_ROOT) -> None:
        self._cur.parallelize(axes, root=root)

    def unroll(self, unrolls: dict[str, int], root: str = DEFAULT_ROOT) -> None:
        self._cur.unroll(unrolls, root=root)

    def buffer_at(self, axis: str, mtype: str | None = None, root: str = DEFAULT_ROOT) -> None:
        self._cur.buffer_at(axis, mtype, root=root)

    def pack_at(self, axis: str, input_idx: int, mtype: str | None = None, pad: bool = False,
                root: str = DEFAULT_ROOT) -> None:
        self._cur.pack_at(axis, input_idx, mtype, pad, root=root)

    def fuse_producer_at(self, axis: str, input_idx: int, root: str = DEFAULT_ROOT) -> None:
        self._cur.fuse_producer_at(axis, input_idx, root=root)

    # The distribution calls of the interface target a multi-memory accelerator
    # extension of the reference (itf/schd/scheduler.py:235-291); GPUs of one box
    # are partitioned by xtc_b200.dist instead.
    def define_memory_mesh(self, axes: dict[str, int]) -> None:
        raise NotImplementedError("memory meshes are not part of the CUDA backend; see xtc_b200.dist")

    def define_processor_mesh(self, axes: dict[str, int]) -> None:
        raise NotImplementedError("processor meshes are not part of the CUDA backend; see xtc_b200.dist")

    def distribute(self, axis: str, processor_axis: str, root: str = DEFAULT_ROOT) -> None:
        raise NotImplementedError("distribute is not part of the CUDA backend; see xtc_b200.dist")

    def distributed_buffer_at(self, axis: str, input_idx: int, memory_axes: list[str],
                              root: str = DEFAULT_ROOT) -> None:
        raise NotImplementedError("distributed buffers are not part of the CUDA backend")

    def get_loop_nest(self) -> LoopNest:
        return self._cur.loop_nest()
