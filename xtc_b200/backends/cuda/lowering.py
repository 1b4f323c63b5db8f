"""Graph -> plan lowering: which kernel runs each node, and what gets fused.

The reference lowers every node to its own loop nest and relies on MLIR fusion
passes (``backends/mlir/MlirGraphBackend.py:96-148``,
``MlirCompilerPasses.py:378-412``).  Here a graph becomes a short list of
``Step`` records for ``libxtc_cuda.so``:

* ``matmul`` / ``conv2d``            -> one tensor-core GEMM / implicit-GEMM step
* a ``relu`` that is their only user -> folded into that step's epilogue
* a zero ``pad`` / ``pad2d`` of H, W feeding only a ``conv2d`` -> folded into
  the convolution's operand fetch
* a 2-D ``transpose`` feeding only a ``matmul`` -> folded into the GEMM as a
  transposed operand when the schedule asks for it (``fuse_producer_at``)
* a ``reshape`` that is not a graph output -> no step: it shares its input's buffer
* everything else -> its own bandwidth kernel (transpose, pad/crop, relu, copy)

Only duck-typed graph attributes are read (``graph.nodes``, ``node.inputs``,
``node.operation.{name, attrs, inputs_types, outputs_types}``), the same
attributes the reference's TVM backend reads (``backends/tvm/TVMOps.py:51-69``),
so a graph built by the reference's own DSL lowers unchanged.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ... import capi


class LoweringError(NotImplementedError):
    """The graph uses something the CUDA kernels do not cover."""


@dataclass
class StepDesc:
    """One kernel launch of a plan, in plain Python data."""

    kind: str                       # "gemm", "conv2d", "transpose", "pad", "relu", "copy"
    node: str                       # name of the graph node that owns the step
    in0: int
    in1: int
    out: int
    flags: int = 0
    relu_threshold: float = 0.0
    pad_value: float = 0.0
    ndim: int = 0
    dims: tuple[int, ...] = ()
    aux0: tuple[int, ...] = ()
    aux1: tuple[int, ...] = ()
    config: dict[str, int] = field(default_factory=dict)
    fused: tuple[str, ...] = ()     # names of the nodes folded into this step
    flops: int = 0                  # 2 * FMAs for contractions, else 0
    bytes: int = 0                  # algorithmic bytes: operands read once + result written once

    KIND_CODES = {"gemm": capi.STEP_GEMM, "conv2d": capi.STEP_CONV2D,
                  "transpose": capi.STEP_TRANSPOSE, "pad": capi.STEP_PAD,
                  "relu": capi.STEP_RELU, "copy": capi.STEP_COPY}

    def to_c(self) -> capi.Step:
        s = capi.Step()
        s.kind = self.KIND_CODES[self.kind]
        s.in0, s.in1, s.out = self.in0, self.in1, self.out
        s.flags = self.flags
        s.ndim = self.ndim
        s.relu_threshold = float(self.relu_threshold)
        s.pad_value = float(self.pad_value)
        for name in ("dims", "aux0", "aux1"):
            arr = getattr(s, name)
            for i, v in enumerate(getattr(self, name)):
                arr[i] = int(v)
        for key, value in self.config.items():
            setattr(s.cfg, key, int(value))
        return s


@dataclass
class Plan:
    """A lowered graph: steps over numbered buffer slots."""

    name: str
    steps: list[StepDesc]
    n_inputs: int
    n_outputs: int
    slot_bytes: list[int]
    slot_shapes: list[tuple[int, ...]]
    input_layouts: list[Any]

    @property
    def flops(self) -> int:
        return sum(s.flops for s in self.steps)

    @property
    def bytes(self) -> int:
        return sum(s.bytes for s in self.steps)


def _shape(t: Any) -> tuple[int, ...]:
    return tuple(int(d) for d in t.shape)


def _prod(values) -> int:
    out = 1
    for v in values:
        out *= int(v)
    return out


def _pad_widths(padding: Any, ndim: int) -> list[tuple[int, int]]:
    if isinstance(padding, dict):
        widths = [(0, 0)] * ndim
        for axis, (lo, hi) in padding.items():
            widths[axis] = (int(lo), int(hi))
        return widths
    return [(int(padding[0]), int(padding[1]))] * ndim


def _conv_stride(attrs) -> tuple[int, int]:
    stride = attrs.get("stride", (1, 1))
    if isinstance(stride, int):
        return (stride, stride)
    stride = tuple(stride)
    return (stride[0], stride[0]) if len(stride) == 1 else (int(stride[0]), int(stride[1]))


PRECISIONS = {"tf32": capi.PRECISION_TF32, "3xtf32": capi.PRECISION_3XTF32,
              "fp32": capi.PRECISION_FP32_SIMT}


def lower(graph: Any, node_configs: dict[str, dict] | None = None,
          fuse_transpose: dict[str, set[int]] | bool = False,
          precision: str = "tf32") -> Plan:
    """Lower ``graph`` to a Plan.

    node_configs: node name -> kernel parameters (tile_m, tile_n, tile_k, stages,
      epilogue) decided by the scheduler.
    fuse_transpose: True to fold every eligible transpose into its matmul, or a
      map node name -> operand indices requested through ``fuse_producer_at``.
    """
    node_configs = node_configs or {}
    if precision not in PRECISIONS:
        raise ValueError(f"precision must be one of {sorted(PRECISIONS)}, got {precision!r}")
    nodes = list(graph.nodes.values())
    inputs, outputs = list(graph.inputs), list(graph.outputs)
    if graph.inputs_types is None:
        raise LoweringError("graph types were not forwarded (inputs need constant shapes)")

    producer = {n.uid: n for n in nodes}
    users: dict[str, list[Any]] = {}
    for n in nodes:
        for u in n.inputs:
            users.setdefault(u, []).append(n)
    out_set = set(outputs)

    shapes: dict[str, tuple[int, ...]] = {}
    layouts: dict[str, Any] = {}
    for uid, t in zip(inputs, graph.inputs_types):
        if str(t.dtype) != "float32":
            raise LoweringError(f"only float32 graphs are supported, input {uid} is {t.dtype}")
        shapes[uid] = _shape(t)
        layouts[uid] = getattr(t, "layout", None)
    for n in nodes:
        t = n.operation.outputs_types[0]
        if str(t.dtype) != "float32":
            raise LoweringError(f"only float32 graphs are supported, node {n.name} is {t.dtype}")
        shapes[n.uid] = _shape(t)

    def only_user(uid: str, user: Any) -> bool:
        us = users.get(uid, [])
        return len(us) == 1 and us[0] is user and uid not in out_set

    def wants_transpose_fusion(node: Any, idx: int) -> bool:
        if fuse_transpose is True:
            return True
        if not fuse_transpose:
            return False
        return idx in fuse_transpose.get(node.name, set())

    # ---- pass 1: decide what is folded into what --------------------------------
    absorbed: set[str] = set()          # node uids that emit no step of their own
    relu_of: dict[str, Any] = {}        # contraction uid -> relu node folded into it
    pad_of: dict[str, Any] = {}         # conv uid -> pad node folded into it
    trans_of: dict[tuple[str, int], Any] = {}  # (matmul uid, operand) -> transpose node
    for n in nodes:
        op = n.operation
        if op.name not in ("matmul", "conv2d"):
            continue
        us = users.get(n.uid, [])
        if len(us) == 1 and us[0].operation.name == "relu" and n.uid not in out_set:
            relu_of[n.uid] = us[0]
            absorbed.add(us[0].uid)
        if op.name == "conv2d":
            p = producer.get(n.inputs[0])
            if p is not None and p.operation.name in ("pad", "pad2d") and only_user(p.uid, n):
                pa = p.operation.attrs
                in_shape = _shape(p.operation.inputs_types[0])
                widths = _pad_widths(pa["padding"], len(in_shape))
                nd = len(in_shape)
                spatial_only = all(w == (0, 0) for i, w in enumerate(widths) if i not in (nd - 3, nd - 2))
                if (nd >= 3 and spatial_only and float(pa.get("constant_value", 0)) == 0.0
                        and all(lo >= 0 and hi >= 0 for lo, hi in widths)):
                    pad_of[n.uid] = p
                    absorbed.add(p.uid)
        else:
            for idx in (0, 1):
                p = producer.get(n.inputs[idx])
                if (p is not None and p.operation.name == "transpose" and only_user(p.uid, n)
                        and wants_transpose_fusion(n, idx)):
                    in_shape = _shape(p.operation.inputs_types[0])
                    axes = tuple(p.operation.attrs.get("axes", ())) or (1, 0)
                    if len(in_shape) == 2 and axes == (1, 0):
                        trans_of[(n.uid, idx)] = p
                        absorbed.add(p.uid)

    # ---- slots --------------------------------------------------------------------
    slot_of: dict[str, int] = {}
    slot_shapes: list[tuple[int, ...]] = []
    for uid in inputs:
        slot_of[uid] = len(slot_shapes)
        slot_shapes.append(shapes[uid])
    out_slots = []
    for uid in outputs:
        out_slots.append(len(slot_shapes))
        if uid not in slot_of:
            slot_of[uid] = len(slot_shapes)
        slot_shapes.append(shapes[uid])

    def slot(uid: str) -> int:
        if uid not in slot_of:
            slot_of[uid] = len(slot_shapes)
            slot_shapes.append(shapes[uid])
        return slot_of[uid]

    def nbytes(uid: str) -> int:
        return 4 * _prod(shapes[uid])

    # ---- pass 2: emit steps ---------------------------------------------------------
    steps: list[StepDesc] = []
    for n in nodes:
        if n.uid in absorbed:
            continue
        op = n.operation
        attrs = dict(op.attrs)
        cfg = dict(node_configs.get(n.name, {}))
        fused: list[str] = []
        if op.name in ("matmul", "conv2d"):
            cfg.setdefault("precision", PRECISIONS[precision])
            if op.name == "conv2d" and cfg["precision"] == capi.PRECISION_3XTF32:
                # the convolution kernels have no operand-split mode: a graph compiled for
                # 3xTF32 runs its convolutions in fp32 FMA, which is at least as accurate
                cfg["precision"] = capi.PRECISION_FP32_SIMT
            if cfg["precision"] == capi.PRECISION_3XTF32 and cfg.get("tile_n", 0) > 128:
                # the 3xTF32 epilogue sums a tile row in registers: at most 128 columns
                cfg["tile_n"] = 128
            if (cfg["precision"] == capi.PRECISION_3XTF32 and cfg.get("tile_k", 0) > 32
                    and cfg.get("tile_n", 128) > 64):
                # a 3xTF32 stage holds hi and lo parts of both operands: at 128 columns and 64
                # of K per stage only one stage would fit
                cfg["tile_k"] = 32
            if cfg["precision"] != capi.PRECISION_TF32 and cfg.get("tile_m", 0) > 128:
                cfg["tile_m"] = 128  # the CTA-pair kernel is a TF32-only configuration
            out_uid, flags, thr = n.uid, 0, 0.0
            relu = relu_of.get(n.uid)
            if relu is not None:
                out_uid = relu.uid
                flags |= capi.FUSE_RELU
                thr = float(relu.operation.attrs.get("threshold", 0))
                fused.append(relu.name)
        if op.name == "matmul":
            srcs = []
            for idx in (0, 1):
                uid = n.inputs[idx]
                t = trans_of.get((n.uid, idx))
                transposed = False
                if t is not None:
                    uid = t.inputs[0]
                    transposed = True
                    fused.append(t.name)
                if uid in layouts and layouts[uid] is not None and list(layouts[uid]) == [1, 0]:
                    transposed = not transposed
                srcs.append((uid, transposed))
            s0, s1 = _shape(op.inputs_types[0]), _shape(op.inputs_types[1])
            M, K, N = s0[0], _prod(s0[1:]), s1[-1]
            a_t, b_t = srcs[0][1], srcs[1][1]
            if a_t:
                flags |= capi.GEMM_A_TRANSPOSED
            if b_t:
                flags |= capi.GEMM_B_TRANSPOSED
            steps.append(StepDesc(
                "gemm", n.name, slot(srcs[0][0]), slot(srcs[1][0]), slot(out_uid), flags, thr,
                dims=(M, N, K, M if a_t else K, K if b_t else N, N), config=cfg,
                fused=tuple(fused), flops=2 * M * N * K, bytes=4 * (M * K + K * N + M * N)))
        elif op.name == "conv2d":
            x_uid = n.inputs[0]
            pads = (0, 0, 0, 0)
            p = pad_of.get(n.uid)
            if p is not None:
                x_uid = p.inputs[0]
                in_shape = _shape(p.operation.inputs_types[0])
                widths = _pad_widths(p.operation.attrs["padding"], len(in_shape))
                nd = len(in_shape)
                pads = (*widths[nd - 3], *widths[nd - 2])
                fused.append(p.name)
            xs = shapes[x_uid]
            R, S, C, F = _shape(op.inputs_types[1])
            B, H, W = _prod(xs[:-3]), xs[-3], xs[-2]
            sh, sw = _conv_stride(attrs)
            os_ = shapes[n.uid]
            steps.append(StepDesc(
                "conv2d", n.name, slot(x_uid), slot(n.inputs[1]), slot(out_uid), flags, thr,
                dims=(B, H, W, C, R, S), aux0=(F, sh, sw), aux1=pads, config=cfg,
                fused=tuple(fused), flops=2 * _prod(os_) * R * S * C,
                bytes=nbytes(x_uid) + 4 * R * S * C * F + 4 * _prod(os_)))
        elif op.name == "relu":
            steps.append(StepDesc("relu", n.name, slot(n.inputs[0]), -1, slot(n.uid),
                                  relu_threshold=float(attrs.get("threshold", 0)),
                                  dims=(_prod(shapes[n.uid]),), bytes=2 * nbytes(n.uid)))
        elif op.name == "transpose":
            in_shape = _shape(op.inputs_types[0])
            if len(in_shape) > capi.MAX_DIMS:
                raise LoweringError(f"transpose of rank {len(in_shape)} > {capi.MAX_DIMS}")
            axes = tuple(attrs.get("axes", ())) or tuple(reversed(range(len(in_shape))))
            steps.append(StepDesc("transpose", n.name, slot(n.inputs[0]), -1, slot(n.uid),
                                  ndim=len(in_shape), dims=in_shape, aux0=axes,
                                  bytes=2 * nbytes(n.uid)))
        elif op.name in ("pad", "pad2d", "unpad"):
            in_shape = _shape(op.inputs_types[0])
            if len(in_shape) > capi.MAX_DIMS:
                raise LoweringError(f"{op.name} of rank {len(in_shape)} > {capi.MAX_DIMS}")
            widths = _pad_widths(attrs["padding"], len(in_shape))
            sign = -1 if op.name == "unpad" else 1
            steps.append(StepDesc("pad", n.name, slot(n.inputs[0]), -1, slot(n.uid),
                                  pad_value=float(attrs.get("constant_value", 0)),
                                  ndim=len(in_shape), dims=in_shape,
                                  aux0=tuple(sign * lo for lo, _ in widths),
                                  aux1=tuple(sign * hi for _, hi in widths),
                                  bytes=nbytes(n.inputs[0]) + nbytes(n.uid)))
        elif op.name == "reshape" and n.uid not in out_set:
            # same bytes under another shape: the result shares its producer's buffer
            slot_of[n.uid] = slot(n.inputs[0])
        elif op.name == "reshape":
            steps.append(StepDesc("copy", n.name, slot(n.inputs[0]), -1, slot(n.uid),
                                  dims=(_prod(shapes[n.uid]),), bytes=2 * nbytes(n.uid)))
        else:
            raise LoweringError(f"operator {op.name!r} has no CUDA lowering")
    # a graph output that is itself a graph input: plain copy
    for uid, s in zip(outputs, out_slots):
        if uid in inputs:
            steps.append(StepDesc("copy", uid, slot_of[uid], -1, s, dims=(_prod(shapes[uid]),),
                                  bytes=2 * nbytes(uid)))
    if not steps:
        raise LoweringError("graph has no operation to run")
    # graph outputs listed twice share a slot with their first occurrence: the C
    # side only knows slots, so alias later duplicates by an extra copy
    seen: dict[str, int] = {}
    for uid, s in zip(outputs, out_slots):
        if uid in seen:
            steps.append(StepDesc("copy", uid, seen[uid], -1, s, dims=(_prod(shapes[uid]),),
                                  bytes=2 * nbytes(uid)))
        else:
            seen[uid] = slot_of[uid]
    return Plan(
        name=graph.name or "payload",
        steps=steps,
        n_inputs=len(inputs),
        n_outputs=len(outputs),
        slot_bytes=[4 * _prod(s) for s in slot_shapes],
        slot_shapes=slot_shapes,
        input_layouts=[layouts.get(u) for u in inputs],
    )
