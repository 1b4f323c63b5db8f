"""Graph DSL of the hot path: tensors, operators, nodes, graphs.

Same surface as the reference's ``xtc.graphs.xtc`` package (op factory
``op_factory.py:38-112``, scopes ``context.py:18-135``, graph ``graph.py:31-205``,
node ``node.py:22-167``, operation ``operation.py:17-99``, operators
``operators.py:35-804``, types ``data.py:31-236``), re-designed around one
operator table instead of a class per operator and per expression.

The NumPy ``forward`` of each operator is the validation reference the
evaluator's ``validate=True`` compares the device results against (as
``utils/evaluation.py:68-75,129-145`` does in the reference); it is never used
to produce a result the backend reports.
"""

from __future__ import annotations

import hashlib
import json
import threading
from collections.abc import Mapping, Sequence
from dataclasses import dataclass, field
from typing import Any, Callable

import numpy as np


def _prod(values: Sequence[int]) -> int:
    out = 1
    for v in values:
        out *= int(v)
    return out


# --------------------------------------------------------------------------- #
# types and values
# --------------------------------------------------------------------------- #
class TensorType:
    """Shape/dtype (+ device, const, layout) of a tensor (data.py:31-174)."""

    def __init__(self, shape=None, dtype=None, device=None, const=False, layout=None):
        self._shape = None if shape is None else tuple(shape)
        self._dtype = dtype
        self._device = device
        self._const = const
        self._layout = layout

    shape = property(lambda self: self._shape)
    dtype = property(lambda self: self._dtype)
    device = property(lambda self: self._device)
    const = property(lambda self: self._const)
    layout = property(lambda self: self._layout)

    @property
    def ndim(self) -> int:
        return 0 if self._shape is None else len(self._shape)

    def is_constant_shape(self) -> bool:
        return self._shape is not None and all(isinstance(d, int) for d in self._shape)

    def is_constant_dtype(self) -> bool:
        return self._dtype is not None

    def is_constant(self) -> bool:
        return self.is_constant_shape() and self.is_constant_dtype()

    @property
    def constant_shape(self) -> tuple[int, ...]:
        assert self.is_constant_shape(), "symbolic shapes are not supported"
        return tuple(int(d) for d in self._shape)

    @property
    def constant_dtype(self) -> str:
        assert self.is_constant_dtype(), "symbolic dtypes are not supported"
        return str(self._dtype)

    @property
    def constant(self) -> "TensorType":
        return TensorType(self.constant_shape, self.constant_dtype, self._device, self._const,
                          self._layout)

    @property
    def size(self) -> int:
        return 0 if self._shape is None else _prod(self.constant_shape)

    @property
    def itemsize(self) -> int:
        return np.dtype(self.constant_dtype).itemsize

    @property
    def nbytes(self) -> int:
        return self.size * self.itemsize

    def __repr__(self) -> str:
        dims = "??" if self._shape is None else "x".join(str(d if d else "?") for d in self._shape)
        text = f"{dims}x{self._dtype if self._dtype else '?'}"
        if self._const:
            text += ", const"
        if self._layout is not None:
            src = ",".join(str(i) for i in range(len(self._shape)))
            dst = ",".join(str(i) for i in self._layout)
            text += f", <({src})->({dst})>"
        return text

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, TensorType):
            return NotImplemented
        return (self._dtype == other._dtype and self._shape == other._shape
                and self._const == other._const and self._layout == other._layout)

    def __hash__(self) -> int:
        return hash((self._shape, self._dtype, self._const))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        if self._shape:
            out["shape"] = list(self._shape)
        if self._dtype:
            out["dtype"] = self._dtype
        return out

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TensorType":
        return cls(tuple(d["shape"]) if "shape" in d else None, d.get("dtype"))


class Tensor:
    """A NumPy-backed value (data.py:202-236)."""

    def __init__(self, data: Any = None, type: TensorType | None = None):
        self._data = None if data is None else np.array(data)
        if self._data is not None:
            self._type = TensorType(self._data.shape, str(self._data.dtype))
        else:
            self._type = type if type is not None else TensorType()

    type = property(lambda self: self._type)
    data = property(lambda self: self._data)

    def numpy(self) -> np.ndarray:
        assert self._data is not None
        return np.array(self._data)

    def __repr__(self) -> str:
        if self._data is None:
            return f"Tensor(type={self._type}, data=None)"
        flat = self._data.reshape(-1)
        if len(flat) > 8:
            text = (" ".join(f"{d:.4g}" for d in flat[:4]) + "..."
                    + " ".join(f"{d:.4g}" for d in flat[-4:]))
        else:
            text = " ".join(f"{d:g}" for d in flat)
        return f"Tensor(type={self._type}, data={text})"


# --------------------------------------------------------------------------- #
# operator table
# --------------------------------------------------------------------------- #
def _pair(value: Any, what: str) -> tuple[int, int]:
    if isinstance(value, int):
        return (value, value)
    value = tuple(value)
    if len(value) == 1:
        return (value[0], value[0])
    assert len(value) == 2, f"{what} of wrong size, expected 1 or 2: {value}"
    return (int(value[0]), int(value[1]))


def _norm_pad_attr(padding: Any) -> Any:
    """O.pad / O.unpad padding forms (operators.py:436-466): int, (lo, hi) for
    all axes, a tuple naming the last axes, or a dict axis -> width(s)."""
    if isinstance(padding, int):
        return (padding, padding)
    if (isinstance(padding, (tuple, list)) and len(padding) == 2
            and all(isinstance(p, int) for p in padding)):
        return tuple(padding)
    if isinstance(padding, (tuple, list)):
        n = len(padding)
        padding = {-(n - i): v for i, v in enumerate(padding)}
    assert isinstance(padding, dict), "padding is either a list of tuple/int or int or a dict"
    padding = {k: ((v, v) if isinstance(v, (int, float)) else tuple(v)) for k, v in padding.items()}
    return {k: v for k, v in padding.items() if v != (0, 0)}


def _norm_pad2d_attr(padding: Any, axes: Sequence[int]) -> dict:
    """O.pad2d padding forms (operators.py:505-561)."""
    a0, a1 = axes
    if isinstance(padding, int):
        out = {a0: (padding, padding), a1: (padding, padding)}
    elif isinstance(padding, dict):
        out = {k: ((v, v) if isinstance(v, int) else tuple(v)) for k, v in padding.items()}
    else:
        padding = tuple(padding)
        if len(padding) == 1:
            out = {a0: (padding[0], padding[0]), a1: (padding[0], padding[0])}
        elif len(padding) == 2 and all(isinstance(p, int) for p in padding):
            out = {a0: (padding[0], padding[1]), a1: (padding[0], padding[1])}
        elif len(padding) == 2:
            out = {a0: tuple(padding[0]), a1: tuple(padding[1])}
        else:
            assert len(padding) == 4, f"padding for pad2d of wrong size, expected 1, 2 or 4: {padding}"
            out = {a0: (padding[0], padding[1]), a1: (padding[2], padding[3])}
    return {k: v for k, v in out.items() if v != (0, 0)}


def pad_widths(padding: Any, ndim: int) -> list[tuple[int, int]]:
    """Per-axis (lo, hi) widths of a normalised padding attribute."""
    if isinstance(padding, dict):
        widths = [(0, 0)] * ndim
        for axis, (lo, hi) in padding.items():
            assert -ndim <= axis < ndim, f"axis: {axis} is out of bound"
            widths[axis] = (int(lo), int(hi))
        return widths
    return [(int(padding[0]), int(padding[1]))] * ndim


@dataclass
class OpDef:
    name: str
    arity: int
    normalize: Callable[[dict], dict]
    infer: Callable[[Sequence[TensorType], dict], tuple[tuple[int, ...], str]]
    forward: Callable[[Sequence[np.ndarray], dict], np.ndarray]
    space: Callable[[Sequence[TensorType], TensorType, dict], tuple]


def _flat_space(ins, out, attrs):
    return ({"i": _prod(ins[0].constant_shape)}, ("P",), (("i",),), (("i",),))


# matmul (operators.py:159-221)
def _mm_dims(ins):
    s0, s1 = ins[0].constant_shape, ins[1].constant_shape
    assert len(s0) >= 2 and len(s1) >= 2
    i, k = s0[0], _prod(s0[1:])
    bk, j = _prod(s1[:-1]), s1[-1]
    assert k == bk, f"incompatible dimension k for matmul inputs shapes: ({i}, {k}) ({bk}, {j})"
    return i, j, k


def _mm_infer(ins, attrs):
    i, j, _ = _mm_dims(ins)
    return (i, j), ins[0].dtype


def _mm_forward(xs, attrs):
    a, b = xs
    return np.dot(a.reshape(a.shape[0], -1), b.reshape(-1, b.shape[-1]))


def _mm_space(ins, out, attrs):
    i, j, k = _mm_dims(ins)
    return ({"i": i, "j": j, "k": k}, ("P", "P", "R"), (("i", "k"), ("k", "j")), (("i", "j"),))


# conv2d (operators.py:252-347)
def _conv_norm(attrs):
    out = dict(attrs)
    return out


def conv_stride(attrs) -> tuple[int, int]:
    return _pair(attrs.get("stride", (1, 1)), "stride for conv2d")


def _conv_dims(ins, attrs):
    xs, ws = ins[0].constant_shape, ins[1].constant_shape
    assert len(xs) >= 3 and len(ws) == 4
    h, w, c = xs[-3:]
    r, s, wc, f = ws
    assert c == wc, f"unexpected with shapes: inp_shape = {xs}, weight_shape = {ws}"
    sh, sw = conv_stride(attrs)
    return xs[:-3], (h - r) // sh + 1, (w - s) // sw + 1, f, r, s, c, sh, sw


def _conv_infer(ins, attrs):
    lead, oh, ow, f, *_ = _conv_dims(ins, attrs)
    return (*lead, oh, ow, f), ins[0].dtype


def _conv_forward(xs, attrs):
    x, w = xs
    sh, sw = conv_stride(attrs)
    h, wd, c = x.shape[-3:]
    r, s, _, f = w.shape
    oh, ow = (h - r) // sh + 1, (wd - s) // sw + 1
    x4 = x.reshape(-1, h, wd, c)
    out = np.zeros((x4.shape[0], oh, ow, f), dtype=x.dtype)
    # one (r, s) filter tap at a time: a strided window view times a [c, f] slab
    for fr in range(r):
        for fs in range(s):
            win = x4[:, fr : fr + (oh - 1) * sh + 1 : sh, fs : fs + (ow - 1) * sw + 1 : sw, :]
            out += np.tensordot(win, w[fr, fs], axes=([3], [0])).astype(x.dtype, copy=False)
    return out.reshape(*x.shape[:-3], oh, ow, f)


def _conv_space(ins, out, attrs):
    lead, oh, ow, f, r, s, c, sh, sw = _conv_dims(ins, attrs)
    dims = {"b": _prod(lead), "h": oh, "w": ow, "f": f, "r": r, "s": s, "c": c}
    return (dims, ("P", "P", "P", "P", "R", "R", "R"),
            (("b", f"h*{sh}+r", f"w*{sw}+s", "c"), ("r", "s", "c", "f")), (("b", "h", "w", "f"),))


# pad / pad2d / unpad (operators.py:350-713)
def _pad_norm(attrs):
    cv = attrs.get("constant_value", 0)
    assert isinstance(cv, (int, float)), "constant_value need to be a number"
    out = {"padding": _norm_pad_attr(attrs.get("padding", 0)), "constant_value": cv}
    if attrs.get("device") is not None:
        out["device"] = attrs["device"]
    return out


def _pad2d_norm(attrs):
    axes = tuple(attrs.get("axes", (-3, -2)))
    assert len(axes) == 2, f"axes for pad2d of wrong size, expected 2: {axes}"
    assert axes[0] != axes[1], f"axes need 2 different dimension to pad: {axes}"
    cv = attrs.get("constant_value", 0)
    assert isinstance(cv, (int, float)), "constant_value need to be a number"
    return {"padding": _norm_pad2d_attr(attrs.get("padding", (0, 0, 0, 0)), axes),
            "constant_value": cv}


def _pad_infer(ins, attrs):
    shape = ins[0].constant_shape
    assert len(shape) >= 2
    widths = pad_widths(attrs["padding"], len(shape))
    return tuple(n + lo + hi for n, (lo, hi) in zip(shape, widths)), ins[0].dtype


def _pad_forward(xs, attrs):
    widths = pad_widths(attrs["padding"], xs[0].ndim)
    return np.pad(xs[0], widths, mode="constant", constant_values=attrs["constant_value"])


def _pad_space(ins, out, attrs):
    shape = ins[0].constant_shape
    widths = pad_widths(attrs["padding"], len(shape))
    names = [f"d{i}" for i in range(len(shape))]
    padded_axes = (set(a % len(shape) for a in attrs["padding"]) if isinstance(attrs["padding"], dict)
                   else set(range(len(shape))))
    in_map = tuple(f"{n}-{widths[i][0]}" if i in padded_axes else n for i, n in enumerate(names))
    dims = {n: s + lo + hi for n, s, (lo, hi) in zip(names, shape, widths)}
    return dims, tuple("P" for _ in shape), (in_map,), (tuple(names),)


def _unpad_norm(attrs):
    return {"padding": _norm_pad_attr(attrs.get("padding", 0))}


def _unpad_infer(ins, attrs):
    shape = ins[0].constant_shape
    assert len(shape) >= 2
    widths = pad_widths(attrs["padding"], len(shape))
    return tuple(n - lo - hi for n, (lo, hi) in zip(shape, widths)), ins[0].dtype


def _unpad_forward(xs, attrs):
    x = xs[0]
    widths = pad_widths(attrs["padding"], x.ndim)
    return x[tuple(slice(lo, n - hi) for (lo, hi), n in zip(widths, x.shape))]


def _unpad_space(ins, out, attrs):
    shape = ins[0].constant_shape
    widths = pad_widths(attrs["padding"], len(shape))
    names = [f"d{i}" for i in range(len(shape))]
    padded_axes = (set(a % len(shape) for a in attrs["padding"]) if isinstance(attrs["padding"], dict)
                   else set(range(len(shape))))
    in_map = tuple(f"{n}+{widths[i][0]}" if i in padded_axes else n for i, n in enumerate(names))
    dims = {n: s - lo - hi for n, s, (lo, hi) in zip(names, shape, widths)}
    return dims, tuple("P" for _ in shape), (in_map,), (tuple(names),)


# reshape / transpose / relu (operators.py:716-804, 224-249)
def _reshape_norm(attrs):
    if "shape" not in attrs:
        return dict(attrs)
    shape = tuple(attrs["shape"])
    assert all(x is not None for x in shape) and sum(1 for x in shape if x == -1) <= 1
    return {**attrs, "shape": shape}


def _reshape_infer(ins, attrs):
    shape = tuple(attrs.get("shape", (-1,)))
    fixed = _prod([x for x in shape if x != -1])
    return tuple(x if x != -1 else ins[0].size // fixed for x in shape), ins[0].dtype


def _transpose_axes(attrs, ndim):
    axes = tuple(attrs.get("axes", ()))
    return tuple(reversed(range(ndim))) if axes == () else axes


def _transpose_infer(ins, attrs):
    shape = ins[0].constant_shape
    axes = _transpose_axes(attrs, len(shape))
    assert len(axes) == len(shape)
    return tuple(shape[a] for a in axes), ins[0].dtype


OPS: dict[str, OpDef] = {
    "matmul": OpDef("matmul", 2, dict, _mm_infer, _mm_forward, _mm_space),
    "relu": OpDef("relu", 1, dict, lambda ins, at: (ins[0].constant_shape, ins[0].dtype),
                  lambda xs, at: np.maximum(xs[0], at.get("threshold", 0)), _flat_space),
    "conv2d": OpDef("conv2d", 2, _conv_norm, _conv_infer, _conv_forward, _conv_space),
    "pad": OpDef("pad", 1, _pad_norm, _pad_infer, _pad_forward, _pad_space),
    "pad2d": OpDef("pad2d", 1, _pad2d_norm, _pad_infer, _pad_forward, _pad_space),
    "unpad": OpDef("unpad", 1, _unpad_norm, _unpad_infer, _unpad_forward, _unpad_space),
    "reshape": OpDef("reshape", 1, _reshape_norm, _reshape_infer,
                     lambda xs, at: xs[0].reshape(tuple(at.get("shape", (-1,)))), _flat_space),
    "transpose": OpDef("transpose", 1, lambda at: {"axes": tuple(at.get("axes", ()))},
                       _transpose_infer,
                       lambda xs, at: xs[0].transpose(_transpose_axes(at, xs[0].ndim)), _flat_space),
}


def ops_version() -> str:
    """Hash of the operator set, stored in serialised graphs (operators.py:129-133)."""
    return hashlib.sha256("|".join(sorted(OPS)).encode()).hexdigest()[:16]


# --------------------------------------------------------------------------- #
# expressions, operations, nodes
# --------------------------------------------------------------------------- #
_counter_lock = threading.Lock()
_counter = [0]


def _next_idx() -> int:
    with _counter_lock:
        idx = _counter[0]
        _counter[0] += 1
    return idx


class Expr:
    """A value of the DSL: a tensor placeholder or the result of an operator."""

    def __init__(self, op_name: str, args: tuple["Expr", ...] = (), attrs: dict | None = None,
                 type: TensorType | None = None, value: Tensor | None = None):
        self._idx = _next_idx()
        self.op_name = op_name
        self.args = args
        self.attrs = dict(attrs or {})
        self.type = type          # tensors only
        self.value = value        # tensors only

    @property
    def uid(self) -> str:
        return f"%{self._idx}"

    @property
    def is_tensor(self) -> bool:
        return self.op_name == "tensor"

    def __str__(self) -> str:
        params = [a.uid for a in self.args] + [f"{k}={v}" for k, v in self.attrs.items()]
        return f"{self.uid} = {self.op_name}({', '.join(params)})"

    def to_dict(self) -> dict[str, Any]:
        if self.is_tensor:
            return {"type": self.type.to_dict()}

        def listify(obj):
            if isinstance(obj, dict):
                return {k: listify(v) for k, v in obj.items()}
            if isinstance(obj, tuple):
                return [listify(v) for v in obj]
            return obj

        return {"op": {"name": self.op_name, "attrs": {k: listify(v) for k, v in self.attrs.items()}},
                "args": [a.uid for a in self.args]}


@dataclass(frozen=True)
class Operation:
    """What a backend reads from a node (operation.py:17-99)."""

    name: str
    attrs: Mapping[str, Any]
    inputs_types: tuple[TensorType, ...]
    outputs_types: tuple[TensorType, ...]
    dims: Mapping[str, int]
    kinds: tuple[str, ...]
    inps_maps: tuple = field(default=())
    outs_maps: tuple = field(default=())

    def dims_kind(self, kind: str) -> list[str]:
        return [d for d, k in zip(self.dims, self.kinds) if k == kind]

    @property
    def accesses_maps(self):
        return (tuple(self.dims.keys()), self.inps_maps, self.outs_maps)

    @property
    def ops_count(self) -> int:
        return _prod(list(self.dims.values()))

    @property
    def ops_dtype(self) -> str:
        return self.outputs_types[0].constant_dtype

    @property
    def signature(self) -> list[Any]:
        return json.loads(json.dumps([self.name, list(self.dims.values()), self.ops_dtype,
                                      dict(self.attrs)], default=str))


class Node:
    """A graph node = one expression with inferred types (node.py:22-167)."""

    _by_uid: dict[str, "Node"] = {}
    _lock = threading.Lock()

    def __init__(self, expr: Expr, name: str | None = None):
        self._expr = expr
        self._name = name if name is not None else expr.uid
        self._inputs_types: list[TensorType] | None = None
        self._outputs_types: list[TensorType] | None = None

    @classmethod
    def of(cls, expr: Expr, name: str | None = None) -> "Node":
        with cls._lock:
            node = cls._by_uid.get(expr.uid)
            if node is None:
                node = cls._by_uid[expr.uid] = Node(expr, name)
        return node

    name = property(lambda self: self._name)
    uid = property(lambda self: self._expr.uid)
    inputs = property(lambda self: [a.uid for a in self._expr.args])
    outputs = property(lambda self: [self._expr.uid])
    preds = property(lambda self: list(dict.fromkeys(a.uid for a in self._expr.args)))
    preds_nodes = property(lambda self: [Node._by_uid[u] for u in self.preds])
    inputs_types = property(lambda self: self._inputs_types)
    outputs_types = property(lambda self: self._outputs_types)
    op_name = property(lambda self: self._expr.op_name)
    attrs = property(lambda self: self._expr.attrs)

    def forward_types(self, inputs_types: Sequence[TensorType]) -> list[TensorType]:
        self._inputs_types = list(inputs_types)
        if self._expr.is_tensor:
            assert self._expr.type.is_constant(), "Tensor type not constant in tensor initializer"
            out = [self._expr.type]
        else:
            op = OPS[self._expr.op_name]
            assert len(inputs_types) == op.arity, (
                f"len of inputs types mismatch : {len(inputs_types)} == {op.arity}")
            shape, dtype = op.infer(inputs_types, self._expr.attrs)
            out = [TensorType(shape, dtype, device=self._expr.attrs.get("device"))]
        self._outputs_types = out
        return out

    def forward(self, inputs: Sequence[Tensor]) -> list[Tensor]:
        if self._expr.is_tensor:
            return [self._expr.value]
        op = OPS[self._expr.op_name]
        assert len(inputs) == op.arity, f"len of inputs mismatch : {len(inputs)} == {op.arity}"
        result = Tensor(op.forward([t.numpy() for t in inputs], self._expr.attrs))
        shape, dtype = op.infer([t.type for t in inputs], self._expr.attrs)
        assert result.type == TensorType(shape, dtype), (
            f"output type mismatch expect: {result.type} != {TensorType(shape, dtype)}")
        return [result]

    @property
    def operation(self) -> Operation:
        assert self._inputs_types is not None and self._outputs_types is not None
        ins = tuple(t.constant for t in self._inputs_types)
        outs = tuple(t.constant for t in self._outputs_types)
        if self._expr.is_tensor:
            return Operation("tensor", {}, ins, outs, {"i": outs[0].size}, ("P",), (), (("i",),))
        dims, kinds, imaps, omaps = OPS[self._expr.op_name].space(ins, outs[0], self._expr.attrs)
        return Operation(self._expr.op_name, dict(self._expr.attrs), ins, outs, dims, tuple(kinds),
                         tuple(imaps), tuple(omaps))

    def __str__(self) -> str:
        text = str(self._expr).split("=", 1)[1].strip()
        if self.uid != self.name:
            text += f" {{name = {self.name!r}}}"
        if self._inputs_types is not None and self._outputs_types is not None:
            text += f" : {self._inputs_types} -> {self._outputs_types}"
        return text

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        if self.uid != self.name:
            out["name"] = self.name
        out["uid"] = self.uid
        out["expr"] = self._expr.to_dict()
        return out


def topological(nodes: Sequence[Node], seeds: Sequence[Node] | None = None) -> list[Node]:
    """Depth-first post-order from the output nodes (utils.py:14-53)."""
    members = set(nodes)
    if seeds is None:
        used = {p for n in nodes for p in n.preds_nodes}
        seeds = [n for n in nodes if n not in used]
    seen: set[Node] = set()
    order: list[Node] = []

    def visit(n: Node) -> None:
        if n in seen or n not in members:
            return
        seen.add(n)
        for p in n.preds_nodes:
            visit(p)
        order.append(n)

    for s in seeds:
        visit(s)
    return order


class Graph:
    """A dataflow graph (graph.py:31-205)."""

    def __init__(self, name: str | None = None):
        self._name = name
        self._nodes: list[Node] = []
        self._inputs: list[Node] = []
        self._outputs: list[Node] = []
        self._inputs_types: list[TensorType] | None = None
        self._outputs_types: list[TensorType] | None = None

    name = property(lambda self: "" if self._name is None else self._name)
    nodes = property(lambda self: {n.uid: n for n in self._nodes})
    inputs = property(lambda self: [n.uid for n in self._inputs])
    outputs = property(lambda self: [n.uid for n in self._outputs])
    inputs_nodes = property(lambda self: self._inputs)
    outputs_nodes = property(lambda self: self._outputs)
    inputs_types = property(lambda self: self._inputs_types)
    outputs_types = property(lambda self: self._outputs_types)

    def forward_types(self, inputs_types: Sequence[TensorType]) -> list[TensorType]:
        assert len(inputs_types) == len(self._inputs), (
            f"forward types inputs size mismatch: {len(inputs_types)} != {len(self._inputs)}")
        self._inputs_types = list(inputs_types)
        env = dict(zip(self.inputs, self._inputs_types))
        for node in topological(self._nodes):
            env[node.uid] = node.forward_types([env[u] for u in node.inputs])[0]
        self._outputs_types = [env[u] for u in self.outputs]
        return self._outputs_types

    def forward(self, inputs: Sequence[Tensor]) -> list[Tensor]:
        assert len(inputs) == len(self._inputs), (
            f"forward types inputs size mismatch: {len(inputs)} != {len(self._inputs)}")
        env = dict(zip(self.inputs, inputs))
        for node in topological(self._nodes):
            env[node.uid] = node.forward([env[u] for u in node.inputs])[0]
        return [env[u] for u in self.outputs]

    def __str__(self) -> str:
        lines = ["graph:"]
        if self.name:
            lines.append(f"  name: {self._name}")
        for title, uids, types in (("inputs", self.inputs, self._inputs_types),
                                   ("outputs", self.outputs, self._outputs_types)):
            if uids:
                lines.append(f"  {title}:")
                for i, uid in enumerate(uids):
                    lines.append(f"  - {uid}" + (f" : {types[i]}" if types else ""))
            else:
                lines.append(f"  {title}: []")
        if self._nodes:
            lines.append("  nodes:")
            for node in topological(self._nodes, self._outputs):
                lines.append(f"  - {node.uid}: {node}")
        else:
            lines.append("  nodes: {}")
        return "\n".join(lines) + "\n"

    def ops_dtype(self) -> str:
        return self._nodes[0].operation.ops_dtype if self._nodes else "float32"

    def ops_count(self) -> int:
        dtype = self.ops_dtype()
        return sum(n.operation.ops_count for n in self._nodes if n.operation.ops_dtype == dtype)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        if self._name:
            out["name"] = self._name
        out["inputs"] = [n.to_dict() for n in self._inputs]
        out["outputs"] = [{"uid": n.uid} for n in self._outputs]
        out["nodes"] = [n.to_dict() for n in self._nodes]
        out["ops_version"] = ops_version()
        base = int(out["inputs"][0]["uid"][1:]) if out["inputs"] else 0

        def compact(obj):
            if isinstance(obj, dict):
                return {k: compact(v) for k, v in obj.items()}
            if isinstance(obj, list):
                return [compact(v) for v in obj]
            if isinstance(obj, str) and obj[:1] == "%":
                return f"%{int(obj[1:]) - base}"
            return obj

        return compact(out)

    def dumps(self) -> str:
        import yaml

        return yaml.safe_dump(self.to_dict())

    def dump(self, file_name) -> None:
        import yaml
        from pathlib import Path

        path = Path(file_name)
        path.parent.mkdir(exist_ok=True, parents=True)
        with open(path, "w") as f:
            yaml.dump(self.to_dict(), f, sort_keys=False)


# --------------------------------------------------------------------------- #
# scopes (context.py:18-135) and the builder (builder.py:16-87)
# --------------------------------------------------------------------------- #
class _Scope:
    def __init__(self, **graph_kwargs: Any):
        self.exprs: list[Expr] = []
        self.names: list[str | None] = []
        self.inputs: list[Expr] = []
        self.outputs: list[Expr] = []
        self.graph_kwargs = graph_kwargs

    def build(self) -> Graph:
        defined = set(self.exprs)
        used = [a for e in self.exprs for a in e.args]
        free = sorted({u._idx: u for u in used if u not in defined}.values(), key=lambda e: e._idx)
        inputs = list({e._idx: e for e in self.inputs + free}.values())
        used_set = set(used)
        outputs = list({e._idx: e for e in
                        self.outputs + [e for e in self.exprs if e not in used_set]}.values())
        graph = Graph(**self.graph_kwargs)
        graph._nodes = [Node.of(e, n) for e, n in zip(self.exprs, self.names)]
        graph._inputs = [Node.of(e) for e in inputs]
        graph._outputs = [Node.of(e) for e in outputs]
        if all(n._expr.is_tensor and n._expr.type.is_constant() for n in graph._inputs):
            graph.forward_types([n._expr.type for n in graph._inputs])
        return graph


class _Scopes(threading.local):
    def __init__(self) -> None:
        self.stack = [_Scope()]

    def append(self, expr: Expr, name: str | None) -> Expr:
        for scope in self.stack:
            scope.exprs.append(expr)
            scope.names.append(name)
        return expr


CONTEXT = _Scopes()


class graph_builder:
    """``with O.graph(name=...) as gb: ...; gb.graph``"""

    def __init__(self, **graph_kwargs: Any):
        self._graph_kwargs = graph_kwargs
        self._graph: Graph | None = None

    def __enter__(self) -> "graph_builder":
        CONTEXT.stack.append(_Scope(**self._graph_kwargs))
        return self

    def __exit__(self, *_: Any) -> None:
        assert len(CONTEXT.stack) > 1
        self._graph = CONTEXT.stack.pop().build()

    @property
    def graph(self) -> Graph:
        assert self._graph is not None, "can't get graph inside builder context"
        return self._graph

    def set_outputs(self, *outs: Expr) -> None:
        CONTEXT.stack[-1].outputs = list(outs)

    def set_inputs(self, *inps: Expr) -> None:
        CONTEXT.stack[-1].inputs = list(inps)

    @classmethod
    def from_dict(cls, graph_dict: Mapping[str, Any]) -> Mapping[str, Any]:
        """Rebuild a serialised graph inside the current scope (builder.py:36-72)."""

        def tuplify(obj):
            if isinstance(obj, dict):
                return {k: tuplify(v) for k, v in obj.items()}
            if isinstance(obj, list):
                return tuple(tuplify(v) for v in obj)
            return obj

        scope = CONTEXT.stack[-1]
        if "name" in graph_dict:
            scope.graph_kwargs["name"] = graph_dict["name"]
        env: dict[str, Expr] = {}
        for inp in graph_dict["inputs"]:
            ttype = TensorType.from_dict(inp["expr"]["type"])
            env[inp["uid"]] = Expr("tensor", type=ttype, value=Tensor(type=ttype))  # not a node
        scope.inputs.extend(env.values())
        for node in graph_dict["nodes"]:
            expr = node["expr"]
            op_name = expr["op"]["name"]
            if op_name not in OPS:
                mismatch = ("version mismatch detected, "
                            if ops_version() != graph_dict.get("ops_version") else "")
                raise ValueError(mismatch + f"serialized op {op_name} is not implemented.")
            args = [env[a] for a in expr["args"]]
            env[node["uid"]] = make_op(op_name, args, node.get("name"),
                                       **tuplify(expr["op"]["attrs"]))
        scope.outputs.extend(env[o["uid"]] for o in graph_dict["outputs"])
        return graph_dict

    @classmethod
    def loads(cls, yaml_str: str) -> None:
        import yaml

        cls.from_dict(yaml.safe_load(yaml_str))

    @classmethod
    def load(cls, file_name) -> None:
        import yaml

        with open(file_name) as f:
            cls.from_dict(yaml.safe_load(f))


def make_tensor(*args: Any, name: str | None = None, **kw: Any) -> Expr:
    """``O.tensor``: (), (shape, dtype), (TensorType) or (Tensor) (expr.py:118-163)."""
    shape = kw.pop("shape", None)
    dtype = kw.pop("dtype", None)
    first = args[0] if args else kw.pop("tensor", None)
    if len(args) > 1:
        assert dtype is None
        dtype = args[1]
    value = None
    if isinstance(first, Tensor):
        value, ttype = first, first.type
    elif isinstance(first, TensorType):
        ttype = first
    else:
        if first is not None:
            shape = first
        assert shape is None or isinstance(shape, tuple)
        assert dtype is None or isinstance(dtype, str)
        ttype = TensorType(shape, dtype, device=kw.get("device"), const=kw.get("const", False),
                           layout=kw.get("layout"))
    expr = Expr("tensor", type=ttype, value=value if value is not None else Tensor(type=ttype))
    return CONTEXT.append(expr, name)


def make_op(op_name: str, args: Sequence[Expr], name: str | None = None, **attrs: Any) -> Expr:
    op = OPS[op_name]
    assert len(args) == op.arity, f"{op_name} takes {op.arity} operands"
    return CONTEXT.append(Expr(op_name, tuple(args), op.normalize(attrs)), name)
