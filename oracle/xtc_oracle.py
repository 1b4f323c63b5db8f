"""CPU oracle for the XTC graph hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A plain NumPy restatement of what the reference (xtc-tools/xtc) defines each
operator of the path to compute.  Only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py may import this module; nothing under
xtc_b200/ does.  Citations are paths inside the reference project.

Pinning: tests/test_oracle.py checks these functions against
  * the known-answer lines of the reference's own graph tests
    (tests/filecheck/graphs/test_matmul_relu.py:56-57, test_conv_relu.py:59-60,
    test_mlp.py, test_matmul.py, test_relu.py), and
  * tests/golden/*.npz, produced by tests/golden/make_golden.py from the
    reference's graph.forward imported from its source tree.

Every function takes and returns NumPy arrays and keeps the dtype of its first
input, as the reference does (operators.py:203-207, 318-324), so calling it on
float64 casts of the inputs gives the float64 reference the tolerances are
stated against.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from typing import Any

import numpy as np


def np_init(shape: Sequence[int], dtype: str = "float32") -> np.ndarray:
    """Default evaluation inputs: 1..9 cycling (src/xtc/utils/numpy.py:12-19)."""
    n = int(np.prod(shape)) if len(shape) else 1
    return (np.arange(n) % 9 + 1).reshape(shape).astype(dtype)


# --------------------------------------------------------------------------- #
# operators
# --------------------------------------------------------------------------- #
def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """src/xtc/graphs/xtc/operators.py:209-221: A is flattened to (i, -1), B to
    (-1, j), then np.dot; output (i, j) in A's dtype."""
    a2 = a.reshape(a.shape[0], -1)
    b2 = b.reshape(-1, b.shape[-1])
    assert a2.shape[1] == b2.shape[0], f"incompatible k: {a2.shape} {b2.shape}"
    return np.dot(a2, b2)


def relu(x: np.ndarray, threshold: float = 0) -> np.ndarray:
    """src/xtc/graphs/xtc/operators.py:224-249: np.maximum(x, threshold)."""
    return np.maximum(x, threshold)


def _stride2(stride: Any) -> tuple[int, int]:
    """src/xtc/graphs/xtc/operators.py:255-272."""
    if isinstance(stride, int):
        return (stride, stride)
    stride = tuple(stride)
    if len(stride) == 1:
        return (stride[0], stride[0])
    assert len(stride) == 2
    return (stride[0], stride[1])


def conv2d(x: np.ndarray, w: np.ndarray, stride: Any = (1, 1)) -> np.ndarray:
    """NHWC x RSCF convolution without implicit padding
    (src/xtc/graphs/xtc/operators.py:326-347): out[b,oh,ow,f] =
    sum_{r,s,c} x[b, oh*sh+r, ow*sw+s, c] * w[r,s,c,f], oh = (h-r)//sh + 1.
    Vectorised; conv2d_loop below is the literal loop."""
    sh, sw = _stride2(stride)
    h, wd, c = x.shape[-3:]
    r, s, wc, f = w.shape
    assert c == wc
    oh, ow = (h - r) // sh + 1, (wd - s) // sw + 1
    lead = x.shape[:-3]
    x4 = x.reshape(-1, h, wd, c)
    win = np.lib.stride_tricks.sliding_window_view(x4, (r, s), axis=(1, 2))
    win = win[:, ::sh, ::sw][:, :oh, :ow]  # (n, oh, ow, c, r, s)
    out = np.einsum("nhwcrs,rscf->nhwf", win, w, optimize=True).astype(x.dtype, copy=False)
    return out.reshape(*lead, oh, ow, f)


def conv2d_loop(x: np.ndarray, w: np.ndarray, stride: Any = (1, 1)) -> np.ndarray:
    """The reference's own element-by-element evaluation
    (src/xtc/graphs/xtc/operators.py:336-341); small cases only."""
    sh, sw = _stride2(stride)
    h, wd, c = x.shape[-3:]
    r, s, _, f = w.shape
    oh, ow = (h - r) // sh + 1, (wd - s) // sw + 1
    out = np.zeros((*x.shape[:-3], oh, ow, f), dtype=x.dtype).reshape(-1, oh, ow, f)
    x4 = x.reshape(-1, h, wd, c)
    for vb, voh, vow, vf in np.ndindex(out.shape):
        view = x4[vb, voh * sh : voh * sh + r, vow * sw : vow * sw + s, 0:c]
        out[vb, voh, vow, vf] = np.sum(view * w[:, :, :, vf])
    return out.reshape(*x.shape[:-3], oh, ow, f)


def normalize_pad(padding: Any, ndim: int) -> Any:
    """Padding normalisation of O.pad (src/xtc/graphs/xtc/operators.py:436-466):
    int -> (p, p) on every axis; 2 ints -> (lo, hi) on every axis; longer
    tuple -> the LAST len(tuple) axes; dict axis -> (lo, hi); zero-width
    entries are dropped."""
    if isinstance(padding, int):
        return (padding, padding)
    if isinstance(padding, (tuple, list)) and len(padding) == 2 and all(
        isinstance(p, int) for p in padding
    ):
        return tuple(padding)
    if isinstance(padding, (tuple, list)):
        n = len(padding)
        padding = {-(n - i): ((v, v) if isinstance(v, int) else tuple(v)) for i, v in enumerate(padding)}
    else:
        padding = {k: ((v, v) if isinstance(v, (int, float)) else tuple(v)) for k, v in padding.items()}
    return {k: v for k, v in padding.items() if tuple(v) != (0, 0)}


def pad_widths(padding: Any, ndim: int) -> list[tuple[int, int]]:
    """Per-axis (lo, hi) list (src/xtc/graphs/xtc/operators.py:413-424)."""
    if isinstance(padding, dict):
        pads = [(0, 0)] * ndim
        for axis, p in padding.items():
            pads[axis] = (int(p[0]), int(p[1]))
        return pads
    return [(int(padding[0]), int(padding[1]))] * ndim


def pad(x: np.ndarray, padding: Any = 0, constant_value: float = 0) -> np.ndarray:
    """src/xtc/graphs/xtc/operators.py:413-433: np.pad(mode="constant")."""
    pads = pad_widths(normalize_pad(padding, x.ndim), x.ndim)
    return np.pad(x, pads, mode="constant", constant_values=constant_value)


def normalize_pad2d(padding: Any, axes: Sequence[int] = (-3, -2)) -> dict:
    """src/xtc/graphs/xtc/operators.py:505-561."""
    a0, a1 = axes
    if isinstance(padding, int):
        d = {a0: (padding, padding), a1: (padding, padding)}
    elif isinstance(padding, dict):
        d = {k: ((v, v) if isinstance(v, int) else tuple(v)) for k, v in padding.items()}
    else:
        padding = tuple(padding)
        if len(padding) == 1:
            d = {a0: (padding[0],) * 2, a1: (padding[0],) * 2}
        elif len(padding) == 2 and all(isinstance(p, int) for p in padding):
            d = {a0: (padding[0], padding[1]), a1: (padding[0], padding[1])}
        elif len(padding) == 2:
            d = {a0: tuple(padding[0]), a1: tuple(padding[1])}
        else:
            assert len(padding) == 4
            d = {a0: (padding[0], padding[1]), a1: (padding[2], padding[3])}
    return {k: v for k, v in d.items() if tuple(v) != (0, 0)}


def pad2d(x: np.ndarray, padding: Any = (0, 0, 0, 0), axes: Sequence[int] = (-3, -2),
          constant_value: float = 0) -> np.ndarray:
    pads = pad_widths(normalize_pad2d(padding, axes), x.ndim)
    return np.pad(x, pads, mode="constant", constant_values=constant_value)


def unpad(x: np.ndarray, padding: Any = 0) -> np.ndarray:
    """src/xtc/graphs/xtc/operators.py:694-713: slice the widths off."""
    pads = pad_widths(normalize_pad(padding, x.ndim), x.ndim)
    return x[tuple(slice(lo, n - hi) for (lo, hi), n in zip(pads, x.shape))]


def reshape(x: np.ndarray, shape: Sequence[int] = (-1,)) -> np.ndarray:
    """src/xtc/graphs/xtc/operators.py:716-754."""
    return x.reshape(tuple(shape))


def transpose(x: np.ndarray, axes: Sequence[int] = ()) -> np.ndarray:
    """src/xtc/graphs/xtc/operators.py:757-787: axes () means reversed."""
    return x.transpose(tuple(axes) if len(axes) else None)


OPS = {
    "matmul": lambda ins, at: matmul(ins[0], ins[1]),
    "relu": lambda ins, at: relu(ins[0], at.get("threshold", 0)),
    "conv2d": lambda ins, at: conv2d(ins[0], ins[1], at.get("stride", (1, 1))),
    "pad": lambda ins, at: pad(ins[0], at.get("padding", 0), at.get("constant_value", 0)),
    "pad2d": lambda ins, at: pad2d(ins[0], at.get("padding", (0, 0, 0, 0)), at.get("axes", (-3, -2)),
                                   at.get("constant_value", 0)),
    "unpad": lambda ins, at: unpad(ins[0], at.get("padding", 0)),
    "reshape": lambda ins, at: reshape(ins[0], at.get("shape", (-1,))),
    "transpose": lambda ins, at: transpose(ins[0], at.get("axes", ())),
}


def run_graph(nodes: Sequence[Mapping[str, Any]], inputs: Mapping[str, np.ndarray],
              outputs: Sequence[str]) -> list[np.ndarray]:
    """Evaluate a graph given as a topologically ordered list of
    {"uid", "op", "args": [uids], "attrs": {}} (the interpreter of
    src/xtc/graphs/xtc/graph.py:109-125)."""
    env = dict(inputs)
    for node in nodes:
        ins = [env[a] for a in node["args"]]
        env[node["uid"]] = OPS[node["op"]](ins, dict(node.get("attrs", {})))
    return [env[o] for o in outputs]


# --------------------------------------------------------------------------- #
# The five benchmark configurations (seeded synthetic inputs)
# --------------------------------------------------------------------------- #
def config_inputs(name: str, scale: int = 1) -> list[np.ndarray]:
    """Inputs of configuration `name` ("c1".."c5"), drawn in graph-input order
    from np.random.default_rng(seed).  `scale` > 1 divides the large extents so
    the oracle finishes in seconds."""
    s = scale
    if name == "c1":
        rng = np.random.default_rng(0)
        return [rng.uniform(-1, 1, (512 // s, 1024 // s)).astype(np.float32),
                rng.uniform(-1, 1, (1024 // s, 256 // s)).astype(np.float32)]
    if name == "c2":
        rng = np.random.default_rng(1)
        n = 4096 // s
        return [rng.uniform(-1, 1, (n, n)).astype(np.float32), rng.uniform(-1, 1, (n, n)).astype(np.float32)]
    if name == "c3":
        rng = np.random.default_rng(2)
        return [rng.uniform(0, 1, (max(32 // s, 1), 56, 56, 64)).astype(np.float32),
                rng.normal(0, np.sqrt(2 / 576), (3, 3, 64, 64)).astype(np.float32)]
    if name == "c4":
        rng = np.random.default_rng(3)
        n = 8192 // s
        return [rng.uniform(-1, 1, (n, n)).astype(np.float32),
                rng.normal(0, 0.02, (n, 1024 // s)).astype(np.float32)]
    if name == "c4a":
        return config_inputs("c4", s)[:1]
    if name == "c5":
        rng = np.random.default_rng(4)
        k = 8192 // s
        return [rng.uniform(-1, 1, (65536 // s, k)).astype(np.float32),
                rng.normal(0, 1 / np.sqrt(8192), (k, k)).astype(np.float32)]
    raise KeyError(name)


def config_forward(name: str, inputs: Sequence[np.ndarray]) -> np.ndarray:
    """Output of configuration `name` on `inputs` in the dtype of the inputs."""
    if name == "c4a":
        return transpose(inputs[0], (1, 0))
    a, b = inputs
    if name == "c1":
        return matmul(a, b)
    if name == "c2":
        return relu(matmul(a, b))
    if name == "c3":
        return relu(conv2d(pad(a, {1: (1, 1), 2: (1, 1)}, 0.0), b, (1, 1)))
    if name == "c4":
        return matmul(transpose(a, (1, 0)), b)
    if name == "c5":
        return matmul(a, b)
    raise KeyError(name)


def rel_err(y: np.ndarray, y64: np.ndarray) -> float:
    """max|y - y64| / max|y64|: the metric the tolerances are stated in."""
    y64 = np.asarray(y64, dtype=np.float64)
    denom = float(np.max(np.abs(y64))) if y64.size else 1.0
    if denom == 0.0:
        denom = 1.0
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - y64))) / denom if y64.size else 0.0
