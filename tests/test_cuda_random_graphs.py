"""Randomised whole-graph parity: seeded random operator chains, built with the
graph DSL, lowered by the CUDA backend (with whatever fusion the lowering
decides on: relu into the producing kernel, zero pads into the convolution,
transposes read in place) and compared with the oracle evaluated step by step in
float64 on the same inputs.

Tolerances as in test_cuda_parity.py (max|y - y64| / max|y64|): TF32 1e-2,
3xTF32 / fp32 2e-5; chains made only of movement operators are bit-exact.
"""

import random

import numpy as np
import pytest

import xtc_b200.graphs.xtc.op as O
from oracle import xtc_oracle as xo
from xtc_b200.backends.cuda import Backend
from xtc_b200.runtimes.cuda import CudaDevice

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(cuda_lib):
    d = CudaDevice(0)
    assert d.detect_accelerator(), "no CUDA device: the gpu tests need one"
    d.activate()
    return d


class Chain:
    """Builds a graph and its float64 oracle value side by side."""

    def __init__(self, rng: random.Random, nprng: np.random.Generator, tensors=None):
        self.rng, self.nprng = rng, nprng
        self.inputs: list[np.ndarray] = []
        self.preset = tensors is not None
        self.tensors = list(tensors or [])
        self.steps: list[str] = []
        self.contractions = 0

    def source(self, shape, lo=-0.5, hi=0.5):
        arr = self.nprng.uniform(lo, hi, shape).astype(np.float32)
        self.inputs.append(arr)
        if not self.preset:
            self.tensors.append(O.tensor(tuple(shape), "float32", name=f"in{len(self.inputs) - 1}"))
        return len(self.inputs) - 1

    def note(self, text: str) -> None:
        self.steps.append(text)


def dim(rng: random.Random, top: int) -> int:
    return rng.choice([1, 3, 4, 8, 17, 32, 64, 100, 128, 129, 4 * rng.randint(1, top // 4), rng.randint(1, top)])


def movement_tail(ch: Chain, expr, val):
    """Zero to two bit-exact operators appended to a chain."""
    rng = ch.rng
    for _ in range(rng.choice([0, 0, 1, 2])):
        kind = rng.choice(["transpose", "pad", "unpad", "reshape", "relu"])
        if kind in ("pad", "unpad") and val.ndim < 2:  # defined from two dimensions up
            kind = "relu"
        if kind == "transpose":
            axes = list(range(val.ndim))
            rng.shuffle(axes)
            expr, val = O.transpose(expr, axes=tuple(axes)), xo.transpose(val, axes)
            ch.note(f"transpose{tuple(axes)}")
        elif kind == "pad":
            widths = tuple((rng.choice([0, 1, 2]), rng.choice([0, 0, 3])) for _ in range(val.ndim))
            value = rng.choice([0.0, -2.5])
            expr, val = O.pad(expr, padding=widths, constant_value=value), xo.pad(val, widths, value)
            ch.note(f"pad{widths}={value}")
        elif kind == "unpad":
            widths = tuple((rng.choice([0, 1]), rng.choice([0, 1])) if n >= 3 else (0, 0) for n in val.shape)
            expr, val = O.unpad(expr, padding=widths), xo.unpad(val, widths)
            ch.note(f"unpad{widths}")
        elif kind == "reshape":
            shape = (-1,) if rng.random() < 0.5 else (val.shape[0], -1)
            expr, val = O.reshape(expr, shape=shape), xo.reshape(np.ascontiguousarray(val), shape)
            ch.note(f"reshape{shape}")
        else:
            thr = rng.choice([0.0, 0.02])
            expr, val = O.relu(expr, threshold=thr), xo.relu(val, thr)
            ch.note(f"relu({thr})")
    return expr, val


def matmul_chain(ch: Chain):
    rng = ch.rng
    m, k = dim(rng, 700), dim(rng, 900)
    a_t = rng.random() < 0.35
    a = ch.source((k, m) if a_t else (m, k))
    val = ch.inputs[a].astype(np.float64)
    expr = ch.tensors[a]
    if a_t:  # a materialised or fused transpose in front of the matmul
        expr, val = O.transpose(expr, axes=(1, 0)), xo.transpose(val, (1, 0))
        ch.note("transpose(1,0)")
    for layer in range(rng.choice([1, 1, 2])):
        n = dim(rng, 700)
        w_t = rng.random() < 0.25
        w = ch.source((n, val.shape[1]) if w_t else (val.shape[1], n))
        wexpr, wval = ch.tensors[w], ch.inputs[w].astype(np.float64)
        if w_t:
            wexpr, wval = O.transpose(wexpr, axes=(1, 0)), xo.transpose(wval, (1, 0))
        expr, val = O.matmul(expr, wexpr, name=f"mm{layer}"), xo.matmul(val, wval)
        ch.contractions += 1
        ch.note(f"matmul[{val.shape[0]}x{wval.shape[0]}x{n}]{'T' if w_t else ''}")
        if rng.random() < 0.6:
            thr = rng.choice([0.0, 0.0, 0.05])
            expr, val = O.relu(expr, threshold=thr), xo.relu(val, thr)
            ch.note(f"relu({thr})")
    return movement_tail(ch, expr, val)


def conv_chain(ch: Chain):
    rng = ch.rng
    b, h, w = rng.randint(1, 3), rng.randint(6, 28), rng.randint(6, 28)
    c = rng.choice([3, 4, 8, 16, 32, 64])
    x = ch.source((b, h, w, c), 0.0, 1.0)
    expr, val = ch.tensors[x], ch.inputs[x].astype(np.float64)
    for layer in range(rng.choice([1, 1, 2])):
        r, s = rng.choice([1, 3, 3, 5, 2]), rng.choice([1, 3, 3, 5, 2])
        how = rng.choice(["none", "pad", "pad", "pad2d", "pad_const"])
        if how in ("pad", "pad_const"):
            widths = {1: (rng.choice([0, 1, 2]), rng.choice([0, 1, 2])), 2: (rng.choice([0, 1, 2]), rng.choice([1, 2]))}
            value = 0.0 if how == "pad" else 0.5  # a non-zero constant cannot fold into the convolution
            expr, val = O.pad(expr, padding=widths, constant_value=value), xo.pad(val, widths, value)
            ch.note(f"pad{widths}={value}")
        elif how == "pad2d":
            p = rng.choice([1, 2])
            expr, val = O.pad2d(expr, padding=p, axes=(1, 2)), xo.pad2d(val, p, (1, 2))
            ch.note(f"pad2d({p})")
        if val.shape[1] < r or val.shape[2] < s:
            r = s = 1
        f = rng.choice([4, 8, 16, 24, 64, 128])
        stride = (rng.choice([1, 1, 2]), rng.choice([1, 1, 2]))
        wt = ch.source((r, s, val.shape[3], f), -0.3, 0.3)
        expr = O.conv2d(expr, ch.tensors[wt], stride=stride, name=f"conv{layer}")
        val = xo.conv2d(val, ch.inputs[wt].astype(np.float64), stride)
        ch.contractions += 1
        ch.note(f"conv{r}x{s}s{stride}->{f}")
        if rng.random() < 0.6:
            thr = rng.choice([0.0, 0.0, 0.1])
            expr, val = O.relu(expr, threshold=thr), xo.relu(val, thr)
            ch.note(f"relu({thr})")
    return movement_tail(ch, expr, val)


def movement_chain(ch: Chain):
    rng = ch.rng
    shape = [rng.choice([1, 2, 3, 5, 8, 16, 33, 64]) for _ in range(rng.randint(2, 4))]
    x = ch.source(shape)
    expr, val = ch.tensors[x], ch.inputs[x].astype(np.float64)
    while not ch.steps:
        expr, val = movement_tail(ch, expr, val)
    return expr, val


def build_case(build, rng, nprng, name):
    """Graph inputs are the tensors created outside the graph scope, so a chain is drawn
    twice from the same generator state: once to learn its input shapes, once for real."""
    state, npstate = rng.getstate(), nprng.bit_generator.state
    with O.graph(name="shapes_only"):
        dry = Chain(rng, nprng)
        build(dry)
    rng.setstate(state)
    nprng.bit_generator.state = npstate
    tensors = [O.tensor(tuple(a.shape), "float32", name=f"in{i}") for i, a in enumerate(dry.inputs)]
    ch = Chain(rng, nprng, tensors)
    with O.graph(name=name) as gb:
        _, val = build(ch)
    return ch, gb, val


def run(graph, ins, precision):
    impl = Backend(graph)
    module = impl.get_compiler(shared_lib=False, precision=precision).compile(impl.get_scheduler().schedule())
    outs = [np.full(tuple(t.shape), np.nan, np.float32) for t in graph.outputs_types]
    results, code, msg = module.get_evaluator(parameters=(ins, outs), repeat=1, number=1,
                                              min_repeat_ms=0).evaluate()
    assert code == 0, msg
    return outs[0]


@pytest.mark.parametrize("family,seed", [(f, s) for f in ("matmul", "conv", "movement") for s in (0, 1)])
def test_random_operator_chains(dev, family, seed):
    rng = random.Random(5000 + 97 * seed + len(family))
    nprng = np.random.default_rng(5000 + seed)
    build = {"matmul": matmul_chain, "conv": conv_chain, "movement": movement_chain}[family]
    for case in range(25):
        ch, gb, val = build_case(build, rng, nprng, f"{family}_{seed}_{case}")
        graph = gb.graph
        precision = rng.choice(["tf32", "tf32", "3xtf32", "fp32"])
        what = f"{family} seed {seed} case {case} [{precision}]: " + " -> ".join(ch.steps)
        y = run(graph, ch.inputs, precision)
        assert y.shape == val.shape, what
        assert dev.status() == 0, what
        if ch.contractions == 0:
            assert np.array_equal(y.view(np.int32), val.astype(np.float32).view(np.int32)), what
            continue
        tol = 1e-2 if precision == "tf32" else 2e-5
        err = np.abs(y - val).max() / max(np.abs(val).max(), 1e-6)
        assert err <= tol, f"{what}: error {err}"
