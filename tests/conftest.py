"""Shared fixtures: the `gpu` marker, golden-vector access, library build."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _unjson(obj):
    if isinstance(obj, dict):
        if "__dict__" in obj:
            return {_unjson(k): _unjson(v) for k, v in obj["__dict__"]}
        if "__tuple__" in obj:
            return tuple(_unjson(v) for v in obj["__tuple__"])
        return {k: _unjson(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_unjson(v) for v in obj]
    return obj


class Golden:
    """tests/golden/reference_forward.{json,npz}: outputs of the reference's own
    graph.forward (float32 and float64) for each described case."""

    def __init__(self) -> None:
        self.meta = json.loads((GOLDEN_DIR / "reference_forward.json").read_text())
        self.arrays = np.load(GOLDEN_DIR / "reference_forward.npz")

    def names(self) -> list[str]:
        return list(self.meta)

    def nodes(self, name: str) -> list[dict]:
        return [{"op": n["op"], "args": n["args"], "attrs": _unjson(n["attrs"])}
                for n in self.meta[name]["nodes"]]

    def inputs(self, name: str) -> list[np.ndarray]:
        specs = self.meta[name]["inputs"]
        out, streams = [], {}
        for spec in specs:
            shape = tuple(spec["shape"])
            if spec["kind"] == "np_init":
                n = int(np.prod(shape))
                out.append(((np.arange(n) % 9 + 1).reshape(shape) + spec.get("offset", 0)).astype(np.float32))
                continue
            rng = streams.setdefault(spec["seed"], np.random.default_rng(spec["seed"]))
            if spec["kind"] == "uniform":
                out.append(rng.uniform(spec["lo"], spec["hi"], shape).astype(np.float32))
            else:
                out.append(rng.normal(0.0, spec["std"], shape).astype(np.float32))
        return out

    def output(self, name: str, dtype: str = "float32") -> np.ndarray:
        return self.arrays[f"{name}.{dtype}"]


GOLDEN = Golden()
GOLDEN_NAMES = GOLDEN.names()


@pytest.fixture(scope="session")
def golden() -> Golden:
    return GOLDEN


def build_dsl_graph(O, name: str, in_specs_shapes, nodes, typed: bool = True):
    """Build a case's graph with an `O`-style operator module."""
    tensors = [O.tensor(tuple(s), "float32", name=f"in{i}") if typed else O.tensor()
               for i, s in enumerate(in_specs_shapes)]
    with O.graph(name=name) as gb:
        vals = []
        for k, node in enumerate(nodes):
            ins = [tensors[int(a[1:])] if a[0] == "i" else vals[int(a[1:])] for a in node["args"]]
            vals.append(getattr(O, node["op"])(*ins, name=f"n{k}", **node["attrs"]))
    return gb.graph


@pytest.fixture(scope="session")
def cuda_lib():
    """The built C-ABI library (compiles it if stale)."""
    from xtc_b200 import build, capi

    build.build()
    return capi.load()


def has_cuda() -> bool:
    try:
        import ctypes

        from xtc_b200 import capi

        n = ctypes.c_int(0)
        return capi.load().xtc_cuda_device_count(ctypes.byref(n)) == 0 and n.value > 0
    except Exception:
        return False
