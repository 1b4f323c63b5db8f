"""Generate tests/golden/reference_forward.{json,npz} from the reference itself.

Run where the reference source tree is available:

    python tests/golden/make_golden.py /path/to/xtc

It imports the reference's ``xtc.graphs.xtc`` (pure Python + NumPy), builds each
case's graph with the reference DSL, evaluates ``graph.forward`` on float32
inputs and on float64 casts of the same inputs, and stores the outputs together
with a plain-data description of the graph and of how the inputs are generated.
Inputs are not stored: they are ``np_init`` patterns or seeded draws that the
tests regenerate.  Nothing in the test-suite imports the reference at run time.
"""

from __future__ import annotations

import importlib.metadata
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def import_reference(root: str):
    sys.path.insert(0, str(Path(root) / "src"))
    real_version = importlib.metadata.version

    def version(name: str) -> str:
        return "0.0.0" if name == "xtc" else real_version(name)

    importlib.metadata.version = version  # the reference asks for its installed dist version
    import xtc.graphs.xtc.op as O  # noqa: E402
    import xtc.graphs.xtc.ty as T  # noqa: E402

    return O, T


def gen_input(spec: dict) -> np.ndarray:
    """Input generators shared with tests/golden_cases.py (kept in sync by test)."""
    shape = tuple(spec["shape"])
    kind = spec["kind"]
    if kind == "np_init":  # 1..9 cycling, plus an offset
        n = int(np.prod(shape))
        return ((np.arange(n) % 9 + 1).reshape(shape) + spec.get("offset", 0)).astype(np.float32)
    rng = np.random.default_rng(spec["seed"])
    for _ in range(spec.get("skip", 0)):  # earlier draws of the same stream
        pass
    if kind == "uniform":
        return rng.uniform(spec["lo"], spec["hi"], shape).astype(np.float32)
    if kind == "normal":
        return rng.normal(0.0, spec["std"], shape).astype(np.float32)
    raise KeyError(kind)


def gen_inputs(specs: list[dict]) -> list[np.ndarray]:
    """Inputs sharing a seed are drawn from ONE stream in order, like the benchmark configs."""
    out = []
    streams: dict[int, np.random.Generator] = {}
    for spec in specs:
        shape = tuple(spec["shape"])
        if spec["kind"] == "np_init":
            out.append(gen_input(spec))
            continue
        rng = streams.setdefault(spec["seed"], np.random.default_rng(spec["seed"]))
        if spec["kind"] == "uniform":
            out.append(rng.uniform(spec["lo"], spec["hi"], shape).astype(np.float32))
        else:
            out.append(rng.normal(0.0, spec["std"], shape).astype(np.float32))
    return out


def ni(shape, offset=-5):
    return {"kind": "np_init", "shape": list(shape), "offset": offset}


def uni(shape, seed, lo=-1.0, hi=1.0):
    return {"kind": "uniform", "shape": list(shape), "seed": seed, "lo": lo, "hi": hi}


def nrm(shape, seed, std):
    return {"kind": "normal", "shape": list(shape), "seed": seed, "std": std}


# name -> (input specs, [(op, arg indices (negative = input -k-1... see below), attrs)])
# Node args refer to earlier values: "i0", "i1" are inputs, "n0", "n1" nodes.
CASES = {
    # tests/filecheck/graphs/test_matmul_relu.py
    "ref_matmul_relu": ([ni((5, 3)), ni((3, 4))],
                        [("matmul", ["i0", "i1"], {}), ("relu", ["n0"], {})]),
    # tests/filecheck/graphs/test_conv_relu.py
    "ref_conv_relu": ([ni((2, 6, 6, 3)), ni((8, 5, 5, 3))],
                      [("pad2d", ["i0"], {"padding": 2, "axes": (1, 2)}),
                       ("transpose", ["i1"], {"axes": (1, 2, 3, 0)}),
                       ("conv2d", ["n0", "n1"], {"stride": (2, 2)}),
                       ("relu", ["n2"], {"threshold": 0.1})]),
    # tests/filecheck/backends/test_matmul_mlir.py shape, default evaluation inputs
    "backend_matmul_4x32x512": ([ni((4, 512), 0), ni((512, 32), 0)], [("matmul", ["i0", "i1"], {})]),
    # tests/filecheck/backends/padding/test_pad_conv2d_mlir.py style graphs
    "backend_pad_conv_5x5_s2": ([ni((1, 8, 8, 3), 0), ni((5, 5, 3, 16), 0)],
                                [("pad", ["i0"], {"padding": {1: (2, 2), 2: (2, 2)}, "constant_value": 0}),
                                 ("conv2d", ["n0", "i1"], {"stride": (2, 2)}), ("relu", ["n1"], {})]),
    "backend_conv_3x3": ([ni((1, 10, 10, 3), 0), ni((3, 3, 3, 16), 0)],
                         [("conv2d", ["i0", "i1"], {}), ("relu", ["n0"], {})]),
    # the pytest backend API shape (tests/pytest/mlir/test_mlir_impl.py)
    "impl_matmul_128x256x91": ([ni((128, 91), 0), ni((91, 256), 0)], [("matmul", ["i0", "i1"], {})]),
    # operator attribute forms
    "pad_int": ([ni((3, 4))], [("pad", ["i0"], {"padding": 2, "constant_value": 1.5})]),
    "pad_pair": ([ni((3, 4, 2))], [("pad", ["i0"], {"padding": (1, 2)})]),
    "pad_tuple_last_axes": ([ni((2, 3, 4))], [("pad", ["i0"], {"padding": (1, (0, 2))})]),
    "pad_dict": ([ni((2, 5, 5, 4))], [("pad", ["i0"], {"padding": {1: (1, 0), -2: 2}, "constant_value": -3})]),
    "pad2d_4": ([ni((1, 4, 5, 2))], [("pad2d", ["i0"], {"padding": (1, 2, 0, 3)})]),
    "unpad_dict": ([ni((2, 6, 7, 3))], [("unpad", ["i0"], {"padding": {1: (1, 2), 2: (0, 3)}})]),
    "unpad_int": ([ni((5, 6))], [("unpad", ["i0"], {"padding": 1})]),
    "reshape": ([ni((2, 3, 4))], [("reshape", ["i0"], {"shape": (4, -1)})]),
    "transpose_default": ([ni((2, 3, 4))], [("transpose", ["i0"], {})]),
    "transpose_3d": ([ni((4, 6, 8))], [("transpose", ["i0"], {"axes": (1, 2, 0)})]),
    "relu_threshold": ([ni((4, 9))], [("relu", ["i0"], {"threshold": 2.5})]),
    "matmul_nd": ([ni((4, 2, 3)), ni((3, 2, 5))], [("matmul", ["i0", "i1"], {})]),
    # the five benchmark configurations at reduced extents, seeded like the full ones
    "c1_small": ([uni((128, 256), 0), uni((256, 64), 0)], [("matmul", ["i0", "i1"], {})]),
    "c2_small": ([uni((128, 128), 1), uni((128, 128), 1)],
                 [("matmul", ["i0", "i1"], {}), ("relu", ["n0"], {})]),
    "c3_small": ([uni((2, 14, 14, 64), 2, 0.0, 1.0), nrm((3, 3, 64, 64), 2, float(np.sqrt(2 / 576)))],
                 [("pad", ["i0"], {"padding": {1: (1, 1), 2: (1, 1)}, "constant_value": 0.0}),
                  ("conv2d", ["n0", "i1"], {"stride": (1, 1)}), ("relu", ["n1"], {})]),
    "c4_small": ([uni((128, 128), 3), nrm((128, 16), 3, 0.02)],
                 [("transpose", ["i0"], {"axes": (1, 0)}), ("matmul", ["n0", "i1"], {})]),
    "c5_small": ([uni((512, 64), 4), nrm((64, 64), 4, float(1 / np.sqrt(8192)))],
                 [("matmul", ["i0", "i1"], {})]),
    "mlp_small": ([ni((1, 96)), ni((96, 32)), ni((32, 8))],
                  [("matmul", ["i0", "i1"], {}), ("relu", ["n0"], {}), ("matmul", ["n1", "i2"], {})]),
}


def jsonable(obj):
    if isinstance(obj, dict):
        return {"__dict__": [[jsonable(k), jsonable(v)] for k, v in obj.items()]}
    if isinstance(obj, tuple):
        return {"__tuple__": [jsonable(v) for v in obj]}
    if isinstance(obj, list):
        return [jsonable(v) for v in obj]
    return obj


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/the/reference/source/tree")
    root = sys.argv[1]
    O, T = import_reference(root)
    arrays = {}
    meta = {}
    for name, (in_specs, nodes) in CASES.items():
        inputs32 = gen_inputs(in_specs)
        for dtype in ("float32", "float64"):
            tensors = [O.tensor() for _ in in_specs]
            with O.graph(name=name) as gb:
                vals = []
                for op, args, attrs in nodes:
                    ins = [tensors[int(a[1:])] if a[0] == "i" else vals[int(a[1:])] for a in args]
                    vals.append(getattr(O, op)(*ins, **attrs))
            graph = gb.graph
            ins = [T.Tensor(x.astype(dtype)) for x in inputs32]
            graph.forward_types([t.type for t in ins])
            outs = graph.forward(ins)
            assert len(outs) == 1
            arrays[f"{name}.{dtype}"] = outs[0].numpy()
        meta[name] = {
            "inputs": in_specs,
            "nodes": [{"op": op, "args": args, "attrs": jsonable(attrs)} for op, args, attrs in nodes],
            "out_shape": list(arrays[f"{name}.float32"].shape),
        }
        print(name, arrays[f"{name}.float32"].shape, arrays[f"{name}.float32"].dtype,
              arrays[f"{name}.float64"].dtype)
    np.savez_compressed(HERE / "reference_forward.npz", **arrays)
    (HERE / "reference_forward.json").write_text(json.dumps(meta, indent=1))


if __name__ == "__main__":
    main()
