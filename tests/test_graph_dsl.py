"""The graph DSL (xtc_b200.graphs.xtc) against the reference's golden outputs
and printed forms (tests/filecheck/graphs/*.py of the reference)."""

import numpy as np
import pytest

import xtc_b200.graphs.xtc.op as O
import xtc_b200.graphs.xtc.ty as T
from conftest import GOLDEN_NAMES, build_dsl_graph
from xtc_b200.graphs.xtc.core import graph_builder
from xtc_b200.utils.numpy import np_init


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_forward_matches_reference(golden, name):
    ins = golden.inputs(name)
    graph = build_dsl_graph(O, name, [x.shape for x in ins], golden.nodes(name))
    for dtype, tol in (("float32", 1e-5), ("float64", 1e-12)):
        outs = graph.forward([T.Tensor(x.astype(dtype)) for x in ins])
        ref = golden.output(name, dtype)
        got = outs[0].numpy()
        assert got.shape == ref.shape and str(got.dtype) == dtype
        scale = max(float(np.abs(ref).max()), 1.0)
        assert float(np.abs(got - ref).max()) <= tol * scale
    assert list(graph.outputs_types[0].shape) == golden.meta[name]["out_shape"]


def test_printed_graph_matmul_relu():
    # expected text: tests/filecheck/graphs/test_matmul_relu.py:33-57 of the reference
    x, y = O.tensor(), O.tensor()
    with O.graph(name="matmul_relu") as gb:
        z = O.matmul(x, y)
        O.relu(z)
    g = gb.graph
    u = [int(v[1:]) for v in g.inputs]
    assert str(g) == (f"graph:\n  name: matmul_relu\n  inputs:\n  - %{u[0]}\n  - %{u[1]}\n  outputs:\n"
                      f"  - %{u[1] + 2}\n  nodes:\n  - %{u[1] + 1}: matmul(%{u[0]}, %{u[1]})\n"
                      f"  - %{u[1] + 2}: relu(%{u[1] + 1})\n")
    out_types = g.forward_types([T.TensorType((5, 3), "float32"), T.TensorType((3, 4), "float32")])
    assert str(out_types) == "[5x4xfloat32]"
    assert (f"  - %{u[1] + 1}: matmul(%{u[0]}, %{u[1]}) : [5x3xfloat32, 3x4xfloat32] -> [5x4xfloat32]"
            in str(g))
    inps = [T.Tensor(np_init(t, "float32") - 5) for t in [(5, 3), (3, 4)]]
    assert str(inps[0]) == "Tensor(type=5x3xfloat32, data=-4 -3 -2 -1...-2 -1 0 1)"
    assert str(g.forward(inps)) == "[Tensor(type=5x4xfloat32, data=8 17 8 0...8 0 0 0)]"


def test_printed_graph_conv_relu():
    # expected text: tests/filecheck/graphs/test_conv_relu.py:35-60 of the reference
    i, k = O.tensor(), O.tensor()
    with O.graph(name="conv_relu") as gb:
        p = O.pad2d(i, padding=2, axes=(1, 2))
        t = O.transpose(k, axes=(1, 2, 3, 0))
        c = O.conv2d(p, t, stride=(2, 2))
        O.relu(c, threshold=0.1)
    g = gb.graph
    text = str(g)
    assert "pad2d(%" in text and ", padding={1: (2, 2), 2: (2, 2)}, constant_value=0)" in text
    assert ", axes=(1, 2, 3, 0))" in text and ", stride=(2, 2))" in text and ", threshold=0.1)" in text
    g.forward_types([T.TensorType((2, 6, 6, 3), "float32"), T.TensorType((8, 5, 5, 3), "float32")])
    assert "[2x6x6x3xfloat32] -> [2x10x10x3xfloat32]" in str(g)
    assert "[2x10x10x3xfloat32, 5x5x3x8xfloat32] -> [2x3x3x8xfloat32]" in str(g)
    inps = [T.Tensor(np_init(s, "float32") - 5) for s in [(2, 6, 6, 3), (8, 5, 5, 3)]]
    assert str(g.forward(inps)) == "[Tensor(type=2x3x3x8xfloat32, data=18 18 18 18...5 113 0.1 5)]"


def test_nested_graph_scopes_and_input_order():
    # tests/filecheck/graphs/test_mlp.py: sub-graphs share expressions with the parent
    img = O.tensor(shape=(1, 12), dtype="float32")
    w1 = O.tensor(shape=(12, 8), dtype="float32")
    w2 = O.tensor(shape=(8, 4), dtype="float32")
    with O.graph(name="mlp2") as gb:
        with O.graph(name="l1") as g1:
            l1 = O.relu(O.matmul(img, w1))
        with O.graph(name="l2") as g2:
            O.matmul(l1, w2)
    g = gb.graph
    assert len(g.nodes) == 3 and len(g.inputs) == 3 and len(g.outputs) == 1
    assert [n.operation.name for n in g.nodes.values()] == ["matmul", "relu", "matmul"]
    assert str(g.outputs_types) == "[1x4xfloat32]"
    assert len(g1.graph.nodes) == 2 and len(g2.graph.nodes) == 1
    assert g1.graph.outputs[0] in g2.graph.inputs


def test_operation_records():
    a = O.tensor((6, 2, 5), "float32", name="A")
    b = O.tensor((10, 7), "float32", name="B")
    with O.graph(name="g") as gb:
        m = O.matmul(a, b, name="mm")
        O.relu(m, name="act")
    g = gb.graph
    mm, act = g.nodes.values()
    op = mm.operation
    assert (mm.name, op.name, dict(op.dims)) == ("mm", "matmul", {"i": 6, "j": 7, "k": 10})
    assert op.dims_kind("P") == ["i", "j"] and op.dims_kind("R") == ["k"]
    assert op.accesses_maps == (("i", "j", "k"), (("i", "k"), ("k", "j")), (("i", "j"),))
    assert op.ops_count == 6 * 7 * 10 and op.ops_dtype == "float32"
    assert dict(act.operation.dims) == {"i": 42}
    assert g.ops_count() == 420 + 42  # the reference also counts elementwise nodes (graph.py:189-200)
    assert "{name = 'mm'}" in str(mm)


def test_conv_operation_dims():
    x = O.tensor((32, 58, 58, 64), "float32")
    w = O.tensor((3, 3, 64, 64), "float32")
    with O.graph(name="c") as gb:
        O.conv2d(x, w, stride=(1, 1))
    op = list(gb.graph.nodes.values())[0].operation
    assert dict(op.dims) == {"b": 32, "h": 56, "w": 56, "f": 64, "r": 3, "s": 3, "c": 64}
    assert op.ops_count * 2 == 7398752256


def test_yaml_round_trip():
    a = O.tensor((4, 6, 6, 3), "float32")
    w = O.tensor((3, 3, 3, 8), "float32")
    with O.graph(name="rt") as gb:
        p = O.pad(a, padding={1: (1, 1), 2: (1, 1)}, constant_value=0.0)
        c = O.conv2d(p, w, stride=(1, 1), name="conv")
        O.relu(c, threshold=0.5)
    g = gb.graph
    text = g.dumps()
    with O.graph() as gb2:
        graph_builder.loads(text)
    g2 = gb2.graph
    assert g2.name == "rt"
    assert [n.operation.name for n in g2.nodes.values()] == ["pad", "conv2d", "relu"]
    assert [n.name for n in g2.nodes.values()][1] == "conv"
    ins = [T.Tensor(np_init(t.constant_shape, "float32")) for t in g.inputs_types]
    assert np.array_equal(g.forward(ins)[0].numpy(), g2.forward(ins)[0].numpy())
    assert g2.to_dict()["nodes"] == g.to_dict()["nodes"]


def test_shape_errors_are_assertions():
    a = O.tensor((4, 5), "float32")
    b = O.tensor((6, 3), "float32")
    with pytest.raises(AssertionError, match="incompatible dimension k"):
        with O.graph(name="bad"):
            O.matmul(a, b)
    with pytest.raises(AssertionError):
        O.pad(a, padding="x")
