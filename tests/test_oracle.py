"""The oracle (oracle/xtc_oracle.py, oracle/cpu_loopnest.c) against the
reference: golden vectors produced by the reference's graph.forward, and the
known-answer lines of the reference's own graph tests."""

import numpy as np
import pytest

from conftest import GOLDEN_NAMES
from oracle import xtc_oracle as xo


def run_case(golden, name, dtype):
    ins = [x.astype(dtype) for x in golden.inputs(name)]
    env = {f"i{k}": x for k, x in enumerate(ins)}
    nodes = [{"uid": f"n{k}", "op": n["op"], "args": n["args"], "attrs": n["attrs"]}
             for k, n in enumerate(golden.nodes(name))]
    return xo.run_graph(nodes, env, [nodes[-1]["uid"]])[0]


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_matches_reference_float64(golden, name):
    got = run_case(golden, name, "float64")
    ref = golden.output(name, "float64")
    assert got.shape == ref.shape and got.dtype == np.float64
    # same arithmetic up to summation order (conv is vectorised here)
    np.testing.assert_allclose(got, ref, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_matches_reference_float32(golden, name):
    got = run_case(golden, name, "float32")
    ref = golden.output(name, "float32")
    assert got.shape == ref.shape and got.dtype == np.float32
    is_movement = all(n["op"] in ("pad", "pad2d", "unpad", "reshape", "transpose", "relu")
                      for n in golden.nodes(name))
    if is_movement:
        assert np.array_equal(got, ref)  # data movement is bit-exact
    else:
        assert xo.rel_err(got, golden.output(name, "float64")) <= 1e-5
        np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4 * np.abs(ref).max())


def _summary(arr):
    flat = arr.reshape(-1)
    return (" ".join(f"{d:.4g}" for d in flat[:4]) + "..." + " ".join(f"{d:.4g}" for d in flat[-4:]))


def test_known_answers_of_reference_graph_tests(golden):
    # tests/filecheck/graphs/test_matmul_relu.py:57 and test_conv_relu.py:60 print
    # the first and last four output values of graph.forward on np_init(...)-5.
    assert _summary(run_case(golden, "ref_matmul_relu", "float32")) == "8 17 8 0...8 0 0 0"
    assert _summary(run_case(golden, "ref_conv_relu", "float32")) == "18 18 18 18...5 113 0.1 5"


def test_known_answer_mlp4():
    # tests/filecheck/graphs/test_mlp.py: 1x3072 image through 3 relu(fc) + 1 fc,
    # np_init(...)-5 inputs; printed output 3.564e+10 5.293e+10 1.027e+10 -2.691e+10...
    # -1.625e+10 1.047e+09 1.834e+10 3.564e+10
    shapes = [(1, 3072), (3072, 512), (512, 256), (256, 128), (128, 10)]
    img, w1, w2, w3, w4 = [xo.np_init(s) - 5 for s in shapes]
    h = xo.relu(xo.matmul(img, w1))
    h = xo.relu(xo.matmul(h, w2))
    h = xo.relu(xo.matmul(h, w3))
    out = xo.matmul(h, w4)
    assert out.shape == (1, 10) and out.dtype == np.float32
    assert _summary(out) == ("3.564e+10 5.293e+10 1.027e+10 -2.691e+10..."
                             "-1.625e+10 1.047e+09 1.834e+10 3.564e+10")


def test_np_init_pattern():
    a = xo.np_init((2, 6))
    assert a.dtype == np.float32
    assert a.reshape(-1).tolist() == [1, 2, 3, 4, 5, 6, 7, 8, 9, 1, 2, 3]


@pytest.mark.parametrize("stride", [(1, 1), (2, 2), (1, 2)])
def test_vectorised_conv_equals_reference_loop(stride):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((2, 9, 8, 5))
    w = rng.standard_normal((3, 2, 5, 4))
    np.testing.assert_allclose(xo.conv2d(x, w, stride), xo.conv2d_loop(x, w, stride), rtol=1e-12, atol=1e-12)


def test_config_generators_are_seeded_and_shaped():
    a, b = xo.config_inputs("c1")
    assert a.shape == (512, 1024) and b.shape == (1024, 256) and a.dtype == np.float32
    a2, _ = xo.config_inputs("c1")
    assert np.array_equal(a, a2)
    x, w = xo.config_inputs("c3", scale=16)
    assert x.shape == (2, 56, 56, 64) and w.shape == (3, 3, 64, 64)
    assert 0.0 <= x.min() and x.max() < 1.0
    assert abs(float(w.std()) - np.sqrt(2 / 576)) < 2e-3


def test_cpu_loopnest_matches_oracle():
    """The C loop nests (the timed CPU baseline) agree with the NumPy oracle."""
    from oracle import cpu_baseline as cb

    for name, scale in [("c1", 4), ("c2", 32), ("c3", 32), ("c4", 64), ("c4a", 64), ("c5", 128)]:
        ins = xo.config_inputs(name, scale)
        y64 = xo.config_forward(name, [x.astype(np.float64) for x in ins])
        got = cb.run_config(name, ins)
        assert got.shape == y64.shape
        assert xo.rel_err(got, y64) <= 1e-5, name
    x = np.random.default_rng(1).standard_normal((3, 5, 6, 4)).astype(np.float32)
    assert np.array_equal(cb.pad_hw(x, 1, 2, 0, 3, 1.5),
                          np.pad(x, ((0, 0), (1, 2), (0, 3), (0, 0)), constant_values=1.5))
    m = np.random.default_rng(2).standard_normal((70, 33)).astype(np.float32)
    assert np.array_equal(cb.transpose2d(m), m.T)


def test_register_blocked_nests_match_oracle():
    """The tuned CPU nests (two-level tiling, packed operands, register tile) on ragged
    shapes and every micro-kernel: same results as the NumPy oracle."""
    from oracle import cpu_baseline as cb

    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (77, 130)).astype(np.float32)
    b = rng.uniform(-1, 1, (130, 101)).astype(np.float32)
    y64 = a.astype(np.float64) @ b.astype(np.float64)
    for micro in range(len(cb.micro_shapes())):
        for mc, nc, kc in ((48, 128, 64), (96, 512, 512)):
            assert xo.rel_err(cb.matmul_blocked(a, b, (mc, nc, kc, micro)), y64) <= 1e-5, (micro, mc)
    assert xo.rel_err(cb.matmul_blocked(a, b, (48, 128, 64, 0), relu=True), np.maximum(y64, 0)) <= 1e-5
    with pytest.raises(ValueError):
        cb.matmul_blocked(a, b, (48, 128, 64, 99))
    for (c, f), stride in (((8, 64), (1, 1)), ((3, 20), (2, 1)), ((16, 33), (2, 2))):
        x = rng.uniform(0, 1, (2, 11, 13, c)).astype(np.float32)
        w = rng.normal(0, 0.1, (3, 3, c, f)).astype(np.float32)
        ref = xo.conv2d(x.astype(np.float64), w.astype(np.float64), stride)
        for micro in range(len(cb.conv_micro_shapes())):
            assert xo.rel_err(cb.conv2d_blocked(x, w, stride, micro), ref) <= 1e-5, (c, f, micro)
            assert xo.rel_err(cb.conv2d_blocked(x, w, stride, micro, relu=True), np.maximum(ref, 0)) <= 1e-5
    assert cb.peak_fma() > 1e9


def test_cpu_nests_are_tuned_through_the_exploration_driver(tmp_path):
    """loop-explore over the CPU backend: the strategy's samples become tile / interchange /
    parallelize / vectorize / unroll calls, an inner tile without a micro-kernel is refused,
    and the best sample reproduces the oracle."""
    from oracle import cpu_backend as cpb
    from oracle import cpu_baseline as cb
    from xtc_b200 import configs
    from xtc_b200.backends.cuda.scheduler import ScheduleError

    for name, scale in (("c2", 16), ("c3", 16)):
        cfg = configs.build(name, scale)
        ins = configs.inputs(name, scale)
        out = tmp_path / f"{name}.csv"
        best, seconds, n = cpb.tune(cfg.graph, trials=5, inputs=ins, output=str(out))
        assert n >= 3 and seconds > 0
        rows = out.read_text().splitlines()
        assert rows[0].split(",")[-4:] == ["X", "time", "peak", "backend"] and "cpu_loopnest" in rows[1]
        y64 = xo.config_forward(name, [x.astype(np.float64) for x in ins])
        assert xo.rel_err(cb.run_config(name, ins, best), y64) <= 1e-5
    cfg = configs.build("c2", 16)
    sch = cpb.Backend(cfg.graph).get_scheduler(strict=True)
    cpb.StrategyCpuTile(cfg.graph).generate(sch, [128, 512, 256, 6])
    text = str(sch.schedule())
    assert "./i2" in text and "./j2" in text
    assert sch.schedule().node_configs()["mm"] == {"mc": 128, "nc": 512, "kc": 256, "micro": 6}
    bad = cpb.Backend(cfg.graph).get_scheduler(strict=True)
    bad.tile("i", {"i1": 64, "i2": 5})
    bad.tile("j", {"j1": 64, "j2": 7})
    bad.tile("k", {"k1": 32})
    bad.vectorize(["j2"])
    with pytest.raises(ScheduleError):
        bad.schedule()
    # validate=True on the CPU evaluator compares with the float64 oracle
    module = cpb.Backend(cfg.graph).get_compiler().compile(sch.schedule())
    assert module.get_evaluator(validate=True, min_repeat_ms=0).evaluate()[1] == 0
