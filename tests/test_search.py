"""The search strategy and the exploration driver (host logic on CPU; one small
exhaustive search on the GPU)."""

import csv

import pytest

from xtc_b200.backends.cuda import Backend
from xtc_b200.search import Exploration, ExplorationConfig, Strategies
from xtc_b200.search.explore import conv2d_graph, matmul_graph


def test_strategy_space_is_legal_and_maps_one_to_one():
    graph = matmul_graph(4096, 4096, 4096)
    strat = Strategies.create("cuda_gemm", graph)
    space = list(strat.exhaustive())
    assert len(space) == len({tuple(s) for s in space}) > 40
    assert strat.sample_names == ["tile_m", "tile_n", "tile_k", "stages", "tma_store", "split_k"]
    for s in space:
        assert strat.is_legal(s)
        sch = Backend(graph).get_scheduler(strict=True)  # strict: an illegal point would raise
        strat.generate(sch, s)
        cfg = sch.schedule().node_configs()["C"]
        assert (cfg["tile_m"], cfg["tile_n"], cfg["tile_k"]) == tuple(s[:3])
        assert cfg.get("stages", 0) == s[3] and cfg.get("epilogue", 0) == (2 if s[4] else 0)
        assert cfg.get("split_k", 1) == s[5]
    # the shared-memory filter: 128x256x64 leaves room for 2 stages, not for 3
    assert strat.is_legal([128, 256, 64, 2, 0, 1]) and not strat.is_legal([128, 256, 64, 3, 0, 1])
    assert not strat.is_legal([128, 96, 32, 0, 0, 1])
    # pieces of the reduction: one CTA per tile, at most 128 columns, K divisible
    assert strat.is_legal([128, 128, 64, 0, 1, 8]) and not strat.is_legal([256, 128, 64, 0, 1, 2])
    assert not strat.is_legal([128, 256, 32, 0, 1, 2]) and not strat.is_legal([128, 64, 32, 0, 0, 3])
    assert strat.sample(5, seed=1) == strat.sample(5, seed=1) and len(strat.sample(5, 1)) == 5
    for level in range(4):
        assert strat.is_legal(strat.default_schedule(level))


def test_o3_default_schedule_is_the_library_choice():
    """default_schedule(3) asks the kernel library what it would run for the product
    (xtc_cuda_gemm_default_config, host arithmetic) and returns it as a legal sample."""
    for dims in ((4096, 4096, 4096), (256, 3072, 8192), (1000, 1104, 1200)):
        st = Strategies.create("cuda_gemm", matmul_graph(*dims))
        sample = st.default_schedule(3)
        assert st.is_legal(sample)
        assert sample == (st.library_default() or [256, 256, 32, 0, 1, 1])
    assert Strategies.create("cuda_gemm", matmul_graph(4096, 4096, 4096)).default_schedule(3)[:3] == [256, 256, 64]


def test_strategy_targets_the_contraction_of_a_fused_graph():
    graph = matmul_graph(256, 256, 256, relu=True)
    strat = Strategies.create("cuda_gemm", graph)
    assert strat.node_name == "C"
    sch = Backend(graph).get_scheduler()
    strat.generate(sch, [128, 128, 64, 3, 1])  # a five-value sample of an older table still works
    assert sch.schedule().node_configs() == {
        "C": {"tile_m": 128, "tile_n": 128, "tile_k": 64, "stages": 3, "epilogue": 2}}
    sch = Backend(graph).get_scheduler(strict=True)
    strat.generate(sch, [128, 64, 64, 0, 1, 4])
    assert sch.schedule().node_configs()["C"]["split_k"] == 4
    assert "k_s3" in str(sch.schedule())
    conv = conv2d_graph(2, 8, 8, 64, 3, 3, 32, 1, 1)
    cs = Strategies.create("cuda_gemm", conv)
    assert {s[0] for s in cs.exhaustive()} == {128, 256}
    sch = Backend(conv).get_scheduler(strict=True)
    assert {s[5] for s in cs.exhaustive()} == {1}  # no split dimension for convolutions
    cs.generate(sch, [128, 64, 64, 0, 0, 1])
    assert sch.schedule().node_configs()["O"] == {"tile_m": 128, "tile_n": 64, "tile_k": 64}
    with pytest.raises(KeyError):
        Strategies.create("nope", graph)


def test_conv_strategy_covers_kernel_variant_slab_and_split():
    """cuda_conv enumerates which kernel runs a convolution as well as its parameters: the
    resident-weights kernel (one CTA or a CTA pair, 16- or 32-channel slabs) and the im2col
    kernels (tiles, epilogue, cluster split-K); every sample maps one to one."""
    from xtc_b200 import configs

    graph = configs.build("c3").graph
    strat = Strategies.create("cuda_conv", graph)
    assert strat.node_name == "conv"
    space = list(strat.exhaustive())
    assert len(space) == len({tuple(s) for s in space}) > 100
    assert {s[0] for s in space} == {1, 2, 3, 4, 5}
    assert [s for s in space if s[0] == 4] == [[4, 128, 64, 32, 0, 0, 1]]  # the sliding input window
    # streamed weights: two stages of a 32-channel halo slab + nine taps' weights fit, not three;
    # four of 16-channel slabs
    assert [s for s in space if s[0] == 5] == [[5, 256, 128, 32, 0, 0, 1], [5, 256, 128, 32, 2, 0, 1],
                                               [5, 256, 128, 16, 0, 0, 1], [5, 256, 128, 16, 2, 0, 1],
                                               [5, 256, 128, 16, 3, 0, 1], [5, 256, 128, 16, 4, 0, 1]]
    resident = [s for s in space if s[0] == 2]
    assert {(s[1], s[3]) for s in resident} == {(128, 16), (128, 32), (256, 32)}
    assert {(s[1], s[3]) for s in space if s[0] == 3} == {(128, 16), (128, 32)}  # two taps per MMA
    assert {s[6] for s in space if s[0] == 1} == set(range(1, 9))
    for s in space:
        assert strat.is_legal(s)
        sch = Backend(graph).get_scheduler(strict=True)
        strat.generate(sch, s)
        cfg = sch.schedule().node_configs()["conv"]
        assert cfg.get("variant", 0) == (s[0] if s[0] in (2, 3, 4, 5) else 0)
        if s[0] == 5:  # the kernel has one tile shape: the slab width and the depth are its parameters
            want = {"variant": 5}
            if s[4]:
                want["stages"] = s[4]
            if s[3] == 16:
                want["tile_k"] = 16
            assert cfg == want
            continue
        assert (cfg["tile_m"], cfg["tile_k"], cfg.get("stages", 0)) == (s[1], s[3], s[4])
        assert cfg.get("split_k", 1) == s[6] and cfg.get("epilogue", 0) == (2 if s[5] else 0)
        if s[0] == 1:
            assert cfg["tile_n"] == s[2]
    # two 32-channel halo stages fit next to the 147 KB filter bank of this layer, not three
    assert strat.is_legal([2, 128, 64, 32, 2, 0, 1]) and not strat.is_legal([2, 128, 64, 32, 3, 0, 1])
    assert strat.default_schedule(2) == [2, 128, 64, 32, 0, 0, 1]
    # a strided layer, or a bank too large to keep on chip, has only the im2col kernels
    strided = Strategies.create("cuda_conv", conv2d_graph(1, 28, 28, 128, 3, 3, 64, 2, 2))
    assert {s[0] for s in strided.exhaustive()} == {1} and strided.default_schedule(3)[0] == 1
    assert strided.streamed_stages() == 0
    big = Strategies.create("cuda_conv", conv2d_graph(1, 14, 14, 256, 3, 3, 256, 1, 1))
    assert {s[0] for s in big.exhaustive()} == {1, 5}  # im2col, or streamed weights beside halo tiles
    # one image is 2 work items: the library keeps it on the im2col kernels; 32 images are 64
    assert not big.library_streams() and big.default_schedule(3)[0] == 1
    batch = Strategies.create("cuda_conv", conv2d_graph(32, 14, 14, 256, 3, 3, 256, 1, 1))
    assert batch.library_streams() and batch.default_schedule(3) == [5, 256, 128, 32, 0, 0, 1]
    assert batch.default_schedule(2)[0] == 1
    deep = Strategies.create("cuda_conv", conv2d_graph(32, 7, 7, 512, 3, 3, 512, 1, 1))
    assert deep.streamed_stages() >= 2 and not deep.library_streams()  # 49 of 81 grid positions are outputs
    half = Strategies.create("cuda_conv", conv2d_graph(1, 28, 28, 128, 3, 3, 64, 1, 1))
    assert {(s[1], s[3]) for s in half.exhaustive() if s[0] == 2} >= {(256, 32)}
    # a halo run of more than 256 positions (112-wide rows) does not go through the ring
    wide = Strategies.create("cuda_conv", conv2d_graph(1, 112, 112, 32, 3, 3, 32, 1, 1))
    assert not wide.sliding_window_fits() and 4 not in {s[0] for s in wide.exhaustive()}
    with pytest.raises(ValueError):
        Strategies.create("cuda_conv", matmul_graph(128, 128, 128))


def test_named_operations_of_the_reference_tables():
    """--op-name serves the reference's benchmark layers (artifacts/operations.py,
    schedules/ttile/prob_sizes.py) under their names, dims then stride parameters."""
    from xtc_b200 import artifacts

    assert artifacts.operation_dims("conv2d", "ResNet18_02") == [1, 56, 56, 64, 3, 3, 64, 1, 1]
    assert artifacts.operation_dims("conv2d", "resnet18_01") == [1, 224, 224, 64, 7, 7, 3, 2, 2]
    assert artifacts.operation_dims("conv2d", "MobilNet_08") == [1, 14, 14, 512, 3, 3, 512, 2, 2]
    assert artifacts.operation_dims("conv2d", "Yolo9000_23") == [1, 17, 17, 28272, 1, 1, 1024, 1, 1]
    assert artifacts.operation_dims("matmul", "Gemma27B_FC") == [4608, 36864, 4608]
    assert artifacts.get_operation("conv2d", "AlexNet_00")["params"] == {"SH": 4, "SW": 4}
    names = dict.fromkeys(n for _, n in artifacts.list_operations("conv2d"))
    assert len(names) >= 49 and len(artifacts.list_operations("matmul")) >= 27
    exp = Exploration(ExplorationConfig(operator="conv2d", op_name="ResNet18_02", peak_flops=1e15))
    assert exp.fma_count() == 56 * 56 * 64 * 9 * 64 and exp.strategy.name == "cuda_conv"
    with pytest.raises(ValueError):
        artifacts.get_operation("conv2d", "ResNet18_99")


def test_exploration_csv_and_resume(tmp_path, monkeypatch):
    out = tmp_path / "res.csv"
    cfg = ExplorationConfig(operator="matmul", dims=[512, 512, 512], search="random", trials=6,
                            output=str(out), peak_flops=1e15, jobs=2,
                            explore_dir=str(tmp_path / "x"))
    calls = []

    def fake_eval(self, module, sample):
        calls.append(list(sample))
        return (sample, 0, 1e-6 * (1 + sample[1] / 64), "cuda")

    monkeypatch.setattr(Exploration, "evaluate_one", fake_eval)
    exp = Exploration(cfg)
    results = exp.run()
    assert len(results) == 6 and len(calls) == 6
    rows = list(csv.DictReader(open(out)))
    assert list(rows[0].keys()) == ["tile_m", "tile_n", "tile_k", "stages", "tma_store", "split_k", "X", "time",
                                    "peak", "backend"]
    assert len(rows) == 6 and all(r["backend"] == "cuda" for r in rows)
    best_sample, best_time = exp.best()
    assert best_time == min(float(r["time"]) for r in rows)
    # peak = (FMAs / peak rate) / time
    assert float(rows[0]["peak"]) == pytest.approx(512 ** 3 / 1e15 / float(rows[0]["time"]))
    # resume: nothing is evaluated twice, new samples are appended
    cfg2 = ExplorationConfig(**{**cfg.__dict__, "trials": 9, "resume": True})
    Exploration(cfg2).run()
    assert len(calls) == 9
    assert len(list(csv.DictReader(open(out)))) == 9


def test_graph_file_and_named_operations(tmp_path, monkeypatch, capsys):
    """``--graph-file`` explores a graph saved as YAML (the reference's
    tests/graphs/*.graph.yaml format); ``--op-name`` takes the dims of a registered
    operation; ``--op-name-list`` prints the registry."""
    from xtc_b200 import artifacts
    from xtc_b200.search import explore

    path = tmp_path / "mm_relu.graph.yaml"
    matmul_graph(384, 640, 256, relu=True).dump(path)
    exp = Exploration(ExplorationConfig(graph_file=str(path), peak_flops=1e15))
    assert [n.operation.name for n in exp.graph.nodes.values()] == ["matmul", "relu"]
    assert exp.fma_count() == 384 * 640 * 256
    assert exp.strategy._node.operation.name == "matmul"

    named = Exploration(ExplorationConfig(operator="conv2d", op_name="c3_conv", peak_flops=1e15))
    assert named.fma_count() == 32 * 56 * 56 * 64 * 3 * 3 * 64
    with pytest.raises(ValueError):
        Exploration(ExplorationConfig(operator="matmul", op_name="no_such_layer"))
    artifacts.register_operation("matmul", "tiny", {"i": 128, "j": 64, "k": 32})
    assert Exploration(ExplorationConfig(operator="matmul", op_name="Tiny", peak_flops=1e15)).fma_count() == 128 * 64 * 32

    assert explore.main(["--op-name-list"]) == 0
    listed = capsys.readouterr().out.split("\n")
    assert "conv2d c3_conv" in listed and "matmul_relu c2" in listed

    seen = []
    monkeypatch.setattr(Exploration, "evaluate_one",
                        lambda self, module, sample: (seen.append(sample) or (sample, 0, 1e-6, "cuda")))
    rc = explore.main(["--graph-file", str(path), "--opt-level", "2", "--peak-flops", "1e15",
                       "--output", str(tmp_path / "r.csv"), "--explore-dir", str(tmp_path / "x")])
    assert rc == 0 and len(seen) == 1


@pytest.mark.gpu
def test_exhaustive_search_on_gpu(tmp_path):
    out = tmp_path / "res.csv"
    cfg = ExplorationConfig(operator="matmul_relu", dims=[1024, 1024, 512], search="exhaustive",
                            output=str(out), validate=True, repeat=2, number=3, min_repeat_ms=1,
                            strategy_options={"tile_k": (32,), "stages": (0, 3)},
                            explore_dir=str(tmp_path / "x"))
    exp = Exploration(cfg)
    results = exp.run()
    assert results and all(code == 0 for _, code, _, _ in results)
    rows = list(csv.DictReader(open(out)))
    assert len(rows) == len(results)
    assert all(0 < float(r["peak"]) <= 1.5 for r in rows)
    assert exp.best() is not None


@pytest.mark.gpu
def test_conv_search_on_gpu_confirms_the_shipped_c3_schedule(tmp_path):
    """Every resident-weights sample of c3 (one tap or two per MMA, one CTA or a pair, 16- or
    32-channel slabs, every depth) and a draw of the im2col samples, measured: the schedule
    the benchmark configuration ships must be the best of them, or within 3 % of it."""
    from xtc_b200 import configs

    cfg = configs.build("c3")
    exp = Exploration(ExplorationConfig(graph=cfg.graph, strategy="cuda_conv", output=str(tmp_path / "c3.csv"),
                                        repeat=3, number=20, min_repeat_ms=5,
                                        explore_dir=str(tmp_path / "x")))
    space = list(exp.strategy.exhaustive())
    resident = [s for s in space if s[0] in (2, 3, 4)]
    im2col = [s for s in exp.strategy.sample(len(space), seed=3) if s[0] == 1][:16]
    shipped = [2, 128, 64, 32, 0, 0, 1]
    assert shipped in resident
    sch = Backend(cfg.graph).get_scheduler(default_node=cfg.contraction)
    cfg.schedule(sch)
    shipped_cfg = sch.schedule().node_configs()[cfg.contraction]
    ref = Backend(cfg.graph).get_scheduler(strict=True)
    exp.strategy.generate(ref, shipped)
    assert ref.schedule().node_configs()[cfg.contraction]["variant"] == shipped_cfg["variant"] == 2
    results = exp.evaluate_batch(resident + im2col, str(tmp_path / "x"), exp.result_callbacks())
    assert all(code == 0 for _, code, _, _ in results), [r for r in results if r[1]]
    times = {tuple(s): t for s, _, t, _ in results}
    best = min(times, key=times.get)
    assert times[tuple(shipped)] <= 1.03 * times[best], (best, times[best], times[tuple(shipped)])


@pytest.mark.gpu
@pytest.mark.parametrize("operator,name", [
    ("conv2d", "ResNet18_01"),    # 7x7 stride 2 on 3 channels: the packed thin-input form
    ("conv2d", "SqueezeNet_03"),  # 16 channels, resident weights
    ("conv2d", "MobilNet_09"),    # 7x7 pixels, K = 9216: split over clusters
    ("matmul", "Gemma2B_QK"),     # 256 rows, K = 8192: few tiles, long K
    ("matmul", "AlexNet_FC8"),    # one row
])
def test_named_layers_with_the_default_schedule_on_gpu(operator, name):
    """Layers of the reference's tables (artifacts/operations.py) compiled with nothing named
    and validated against the NumPy semantics of the graph."""
    exp = Exploration(ExplorationConfig(operator=operator, op_name=name, peak_flops=1e15))
    impl = Backend(exp.graph)
    module = impl.get_compiler(shared_lib=False).compile(impl.get_scheduler().schedule())
    results, code, msg = module.get_evaluator(validate=True, repeat=2, number=2, min_repeat_ms=0).evaluate()
    assert code == 0, msg
    assert all(t > 0 for t in results)


@pytest.mark.gpu
def test_iterative_search_and_database_on_gpu(tmp_path):
    from xtc_b200.search import read_db

    cfg = ExplorationConfig(operator="matmul", dims=[1024, 1024, 1024], search="iterative", trials=8,
                            batch=4, optimizer="random-forest-default", output=str(tmp_path / "it.csv"),
                            db_file=str(tmp_path / "db.jsonl"), repeat=2, number=3, min_repeat_ms=1,
                            validate=True, explore_dir=str(tmp_path / "x"))
    exp = Exploration(cfg)
    results = exp.run()
    assert len(results) == 8 and all(code == 0 for _, code, _, _ in results)
    recs = read_db(cfg.db_file, graph=exp.graph, backend="cuda")
    assert len(recs) == 8 and all(r["results"][0] == 0 and r["results"][1][0] > 0 for r in recs)
    assert "B200" in recs[0]["compiler"][2]
    # the table of this run drives a data search
    replay = Exploration(ExplorationConfig(**{**cfg.__dict__, "search": "data", "data": cfg.output,
                                              "output": str(tmp_path / "replay.csv"), "db_file": None}))
    assert [r[0] for r in replay.run()] == [r[0] for r in results]


def _fake_timer(monkeypatch, calls=None):
    """Replaces compile and execute by a cost model: time falls with the tile area."""
    def fake_eval(self, module, sample):
        if calls is not None:
            calls.append(list(sample))
        if sample[3] == 6:  # pretend the deepest pipeline fails to run
            return (list(sample), 7, float("inf"), "cuda")
        return (list(sample), 0, 1.0 / (sample[0] * sample[1] * (1 + sample[4])), "cuda")

    monkeypatch.setattr(Exploration, "compile_one", lambda self, ident, sample, d: None)
    monkeypatch.setattr(Exploration, "evaluate_one", fake_eval)


def test_callbacks_write_table_database_and_manifest(tmp_path, monkeypatch):
    import csv
    import json

    from xtc_b200.search import DBCallback, read_db
    from xtc_b200.search.explore import matmul_graph

    _fake_timer(monkeypatch)
    out = tmp_path / "t.csv"
    cfg = ExplorationConfig(operator="matmul", dims=[512, 512, 512], search="exhaustive", trials=0,
                            output=str(out), peak_flops=1e15)
    exp = Exploration(cfg)
    results = exp.run()
    space = list(exp.strategy.exhaustive())
    assert [r[0] for r in results] == space
    failed = [r for r in results if r[1] != 0]
    assert failed and all(r[0][3] == 6 for r in failed)
    rows = list(csv.DictReader(open(out)))
    assert len(rows) == len(space) - len(failed)  # failures stay out of the table
    assert list(rows[0])[-4:] == ["X", "time", "peak", "backend"]
    assert float(rows[0]["peak"]) == pytest.approx(exp.peak_time() / float(rows[0]["time"]))
    meta = json.load(open(f"{out}.meta.json"))
    assert meta["sampleNames"] == exp.strategy.sample_names and meta["args"]["search"] == "exhaustive"

    # append adds rows without a second header; a data search replays the table's X column
    cfg_data = ExplorationConfig(**{**cfg.__dict__, "search": "data", "data": str(out),
                                    "output": str(tmp_path / "replay.csv")})
    replay = Exploration(cfg_data)
    assert replay.samples() == [r[0] for r in results if r[1] == 0]
    cfg_app = ExplorationConfig(**{**cfg.__dict__, "append": True, "search": "random", "trials": 2})
    added = sum(r[1] == 0 for r in Exploration(cfg_app).run())
    lines = open(out).read().strip().splitlines()
    assert len(lines) == 1 + len(rows) + added and sum(l.startswith("tile_m") for l in lines) == 1

    # the results database: one JSON line per sample, failures with time 0, matched by graph digest
    graph = matmul_graph(512, 512, 512)
    db = DBCallback(str(tmp_path / "db.jsonl"), "NVIDIA B200", 1, "cuda_gemm")
    db.set_graph(graph)
    for r in results[:5] + failed[:1]:
        db(r)
    recs = read_db(str(tmp_path / "db.jsonl"), graph=matmul_graph(512, 512, 512, name="other_name"),
                   target="NVIDIA B200", backend="cuda")
    assert len(recs) == 6 and recs[-1]["results"] == [7, [0.0]]
    assert recs[0]["compiler"][:1] == ["xtc"] and recs[0]["compiler"][2:] == ["NVIDIA B200", 1, "cuda"]
    assert recs[0]["schedule"] == results[0][0] and recs[0]["operator"][0] == "xtc.graph"
    assert read_db(str(tmp_path / "db.jsonl"), graph=matmul_graph(512, 512, 256)) == []


@pytest.mark.parametrize("optimizer", ["random", "random-forest-default", "random-forest-aggressive"])
def test_iterative_search_with_optimizers(tmp_path, monkeypatch, optimizer):
    from xtc_b200.search import Optimizers

    calls: list[list[int]] = []
    _fake_timer(monkeypatch, calls)
    cfg = ExplorationConfig(operator="matmul", dims=[1024, 1024, 1024], search="iterative", trials=24,
                            batch=6, optimizer=optimizer, output=str(tmp_path / "it.csv"),
                            peak_flops=1e15, seed=3)
    exp = Exploration(cfg)
    results = exp.run()
    assert len(results) == 24 and len(calls) == 24
    assert len({tuple(c) for c in calls}) == 24  # nothing is measured twice while unseen samples remain
    assert all(exp.strategy.is_legal(c) for c in calls)
    best = exp.best()
    assert best is not None
    if optimizer != "random":  # the surrogate finds the widest tile with the TMA epilogue
        assert best[0][0] * best[0][1] == 256 * 256 and best[0][4] == 1
    with pytest.raises(ValueError):
        Optimizers.create("no-such-optimizer", exp.strategy.sample, 4, 0)


def test_optimizer_refit_schedule_and_config_file(tmp_path):
    from xtc_b200.search import Optimizers
    from xtc_b200.search.explore import matmul_graph

    strategy = Strategies.create("cuda_gemm", matmul_graph(512, 512, 512))
    cfgfile = tmp_path / "opt.yaml"
    cfgfile.write_text("n_estimators: 10\nupdate_first: 8\nupdate_period: 4\nbeta: 1.0\n")
    opt = Optimizers.create("random-forest-explore", strategy.sample, 4, 0, str(cfgfile))
    assert opt.forest.n_estimators == 10 and opt.beta0 == 1.0 and opt.alpha == 0.6
    for step in range(4):
        batch = opt.suggest()
        assert len(batch) == 4
        opt.observe(batch, [s[0] * s[1] / 65536 for s in batch])
        assert opt.fitted_on == (0 if step == 0 else 8 + (4 * (step + 1) - 8) // 4 * 4)
    assert opt.beta() == pytest.approx(max(0.05, 1.0 / 16 ** 0.6))
    assert opt.best_y == max(opt.y)
