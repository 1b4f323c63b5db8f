"""Host-side logic of the CUDA backend that needs no GPU: schedule recording
and mapping, graph lowering and fusion decisions, the payload library, the
C-ABI library's exported symbols and its error behaviour without a device."""

import ctypes
import re
import threading
from pathlib import Path

import pytest

import xtc_b200.graphs.xtc.op as O
from conftest import ROOT, build_dsl_graph, has_cuda
from xtc_b200 import capi
from xtc_b200.backends.cuda import Backend, ScheduleError
from xtc_b200.backends.cuda.compiler import payload_source
from xtc_b200.backends.cuda.lowering import LoweringError


def matmul_impl(i, j, k, name="matmul"):
    a = O.tensor((i, k), "float32", name="A")
    b = O.tensor((k, j), "float32", name="B")
    with O.graph(name=name) as gb:
        O.matmul(a, b, name="C")
    return Backend(gb.graph)


# The four schedules and the expected substrings of str(schedule) are those of the
# reference's backend API tests (tests/pytest/mlir/test_mlir_impl.py:9-67).
def sched_nop(sch):
    return ["permutation={'.': ['./i', './j', './k']}"]


def sched_tile2(sch):
    sch.tile("i", {"i1": 64, "i2": 4})
    sch.tile("j", {"j1": 64, "j2": 64})
    sch.tile("k", {"k1": 13})
    return ["permutation={'.': ['./i', './j', './k', './i1', './j1', './k1', './i2', './j2']}",
            "'j': {'./j1': 64, './j2': 64}"]


def sched_tile2p(sch):
    sch.tile("i", {"i1": 64, "i2": 4})
    sch.tile("j", {"j1": 64, "j2": 64})
    sch.tile("k", {"k1": 13})
    sch.interchange(["i", "i1", "j", "k", "j1", "k1", "i2", "j2"])
    sch.parallelize(["i", "i1"])
    sch.unroll({"j2": 64, "k1": 13, "i2": 4})
    sch.vectorize(["j2"])
    return ["permutation={'.': ['./i', './i1', './j', './k', './j1', './k1', './i2', './j2']}",
            "unrolling={'./j2': 64, './k1': 13, './i2': 4}", "vectorization=['./j2']",
            "parallelization=['./i', './i1']"]


def sched_tile3wc(sch):
    sch.tile("i", {"i1": 64, "i2": 32, "i3": 4})
    sch.tile("j", {"j1": 256, "j2": 64, "j3": 64})
    sch.tile("k", {"k1": 13})
    sch.interchange(["i", "j", "i1", "j1", "k", "i2", "j2", "k1", "i3", "j3"])
    sch.parallelize(["i", "j"])
    sch.unroll({"k1": 13, "i3": 4, "j3": 64})
    sch.vectorize(["j3"])
    sch.buffer_at("j")
    sch.buffer_at("j1")
    return ["permutation={'.': ['./i', './j', './i1', './j1', './k', './i2', './j2', './k1', './i3', './j3']",
            "vectorization=['./j3']", "parallelization=['./i', './j']",
            "unrolling={'./k1': 13, './i3': 4, './j3': 64}"]


SCHEDULES = [sched_nop, sched_tile2, sched_tile2p, sched_tile3wc]


@pytest.mark.parametrize("sched", SCHEDULES, ids=lambda f: f.__name__)
def test_schedule_text(sched):
    impl = matmul_impl(128, 256, 91)
    sch = impl.get_scheduler()
    expected = sched(sch)
    text = str(sch.schedule())
    for sub in expected:
        assert sub in text


def test_schedule_maps_to_kernel_parameters():
    impl = matmul_impl(4096, 4096, 4096)
    sch = impl.get_scheduler()
    sch.tile("i", {"i1": 128})
    sch.tile("j", {"j1": 256, "j2": 32})
    sch.tile("k", {"k1": 64})
    sch.unroll({"k1": 3})
    sch.vectorize(["j2"])
    sch.parallelize(["i", "j"])
    cfg = sch.schedule().node_configs()["C"]
    assert cfg == {"tile_m": 128, "tile_n": 256, "tile_k": 64, "stages": 3, "epilogue": 2}
    plan = impl.get_compiler(shared_lib=False).lower(sch.schedule())
    assert plan.steps[0].config["tile_n"] == 256 and plan.steps[0].config["precision"] == 0


def test_illegal_tiles_snap_or_raise():
    impl = matmul_impl(128, 256, 91)
    sch = impl.get_scheduler()
    sched_tile2(sch)
    cfg = sch.schedule().node_configs()["C"]
    assert cfg["tile_m"] == 128 and cfg["tile_n"] == 64 and cfg["tile_k"] == 32
    strict = impl.get_scheduler(strict=True)
    sched_tile2(strict)
    with pytest.raises(ScheduleError):
        strict.schedule()


def test_precision_modes_snap_the_benchmark_schedules():
    """The 3xTF32 and fp32 modes cannot use every TF32 tile: CTA-pair rows, 256 columns and
    (at 128 columns) 64 of K per stage are snapped to what the single-CTA 3xTF32 kernel runs."""
    from xtc_b200 import capi, configs

    for name in ("c2", "c4", "c5"):
        cfg = configs.build(name, 8)
        step = configs.compile_config(cfg, precision="3xtf32").plan.steps[-1]
        assert step.config["precision"] == capi.PRECISION_3XTF32
        assert step.config["tile_m"] == 128 and step.config["tile_n"] == 128
        assert step.config["tile_k"] == 32
        tf32 = configs.compile_config(cfg).plan.steps[-1].config
        assert tf32["tile_m"] == 256 and tf32["tile_n"] == 256
    c1 = configs.compile_config(configs.build("c1"), precision="3xtf32").plan.steps[-1].config
    assert (c1["tile_n"], c1["tile_k"]) == (64, 64)  # two stages of it do fit
    # convolutions have no operand-split mode: a 3xTF32 graph runs them in fp32 FMA
    c3 = configs.compile_config(configs.build("c3", 8), precision="3xtf32").plan.steps[-1]
    assert c3.kind == "conv2d" and c3.config["precision"] == capi.PRECISION_FP32_SIMT


def test_default_node_is_the_contraction():
    a = O.tensor((64, 64), "float32")
    b = O.tensor((64, 64), "float32")
    with O.graph(name="mr") as gb:
        O.relu(O.matmul(a, b, name="mm"), name="act")
    impl = Backend(gb.graph)
    sch = impl.get_scheduler()
    sch.tile("j", {"j1": 64})  # would fail on the relu node: it has no j
    assert sch.schedule().node_configs() == {"mm": {"tile_n": 64}}
    relu_sch = impl.get_scheduler(default_node="act")
    with pytest.raises(AssertionError):
        relu_sch.tile("j", {"j1": 64})
    assert "loop i" in sch.get_loop_nest().pretty_print()


def test_lowering_fuses_relu_pad_and_optional_transpose():
    x = O.tensor((2, 8, 8, 32), "float32")
    w = O.tensor((3, 3, 32, 64), "float32")
    with O.graph(name="c3ish") as gb:
        p = O.pad(x, padding={1: (1, 1), 2: (1, 1)}, constant_value=0.0, name="pad")
        c = O.conv2d(p, w, stride=(1, 1), name="conv")
        O.relu(c, name="relu")
    plan = Backend(gb.graph).get_compiler(shared_lib=False).lower(None)
    assert [s.kind for s in plan.steps] == ["conv2d"]
    s = plan.steps[0]
    assert set(s.fused) == {"pad", "relu"} and s.flags == capi.FUSE_RELU
    assert s.dims == (2, 8, 8, 32, 3, 3) and s.aux0 == (64, 1, 1) and s.aux1 == (1, 1, 1, 1)
    assert len(plan.slot_bytes) == 3  # no intermediate buffer at all

    # a non-zero pad constant cannot be folded into the operand fetch
    with O.graph(name="padval") as gb:
        p = O.pad(x, padding={1: (1, 1), 2: (1, 1)}, constant_value=1.0)
        O.conv2d(p, w)
    plan = Backend(gb.graph).get_compiler(shared_lib=False).lower(None)
    assert [s.kind for s in plan.steps] == ["pad", "conv2d"]

    xt = O.tensor((96, 64), "float32")
    w2 = O.tensor((96, 32), "float32")
    with O.graph(name="c4ish") as gb:
        t = O.transpose(xt, axes=(1, 0), name="xt")
        O.matmul(t, w2, name="mm")
    impl = Backend(gb.graph)
    plan = impl.get_compiler(shared_lib=False).lower(None)
    assert [s.kind for s in plan.steps] == ["transpose", "gemm"]
    sch = impl.get_scheduler()
    sch.fuse_producer_at("i", 0)
    plan = impl.get_compiler(shared_lib=False).lower(sch.schedule())
    assert [s.kind for s in plan.steps] == ["gemm"]
    assert plan.steps[0].flags == capi.GEMM_A_TRANSPOSED
    assert plan.steps[0].dims == (64, 32, 96, 64, 32, 32)


def test_lowering_keeps_a_relu_whose_input_is_also_an_output():
    a = O.tensor((8, 8), "float32")
    b = O.tensor((8, 8), "float32")
    with O.graph(name="two_out") as gb:
        m = O.matmul(a, b)
        r = O.relu(m)
        O.outputs(m, r)
    plan = Backend(gb.graph).get_compiler(shared_lib=False).lower(None)
    assert [s.kind for s in plan.steps] == ["gemm", "relu"] and plan.n_outputs == 2


def test_lowering_rejects_other_dtypes():
    a = O.tensor((8, 8), "float64")
    b = O.tensor((8, 8), "float64")
    with O.graph(name="f64") as gb:
        O.matmul(a, b)
    with pytest.raises(LoweringError):
        Backend(gb.graph).get_compiler(shared_lib=False).lower(None)


@pytest.mark.parametrize("name", ["ref_conv_relu", "pad_dict", "unpad_dict", "reshape", "mlp_small"])
def test_every_golden_graph_lowers(golden, name):
    ins = golden.inputs(name)
    graph = build_dsl_graph(O, name, [x.shape for x in ins], golden.nodes(name))
    plan = Backend(graph).get_compiler(shared_lib=False).lower(None)
    assert plan.n_inputs == len(ins) and plan.steps
    for s in plan.steps:
        s.to_c()  # fits the fixed-size C record


def test_payload_library_builds_and_exports_the_graph_symbol(tmp_path, cuda_lib):
    impl = matmul_impl(128, 256, 64, name="payload_fn")
    module = impl.get_compiler(dump_file=str(tmp_path / "payload_x"), shared_lib=True).compile(
        impl.get_scheduler().schedule())
    assert module.file_type == "shlib" and module.payload_name == "payload_fn"
    assert Path(module.file_name).exists()
    lib = ctypes.CDLL(module.file_name)
    assert hasattr(lib, "payload_fn")
    Path(module.file_name).unlink()  # the reference's search driver deletes it after use
    assert "xtc_cuda_plan_run_host" in payload_source(module.plan)


def test_compile_is_thread_safe(tmp_path, cuda_lib):
    impl = matmul_impl(256, 256, 256, name="mt")
    errors = []

    def work(i):
        try:
            sch = impl.get_scheduler()
            sch.tile("j", {"j1": [64, 128, 256][i % 3]})
            m = impl.get_compiler(dump_file=str(tmp_path / f"p{i}"), shared_lib=True).compile(sch.schedule())
            assert m.plan.steps[0].config["tile_n"] == [64, 128, 256][i % 3]
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(6)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors


def test_library_exports_every_declared_symbol(cuda_lib):
    header = (ROOT / "include" / "xtc_cuda.h").read_text()
    declared = set(re.findall(r"\b(xtc_cuda_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    assert declared == set(capi.SIGNATURES), declared ^ set(capi.SIGNATURES)
    for name in declared:
        assert hasattr(cuda_lib, name), name
    assert cuda_lib.xtc_cuda_abi_version() == 1


def test_plan_clears_every_split_k_counter(cuda_lib):
    """A split-K step keeps one int per output tile at the start of its workspace.  With
    more than 16384 tiles those counters pass 64 KiB: the bytes a plan clears must cover
    all of them (needs no device: the sizes are host arithmetic)."""
    from xtc_b200.backends.cuda.lowering import StepDesc

    m, n, k = 128 * 130, 64 * 128, 96  # 130 x 128 = 16640 tiles of 128 x 64
    step = StepDesc("gemm", "mm", 0, 1, 2, dims=(m, n, k, k, n, n),
                    config={"tile_m": 128, "tile_n": 64, "tile_k": 32, "split_k": 3, "variant": 1}).to_c()
    total, zeroed = ctypes.c_size_t(0), ctypes.c_size_t(0)
    capi.check(cuda_lib.xtc_cuda_step_workspace_bytes(ctypes.byref(step), ctypes.byref(total),
                                                      ctypes.byref(zeroed)))
    tiles = (m // 128) * (n // 64)
    counters = (tiles * 4 + 255) // 256 * 256
    assert counters > 65536
    assert total.value == counters + 3 * tiles * 128 * 64 * 4
    assert zeroed.value >= counters
    # the 3xTF32 operand split is rewritten by every run: nothing to clear
    step.cfg.precision = capi.PRECISION_3XTF32
    capi.check(cuda_lib.xtc_cuda_step_workspace_bytes(ctypes.byref(step), ctypes.byref(total),
                                                      ctypes.byref(zeroed)))
    assert total.value > 0 and zeroed.value == 0


def test_row_exchange_entry_points_check_their_arguments(cuda_lib):
    """xtc_cuda_comm_* / xtc_cuda_allgather_rows refuse bad arguments before NCCL is loaded
    or a device is touched."""
    handle = ctypes.c_void_p()
    ident = ctypes.create_string_buffer(128)
    assert cuda_lib.xtc_cuda_comm_unique_id(None) == capi.ERR_INVALID
    assert cuda_lib.xtc_cuda_comm_init(None, 2, 0, ident) == capi.ERR_INVALID
    assert cuda_lib.xtc_cuda_comm_init(ctypes.byref(handle), 2, 2, ident) == capi.ERR_INVALID
    assert "rank 2 of 2" in capi.last_error() and not handle.value
    assert cuda_lib.xtc_cuda_comm_init(ctypes.byref(handle), 2, 0, None) == capi.ERR_INVALID
    assert cuda_lib.xtc_cuda_allgather_rows(None, 1, 4, 16, 0, 4, None) == capi.ERR_INVALID
    assert "NULL communicator" in capi.last_error()
    assert cuda_lib.xtc_cuda_comm_destroy(None) == capi.OK
    # the one-warp barrier: no peers is a no-op, more than 7 or a rank outside [0, 8) is refused
    flags = (ctypes.c_void_p * 8)()
    ranks = (ctypes.c_int * 8)(*range(1, 9))
    assert cuda_lib.xtc_cuda_peer_barrier(None, flags, ranks, 0, 0, 1, None) == capi.OK
    assert cuda_lib.xtc_cuda_peer_barrier(None, flags, ranks, 8, 0, 1, None) == capi.ERR_INVALID
    assert cuda_lib.xtc_cuda_peer_barrier(None, flags, ranks, 2, 0, 1, None) == capi.ERR_INVALID
    assert "NULL argument" in capi.last_error()


def test_plan_run_sets_checks_its_arguments(cuda_lib):
    """xtc_cuda_plan_run_sets refuses a missing plan or table and an empty or negative
    rotation before anything is launched."""
    table = (ctypes.c_void_p * 3)()
    assert cuda_lib.xtc_cuda_plan_run_sets(None, table, 1, 0, 1, None) == capi.ERR_INVALID
    assert "NULL plan" in capi.last_error()
    fake = ctypes.c_void_p(1)  # never dereferenced: the table is checked first
    assert cuda_lib.xtc_cuda_plan_run_sets(fake, None, 1, 0, 1, None) == capi.ERR_INVALID


def test_conv_workspace_of_the_balanced_streamed_kernel(cuda_lib):
    """xtc_cuda_conv2d_workspace_bytes, callable without a device: a stride-1 layer whose filter
    bank does not fit in shared memory gets the flags and partial sums of the streamed-weights
    kernel's balanced form where dealing out (work item, slab) units evenly pays (16x28x28x256 ->
    512: 25 units for the busiest CTA pair instead of 32), asked for by name or not, and nothing
    where it does not (one unit in eight saved, or items cut into many pieces)."""
    def ask(B, H, W, C, F, variant):
        c = capi.GemmConfig(variant=variant)
        ws = ctypes.c_size_t(7)
        capi.check(cuda_lib.xtc_cuda_conv2d_workspace_bytes(B, H, W, C, 3, 3, F, 1, 1, 1, 1, 1, 1,
                                                            ctypes.byref(c), ctypes.byref(ws)))
        return ws.value

    pairs = 74  # of a 148-SM device, which is also what the library assumes without one
    flags = (pairs * 8 * 4 + 255) // 256 * 256
    want = flags + pairs * 8 * 32 * 128 * 4  # one flag and one 32 x 128 block per (pair, CTA, warp)
    assert ask(16, 28, 28, 256, 512, 5) == ask(16, 28, 28, 256, 512, 0) == want
    assert ask(32, 28, 28, 128, 128, 5) == ask(32, 28, 28, 128, 128, 0) == 0  # 7 units against 8
    assert ask(8, 14, 14, 256, 256, 5) == 0  # 128 units on 74 pairs: every item would be cut in pieces
    assert ask(32, 56, 56, 64, 64, 0) == 0   # the filter bank fits: resident weights


def test_default_gemm_config_is_a_legal_config(cuda_lib):
    """xtc_cuda_gemm_default_config: host arithmetic, callable without a device; what it returns
    is a configuration the GEMM entry point accepts (legal tile, K stage and split)."""
    for shape in ((4096, 4096, 4096), (512, 1024, 256), (256, 3072, 8192), (100352, 64, 256), (7, 9, 11)):
        c = capi.GemmConfig()
        capi.check(cuda_lib.xtc_cuda_gemm_default_config(*shape, ctypes.byref(c)))
        assert c.tile_m in (128, 256) and c.tile_n in (64, 128, 256) and c.tile_k in (32, 64), shape
        assert c.split_k >= 0 and (c.tile_m == 128 or c.split_k == 0)
    assert cuda_lib.xtc_cuda_gemm_default_config(0, 4, 4, ctypes.byref(capi.GemmConfig())) == capi.ERR_INVALID
    assert cuda_lib.xtc_cuda_gemm_default_config(4, 4, 4, None) == capi.ERR_INVALID


def test_counters_library_exports_every_declared_symbol(cuda_lib):
    """include/xtc_cuda_counters.h against the built CUPTI module and its ctypes binding."""
    from xtc_b200.runtimes import counters as gc

    header = (ROOT / "include" / "xtc_cuda_counters.h").read_text()
    declared = set(re.findall(r"\b(xtc_cuda_counters_[a-z0-9_]+)\s*\(", header))
    assert declared == set(gc.SIGNATURES), declared ^ set(gc.SIGNATURES)
    lib = gc.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert gc.split_counter_names(["cycles", "gpu.clocks", "gpu.dram__bytes_read.sum"]) == (
        [1, 2], ["clocks", "dram__bytes_read.sum"])
    # bad arguments are refused before the profiler is touched
    h = ctypes.c_void_p()
    assert lib.xtc_cuda_counters_open(ctypes.byref(h), None, 0) == gc.ERR_INVALID
    names = (ctypes.c_char_p * 1)(b"")
    assert lib.xtc_cuda_counters_open(ctypes.byref(h), names, 1) in (gc.ERR_INVALID, gc.ERR_UNAVAILABLE)
    assert lib.xtc_cuda_counters_last_error()


@pytest.mark.skipif(has_cuda(), reason="checks behaviour on a machine without a GPU")
def test_counters_say_unavailable_without_a_device(cuda_lib):
    from xtc_b200.runtimes import counters as gc

    with pytest.raises(gc.CountersError, match="no current CUDA context"):
        gc.GpuCounters(["clocks"])


def test_struct_layout_matches_the_header(cuda_lib):
    # sizeof(xtc_cuda_gemm_config) = 8 int32; sizeof(xtc_cuda_step) = 8*4 + 3*6*8 + 32
    assert ctypes.sizeof(capi.GemmConfig) == 32
    assert ctypes.sizeof(capi.Step) == 32 + 144 + 32


@pytest.mark.skipif(has_cuda(), reason="checks behaviour on a machine without a GPU")
def test_no_cpu_fallback_without_a_device(cuda_lib):
    n = ctypes.c_int(-1)
    rc = cuda_lib.xtc_cuda_device_count(ctypes.byref(n))
    assert rc == capi.ERR_RUNTIME and capi.last_error()
    impl = matmul_impl(128, 256, 64)
    result = impl.evaluate(impl.get_scheduler().schedule())
    assert isinstance(result, str) and "no CUDA device" in result
    module = impl.get_compiler(shared_lib=False).compile(None)
    assert module.get_executor().execute() != 0


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError, match="no fallback"):
        capi.load(tmp_path / "libxtc_cuda.so")
