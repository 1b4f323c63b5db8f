"""The declarative schedule front end: the reference's descript specifications
(tests/filecheck/schedules/test_matmul_descript_mlir.py and its neighbours) turn into
the same scheduler calls a hand-written schedule makes."""

import pytest

import xtc_b200.graphs.xtc.op as O
from xtc_b200.backends.cuda import Backend
from xtc_b200.schedules.descript import (ScheduleInterpretError, ScheduleParseError,
                                         descript_scheduler)


def matmul_backend(i=4, j=32, k=512):
    a = O.tensor((i, k), "float32", name="A")
    b = O.tensor((k, j), "float32", name="B")
    with O.graph(name="matmul") as gb:
        O.matmul(a, b, name="C")
    return Backend(gb.graph)


class Recorder:
    """A scheduler that only records the calls it gets."""

    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        def record(*args, **kwargs):
            self.calls.append((name, args, kwargs))
        return record


def test_reference_example_equals_direct_calls():
    """The specification of test_matmul_descript_mlir.py:19-31."""
    spec = {"K": {}, "I": {}, "J": {}, "I#2": {"unroll": True}, "J#16": {"vectorize": True}}
    sch = matmul_backend().get_scheduler()
    descript_scheduler(scheduler=sch, node_name="C", abstract_dims=["I", "J", "K"], spec=spec)
    direct = matmul_backend().get_scheduler()
    direct.set_dims(["I", "J", "K"])
    direct.tile("I", {"I0": 2}, root="C")
    direct.tile("J", {"J0": 16}, root="C")
    direct.interchange(["K", "I", "J", "I0", "J0"], root="C")
    direct.vectorize(["J0"], root="C")
    direct.unroll({"I0": 2}, root="C")
    assert str(sch.schedule()) == str(direct.schedule())
    assert sch.schedule().node_configs() == direct.schedule().node_configs()


def test_call_sequence_with_splits_packs_and_yaml():
    spec = """
    J[0:256]:
      K: {}
      K#8: {unroll: 4}
      J#64: {parallelize: true, pack: [1, shared, false]}
    J[256:]:
      K#T: {buffer: default}
      J#16: {vectorize: null}
    I: {}
    """
    rec = Recorder()
    descript_scheduler(rec, "mm", ["I", "J", "K"], spec, abstract_dim_sizes={"I": 64, "J": 320, "K": 128},
                       sample={"T": 32})
    names = [c[0] for c in rec.calls]
    assert names[0] == "set_dims" and rec.calls[0][1] == (["I", "J", "K"],)
    # the root nest: one split of J into two segments, then I
    assert ("split", ("J", {"J[0]": 0, "J[1]": 256}), {"root": "mm"}) in rec.calls
    assert ("interchange", (["J[0]", "J[1]", "I"],), {"root": "mm"}) in rec.calls
    # first segment
    assert ("tile", ("K", {"K0": 8}), {"root": "mm/J[0]"}) in rec.calls
    assert ("tile", ("J", {"J0": 64}), {"root": "mm/J[0]"}) in rec.calls
    assert ("interchange", (["J", "K", "K0", "J0"],), {"root": "mm/J[0]"}) in rec.calls
    assert ("unroll", ({"K0": 4},), {"root": "mm/J[0]"}) in rec.calls
    assert ("parallelize", (["J0"],), {"root": "mm/J[0]"}) in rec.calls
    assert ("pack_at", ("J0", 1), {"mtype": "shared", "pad": False, "root": "mm/J[0]"}) in rec.calls
    # second segment: the tile size comes from the sample, `vectorize: null` means yes
    assert ("tile", ("K", {"K0": 32}), {"root": "mm/J[1]"}) in rec.calls
    assert ("buffer_at", ("K0",), {"mtype": None, "root": "mm/J[1]"}) in rec.calls
    assert ("vectorize", (["J0"],), {"root": "mm/J[1]"}) in rec.calls
    # parents are applied before their children
    assert names.index("split") < [i for i, c in enumerate(rec.calls) if c[2].get("root") == "mm/J[0]"][0]


def test_sized_segments_and_matrix_names():
    rec = Recorder()
    descript_scheduler(rec, "n", ["i", "j"],
                       {"i[:32:]": {"j": {}},                       # the next 32 iterations
                        "i[32:]": {"j": {"pack": ("A", "default", True)}, "C": {"pack": None}}},
                       abstract_dim_sizes={"i": 64, "j": 8}, abstract_matrix=["A", "B", "C"])
    assert ("split", ("i", {"i[0]": 0, "i[1]": 32}), {"root": "n"}) in rec.calls
    assert ("pack_at", ("j", 0), {"mtype": None, "pad": True, "root": "n/i[1]"}) in rec.calls
    # packing the last matrix (the output) is a write buffer
    assert ("buffer_at", ("j",), {"mtype": None, "root": "n/i[1]"}) in rec.calls


@pytest.mark.parametrize("spec,error", [
    ({"Z": {}}, ScheduleInterpretError),                                  # unknown axis
    ({"I#0": {}}, ScheduleInterpretError),                                # empty tile
    ({"I#2#3": {}}, ScheduleParseError),                                  # tile syntax
    ({"I": {"unrol": True}}, ScheduleParseError),                         # unknown annotation
    ({"I": {"unroll": True}}, ScheduleInterpretError),                    # full unroll of an unsized loop
    ({"I#4": {"unroll": -1}}, ScheduleInterpretError),
    ({"I#4": {"partial": True, "full": True}}, ScheduleParseError),
    ({"I#T": {}}, ScheduleInterpretError),                                # unbound parameter
    ({"I[0:4]": {}, "I[8:]": {}}, ScheduleInterpretError),                # gap between segments
    ({"I[0:4]": {}, "I[2:]": {}}, ScheduleInterpretError),                # overlap
    ({"I[4:4]": {}}, ScheduleInterpretError),
    ({"I[0:4]": {}}, ScheduleInterpretError),                             # stops before the end
    ({"I[0:]": {}, "I[4:]": {}}, ScheduleInterpretError),                 # already covered
    ({"I": {"buffer": True}}, ScheduleParseError),
    ({"I": {"pack": (1, 2)}}, ScheduleParseError),
    ({"I": 3}, ScheduleParseError),
])
def test_errors(spec, error):
    with pytest.raises(error):
        descript_scheduler(Recorder(), "n", ["I", "J"], spec,
                           abstract_dim_sizes={"I": 16} if any("[" in k for k in spec) else {})


def test_axis_scheduled_twice_in_a_segment():
    with pytest.raises(ScheduleInterpretError):
        descript_scheduler(Recorder(), "n", ["I", "J"], {"I[0:]": {"I": {}}})


@pytest.mark.gpu
def test_descript_schedule_runs_and_validates(cuda_lib):
    """The reference's script end to end with only the imports changed, plus a
    schedule that names the CTA-pair tile."""
    impl = matmul_backend()
    sch = impl.get_scheduler()
    descript_scheduler(scheduler=sch, node_name="C", abstract_dims=["I", "J", "K"],
                       spec={"K": {}, "I": {}, "J": {}, "I#2": {"unroll": True}, "J#16": {"vectorize": True}})
    module = impl.get_compiler(shared_lib=False).compile(sch.schedule())
    assert module.get_executor(validate=True).execute() == 0

    impl = matmul_backend(512, 512, 256)
    sch = impl.get_scheduler(strict=True)
    descript_scheduler(sch, "C", ["m", "n", "k"],
                       {"m": {"parallelize": True}, "n": {"parallelize": True}, "k": {},
                        "k#64": {"unroll": 3}, "m#256": {}, "n#128": {"vectorize": True}})
    schedule = sch.schedule()
    assert schedule.node_configs()["C"] == {"tile_m": 256, "tile_n": 128, "tile_k": 64, "stages": 3,
                                            "epilogue": 2}
    module = impl.get_compiler(shared_lib=False).compile(schedule)
    assert module.get_executor(validate=True).execute() == 0
