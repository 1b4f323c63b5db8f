"""A Backend over the CPU loop nests of oracle/cpu_loopnest.c, and its search strategy.

TEST / BASELINE INFRASTRUCTURE: used only by tests/ and by the cpu_baseline /
reference legs of bench.py, never by the product path.

The reference tunes its CPU schedules with loop-explore: a strategy turns a sample
into tile / interchange / parallelize / vectorize / unroll calls on a Scheduler and
the driver compiles and times every sample (src/xtc/search/explore.py:339-438,
strategies src/xtc/search/strategies.py:638-670 "tile_oo", :772-781
"tile_pprprp_vr").  This module lets this repository's own exploration driver
(xtc_b200.search.explore.Exploration, `backend=` plug-in point) do the same for the
CPU restatement, so that the CPU baseline is a *tuned* schedule:

  StrategyCpuTile   sample [mc, nc, kc, micro] (matmul) or [micro] (conv2d) ->
                    tile(i, {i1: mc, i2: MR}); tile(j, {j1: nc, j2: NR}); tile(k, {k1: kc});
                    interchange; parallelize [i, j]; pack_at; vectorize [j2]; unroll {i2: MR}
  CpuScheduler      records the directives (the recorder of the CUDA backend, whose
                    fields are the reference's) and maps them back onto the nest's
                    arguments; an inner tile that no micro-kernel implements is
                    refused in strict mode
  CpuCompiler       nothing to generate: the nests are prebuilt with their tile sizes
                    as arguments (the reference generates and compiles code per sample)
  CpuEvaluator      (results, code, message) with host wall-clock seconds per run, the
                    reference's host evaluator contract
                    (src/xtc/targets/host/HostEvaluator.py:28-120)
"""

from __future__ import annotations

import itertools
import json
import random
import tempfile
import time
from pathlib import Path
from typing import Any

import numpy as np

from xtc_b200.backends.cuda.scheduler import (CudaNodeScheduler, CudaScheduler, ScheduleError,
                                              make_loop_name)

from . import cpu_baseline as cb
from . import xtc_oracle as xo

DEFAULT_MATMUL_SAMPLE = (128, 512, 256, 7)


class CpuNodeScheduler(CudaNodeScheduler):
    """Same recording; the mapping targets the CPU nests' arguments."""

    def kernel_config(self, strict: bool) -> dict[str, int]:
        def levels(dim: str) -> list[int]:
            return list(self.tiles.get(dim, {}).values())

        def lookup(shapes: list[tuple[int, int]], want: tuple[int, int], what: str) -> int:
            if want in shapes:
                return shapes.index(want)
            if strict:
                raise ScheduleError(f"{self.node_name}: no {what} micro-kernel for an inner tile of "
                                    f"{want[0]} x {want[1]} (have {shapes})")
            return min(range(len(shapes)),
                       key=lambda i: abs(shapes[i][0] - want[0]) + abs(shapes[i][1] - want[1]))

        if self.op_name == "matmul" and len(self.dims) == 3:
            i, j, k = self.dims
            ti, tj, tk = levels(i), levels(j), levels(k)
            if len(ti) < 2 or len(tj) < 2 or not tk:
                return {}
            inner_j = list(self.tiles[j])[-1]
            if strict and inner_j not in self.vectorization:
                raise ScheduleError(f"{self.node_name}: the innermost column tile must be vectorized")
            return {"mc": ti[0], "nc": tj[0], "kc": tk[0],
                    "micro": lookup(cb.micro_shapes(), (ti[1], tj[1]), "matmul")}
        if self.op_name == "conv2d" and len(self.dims) == 7:
            w, f = self.dims[2], self.dims[3]
            tw, tf = levels(w), levels(f)
            if not tw or not tf:
                return {}
            return {"micro": lookup(cb.conv_micro_shapes(), (tw[0], tf[0]), "conv2d")}
        return {}


class CpuScheduler(CudaScheduler):
    node_scheduler = CpuNodeScheduler


class CpuModule:
    file_type = "plan"

    def __init__(self, graph: Any, configs: dict[str, dict[str, int]], file_name: str) -> None:
        self.graph, self.configs, self.file_name = graph, configs, file_name
        self.name = self.payload_name = graph.name or "payload"

    def export(self) -> None:
        pass

    def get_evaluator(self, **kwargs: Any) -> "CpuEvaluator":
        return CpuEvaluator(self, **kwargs)

    def get_executor(self, **kwargs: Any) -> "CpuEvaluator":
        return CpuEvaluator(self, repeat=1, number=1, min_repeat_ms=0, **kwargs)


class CpuCompiler:
    def __init__(self, backend: "Backend", dump_file: str | None = None, **_ignored: Any) -> None:
        self._backend, self.dump_file = backend, dump_file

    def compile(self, schedule: Any = None) -> CpuModule:
        configs = schedule.node_configs() if schedule is not None else {}
        dump = self.dump_file or str(Path(tempfile.mkdtemp(prefix="xtc_cpu_")) / "payload")
        Path(dump).parent.mkdir(parents=True, exist_ok=True)
        file_name = f"{dump}.plan.json"
        Path(file_name).write_text(json.dumps(configs))
        return CpuModule(self._backend.graph, configs, file_name)


def run_nodes(graph: Any, configs: dict[str, dict[str, int]], inputs: list[np.ndarray]) -> list[np.ndarray]:
    """The graph's nodes in order on the CPU nests (matmul and conv2d on the register-blocked
    nests with their node's sample, the data movement on the one-pass loops or NumPy)."""
    vals: dict[str, np.ndarray] = dict(zip(graph.inputs, inputs))
    for node in graph.nodes.values():
        op, attrs = node.operation, dict(node.operation.attrs)
        args = [vals[u] for u in node.inputs]
        cfg = configs.get(node.name, {})
        if op.name == "matmul":
            a = np.ascontiguousarray(args[0].reshape(args[0].shape[0], -1))
            b = np.ascontiguousarray(args[1].reshape(-1, args[1].shape[-1]))
            sample = ((cfg["mc"], cfg["nc"], cfg["kc"], cfg["micro"]) if cfg else DEFAULT_MATMUL_SAMPLE)
            out = cb.matmul_blocked(a, b, sample)
        elif op.name == "conv2d":
            stride = xo._stride2(attrs.get("stride", (1, 1)))
            x = np.ascontiguousarray(args[0].reshape((-1,) + args[0].shape[-3:]))
            out = cb.conv2d_blocked(x, np.ascontiguousarray(args[1]), stride, cfg.get("micro", 2))
            out = out.reshape(tuple(op.outputs_types[0].shape))
        elif op.name == "relu":
            out = cb.relu(np.ascontiguousarray(args[0]), float(attrs.get("threshold", 0)))
        elif op.name == "transpose" and args[0].ndim == 2:
            out = cb.transpose2d(np.ascontiguousarray(args[0]))
        elif op.name == "pad":
            widths = xo.pad_widths(attrs.get("padding", 0), args[0].ndim)
            if args[0].ndim == 4 and widths[0] == (0, 0) and widths[3] == (0, 0):
                out = cb.pad_hw(np.ascontiguousarray(args[0]), *widths[1], *widths[2],
                                float(attrs.get("constant_value", 0)))
            else:
                out = xo.pad(args[0], attrs.get("padding", 0), attrs.get("constant_value", 0))
        else:
            out = getattr(xo, op.name)(*args, **attrs)
        vals[node.uid] = out
    return [vals[u] for u in graph.outputs]


class CpuEvaluator:
    def __init__(self, module: CpuModule, repeat: int = 1, number: int = 1, min_repeat_ms: int = 100,
                 validate: bool = False, parameters: Any = None, **_ignored: Any) -> None:
        self.module, self.repeat, self.number = module, repeat, max(number, 1)
        self.min_repeat_ms, self.validate, self.parameters = min_repeat_ms, validate, parameters

    def evaluate(self) -> tuple[list[float], int, str]:
        graph = self.module.graph
        try:
            if self.parameters is not None:
                ins = [np.asarray(a) for a in self.parameters[0]]
            else:
                ins = [xo.np_init(tuple(t.shape), str(t.dtype)) for t in graph.inputs_types]
            outs = run_nodes(graph, self.module.configs, ins)  # warm-up (and validation) run
            if self.validate:
                nodes = [{"op": n.operation.name, "inputs": list(n.inputs), "uid": n.uid,
                          "attrs": dict(n.operation.attrs)} for n in graph.nodes.values()]
                vals = dict(zip(graph.inputs, [a.astype(np.float64) for a in ins]))
                for n in nodes:
                    vals[n["uid"]] = getattr(xo, n["op"])(*[vals[u] for u in n["inputs"]], **n["attrs"])
                for got, uid in zip(outs, graph.outputs):
                    if xo.rel_err(got, vals[uid]) > 1e-5:
                        return ([], 1, "Error in validation: outputs differ")
            results = []
            for _ in range(self.repeat):
                attempts = self.number
                while True:  # the doubling loop of csrcs/runtimes/host/evaluate_perf.c:92-120
                    t0 = time.perf_counter()
                    for _ in range(attempts):
                        outs = run_nodes(graph, self.module.configs, ins)
                    t = time.perf_counter() - t0
                    if t * 1e3 >= self.min_repeat_ms or attempts >= 1 << 20:
                        results.append(t / attempts)
                        break
                    attempts *= 2
            if self.parameters is not None:
                for dst, src in zip(self.parameters[1], outs):
                    np.copyto(dst, src.reshape(dst.shape))
            return (results, 0, "")
        except (ValueError, AssertionError) as exc:
            return ([], 1, f"Error in execution: {exc}")

    def execute(self) -> int:
        return self.evaluate()[1]


class Backend:
    """``Backend(graph)`` over the CPU nests: what ``Exploration(backend=...)`` instantiates."""

    def __init__(self, graph: Any, **_ignored: Any) -> None:
        self._graph = graph

    @property
    def graph(self) -> Any:
        return self._graph

    def get_scheduler(self, **kwargs: Any) -> CpuScheduler:
        return CpuScheduler(self, **kwargs)

    def get_compiler(self, **kwargs: Any) -> CpuCompiler:
        return CpuCompiler(self, **kwargs)


class StrategyCpuTile:
    """Two-level tiling with a register-blocked, vectorized inner tile: the shape of the
    reference's "tile_oo" / "tile_pprprp_vr" strategies, over the sizes the nests implement."""

    name = "cpu_tile"
    MC = (48, 96, 128, 192, 256, 384)
    NC = (128, 256, 512, 1024, 2048)
    KC = (64, 128, 256, 512)

    def __init__(self, graph: Any, **_ignored: Any) -> None:
        nodes = [n for n in graph.nodes.values() if n.operation.name in ("matmul", "conv2d")]
        if not nodes:
            raise ValueError("the graph has no matmul or conv2d node to schedule")
        self._graph, self._node = graph, nodes[-1]
        self._op = self._node.operation
        self._is_conv = self._op.name == "conv2d"
        self.sample_names = ["micro"] if self._is_conv else ["mc", "nc", "kc", "micro"]

    @property
    def graph(self) -> Any:
        return self._graph

    def exhaustive(self):
        if self._is_conv:
            f = int(list(self._op.dims.values())[3])
            for idx, (_, ft) in enumerate(cb.conv_micro_shapes()):
                if ft <= max(f, cb.conv_micro_shapes()[0][1]):
                    yield [idx]
            return
        m, n, k = (int(v) for v in self._op.dims.values())
        for mc, nc, kc, micro in itertools.product(self.MC, self.NC, self.KC,
                                                   range(len(cb.micro_shapes()))):
            mr, nr = cb.micro_shapes()[micro]
            if mc % mr or nc % nr or mc > max(m, mr) * 2 or nc > max(n, nr) * 2 or kc > max(k, 64):
                continue
            if (mc * kc + kc * nc) * 4 > 2 << 20:  # the packed blocks of one thread stay in L2
                continue
            yield [mc, nc, kc, micro]

    def sample(self, num: int, seed: int | None = 0) -> list[list[int]]:
        space = list(self.exhaustive())
        random.Random(seed).shuffle(space)
        return space[: max(num, 0)]

    def default_schedule(self, opt_level: int = 2) -> list[int]:
        return [2] if self._is_conv else list(DEFAULT_MATMUL_SAMPLE)

    def generate(self, scheduler: Any, sample: list[int]) -> None:
        dims = list(self._op.dims)
        target = scheduler.node(self._node.name) if hasattr(scheduler, "node") else scheduler
        if self._is_conv:
            wt, ft = cb.conv_micro_shapes()[int(sample[0])]
            b, h, w, f, r, s, c = dims
            target.tile(w, {f"{w}1": wt})
            target.tile(f, {f"{f}1": ft})
            target.interchange([b, h, w, f, r, s, c, f"{w}1", f"{f}1"])
            target.parallelize([b, h])
            target.vectorize([f"{f}1"])
            target.unroll({f"{w}1": wt})
            return
        mc, nc, kc, micro = (int(v) for v in sample)
        mr, nr = cb.micro_shapes()[micro]
        i, j, k = dims
        target.tile(i, {f"{i}1": mc, f"{i}2": mr})
        target.tile(j, {f"{j}1": nc, f"{j}2": nr})
        target.tile(k, {f"{k}1": kc})
        target.interchange([i, j, k, f"{j}1", f"{i}1", f"{k}1", f"{i}2", f"{j}2"])
        target.parallelize([i, j])
        target.pack_at(k, 0)
        target.pack_at(k, 1)
        target.vectorize([f"{j}2"])
        target.unroll({f"{i}2": mr})


def tune(graph: Any, trials: int = 20, seed: int = 0, inputs: list[np.ndarray] | None = None,
         output: str | None = None) -> tuple[list[int], float, int]:
    """Random search with this repository's exploration driver over the CPU nests.
    Returns (best sample, its seconds per run, samples measured)."""
    from xtc_b200.search.explore import Exploration, ExplorationConfig
    from xtc_b200.search.strategies import Strategies

    Strategies.register(StrategyCpuTile.name, StrategyCpuTile)
    cfg = ExplorationConfig(graph=graph, strategy=StrategyCpuTile.name, search="random", trials=trials,
                            seed=seed, output=output or "", repeat=1, number=1, min_repeat_ms=0,
                            jobs=1, peak_flops=cb.peak_fma(), backend=_backend_with(inputs),
                            backend_name="cpu_loopnest")
    exp = Exploration(cfg)
    exp.run()
    best = exp.best()
    if best is None:
        raise RuntimeError("no CPU sample could be measured")
    return list(best[0]), float(best[1]), len(exp.results)


def _backend_with(inputs: list[np.ndarray] | None) -> Any:
    """The Backend class, or one whose evaluators run on the given inputs."""
    if inputs is None:
        return Backend

    class BoundBackend(Backend):
        def get_compiler(self, **kwargs: Any) -> CpuCompiler:
            comp = CpuCompiler(self, **kwargs)
            compile_ = comp.compile

            def compile_bound(schedule: Any = None) -> CpuModule:
                module = compile_(schedule)
                get = module.get_evaluator
                module.get_evaluator = lambda **kw: get(**{**kw, "parameters": (
                    inputs, [np.empty(tuple(t.shape), np.float32) for t in self.graph.outputs_types])})
                return module

            comp.compile = compile_bound
            return comp

    return BoundBackend
