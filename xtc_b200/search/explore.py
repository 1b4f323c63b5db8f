"""``loop-explore`` for the CUDA backend: search the kernels' parameter space.

Mirrors the reference's exploration driver (``search/explore.py:200-873`` and
its CLI ``cli/explore.py:52-355``): build the operator's graph, draw samples
from a strategy (``--search random | exhaustive``, or one default schedule with
``--opt-level``), and for every sample run the chain
``Backend -> get_scheduler -> strategy.generate -> schedule -> get_compiler ->
compile -> get_evaluator -> evaluate`` (``search/explore.py:339-438``), compile
stage in a thread pool, execute stage serial (``search/pipeline.py:28-117``).
Results go to a CSV with the reference's columns ``<sample names>, X, time,
peak, backend`` (``search/callback.py:149-165``); ``--resume`` skips samples
already present.  ``peak`` = peak_time / time with peak_time = FMAs / peak FMA
rate, the reference's definition (``search/explore.py:619-625``); the peak
rate defaults to the tensor-pipe probe of the device.

    python -m xtc_b200.search.explore --operator matmul --dims 4096 4096 4096 \
        --search exhaustive --output results.csv
"""

from __future__ import annotations

import argparse
import csv
import logging
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..graphs.xtc import op as O
from .strategies import Strategies

logger = logging.getLogger("xtc_b200.search")

OPERATORS = {
    "matmul": {"dims": ["i", "j", "k"], "default_dims": [512, 1024, 128],
               "default_strategy": "cuda_gemm"},
    "matmul_relu": {"dims": ["i", "j", "k"], "default_dims": [4096, 4096, 4096],
                    "default_strategy": "cuda_gemm"},
    "conv2d": {"dims": ["n", "h", "w", "f", "r", "s", "c", "SH", "SW"],
               "default_dims": [1, 112, 112, 64, 7, 7, 4, 2, 2], "default_strategy": "cuda_gemm"},
}


def matmul_graph(i: int, j: int, k: int, dtype: str = "float32", name: str = "matmul", relu=False):
    a = O.tensor((i, k), dtype, name="A")
    b = O.tensor((k, j), dtype, name="B")
    with O.graph(name=name) as gb:
        c = O.matmul(a, b, name="C")
        if relu:
            O.relu(c, name="R")
    return gb.graph


def conv2d_graph(n, h, w, f, r, s, c, SH, SW, dtype: str = "float32", name: str = "conv2d"):
    a = O.tensor((n, h * SH + r - 1, w * SW + s - 1, c), dtype, name="A")
    b = O.tensor((r, s, c, f), dtype, name="B")
    with O.graph(name=name) as gb:
        O.conv2d(a, b, stride=(SH, SW), name="O")
    return gb.graph


@dataclass
class ExplorationConfig:
    operator: str = "matmul"
    dims: list[int] | None = None
    graph: Any = None               # an already built graph overrides operator/dims
    graph_file: str | None = None   # a graph saved with Graph.dump (YAML) overrides operator/dims
    op_name: str | None = None      # dims of a registered operation (xtc_b200.artifacts)
    strategy: str | None = None
    search: str = "random"          # random | exhaustive
    trials: int = 20
    seed: int = 0
    opt_level: int | None = None    # evaluate one default schedule instead of searching
    output: str = "results.csv"
    resume: bool = False
    repeat: int = 3
    number: int = 10
    min_repeat_ms: int = 20
    validate: bool = False
    jobs: int = 4
    peak_flops: float | None = None  # FMA/s; default: probe the device
    precision: str = "tf32"
    device: int = 0
    explore_dir: str | None = None
    save_temps: bool = False
    strategy_options: dict = field(default_factory=dict)


class Exploration:
    def __init__(self, config: ExplorationConfig) -> None:
        self.config = config
        if config.graph is not None:
            self.graph = config.graph
        elif config.graph_file is not None:
            self.graph = self.load_graph(config.graph_file)
        else:
            spec = OPERATORS[config.operator]
            dims = config.dims or spec["default_dims"]
            if config.op_name:
                from .. import artifacts

                named = artifacts.get_operation(config.operator, config.op_name)["dims"]
                dims = [named[d] for d in spec["dims"]]
            assert len(dims) == len(spec["dims"]), (
                f"{config.operator} takes dims {spec['dims']}, got {dims}")
            if config.operator == "conv2d":
                self.graph = conv2d_graph(*dims)
            else:
                self.graph = matmul_graph(*dims, relu=config.operator == "matmul_relu")
        name = config.strategy or OPERATORS.get(config.operator, {}).get("default_strategy", "cuda_gemm")
        self.strategy = Strategies.create(name, self.graph, **config.strategy_options)
        self.results: list[tuple[list[int], int, float, str]] = []
        self._peak_time: float | None = None

    @staticmethod
    def load_graph(graph_file: str) -> Any:
        """A graph written by ``Graph.dump`` (the reference's ``--graph-file``,
        ``search/explore.py:211-217``)."""
        with O.graph() as gb:
            gb.load(graph_file)
        return gb.graph

    # -- peak -----------------------------------------------------------------------
    def fma_count(self) -> int:
        return sum(n.operation.ops_count for n in self.graph.nodes.values()
                   if n.operation.name in ("matmul", "conv2d"))

    def peak_time(self) -> float:
        if self._peak_time is None:
            peak = self.config.peak_flops
            if peak is None:
                from ..runtimes.cuda import CudaDevice

                peak = CudaDevice(self.config.device).evaluate_flops("float32")
            self._peak_time = self.fma_count() / peak
        return self._peak_time

    # -- one sample -------------------------------------------------------------------
    def compile_one(self, ident: str, sample: list[int], explore_dir: str):
        from ..backends.cuda import Backend

        impl = Backend(self.graph)
        scheduler = impl.get_scheduler(strict=True)
        self.strategy.generate(scheduler, sample)
        schedule = scheduler.schedule()
        compiler = impl.get_compiler(shared_lib=self.config.save_temps,
                                     dump_file=f"{explore_dir}/payload_{ident}",
                                     precision=self.config.precision)
        return compiler.compile(schedule)

    def evaluate_one(self, module: Any, sample: list[int]) -> tuple[list[int], int, float, str]:
        cfg = self.config
        evaluator = module.get_evaluator(repeat=cfg.repeat, number=cfg.number,
                                         min_repeat_ms=cfg.min_repeat_ms, validate=cfg.validate,
                                         device=cfg.device)
        results, code, msg = evaluator.evaluate()
        if code != 0:
            logger.error("error evaluating %s: %s", sample, msg)
            return (sample, code, float("inf"), "cuda")
        path = Path(module.file_name)
        if not cfg.save_temps and path.exists():
            path.unlink()
        return (sample, 0, min(results), "cuda")

    # -- the search ---------------------------------------------------------------------
    def samples(self) -> list[list[int]]:
        cfg = self.config
        if cfg.opt_level is not None:
            return [self.strategy.default_schedule(cfg.opt_level)]
        if cfg.search == "exhaustive":
            return list(self.strategy.exhaustive())
        if cfg.search == "random":
            return self.strategy.sample(cfg.trials, cfg.seed)
        raise ValueError(f"unknown search {cfg.search!r} (random, exhaustive)")

    def run(self) -> list[tuple[list[int], int, float, str]]:
        cfg = self.config
        samples = self.samples()
        names = list(self.strategy.sample_names)
        seen: set[tuple[int, ...]] = set()
        out_path = Path(cfg.output)
        if cfg.resume and out_path.exists() and out_path.stat().st_size > 0:
            with open(out_path, newline="") as f:
                for row in csv.DictReader(f):
                    try:
                        seen.add(tuple(int(row[n]) for n in names))
                    except (KeyError, ValueError, TypeError):
                        continue
        mode = "a" if (cfg.resume and seen) else "w"
        out_path.parent.mkdir(parents=True, exist_ok=True)
        explore_dir = cfg.explore_dir or tempfile.mkdtemp(prefix="xtc_explore_")
        Path(explore_dir).mkdir(parents=True, exist_ok=True)
        todo = [s for s in samples if tuple(s) not in seen]
        t0 = time.time()
        with open(out_path, mode, newline="") as f:
            writer = csv.writer(f)
            if mode == "w":
                writer.writerow(names + ["X", "time", "peak", "backend"])
            with ThreadPoolExecutor(max_workers=max(cfg.jobs, 1)) as pool:
                futures = [pool.submit(self.compile_one, f"{i}", s, explore_dir)
                           for i, s in enumerate(todo)]
                for sample, fut in zip(todo, futures):  # execute stage: serial, in order
                    module = fut.result()
                    result = self.evaluate_one(module, sample)
                    self.results.append(result)
                    if result[1] == 0:
                        writer.writerow(list(sample) + [str(list(sample)).replace(",", ";"), result[2],
                                                        self.peak_time() / result[2], "cuda"])
                        f.flush()
        elapsed = time.time() - t0
        ok = [r for r in self.results if r[1] == 0]
        if todo:
            logger.info("%d samples in %.1f s (%.3f s/sample)", len(todo), elapsed, elapsed / len(todo))
        if ok:
            best = min(ok, key=lambda r: r[2])
            print(f"Schedule: cuda: {best[0]}: time: {best[2] * 1e3:.4f} msecs, "
                  f"peak perf: {100 * self.peak_time() / best[2]:.2f}%")
        return self.results

    def best(self) -> tuple[list[int], float] | None:
        ok = [r for r in self.results if r[1] == 0]
        if not ok:
            return None
        b = min(ok, key=lambda r: r[2])
        return b[0], b[2]


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="loop-explore (cuda)", description=__doc__.split("\n")[0])
    ap.add_argument("--operator", default="matmul", choices=sorted(OPERATORS))
    ap.add_argument("--dims", nargs="+", type=int, help="dimensions, default to the operator's default")
    ap.add_argument("--graph-file", default=None, help="explore a graph saved as YAML instead of an operator")
    ap.add_argument("--op-name", default=None, help="dims of a registered operation, see --op-name-list")
    ap.add_argument("--op-name-list", action="store_true", help="list the registered operations and exit")
    ap.add_argument("--strategy", default=None, choices=Strategies.names())
    ap.add_argument("--search", default="random", choices=["random", "exhaustive"])
    ap.add_argument("--backends", nargs="+", default=["cuda"], choices=["cuda"])
    ap.add_argument("--trials", type=int, default=20)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--opt-level", type=int, default=None, choices=[0, 1, 2, 3])
    ap.add_argument("--output", default="results.csv")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--number", type=int, default=10)
    ap.add_argument("--min-repeat-ms", type=int, default=20)
    ap.add_argument("--validate", action="store_true")
    ap.add_argument("--jobs", type=int, default=4)
    ap.add_argument("--peak-flops", type=float, default=None, help="peak FMA/s (default: probe the device)")
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--explore-dir", default=None)
    ap.add_argument("--save-temps", action="store_true")
    ap.add_argument("--debug", action="store_true")
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.DEBUG if args.debug else logging.INFO)
    if args.op_name_list:
        from .. import artifacts

        for operator, name in artifacts.list_operations():
            print(f"{operator} {name}")
        return 0
    cfg = ExplorationConfig(
        graph_file=args.graph_file, op_name=args.op_name,
        operator=args.operator, dims=args.dims, strategy=args.strategy, search=args.search,
        trials=args.trials, seed=args.seed, opt_level=args.opt_level, output=args.output,
        resume=args.resume, repeat=args.repeat, number=args.number,
        min_repeat_ms=args.min_repeat_ms, validate=args.validate, jobs=args.jobs,
        peak_flops=args.peak_flops, precision=args.precision, device=args.device,
        explore_dir=args.explore_dir, save_temps=args.save_temps)
    results = Exploration(cfg).run()
    return 0 if any(r[1] == 0 for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
