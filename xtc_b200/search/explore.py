"""``loop-explore`` for the CUDA backend: search the kernels' parameter space.

Mirrors the reference's exploration driver (``search/explore.py:200-873`` and
its CLI ``cli/explore.py:52-355``): build the operator's graph, draw samples
from a strategy (``--search random | exhaustive``, the samples of an earlier
table with ``--search data --data table.csv``, batches proposed by an optimizer
with ``--search iterative --optimizer ... --batch n``, or one default schedule
with ``--opt-level``), and for every sample run the chain
``Backend -> get_scheduler -> strategy.generate -> schedule -> get_compiler ->
compile -> get_evaluator -> evaluate`` (``search/explore.py:339-438``), compile
stage in a thread pool, execute stage serial (``search/pipeline.py:28-117``).
Results go to a CSV with the reference's columns ``<sample names>, X, time,
peak, backend`` (``search/callback.py:149-165``); ``--resume`` skips samples
already present, ``--append`` adds to the file, ``--db-file`` also appends JSON
lines to a results database, and ``<output>.meta.json`` records the arguments.  ``peak`` = peak_time / time with peak_time = FMAs / peak FMA
rate, the reference's definition (``search/explore.py:619-625``); the peak
rate defaults to the tensor-pipe probe of the device.

    python -m xtc_b200.search.explore --operator matmul --dims 4096 4096 4096 \
        --search exhaustive --output results.csv
"""

from __future__ import annotations

import argparse
import csv
import itertools
import json
import logging
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

from ..graphs.xtc import op as O
from .callback import CSVCallback, DBCallback, MemoryCallback
from .optimizers import Optimizers
from .strategies import Strategies

logger = logging.getLogger("xtc_b200.search")

OPERATORS = {
    "matmul": {"dims": ["i", "j", "k"], "default_dims": [512, 1024, 128],
               "default_strategy": "cuda_gemm"},
    "matmul_relu": {"dims": ["i", "j", "k"], "default_dims": [4096, 4096, 4096],
                    "default_strategy": "cuda_gemm"},
    "conv2d": {"dims": ["n", "h", "w", "f", "r", "s", "c", "SH", "SW"],
               "default_dims": [1, 112, 112, 64, 7, 7, 4, 2, 2], "default_strategy": "cuda_conv"},
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
    search: str = "random"          # random | exhaustive | data | iterative
    data: str | None = None         # CSV table whose X column lists the samples of a "data" search
    optimizer: str = "random-forest-default"  # proposes the batches of an "iterative" search
    optimizer_config: str | None = None       # YAML file overriding single optimizer settings
    batch: int = 1                  # samples per optimizer step
    trials: int = 20
    seed: int = 0
    opt_level: int | None = None    # evaluate one default schedule instead of searching
    output: str = "results.csv"
    db_file: str | None = None      # also append JSON lines to this results database
    resume: bool = False
    append: bool = False
    repeat: int = 3
    number: int = 10
    min_repeat_ms: int = 20
    validate: bool = False
    jobs: int = 4
    peak_flops: float | None = None  # FMA/s; default: probe the device
    precision: str = "tf32"
    device: int = 0
    # Backend class to explore with: Backend(graph) with get_scheduler / get_compiler, the
    # plug-in point of the reference's driver (search/explore.py:262-268).  None = the CUDA
    # backend; `backend_name` is what the result rows carry.
    backend: Any = None
    backend_name: str = "cuda"
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

                dims = artifacts.operation_dims(config.operator, config.op_name)
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
        Backend = self.config.backend
        if Backend is None:
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
            return (sample, code, float("inf"), cfg.backend_name)
        path = Path(module.file_name)
        if not cfg.save_temps and path.exists():
            path.unlink()
        return (sample, 0, min(results), cfg.backend_name)

    # -- the search ---------------------------------------------------------------------
    @staticmethod
    def read_input(fname: str) -> list[list[int]]:
        """Samples of a results table: its ``X`` column holds each sample as a list
        printed with ``;`` between the values (the table ``CSVCallback`` writes; the
        reference reads the same column, ``search/explore.py:607-617``)."""
        out: list[list[int]] = []
        with open(fname, newline="") as f:
            for row in csv.DictReader(f):
                text = (row.get("X") or "").strip().strip("[]")
                if text:
                    out.append([int(v) for v in text.replace(";", ",").split(",")])
        return out

    def samples(self) -> list[list[int]]:
        """The fixed sample list of every search but the iterative one."""
        cfg = self.config
        if cfg.opt_level is not None:
            return [self.strategy.default_schedule(cfg.opt_level)]
        if cfg.search == "exhaustive":
            space = self.strategy.exhaustive()
            return list(itertools.islice(space, cfg.trials)) if cfg.trials else list(space)
        if cfg.search == "random":
            return self.strategy.sample(cfg.trials, cfg.seed)
        if cfg.search == "data":
            assert cfg.data, "a data search needs the table to read (--data)"
            return self.read_input(cfg.data)
        raise ValueError(f"unknown search {cfg.search!r} (random, exhaustive, data, iterative)")

    def result_callbacks(self) -> list[Any]:
        cfg = self.config
        self.memory = MemoryCallback()
        callbacks: list[Any] = [self.memory]
        self.csv = None
        if cfg.output:
            self.csv = CSVCallback(cfg.output, self.peak_time(), list(self.strategy.sample_names),
                                   resume=cfg.resume, append=cfg.append)
            callbacks.append(self.csv)
        if cfg.db_file:
            from ..runtimes.cuda import CudaDevice

            device = CudaDevice(cfg.device)
            db = DBCallback(cfg.db_file, device.device_name(), 1, self.strategy.name)
            db.set_graph(self.graph)
            callbacks.append(db)
        return callbacks

    def evaluate_batch(self, batch: list[list[int]], explore_dir: str, callbacks: list[Any],
                       first_ident: int = 0) -> list[tuple[list[int], int, float, str]]:
        """Compile stage in a thread pool, execute stage serial and in order."""
        out = []
        with ThreadPoolExecutor(max_workers=max(self.config.jobs, 1)) as pool:
            futures = [pool.submit(self.compile_one, f"{first_ident + i}", s, explore_dir)
                       for i, s in enumerate(batch)]
            for sample, fut in zip(batch, futures):
                try:
                    result = self.evaluate_one(fut.result(), sample)
                except Exception as exc:  # an illegal sample is a failed result, not the end
                    logger.error("error compiling %s: %s", sample, exc)
                    result = (list(sample), 1, float("inf"), self.config.backend_name)
                out.append(result)
                for cb in callbacks:
                    cb(result)
        return out

    def write_run_manifest(self) -> None:
        """``<output>.meta.json``: when, with which arguments and sample names a table
        was made (``search/explore.py:656-677``)."""
        cfg = self.config
        args = {k: (v if isinstance(v, (str, int, float, bool, list, dict)) or v is None else str(v))
                for k, v in vars(cfg).items() if k != "graph"}
        payload = {"generatedAt": datetime.now(timezone.utc).isoformat(), "output": cfg.output,
                   "resume": cfg.resume, "append": cfg.append,
                   "sampleNames": list(self.strategy.sample_names),
                   "python": {"version": sys.version, "executable": sys.executable},
                   "platform": {"platform": sys.platform}, "args": args}
        with open(f"{cfg.output}.meta.json", "w", encoding="utf-8") as f:
            json.dump(payload, f, indent=2, sort_keys=True)
            f.write("\n")

    def run(self) -> list[tuple[list[int], int, float, str]]:
        cfg = self.config
        callbacks = self.result_callbacks()
        if cfg.output:
            self.write_run_manifest()
        explore_dir = cfg.explore_dir or tempfile.mkdtemp(prefix="xtc_explore_")
        Path(explore_dir).mkdir(parents=True, exist_ok=True)
        t0 = time.time()
        if cfg.search == "iterative" and cfg.opt_level is None:
            done = self.run_iterative(explore_dir, callbacks)
        else:
            todo = [s for s in self.samples()
                    if not (cfg.resume and self.csv is not None and self.csv.is_recorded(s))]
            done = len(self.evaluate_batch(todo, explore_dir, callbacks))
        elapsed = time.time() - t0
        if self.csv is not None:
            self.csv.close()
        self.results = list(self.memory.results)
        ok = [r for r in self.results if r[1] == 0]
        if done:
            logger.info("%d samples in %.1f s (%.3f s/sample)", done, elapsed, elapsed / done)
        if ok:
            best = min(ok, key=lambda r: r[2])
            print(f"Schedule: {cfg.backend_name}: {best[0]}: time: {best[2] * 1e3:.4f} msecs, "
                  f"peak perf: {100 * self.peak_time() / best[2]:.2f}%")
        return self.results

    def run_iterative(self, explore_dir: str, callbacks: list[Any]) -> int:
        """Optimizer-driven search: suggest a batch, measure it, report fractions of peak
        (``search/explore.py:515-541``; a failed sample scores 0 instead of dividing by
        its zero time)."""
        cfg = self.config
        opt = Optimizers.create(cfg.optimizer, self.strategy.sample, cfg.batch, cfg.seed,
                                cfg.optimizer_config)
        done = 0
        while done < cfg.trials:
            batch = opt.suggest()[: min(cfg.batch, cfg.trials - done)]
            if not batch:
                break
            results = self.evaluate_batch(batch, explore_dir, callbacks, first_ident=done)
            opt.observe(batch, [self.peak_time() / r[2] if r[1] == 0 else 0.0 for r in results])
            done += len(batch)
        opt.finished()
        return done

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
    ap.add_argument("--search", default="random", choices=["random", "exhaustive", "data", "iterative"])
    ap.add_argument("--data", default=None, help="results table whose samples a data search re-evaluates")
    ap.add_argument("--optimizer", default="random-forest-default", choices=Optimizers.names())
    ap.add_argument("--optimizer-list", action="store_true", help="list the optimizers and exit")
    ap.add_argument("--optimizer-config", default=None, help="YAML file overriding optimizer settings")
    ap.add_argument("--batch", type=int, default=1, help="samples per optimizer step")
    ap.add_argument("--backends", nargs="+", default=["cuda"], choices=["cuda"])
    ap.add_argument("--trials", type=int, default=20)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--opt-level", type=int, default=None, choices=[0, 1, 2, 3])
    ap.add_argument("--output", default="results.csv")
    ap.add_argument("--db-file", default=None, help="also append results to this JSON-lines database")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--append", action="store_true")
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
    if args.optimizer_list:
        print("\n".join(Optimizers.names()))
        return 0
    if args.op_name_list:
        from .. import artifacts

        for operator, name in artifacts.list_operations():
            print(f"{operator} {name}")
        return 0
    cfg = ExplorationConfig(
        graph_file=args.graph_file, op_name=args.op_name,
        operator=args.operator, dims=args.dims, strategy=args.strategy, search=args.search,
        trials=args.trials, seed=args.seed, opt_level=args.opt_level, output=args.output,
        resume=args.resume, append=args.append, db_file=args.db_file, data=args.data,
        optimizer=args.optimizer, optimizer_config=args.optimizer_config, batch=args.batch,
        repeat=args.repeat, number=args.number,
        min_repeat_ms=args.min_repeat_ms, validate=args.validate, jobs=args.jobs,
        peak_flops=args.peak_flops, precision=args.precision, device=args.device,
        explore_dir=args.explore_dir, save_temps=args.save_temps)
    results = Exploration(cfg).run()
    return 0 if any(r[1] == 0 for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
