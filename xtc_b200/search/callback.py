"""Result sinks of an exploration.

Every evaluated sample is handed, as ``(sample, code, seconds, backend)``, to
a list of callbacks: one keeps results in memory, one writes the CSV table
that ``--search data`` reads back, one appends JSON lines to a results
database.  The three mirror ``MemoryCallback``, ``CSVCallback`` and
``DBCallback`` of the reference (``search/callback.py:22-176``) with the same
file formats, so tables written by either side can be read by the other: the
CSV header is the strategy's sample names followed by ``X, time, peak,
backend`` and the database record has the keys ``version, platform, compiler,
operator, strategy, schedule, results`` of ``cli/query_results.py:60-125``
with the compiler entry ``["xtc", <version>, <target>, <threads>, <backend>]``
(target is the device name here, threads 1: one GPU).
"""

from __future__ import annotations

import csv
import hashlib
import json
import os
import platform
from pathlib import Path
from typing import Any, Protocol, Sequence

Result = Sequence[Any]  # (sample, code, seconds, backend)

DB_FORMAT_VERSION = 1


class ResultCallback(Protocol):
    def __call__(self, result: Result) -> None: ...


class MemoryCallback:
    """Keeps every result, failed ones included."""

    def __init__(self) -> None:
        self.results: list[Result] = []

    def __call__(self, result: Result) -> None:
        self.results.append(result)


class CSVCallback:
    """One row per successful sample; ``resume`` skips samples already in the file,
    ``append`` adds to an existing file without reading it."""

    def __init__(self, fname: str, peak_time: float, sample_names: list[str], *,
                 resume: bool = False, append: bool = False) -> None:
        self.fname = fname
        self.peak_time = peak_time
        self.sample_names = list(sample_names)
        self.seen: set[tuple[str, tuple[int, ...]]] = set()
        path = Path(fname)
        path.parent.mkdir(parents=True, exist_ok=True)
        has_rows = path.exists() and path.stat().st_size > 0
        if resume and has_rows:
            self.seen = self.read_keys(fname, self.sample_names)
        mode = "a" if (resume or append) else "w"
        self._file = open(fname, mode, newline="")
        self._writer = csv.writer(self._file)
        if mode == "w" or not has_rows:
            self._writer.writerow(self.sample_names + ["X", "time", "peak", "backend"])
            self._file.flush()

    @staticmethod
    def read_keys(fname: str, sample_names: list[str]) -> set[tuple[str, tuple[int, ...]]]:
        keys: set[tuple[str, tuple[int, ...]]] = set()
        with open(fname, newline="") as f:
            for row in csv.DictReader(f):
                try:
                    keys.add((row["backend"], tuple(int(row[n]) for n in sample_names)))
                except (KeyError, ValueError, TypeError):
                    continue  # a foreign or damaged row does not stop a resume
        return keys

    def is_recorded(self, sample: Sequence[int], backend: str = "cuda") -> bool:
        return (backend, tuple(int(v) for v in sample)) in self.seen

    def __call__(self, result: Result) -> None:
        sample, code, seconds, backend = result
        if code != 0:
            return
        key = (backend, tuple(int(v) for v in sample))
        if key in self.seen:
            return
        values = [int(v) for v in sample]
        peak = self.peak_time / seconds if seconds > 0 else 0.0
        self._writer.writerow(values + [str(values).replace(",", ";"), seconds, peak, backend])
        self._file.flush()
        try:
            os.fsync(self._file.fileno())
        except OSError:
            pass
        self.seen.add(key)

    def close(self) -> None:
        if not self._file.closed:
            self._file.close()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


def _digest(obj: Any) -> str:
    return hashlib.sha1(json.dumps(obj).encode()).hexdigest()


class DBCallback:
    """Appends one JSON line per sample (failed ones with time 0) to ``dbfile``."""

    def __init__(self, dbfile: str, target: str, threads: int, strategy: str,
                 version: str | None = None) -> None:
        if version is None:
            from .. import __version__ as version  # type: ignore[no-redef]
        self.dbfile = dbfile
        self.target = target
        self.threads = threads
        self.xtc_version = f"v{version}"
        self.platform = [platform.node().split(".")[0], platform.system(), platform.machine()]
        self.strategy = ["xtc.strategy", _digest(strategy), strategy]
        self.operator: list[Any] | None = None
        Path(dbfile).parent.mkdir(parents=True, exist_ok=True)

    def set_graph(self, graph: Any) -> None:
        """The operator key is the graph's dictionary without its name, and its SHA-1."""
        obj = graph.to_dict() if not isinstance(graph, (str, dict)) else graph
        if isinstance(obj, dict):
            obj = {k: v for k, v in obj.items() if k != "name"}
        self.operator = ["xtc.graph", _digest(obj), obj]

    def record(self, result: Result) -> dict[str, Any]:
        sample, code, seconds, backend = result
        return dict(
            version=[DB_FORMAT_VERSION],
            platform=self.platform,
            compiler=["xtc", self.xtc_version, self.target, self.threads, backend],
            operator=self.operator,
            strategy=self.strategy,
            schedule=[int(v) for v in sample],
            results=[int(code), [float(seconds) if code == 0 else 0.0]],
        )

    def __call__(self, result: Result) -> None:
        with open(self.dbfile, "a") as f:
            print(json.dumps(self.record(result)), file=f, flush=True)


def read_db(dbfile: str, graph: Any = None, target: str | None = None,
            backend: str | None = None) -> list[dict[str, Any]]:
    """Records of a results database, optionally only those of one graph, target and
    backend (the matching rule of ``cli/query_results.py:43-75``: equal operator
    digest, compiler entries compared as prefixes)."""
    want_op = None
    if graph is not None:
        probe = DBCallback(os.devnull, target or "", 0, "", version="0")
        probe.set_graph(graph)
        assert probe.operator is not None
        want_op = probe.operator[1]
    out = []
    with open(dbfile) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            if want_op is not None and rec["operator"][1] != want_op:
                continue
            if target is not None and rec["compiler"][2] != target:
                continue
            if backend is not None and (len(rec["compiler"]) < 5 or rec["compiler"][4] != backend):
                continue
            out.append(rec)
    return out
