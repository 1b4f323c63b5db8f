"""Compiler of the CUDA backend: schedule -> plan -> module on disk.

Takes the place of ``backends/mlir/MlirCompiler.py:36-110`` and of the
llvmir target's four-subprocess toolchain (``MlirLLVMTarget.py:62-166``).
Nothing is generated per schedule except a table: the kernels are prebuilt in
``libxtc_cuda.so`` and a schedule only selects their parameters, so compiling
costs milliseconds instead of the reference's ~3 s per sample.

With ``shared_lib=True`` a small payload library is written to
``<dump_file>.so``.  It exports ``void <graph.name>(void* in0.., void* out0..)``
taking HOST pointers -- the signature of the reference's own payloads
(``MlirGraphBackend.py:144-148``) -- and forwards to ``xtc_cuda_plan_run_host``.
"""

from __future__ import annotations

import json
import subprocess
import tempfile
from pathlib import Path
from typing import Any

from ... import capi
from .lowering import Plan, lower
from .module import CudaModule
from .scheduler import CudaSchedule

# Compiler options of other backends that the search driver always passes
# (search/explore.py:365-389, backends/mlir/MlirConfig.py:12-36); accepted, unused.
_TOLERATED = {"bare_ptr", "debug", "print_source_ir", "print_transformed_ir",
              "print_bufferization_ir", "print_lowered_ir", "print_assembly", "color",
              "to_disassemble", "save_temps", "save_temps_dir", "target", "executable", "arch",
              "cpu", "selected_device", "concluding_passes", "always_vectorize", "no_alias",
              "vectors_size", "mlir_extensions"}


class CudaCompiler:
    def __init__(self, backend: Any, shared_lib: bool = True, dump_file: str | None = None,
                 precision: str = "tf32", fuse_transpose: bool | None = None,
                 print_plan: bool = False, **kwargs: Any) -> None:
        unknown = set(kwargs) - _TOLERATED
        assert not unknown, f"unknown compiler options: {sorted(unknown)}"
        self._backend = backend
        self.shared_lib = shared_lib
        self.dump_file = dump_file
        self.precision = precision
        self.fuse_transpose = fuse_transpose
        self.print_plan = print_plan or bool(kwargs.get("print_source_ir"))
        self.options = kwargs

    @property
    def backend(self) -> Any:
        return self._backend

    def lower(self, schedule: CudaSchedule | None) -> Plan:
        configs = schedule.node_configs() if schedule is not None else {}
        fuse: Any = self.fuse_transpose
        if fuse is None:
            fuse = schedule.fused_transposes() if schedule is not None else False
        return lower(self._backend.graph, configs, fuse, self.precision)

    def compile(self, schedule: CudaSchedule | None = None) -> CudaModule:
        plan = self.lower(schedule)
        if self.print_plan:
            print(describe(plan))
        dump_file = self.dump_file
        if dump_file is None:
            tmp = tempfile.mkdtemp(prefix="xtc_cuda_")
            dump_file = str(Path(tmp) / f"payload_{plan.name}")
        Path(dump_file).parent.mkdir(parents=True, exist_ok=True)
        file_name = f"{dump_file}.so" if self.shared_lib else f"{dump_file}.plan.json"
        if self.shared_lib:
            write_payload_library(plan, file_name)
        else:
            Path(file_name).write_text(json.dumps(plan_to_json(plan), indent=1))
        return CudaModule(plan.name, plan.name, file_name, "shlib" if self.shared_lib else "plan",
                          plan=plan, graph=self._backend.graph, backend=self._backend)


def describe(plan: Plan) -> str:
    lines = [f"plan {plan.name}: {plan.n_inputs} inputs, {plan.n_outputs} outputs, "
             f"{len(plan.slot_bytes)} slots"]
    for s in plan.steps:
        fused = f" fused={list(s.fused)}" if s.fused else ""
        lines.append(f"  {s.kind:9s} {s.node}: in=({s.in0},{s.in1}) out={s.out} dims={s.dims} "
                     f"flags={s.flags} cfg={s.config}{fused}")
    return "\n".join(lines)


def plan_to_json(plan: Plan) -> dict[str, Any]:
    return {
        "name": plan.name, "n_inputs": plan.n_inputs, "n_outputs": plan.n_outputs,
        "slot_bytes": plan.slot_bytes,
        "steps": [{k: getattr(s, k) for k in ("kind", "node", "in0", "in1", "out", "flags",
                                                "relu_threshold", "pad_value", "ndim", "dims", "aux0",
                                                "aux1", "config", "fused")} for s in plan.steps],
    }


def _c_array(values, n: int) -> str:
    vals = list(values) + [0] * (n - len(values))
    return "{" + ", ".join(str(int(v)) for v in vals) + "}"


def payload_source(plan: Plan) -> str:
    """C source of the per-module payload library."""
    n_io = plan.n_inputs + plan.n_outputs
    steps = []
    for s in plan.steps:
        cfg = s.to_c().cfg
        steps.append(
            "  {%d, %d, %d, %d, %d, %d, (float)%r, (float)%r, %s, %s, %s, {%d, %d, %d, %d, %d, %d, %d, %d}}"
            % (s.KIND_CODES[s.kind], s.in0, s.in1, s.out, s.flags, s.ndim, float(s.relu_threshold),
               float(s.pad_value), _c_array(s.dims, capi.MAX_DIMS), _c_array(s.aux0, capi.MAX_DIMS),
               _c_array(s.aux1, capi.MAX_DIMS), cfg.tile_m, cfg.tile_n, cfg.tile_k, cfg.stages,
               cfg.precision, cfg.epilogue, cfg.variant, cfg.split_k))
    params = ", ".join(f"void* a{i}" for i in range(n_io))
    args = ", ".join(f"a{i}" for i in range(n_io))
    name = "".join(c if c.isalnum() or c == "_" else "_" for c in plan.name)
    return f"""/* generated by xtc_b200.backends.cuda: payload of graph {plan.name} */
#include <pthread.h>
#include <stdio.h>
#include "xtc_cuda.h"
static const xtc_cuda_step steps[] = {{
{(',' + chr(10)).join(steps)}
}};
static const size_t slot_bytes[] = {_c_array(plan.slot_bytes, len(plan.slot_bytes))};
static xtc_cuda_plan* plan;
static pthread_once_t plan_once = PTHREAD_ONCE_INIT;
static pthread_mutex_t run_lock = PTHREAD_MUTEX_INITIALIZER;
static void create_plan(void) {{ /* once, whichever thread calls first */
  if (xtc_cuda_plan_create(&plan, steps, {len(plan.steps)}, {plan.n_inputs}, {plan.n_outputs},
                           {len(plan.slot_bytes)}, slot_bytes) != XTC_CUDA_OK) {{
    fprintf(stderr, "{name}: %s\\n", xtc_cuda_last_error());
    plan = NULL;
  }}
}}
void {name}({params}) {{
  void* io[] = {{{args}}};
  pthread_once(&plan_once, create_plan);
  if (!plan) return;
  pthread_mutex_lock(&run_lock); /* one plan, one set of staging buffers */
  if (xtc_cuda_plan_run_host(plan, io) != XTC_CUDA_OK)
    fprintf(stderr, "{name}: %s\\n", xtc_cuda_last_error());
  pthread_mutex_unlock(&run_lock);
}}
"""


def write_payload_library(plan: Plan, file_name: str) -> None:
    lib = capi.LIB_PATH
    if not lib.exists():
        raise RuntimeError(f"{lib} is missing: build it with `python -m xtc_b200.build`")
    include = Path(__file__).resolve().parents[3] / "include"
    src = Path(file_name).with_suffix(".c")
    src.write_text(payload_source(plan))
    cmd = ["cc", "-shared", "-fPIC", "-O1", "-pthread", "-I", str(include), str(src), "-o", file_name,
           f"-L{lib.parent}", "-lxtc_cuda", f"-Wl,-rpath,{lib.parent}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    src.unlink(missing_ok=True)
    if proc.returncode != 0:
        raise RuntimeError(f"payload library build failed: {proc.stderr}")
