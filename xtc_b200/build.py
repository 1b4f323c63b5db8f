"""Build recipe of libxtc_cuda.so (the C-ABI library declared in include/xtc_cuda.h).

The library is compiled in-tree with nvcc for sm_100a only and lands in
``xtc_b200/lib/``.  ``python -m xtc_b200.build`` rebuilds it; ``build()`` is a
no-op when the library is newer than every source.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libxtc_cuda.so"
# GPU hardware counters (CUPTI range profiler): a library of its own, so that the kernel
# library does not depend on CUPTI (include/xtc_cuda_counters.h)
COUNTERS_SRC = CSRC_DIR / "counters" / "cupti_counters.cpp"
COUNTERS_LIB_PATH = LIB_DIR / "libxtc_cuda_counters.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for cand in (
        os.environ.get("XTC_CUDA_NVCC"),
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set XTC_CUDA_NVCC)")


def sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def _deps() -> list[Path]:
    return sources() + sorted(CSRC_DIR.glob("*.cuh")) + sorted(INCLUDE_DIR.glob("*.h"))


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in _deps())


def build_counters(force: bool = False) -> Path | None:
    """Compile the CUPTI counters library.  Returns None (with a note on stderr) when this
    CUDA installation ships no CUPTI range-profiler headers; counters are then unavailable
    and the evaluator says so."""
    nvcc = find_nvcc()
    cuda_root = Path(nvcc).resolve().parent.parent
    include = next((d for d in (cuda_root / "include", cuda_root / "extras" / "CUPTI" / "include")
                    if (d / "cupti_range_profiler.h").exists()), None)
    libdir = next((d for d in (cuda_root / "lib64", cuda_root / "extras" / "CUPTI" / "lib64")
                   if (d / "libcupti.so").exists()), None)
    if include is None or libdir is None:
        sys.stderr.write("CUPTI range profiler not found: libxtc_cuda_counters.so not built\n")
        return None
    deps = [COUNTERS_SRC, INCLUDE_DIR / "xtc_cuda_counters.h"]
    if (not force and COUNTERS_LIB_PATH.exists()
            and COUNTERS_LIB_PATH.stat().st_mtime > max(p.stat().st_mtime for p in deps)):
        return COUNTERS_LIB_PATH
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, "-shared", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-I", str(include),
           "-I", str(cuda_root / "include"), str(COUNTERS_SRC), "-o", str(COUNTERS_LIB_PATH),
           f"-L{libdir}", "-lcupti", "-ldl", "-Xlinker", f"-rpath={libdir}", "--cudart", "none"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"building libxtc_cuda_counters.so failed:\n{proc.stdout}{proc.stderr}")
    return COUNTERS_LIB_PATH


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile every .cu under csrc/ into objects (in parallel) and link the .so."""
    build_counters(force)
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(parents=True, exist_ok=True)
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    procs = []
    objs = []
    deps_mtime = max(
        p.stat().st_mtime
        for p in sorted(CSRC_DIR.glob("*.cuh")) + sorted(INCLUDE_DIR.glob("*.h"))
    )
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        if (
            not force
            and obj.exists()
            and obj.stat().st_mtime > max(src.stat().st_mtime, deps_mtime)
        ):
            continue
        cmd = [nvcc, *flags, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        text = out.decode(errors="replace")
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src.name}:\n{text}\n")
        elif verbose or text.strip():
            sys.stderr.write(text)
    if failed:
        raise RuntimeError("building libxtc_cuda.so failed")
    link = [
        nvcc,
        "-shared",
        "-gencode",
        "arch=compute_100a,code=sm_100a",
        "-o",
        str(LIB_PATH),
        *[str(o) for o in objs],
    ]
    subprocess.run(link, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
