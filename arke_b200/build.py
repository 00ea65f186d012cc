"""Ahead-of-time build of the sm_100a kernel library (``libarke_b200.so``) with nvcc.

The shared object is written next to this file so it is found in-tree; nothing is JIT-compiled
at import time and nothing is installed into site-packages.  ``python -m arke_b200.build``
rebuilds out-of-date objects; ``--force`` rebuilds everything; ``--verbose`` prints the ptxas
register / shared-memory report.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "libarke_b200.so"

SOURCES = ["capi.cu", "rowops.cu", "rope.cu", "gemm.cu", "flce.cu", "flce_bwd.cu", "attention.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("ARKE_B200_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set ARKE_B200_NVCC)")
    return cand


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=None, out: Path | None = None) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libarke_b200.so``; returns its path.

    ``extra_flags`` (or ``ARKE_B200_NVCC_FLAGS``) are appended to the nvcc command line and ``out``
    names an alternative shared object (select it at run time with ``ARKE_B200_SO``): together
    they build tuning variants next to the default library without touching it.
    """
    nvcc = _nvcc()
    extra = list(extra_flags or []) + os.environ.get("ARKE_B200_NVCC_FLAGS", "").split()
    global OBJ_DIR, LIB_PATH
    obj_dir, lib_path = OBJ_DIR, LIB_PATH
    if out is not None:
        lib_path = Path(out).resolve()
        obj_dir = OBJ_DIR / lib_path.stem
    # objects are reused only when they were compiled with the same extra flags
    obj_dir.mkdir(parents=True, exist_ok=True)
    stamp = obj_dir / "flags.txt"
    if not stamp.exists() or stamp.read_text() != " ".join(extra):
        force = True
    lib = _build(nvcc, extra, obj_dir, lib_path, force, verbose)
    stamp.write_text(" ".join(extra))
    return lib


def _build(nvcc, extra, OBJ_DIR, LIB_PATH, force, verbose) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "arke_b200.h"]
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers, Path(__file__)]):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, p in ex.map(run, jobs):
            if verbose or p.returncode != 0:
                sys.stderr.write(p.stdout + p.stderr)
            if p.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-cudart", "static",
               "-Xlinker", "--no-undefined"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link of libarke_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--out", default=None, help="write the library to this path instead (tuning variants)")
    ap.add_argument("--flag", action="append", default=[], help="extra nvcc flag, e.g. --flag=-DARKE_ATT_EMU_MASK=7")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, extra_flags=a.flag, out=Path(a.out) if a.out else None))
