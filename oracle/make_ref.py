"""Test infrastructure: stage the reference checkout (pure Python) next to the oracle.

The reference's own drivers — ``benchmarks.bench_l1.run_op``, ``benchmarks.bench_l2``,
``arke.agent.backends.run_backend``, the façade tools of ``arke.agent.tools`` — are what the
parity tests point at the B200 backend.  They live in the reference checkout, which is not a
dependency of the product package and is not part of this repository's history.  This recipe
copies the importable part of a checkout (``arke/``, the Python files of ``benchmarks/``, the two
markdown tables its registries parse, the example operators) into ``oracle/_ref/``, a git-ignored
folder beside the oracle, so that a test host without the checkout can still import it.

Usage::

    python oracle/make_ref.py [--src <reference checkout>] [--dst oracle/_ref]

Nothing under ``arke_b200/`` imports ``oracle`` or ``oracle/_ref``; only ``tests/`` and
``bench.py --impl reference`` put the folder on ``sys.path`` (``oracle.ref_path()``).
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_DST = HERE / "_ref"
# default source: ARKE_REFERENCE_DIR, else a checkout named "reference" beside this repository
DEFAULT_SRC = os.environ.get("ARKE_REFERENCE_DIR", str(HERE.parent.parent / "reference"))

# (sub-tree, predicate on the relative path) — what the drivers import or parse at run time
_KEEP_SUFFIX = {".py", ".j2", ".lark", ".toml", ".ak", ".yaml", ".yml"}
_SKIP_DIRS = {"__pycache__", "results", "probes", ".git"}


def _want(rel: Path) -> bool:
    parts = set(rel.parts)
    if parts & _SKIP_DIRS or any(p.startswith("results_") for p in rel.parts):
        return False
    return rel.suffix in _KEEP_SUFFIX


def stage(src: Path, dst: Path) -> dict:
    """Copy the importable part of ``src`` into ``dst`` (replacing it).  Returns counts."""
    src, dst = Path(src), Path(dst)
    if not (src / "arke" / "ir" / "ops" / "interpreter.py").is_file():
        raise FileNotFoundError(f"{src} is not a reference checkout (arke/ir/ops/interpreter.py missing)")
    tmp = dst.with_name(dst.name + ".tmp")
    if tmp.exists():
        shutil.rmtree(tmp)
    n_files = n_bytes = 0
    for top in ("arke", "benchmarks", "examples"):
        for path in sorted((src / top).rglob("*")):
            if not path.is_file():
                continue
            rel = path.relative_to(src)
            if not _want(rel):
                continue
            out = tmp / rel
            out.parent.mkdir(parents=True, exist_ok=True)
            shutil.copyfile(path, out)
            n_files += 1
            n_bytes += path.stat().st_size
    for rel in ("docs/benchmark/benchmark-shapes.md", "docs/benchmark/benchmark-ops.md"):
        if (src / rel).is_file():
            (tmp / rel).parent.mkdir(parents=True, exist_ok=True)
            shutil.copyfile(src / rel, tmp / rel)
            n_files += 1
            n_bytes += (src / rel).stat().st_size
    (tmp / "STAGED_FROM").write_text(f"{src}\n")
    if dst.exists():
        shutil.rmtree(dst)
    tmp.rename(dst)
    return {"files": n_files, "bytes": n_bytes, "dst": str(dst)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--src", default=DEFAULT_SRC)
    ap.add_argument("--dst", default=str(DEFAULT_DST))
    args = ap.parse_args(argv)
    info = stage(Path(args.src), Path(args.dst))
    print(f"staged {info['files']} files ({info['bytes'] / 1e6:.1f} MB) into {info['dst']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
