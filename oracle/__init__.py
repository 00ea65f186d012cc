"""Test infrastructure (checker side only): the CPU restatement in ``oracle.ops`` and, when it
has been staged by ``oracle/make_ref.py``, the reference's own Python package under
``oracle/_ref``.  The product package ``arke_b200`` never imports anything from here."""
from __future__ import annotations

import os
import sys
from pathlib import Path
from typing import Optional

_HERE = Path(__file__).resolve().parent


def ref_path() -> Optional[Path]:
    """Folder holding an importable copy of the reference (``arke/``, ``benchmarks/``), or None.

    ``ARKE_REFERENCE_DIR`` (a full checkout) wins; otherwise the staged copy ``oracle/_ref``."""
    env = os.environ.get("ARKE_REFERENCE_DIR")
    for cand in ([Path(env)] if env else []) + [_HERE / "_ref"]:
        if (cand / "arke" / "ir" / "ops" / "interpreter.py").is_file():
            return cand
    return None


def use_reference() -> Optional[Path]:
    """Put the reference on ``sys.path`` (once) and return its folder; None if it is absent."""
    path = ref_path()
    if path is None:
        return None
    sys.dont_write_bytecode = True
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))
    return path
