"""arke_b200 — B200 (sm_100a) execution backend for the data-parallel hot path of Arke's op
registry: per-token quantisation, W8A8/FP8 GEMM, packed SwiGLU with FP8 re-quantisation, causal
GQA flash-attention forward and fused linear + cross-entropy.

``arke_b200.ops`` (and everything built on it) loads ``libarke_b200.so``, which
``python -m arke_b200.build`` compiles in-tree; a missing library or symbol is an ImportError —
there is no CPU, eager or Triton fallback.  Sub-modules are imported on first use so that the
build module itself can run before the library exists.
"""
from __future__ import annotations

import importlib

_SUBMODULES = ("_lib", "ops", "backend", "runner", "bridge", "install", "sharding", "hardware", "build")
__all__ = ["ops", "backend", "runner", "bridge", "install", "sharding", "hardware", "version",
           "ArkeB200Error", "UnsupportedError"]


def __getattr__(name: str):
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    if name in ("ArkeB200Error", "UnsupportedError", "version"):
        return getattr(importlib.import_module(f"{__name__}._lib"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
