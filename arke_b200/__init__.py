"""arke_b200 — B200 (sm_100a) execution backend for the data-parallel hot path of Arke's op
registry: per-token quantisation, W8A8/FP8 GEMM, packed SwiGLU with FP8 re-quantisation, causal
GQA flash-attention forward and fused linear + cross-entropy.

Importing the package loads ``libarke_b200.so`` (built by ``python -m arke_b200.build``); a missing
library is an ImportError — there is no CPU, eager or Triton fallback.
"""
from . import _lib  # noqa: F401  (loads the kernel library, raises if absent)
from . import ops  # noqa: F401
from ._lib import ArkeB200Error, UnsupportedError, version  # noqa: F401

__all__ = ["ops", "ArkeB200Error", "UnsupportedError", "version"]
