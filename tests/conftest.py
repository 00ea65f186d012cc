"""pytest configuration: the ``gpu`` marker (tests that need a B200) and shared helpers."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))

GOLDEN = ROOT / "tests" / "golden"

import oracle  # noqa: E402  (test infrastructure)

# The reference's Python package, when it has been staged beside the oracle (oracle/make_ref.py),
# is importable in every test: arke_b200 then subclasses the reference's own ABC / dataclasses and
# the driver tests can import ``arke`` and ``benchmarks``.  Absent -> those tests skip.
REFERENCE = oracle.use_reference()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    return np.load(GOLDEN / name)


def from_bits(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(arr)).view(dtype)
