"""CPU: the C-ABI library loads and exports every symbol the public header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def header_symbols():
    text = (ROOT / "include" / "arke_b200.h").read_text()
    return sorted(set(re.findall(r"ARKE_B200_API[^;]*?\b(arke_b200_\w+)\s*\(", text)))


def test_header_declares_symbols():
    syms = header_symbols()
    assert "arke_b200_quantize_per_token" in syms and "arke_b200_gqa_fwd" in syms
    assert len(syms) >= 10


def test_library_exports_every_declared_symbol():
    from arke_b200 import _lib
    lib = ctypes.CDLL(str(_lib.lib_path()))
    for s in header_symbols():
        assert hasattr(lib, s), f"{s} declared in include/arke_b200.h but not exported"
    assert set(header_symbols()) == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_error_string_without_gpu():
    from arke_b200 import _lib
    assert _lib.version().startswith("arke_b200")
    assert isinstance(_lib.last_error(), str)


def test_cpu_tensors_are_rejected_not_silently_computed():
    import torch
    from arke_b200 import ops, _lib
    with pytest.raises(_lib.ArkeB200Error):
        ops.quantize_per_token(torch.randn(4, 64).bfloat16())
    with pytest.raises(_lib.ArkeB200Error):
        ops.silu_and_mul(torch.randn(4, 64).bfloat16())
