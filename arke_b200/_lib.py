"""ctypes binding of ``libarke_b200.so`` (the C ABI declared in ``include/arke_b200.h``).

There is no fallback: if the shared object is missing or a symbol cannot be resolved the import
of this module raises, and every op raises :class:`ArkeB200Error` when the library reports a
failure.  ``ARKE_B200_SO`` overrides the library path.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
DEFAULT_LIB = PKG_DIR / "libarke_b200.so"

# element type codes (include/arke_b200.h)
BF16, F16, F32, I8, E4M3, I32, I64 = range(7)
QUANT_INT8, QUANT_E4M3 = 0, 1
W_KN, W_NK = 0, 1

ERR_NAMES = {
    0: "OK", -1: "ARG", -2: "DTYPE", -3: "SHAPE", -4: "ALIGN", -5: "CUDA", -6: "WORKSPACE",
    -7: "DEVICE", -8: "KERNEL",
}


class ArkeB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"arke_b200 error {code} ({ERR_NAMES.get(code, '?')}): {message}")
        self.code = code
        self.message = message


class UnsupportedError(ArkeB200Error):
    """The library rejected the dtype / shape / alignment (typed 'unsupported', not a crash)."""


# name -> (restype, argtypes); must list every symbol the public header declares.
SIGNATURES = {
    "arke_b200_version": (c_char_p, []),
    "arke_b200_last_error": (c_char_p, []),
    "arke_b200_kernel_status": (c_int, [c_void_p]),
    "arke_b200_selftest_wait_timeout": (c_int, [c_int64, c_void_p]),
    "arke_b200_selftest_bounds_check": (c_int, [c_void_p]),
    "arke_b200_quantize_per_token": (
        c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int,
                c_int, c_void_p]),
    "arke_b200_dequantize_per_channel": (
        c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "arke_b200_rmsnorm": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p,
                c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p]),
    "arke_b200_set_option": (c_int, [c_char_p, c_int64]),
    "arke_b200_get_option": (c_int64, [c_char_p]),
    "arke_b200_matmul_tn": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                c_int64, c_void_p]),
    "arke_b200_fused_linear_ce_backward_workspace": (c_size_t, [c_int64, c_int64]),
    "arke_b200_fused_linear_ce_backward": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "arke_b200_rope": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "arke_b200_qkv_rope_split": (
        c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                c_int64, c_int64, c_int64, c_void_p]),
    "arke_b200_selftest_quant_division": (c_int, [c_int, c_int, c_void_p, c_void_p]),
    "arke_b200_silu_and_mul": (
        c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                c_void_p, c_void_p]),
    "arke_b200_quant_gemm": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64,
                c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p]),
    "arke_b200_matmul": (
        c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int64, c_int64, c_int64,
                c_void_p, c_int64, c_void_p]),
    "arke_b200_gqa_fwd": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                c_int64, c_int64, c_int64, c_int64, c_int, c_float, c_void_p]),
    "arke_b200_fused_linear_ce_workspace": (c_size_t, [c_int64, c_int64, c_int64]),
    "arke_b200_fused_linear_ce": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "arke_b200_fused_linear_ce_static": (
        c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                c_void_p, c_void_p, c_void_p, c_void_p]),
    "arke_b200_ce_combine": (
        c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
}


def lib_path() -> Path:
    return Path(os.environ.get("ARKE_B200_SO", str(DEFAULT_LIB)))


def _load() -> ctypes.CDLL:
    path = lib_path()
    if not path.exists():
        raise ImportError(
            f"arke_b200: kernel library {path} not found; build it with `python -m arke_b200.build` "
            "(there is no CPU or eager fallback)")
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing: fail loudly
        fn.restype = res
        fn.argtypes = args
    return lib


LIB = _load()


def last_error() -> str:
    return LIB.arke_b200_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Raise on a non-zero status from the library."""
    if rc == 0:
        return
    msg = last_error()
    if rc in (-2, -3, -4):
        raise UnsupportedError(rc, msg)
    raise ArkeB200Error(rc, msg)


def version() -> str:
    return LIB.arke_b200_version().decode()
