"""Python front door of the B200 kernels: torch tensors in, torch tensors out.

Each function validates its arguments, allocates the outputs with ``torch.empty`` on the caller's
device, and enqueues one C-ABI call on the caller's current CUDA stream.  PyTorch is used for
device memory and streams only; there is no eager or CPU fallback — a CPU tensor, a missing
library or an unsupported dtype raises.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import LIB, check

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}
FP8 = torch.float8_e4m3fn


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: torch.Tensor) -> int:
    """Handle of the caller's current CUDA stream on ``t``'s device (the raw-handle query when
    this torch has it: building a ``torch.cuda.Stream`` object costs microseconds per call)."""
    if _raw_stream is not None:
        idx = t.device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(t.device).cuda_stream


class _dev:
    """``with _dev(tensor.device):`` — the library call runs with that device current.  Unlike
    ``torch.cuda.device`` it does nothing when the device is current already (the usual case:
    one process per GPU), which keeps the per-call host overhead low."""
    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and self.idx != cur:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _need_cuda(*ts: torch.Tensor) -> None:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"expected torch.Tensor, got {type(t).__name__}")
        if not t.is_cuda:
            raise _lib.ArkeB200Error(-7, "arke_b200 ops run on CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise _lib.ArkeB200Error(-1, "all tensors must be on the same device")


def _dt(t: torch.Tensor, allowed=(torch.bfloat16, torch.float16, torch.float32)) -> int:
    if t.dtype not in allowed:
        raise _lib.UnsupportedError(-2, f"unsupported dtype {t.dtype}; expected one of {allowed}")
    return _DT[t.dtype]


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    """View as [rows, cols] with unit inner stride (copies only if the layout forces it)."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1:
        t2 = t2.contiguous()
    return t2


# ---------------------------------------------------------------------------------------------
# quantize_per_token
# ---------------------------------------------------------------------------------------------
def quantize_per_token(x: torch.Tensor, out_dtype: str = "int8", formula: str = "interp",
                       out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric quantisation → ``(q, scale)``.

    ``out_dtype``: ``"int8"`` (scale = amax/127) or ``"fp8"`` (e4m3, scale = amax/448).
    ``formula``: ``"interp"`` follows ``ref_quantize_per_token`` evaluated on ``x.float()``
    (arke/ir/ops/reference_impls.py:215-218); ``"bench_l1"`` follows the benchmark driver's golden
    (benchmarks/bench_l1.py:443-448) and returns ``amax`` as the scale.
    ``out=(q, scale)`` reuses caller-owned contiguous buffers instead of allocating.
    """
    _need_cuda(x)
    if x.dim() < 1:
        raise _lib.UnsupportedError(-3, "quantize_per_token needs at least one dimension")
    x2 = _rows2d(x)
    M, N = x2.shape
    kind = {"int8": _lib.QUANT_INT8, "fp8": _lib.QUANT_E4M3}[out_dtype]
    form = {"interp": 0, "bench_l1": 1}[formula]
    qdt = torch.int8 if kind == 0 else FP8
    if out is not None:
        q, scale = out
        if (q.dtype != qdt or q.numel() != M * N or not q.is_contiguous() or scale.dtype != torch.float32
                or scale.numel() != M or not scale.is_contiguous() or q.device != x.device):
            raise _lib.UnsupportedError(-3, "quantize_per_token: out buffers have the wrong dtype/shape/device")
    else:
        q = torch.empty((M, N), dtype=qdt, device=x.device)
        scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    with _dev(x.device):
        check(LIB.arke_b200_quantize_per_token(x2.data_ptr(), _dt(x2), M, N, x2.stride(0) if M > 0 else N,
                                               q.data_ptr(), N, scale.data_ptr(), kind, form,
                                               _stream(x)))
    return q.reshape(x.shape), scale.reshape(x.shape[:-1])


# ---------------------------------------------------------------------------------------------
# silu_and_mul (+ fused FP8 re-quantisation)
# ---------------------------------------------------------------------------------------------
def silu_and_mul(x: torch.Tensor, quantize_fp8: bool = False, return_y: bool = True):
    """``silu(x[..., :N]) * x[..., N:]`` on a packed gate|up tensor
    (arke/ir/ops/reference_impls.py:167-171).

    Returns ``y`` when ``quantize_fp8`` is false; ``(y, yq, scale)`` when both are requested;
    ``(yq, scale)`` when ``return_y`` is false.  ``yq`` is e4m3 with ``scale = amax|y|/448`` per row.
    """
    _need_cuda(x)
    if x.shape[-1] % 2 != 0:
        raise _lib.UnsupportedError(-3, "silu_and_mul needs an even last dimension (gate|up packed)")
    if not quantize_fp8 and not return_y:
        raise ValueError("nothing to compute: request y and/or the fp8 output")
    x2 = _rows2d(x)
    M, N2 = x2.shape
    N = N2 // 2
    out_shape = (*x.shape[:-1], N)
    y = torch.empty((M, N), dtype=x.dtype, device=x.device) if return_y else None
    yq = torch.empty((M, N), dtype=FP8, device=x.device) if quantize_fp8 else None
    sc = torch.empty((M,), dtype=torch.float32, device=x.device) if quantize_fp8 else None
    with _dev(x.device):
        check(LIB.arke_b200_silu_and_mul(x2.data_ptr(), _dt(x2), M, N, x2.stride(0) if M > 0 else N2,
                                         y.data_ptr() if y is not None else None, N,
                                         yq.data_ptr() if yq is not None else None, N,
                                         sc.data_ptr() if sc is not None else None, _stream(x)))
    if not quantize_fp8:
        return y.reshape(out_shape)
    if return_y:
        return y.reshape(out_shape), yq.reshape(out_shape), sc.reshape(x.shape[:-1])
    return yq.reshape(out_shape), sc.reshape(x.shape[:-1])


def dequantize_per_channel(x_int8: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
                           out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``(x_int8.float() - zero_point.float()) * scale`` per output channel
    (``ref_dequantize_per_channel``, arke/ir/ops/reference_impls.py:220-224)."""
    _need_cuda(x_int8, scale, zero_point)
    if x_int8.dtype != torch.int8 or x_int8.dim() != 2:
        raise _lib.UnsupportedError(-2, "dequantize_per_channel: x must be a 2-D int8 tensor")
    M, N = x_int8.shape
    if scale.numel() != N or (zero_point is not None and zero_point.numel() != N):
        raise _lib.UnsupportedError(-3, "dequantize_per_channel: scale / zero_point must have N entries")
    if x_int8.stride(1) != 1:
        x_int8 = x_int8.contiguous()
    scale = scale.to(torch.float32).contiguous()
    zp = zero_point.to(torch.float32).contiguous() if zero_point is not None else None
    y = torch.empty((M, N), dtype=out_dtype, device=x_int8.device)
    with _dev(x_int8.device):
        check(LIB.arke_b200_dequantize_per_channel(x_int8.data_ptr(), M, N, x_int8.stride(0) if M > 0 else N,
                                                   scale.data_ptr(), zp.data_ptr() if zp is not None else None,
                                                   y.data_ptr(), _dt(y), N, _stream(x_int8)))
    return y


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
            quantize: Optional[str] = None, return_y: bool = True):
    """``(h / sqrt(mean(h**2) + eps) * w)`` with ``h = x (+ residual)``, fp32 math, result in the
    input dtype (``ref_rmsnorm`` arke/ir/ops/reference_impls.py:85-90, ``ref_rmsnorm_residual``).

    ``quantize="int8"`` / ``"fp8"`` additionally returns the per-token quantisation of the rounded
    result — bit-identical to ``quantize_per_token(y)`` — without writing/re-reading ``y``:
    returns ``y``; ``(y, q, scale)``; or ``(q, scale)`` with ``return_y=False``.
    """
    _need_cuda(x, w, residual)
    if w.dtype != x.dtype or (residual is not None and residual.dtype != x.dtype):
        raise _lib.UnsupportedError(-2, "rmsnorm: x, w and residual must share one dtype")
    if w.dim() != 1 or w.shape[0] != x.shape[-1] or (residual is not None and residual.shape != x.shape):
        raise _lib.UnsupportedError(-3, "rmsnorm: w must be [N] and residual must match x")
    if quantize is None and not return_y:
        raise ValueError("nothing to compute")
    x2 = _rows2d(x)
    r2 = _rows2d(residual) if residual is not None else None
    w = w.contiguous()
    M, N = x2.shape
    y = torch.empty((M, N), dtype=x.dtype, device=x.device) if return_y else None
    q = sc = None
    kind = 0
    if quantize is not None:
        kind = {"int8": _lib.QUANT_INT8, "fp8": _lib.QUANT_E4M3}[quantize]
        q = torch.empty((M, N), dtype=torch.int8 if kind == 0 else FP8, device=x.device)
        sc = torch.empty((M,), dtype=torch.float32, device=x.device)
    with _dev(x.device):
        check(LIB.arke_b200_rmsnorm(x2.data_ptr(), r2.data_ptr() if r2 is not None else None, w.data_ptr(), _dt(x2),
                                    M, N, x2.stride(0) if M > 0 else N, r2.stride(0) if r2 is not None and M > 0 else N,
                                    float(eps), y.data_ptr() if y is not None else None, N,
                                    q.data_ptr() if q is not None else None, N,
                                    sc.data_ptr() if sc is not None else None, kind, _stream(x)))
    if quantize is None:
        return y.reshape(x.shape)
    if return_y:
        return y.reshape(x.shape), q.reshape(x.shape), sc.reshape(x.shape[:-1])
    return q.reshape(x.shape), sc.reshape(x.shape[:-1])


class options:
    """Context manager for the per-thread tuning options of the library (``arke_b200_set_option``):
    ``with ops.options(gemm_tile_m=256): ...``; the previous values are restored on exit.
    Results do not depend on them."""

    def __init__(self, **kv: int):
        self.kv = {k: int(v) for k, v in kv.items()}
        self.old: dict = {}

    def __enter__(self):
        for k, v in self.kv.items():
            self.old[k] = int(LIB.arke_b200_get_option(k.encode()))
            check(LIB.arke_b200_set_option(k.encode(), v))
        return self

    def __exit__(self, *exc):
        for k, v in self.old.items():
            LIB.arke_b200_set_option(k.encode(), max(v, 0))
        return False


def _check_rope_tables(name: str, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, S: int, D: int):
    if cos.dtype != x.dtype or sin.dtype != x.dtype:
        raise _lib.UnsupportedError(-2, f"{name}: cos and sin must have the dtype of x")
    if D % 2 or tuple(cos.shape) != (S, D // 2) or tuple(sin.shape) != (S, D // 2):
        raise _lib.UnsupportedError(-3, f"{name}: cos and sin must be [S, D/2] = [{S}, {D // 2}] and D even")


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding, rotate-half form: ``x [B,H,S,D]`` (or ``[H,S,D]`` / ``[S,D]``), ``cos`` /
    ``sin`` ``[S, D/2]`` → same shape and dtype, bit-identical to the interpreter's ``ref_rope``
    (arke/ir/ops/reference_impls.py:197-206)."""
    _need_cuda(x, cos, sin)
    if x.dim() < 2 or x.dim() > 4:
        raise _lib.UnsupportedError(-3, "rope: x must be [B,H,S,D], [H,S,D] or [S,D]")
    S, D = x.shape[-2], x.shape[-1]
    _check_rope_tables("rope", x, cos, sin, S, D)
    xc = x.contiguous()
    y = torch.empty_like(xc)
    lead = 1
    for d in x.shape[:-2]:
        lead *= d
    with _dev(x.device):
        check(LIB.arke_b200_rope(xc.data_ptr(), cos.contiguous().data_ptr(), sin.contiguous().data_ptr(), y.data_ptr(),
                                 _dt(xc), lead, 1, S, D, _stream(x)))
    return y


def qkv_rope_split(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, S: int, Hq: int, Hkv: int,
                   D: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Packed projection output ``qkv [B*S, (Hq + 2*Hkv)*D]`` (row stride free) → rotated
    ``q [B,Hq,S,D]``, rotated ``k [B,Hkv,S,D]`` and ``v [B,Hkv,S,D]`` in one pass."""
    _need_cuda(qkv, cos, sin)
    W = (Hq + 2 * Hkv) * D
    if qkv.dim() != 2 or qkv.shape[0] != B * S or qkv.shape[1] != W or (qkv.shape[0] > 1 and qkv.stride(1) != 1):
        raise _lib.UnsupportedError(-3, f"qkv_rope_split: qkv must be [B*S, (Hq + 2*Hkv)*D] = [{B * S}, {W}] with unit column stride")
    _check_rope_tables("qkv_rope_split", qkv, cos, sin, S, D)
    q = torch.empty((B, Hq, S, D), dtype=qkv.dtype, device=qkv.device)
    k = torch.empty((B, Hkv, S, D), dtype=qkv.dtype, device=qkv.device)
    v = torch.empty((B, Hkv, S, D), dtype=qkv.dtype, device=qkv.device)
    with _dev(qkv.device):
        check(LIB.arke_b200_qkv_rope_split(qkv.data_ptr(), qkv.stride(0) if qkv.shape[0] > 1 else W,
                                           cos.contiguous().data_ptr(), sin.contiguous().data_ptr(),
                                           q.data_ptr(), k.data_ptr(), v.data_ptr(), _dt(qkv), B, S, Hq, Hkv, D,
                                           _stream(qkv)))
    return q, k, v


def qkv_rope_attention(x: torch.Tensor, w_qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, S: int,
                       Hq: int, Hkv: int, D: int, causal: bool = True, w_layout: str = "kn",
                       return_lse: bool = False):  # noqa: D401
    """QKV projection → rotary embedding → grouped-query attention: ``x [B*S, hidden]`` times
    ``w_qkv`` (``[hidden, (Hq+2Hkv)*D]`` for ``w_layout="kn"``, its transpose for ``"nk"``) on the
    tcgen05 GEMM, one :func:`qkv_rope_split` pass, then :func:`gqa_fwd`.  Returns ``O [B,Hq,S,D]``."""
    qkv = matmul(x, w_qkv, b_layout=w_layout)
    q, k, v = qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D)
    return gqa_fwd(q, k, v, causal=causal, return_lse=return_lse)


def swiglu_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packed SwiGLU fused with per-row e4m3 re-quantisation → ``(yq, scale)``."""
    return silu_and_mul(x, quantize_fp8=True, return_y=False)


# ---------------------------------------------------------------------------------------------
# quantised GEMM (W8A8 / FP8) and dense 16-bit GEMM
# ---------------------------------------------------------------------------------------------
def quant_gemm(a: torch.Tensor, sa: Optional[torch.Tensor], w: torch.Tensor,
               sw: Optional[torch.Tensor], out_dtype: Optional[torch.dtype] = torch.bfloat16,
               w_layout: str = "kn", return_acc: bool = False, out: Optional[torch.Tensor] = None):
    """``out_dtype((acc * sa[:, None]) * sw[None, :])`` with ``acc = a @ w`` accumulated exactly
    in int32 (int8 operands) or in fp32 (e4m3 operands).

    ``a`` [M,K]; ``w`` [K,N] for ``w_layout="kn"`` or [N,K] for ``"nk"``.  With ``return_acc`` the
    raw accumulators (int32 / fp32) are returned as well; ``out_dtype=None`` skips Y.
    """
    _need_cuda(a, w, sa, sw)
    if a.dtype != w.dtype or a.dtype not in (torch.int8, FP8):
        raise _lib.UnsupportedError(-2, f"quant_gemm operands must both be int8 or e4m3, got {a.dtype}/{w.dtype}")
    if a.dim() != 2 or w.dim() != 2:
        raise _lib.UnsupportedError(-3, "quant_gemm takes 2-D operands")
    if a.stride(1) != 1:
        a = a.contiguous()
    if w.stride(1) != 1:
        w = w.contiguous()
    M, K = a.shape
    layout = {"kn": _lib.W_KN, "nk": _lib.W_NK}[w_layout]
    N = w.shape[1] if layout == _lib.W_KN else w.shape[0]
    if (w.shape[0] if layout == _lib.W_KN else w.shape[1]) != K:
        raise _lib.UnsupportedError(-3, f"quant_gemm inner dimensions differ: a {tuple(a.shape)}, w {tuple(w.shape)} ({w_layout})")
    for s, n, nm in ((sa, M, "sa"), (sw, N, "sw")):
        if s is not None and (s.dtype != torch.float32 or s.numel() != n or not s.is_contiguous()):
            raise _lib.UnsupportedError(-3, f"{nm} must be a contiguous fp32 vector of length {n}")
    is_i8 = a.dtype == torch.int8
    if out is not None:
        if out.shape != (M, N) or not out.is_contiguous() or out.device != a.device:
            raise _lib.UnsupportedError(-3, "quant_gemm: out must be a contiguous [M,N] tensor on the operands' device")
        y = out
    else:
        y = torch.empty((M, N), dtype=out_dtype, device=a.device) if out_dtype is not None else None
    acc = torch.empty((M, N), dtype=torch.int32 if is_i8 else torch.float32, device=a.device) if return_acc else None
    if y is None and acc is None:
        raise ValueError("nothing to compute: request Y and/or the accumulators")
    with _dev(a.device):
        check(LIB.arke_b200_quant_gemm(
            a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), layout,
            _lib.I8 if is_i8 else _lib.E4M3,
            sa.data_ptr() if sa is not None else None, sw.data_ptr() if sw is not None else None,
            M, N, K, y.data_ptr() if y is not None else None, _dt(y) if y is not None else _lib.BF16, N,
            acc.data_ptr() if acc is not None else None, N, _stream(a)))
    if y is not None and acc is not None:
        return y, acc
    return y if y is not None else acc


def w8a8_gemm(xq, sx, w, sw, out_dtype=torch.bfloat16, w_layout="kn", return_acc=False, out=None):
    """INT8 × INT8 → int32 GEMM with per-token × per-channel dequantisation."""
    if xq.dtype != torch.int8:
        raise _lib.UnsupportedError(-2, "w8a8_gemm needs int8 operands")
    return quant_gemm(xq, sx, w, sw, out_dtype, w_layout, return_acc, out)


def fp8_gemm(xq, sx, w, sw, out_dtype=torch.bfloat16, w_layout="kn", return_acc=False, out=None):
    """e4m3 × e4m3 → fp32 GEMM with per-token × per-channel dequantisation."""
    if xq.dtype != FP8:
        raise _lib.UnsupportedError(-2, "fp8_gemm needs float8_e4m3fn operands")
    return quant_gemm(xq, sx, w, sw, out_dtype, w_layout, return_acc, out)


def matmul(a: torch.Tensor, b: torch.Tensor, b_layout: str = "kn") -> torch.Tensor:
    """Dense GEMM with fp32 accumulation (arke/ir/ops/reference_impls.py:118-119): bf16 / fp16
    operands, or fp32 operands multiplied as TF32 on the tensor cores."""
    _need_cuda(a, b)
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise _lib.UnsupportedError(-2, f"matmul operands must both be bf16, f16 or f32, got {a.dtype}/{b.dtype}")
    if a.dim() != 2 or b.dim() != 2:
        raise _lib.UnsupportedError(-3, "matmul takes 2-D operands")
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    M, K = a.shape
    layout = {"kn": _lib.W_KN, "nk": _lib.W_NK}[b_layout]
    N = b.shape[1] if layout == _lib.W_KN else b.shape[0]
    if (b.shape[0] if layout == _lib.W_KN else b.shape[1]) != K:
        raise _lib.UnsupportedError(-3, "matmul inner dimensions differ")
    if a.dtype == torch.float32 and layout == _lib.W_KN:
        # the TF32 kernel takes K-contiguous operands only: one layout copy of B ([K,N] -> [N,K])
        b = b.t().contiguous()
        layout = _lib.W_NK
    c = torch.empty((M, N), dtype=a.dtype, device=a.device)
    with _dev(a.device):
        check(LIB.arke_b200_matmul(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), layout,
                                   _dt(a), M, N, K, c.data_ptr(), N, _stream(a)))
    return c


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
def gqa_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
            softmax_scale: Optional[float] = None, return_lse: bool = True):
    """Grouped-query flash-attention forward (arke/ir/ops/reference_impls.py:236-244).

    ``q`` [B,Hq,S,D], ``k``/``v`` [B,Hkv,Skv,D] (3-D inputs are read as B=1).  Returns ``(o, lse)``
    with ``lse`` the fp32 natural-log logsumexp of the scaled masked scores, or ``o`` alone.
    """
    _need_cuda(q, k, v)
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise _lib.UnsupportedError(-2, f"gqa_fwd needs bf16/f16 q,k,v of one dtype, got {q.dtype}/{k.dtype}/{v.dtype}")
    squeeze = q.dim() == 3
    if squeeze:
        q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape:
        raise _lib.UnsupportedError(-3, "gqa_fwd takes [B,H,S,D] tensors with k.shape == v.shape")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, Hq, S, D = q.shape
    Bk, Hkv, Skv, Dk = k.shape
    if Bk != B or Dk != D or Hkv == 0 or Hq % Hkv != 0:
        raise _lib.UnsupportedError(-3, f"gqa_fwd shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}")
    o = torch.empty_like(q)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device) if return_lse else None
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    with _dev(q.device):
        check(LIB.arke_b200_gqa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                    lse.data_ptr() if lse is not None else None, _dt(q), B, Hq, Hkv,
                                    S, Skv, D, 1 if causal else 0, scale, _stream(q)))
    if squeeze:
        o = o.squeeze(0)
        lse = lse.squeeze(0) if lse is not None else None
    return (o, lse) if return_lse else o


# ---------------------------------------------------------------------------------------------
# fused linear + cross-entropy
# ---------------------------------------------------------------------------------------------
def fused_linear_ce_workspace_bytes(M: int, V: int, D: int) -> int:
    return int(LIB.arke_b200_fused_linear_ce_workspace(M, V, D))


def fused_linear_ce(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                    ignore_index: int = -100, vocab_offset: int = 0, want_partials: bool = False,
                    workspace: Optional[torch.Tensor] = None):
    """Fused ``cross_entropy(x.float() @ w.float().T, labels)`` that never materialises logits
    (arke/ir/ops/reference_impls.py:211-213).

    Returns ``(loss_tok [M] fp32, mean fp32 scalar)``; with ``want_partials`` returns the per-row
    ``(max, sumexp, target_logit)`` triple [M,3] of this vocabulary slice instead (see
    :mod:`arke_b200.sharding`).
    """
    _need_cuda(x, w, labels)
    if x.dtype not in (torch.bfloat16, torch.float16) or w.dtype != x.dtype:
        raise _lib.UnsupportedError(-2, f"fused_linear_ce needs bf16/f16 x and w of one dtype, got {x.dtype}/{w.dtype}")
    if labels.dtype != torch.int64:
        raise _lib.UnsupportedError(-2, f"fused_linear_ce labels must be int64, got {labels.dtype}")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or labels.shape != (x.shape[0],):
        raise _lib.UnsupportedError(-3, f"fused_linear_ce shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, labels {tuple(labels.shape)}")
    x, w, labels = x.contiguous(), w.contiguous(), labels.contiguous()
    M, D = x.shape
    V = w.shape[0]
    need = fused_linear_ce_workspace_bytes(M, V, D)
    if workspace is None:
        workspace = torch.empty((max(need, 16),), dtype=torch.uint8, device=x.device)
    elif workspace.numel() * workspace.element_size() < need:
        raise _lib.ArkeB200Error(-6, f"workspace too small: {workspace.numel() * workspace.element_size()} < {need}")
    loss = mean = part = None
    if want_partials:
        part = torch.empty((M, 3), dtype=torch.float32, device=x.device)
    else:
        loss = torch.empty((M,), dtype=torch.float32, device=x.device)
        mean = torch.empty((), dtype=torch.float32, device=x.device)
    with _dev(x.device):
        check(LIB.arke_b200_fused_linear_ce(
            x.data_ptr(), w.data_ptr(), labels.data_ptr(), _dt(x), M, V, D, int(vocab_offset),
            int(ignore_index), loss.data_ptr() if loss is not None else None,
            mean.data_ptr() if mean is not None else None,
            part.data_ptr() if part is not None else None, workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _stream(x)))
    return part if want_partials else (loss, mean)


def fused_linear_ce_backward_workspace_bytes(M: int, V: int) -> int:
    return int(LIB.arke_b200_fused_linear_ce_backward_workspace(M, V))


def fused_linear_ce_backward(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, lse: Optional[torch.Tensor] = None,
                             grad=1.0, ignore_index: int = -100, vocab_offset: int = 0,
                             want_dx: bool = True, want_dw: bool = True, workspace: Optional[torch.Tensor] = None,
                             dx_dtype: Optional[torch.dtype] = None):
    """Gradients of the mean loss of :func:`fused_linear_ce` → ``(dx [M,D], dw [V,D])`` in the
    operands' dtype (either may be skipped → ``None``); ``dx_dtype=torch.float32`` returns ``dx``
    unrounded (what a vocabulary-sharded caller sums over ranks).  ``grad`` is the upstream
    gradient: a Python number, or an fp32 CUDA scalar tensor that is read on the device (no
    host synchronisation).  ``lse`` is the per-row natural-log
    logsumexp over the whole vocabulary; when omitted it is taken from a forward pass of this slice
    (``want_partials``), which is only right for an unsharded vocabulary.  The one intermediate is
    the 16-bit logits gradient ``[M,V]`` in ``workspace`` (:func:`fused_linear_ce_backward_workspace_bytes`).
    """
    _need_cuda(x, w, labels)
    if x.dtype not in (torch.bfloat16, torch.float16) or w.dtype != x.dtype:
        raise _lib.UnsupportedError(-2, f"fused_linear_ce_backward needs bf16/f16 x and w of one dtype, got {x.dtype}/{w.dtype}")
    if labels.dtype != torch.int64:
        raise _lib.UnsupportedError(-2, f"fused_linear_ce_backward labels must be int64, got {labels.dtype}")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or labels.shape != (x.shape[0],):
        raise _lib.UnsupportedError(-3, f"fused_linear_ce_backward shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, labels {tuple(labels.shape)}")
    x, w, labels = x.contiguous(), w.contiguous(), labels.contiguous()
    M, D = x.shape
    V = w.shape[0]
    if lse is None:
        if vocab_offset != 0:
            raise ValueError("a vocabulary slice needs the global lse (combine the slices' partials first)")
        part = fused_linear_ce(x, w, labels, ignore_index=ignore_index, want_partials=True)
        lse = part[:, 0] + torch.log(part[:, 1])
    if lse.dtype != torch.float32 or lse.shape != (M,):
        raise _lib.UnsupportedError(-3, "fused_linear_ce_backward: lse must be fp32 [M]")
    lse = lse.contiguous()
    need = fused_linear_ce_backward_workspace_bytes(M, V)
    if workspace is None:
        workspace = torch.empty((max(need, 256),), dtype=torch.uint8, device=x.device)
    elif workspace.numel() * workspace.element_size() < need:
        raise _lib.ArkeB200Error(-6, f"workspace too small: {workspace.numel() * workspace.element_size()} < {need}")
    if dx_dtype not in (None, x.dtype, torch.float32):
        raise _lib.UnsupportedError(-2, f"fused_linear_ce_backward: dx_dtype must be {x.dtype} or float32")
    dxt = dx_dtype or x.dtype
    dx = torch.empty((M, D), dtype=dxt, device=x.device) if want_dx else None
    dw = torch.empty((V, D), dtype=x.dtype, device=x.device) if want_dw else None
    grad_dev = None
    if isinstance(grad, torch.Tensor):
        if not grad.is_cuda or grad.numel() != 1:
            raise ValueError("fused_linear_ce_backward: a tensor grad must be a CUDA scalar")
        grad_dev = grad.detach().reshape(1).to(torch.float32)      # stays on the device
        grad = 1.0
    with _dev(x.device):
        check(LIB.arke_b200_fused_linear_ce_backward(
            x.data_ptr(), w.data_ptr(), labels.data_ptr(), lse.data_ptr(), _dt(x), M, V, D, int(vocab_offset),
            int(ignore_index), float(grad), grad_dev.data_ptr() if grad_dev is not None else None,
            dx.data_ptr() if dx is not None else None, _lib.F32 if dxt == torch.float32 else _dt(x),
            dw.data_ptr() if dw is not None else None, workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _stream(x)))
    return dx, dw


def matmul_tn(a_t: torch.Tensor, b: torch.Tensor, b_layout: str = "kn", out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``a_t.T @ b`` with ``a_t`` given as ``[K, M]`` (no transposed copy: the tensor core reads it
    as an M-contiguous operand); bf16 / f16 operands, fp32 accumulation."""
    _need_cuda(a_t, b)
    if a_t.dtype != b.dtype or a_t.dtype not in (torch.bfloat16, torch.float16):
        raise _lib.UnsupportedError(-2, f"matmul_tn operands must both be bf16 or f16, got {a_t.dtype}/{b.dtype}")
    if a_t.dim() != 2 or b.dim() != 2:
        raise _lib.UnsupportedError(-3, "matmul_tn takes 2-D operands")
    if a_t.stride(1) != 1:
        a_t = a_t.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    K, M = a_t.shape
    layout = {"kn": _lib.W_KN, "nk": _lib.W_NK}[b_layout]
    N = b.shape[1] if layout == _lib.W_KN else b.shape[0]
    if (b.shape[0] if layout == _lib.W_KN else b.shape[1]) != K:
        raise _lib.UnsupportedError(-3, "matmul_tn inner dimensions differ")
    od = out_dtype or a_t.dtype
    c = torch.empty((M, N), dtype=od, device=a_t.device)
    with _dev(a_t.device):
        check(LIB.arke_b200_matmul_tn(a_t.data_ptr(), a_t.stride(0), b.data_ptr(), b.stride(0), layout, _dt(a_t),
                                      M, N, K, c.data_ptr(), _DT[od], N, _stream(a_t)))
    return c


STATIC_SCRATCH_BYTES = 8 << 20


def fused_linear_ce_static(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                           loss_tok: torch.Tensor, mean: torch.Tensor, ignore_index: int = -100,
                           vocab_offset: int = 0) -> None:
    """:func:`fused_linear_ce` without any allocation: the scratch is the 8 MiB array built into
    the kernel library and the caller passes the outputs (``loss_tok`` fp32 [M], ``mean`` fp32
    scalar tensor).  For hosts whose device memory is fully owned by their own pool or that must
    not allocate where this op runs.  Problems whose workspace
    (:func:`fused_linear_ce_workspace_bytes`) exceeds ``STATIC_SCRATCH_BYTES`` are rejected.
    Inputs must already be contiguous; calls share the scratch, so keep them ordered on one stream.
    """
    _need_cuda(x, w, labels, loss_tok, mean)
    if x.dtype not in (torch.bfloat16, torch.float16) or w.dtype != x.dtype or labels.dtype != torch.int64:
        raise _lib.UnsupportedError(-2, "fused_linear_ce_static needs bf16/f16 x, w and int64 labels")
    if not (x.is_contiguous() and w.is_contiguous() and labels.is_contiguous() and loss_tok.is_contiguous()):
        raise _lib.UnsupportedError(-3, "fused_linear_ce_static takes contiguous tensors (it never copies)")
    M, D = x.shape
    V = w.shape[0]
    if w.shape[1] != D or labels.shape != (M,) or loss_tok.shape != (M,) or loss_tok.dtype != torch.float32 \
            or mean.dtype != torch.float32 or mean.numel() != 1:
        raise _lib.UnsupportedError(-3, "fused_linear_ce_static: shape/dtype mismatch")
    with _dev(x.device):
        check(LIB.arke_b200_fused_linear_ce_static(
            x.data_ptr(), w.data_ptr(), labels.data_ptr(), _dt(x), M, V, D, int(vocab_offset),
            int(ignore_index), loss_tok.data_ptr(), mean.data_ptr(), None, _stream(x)))


def ce_combine(partials: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Merge vocabulary-shard partials [G,M,3] → ``(loss_tok [M], mean)``."""
    _need_cuda(partials, labels)
    if partials.dtype != torch.float32 or partials.dim() != 3 or partials.shape[2] != 3:
        raise _lib.UnsupportedError(-3, "ce_combine takes fp32 partials of shape [G,M,3]")
    partials, labels = partials.contiguous(), labels.contiguous()
    G, M, _ = partials.shape
    loss = torch.empty((M,), dtype=torch.float32, device=partials.device)
    mean = torch.empty((), dtype=torch.float32, device=partials.device)
    with _dev(partials.device):
        check(LIB.arke_b200_ce_combine(partials.data_ptr(), G, M, labels.data_ptr(), int(ignore_index),
                                       loss.data_ptr(), mean.data_ptr(), _stream(partials)))
    return loss, mean


def selftest_quant_division(dtype: torch.dtype = torch.bfloat16, out_dtype: str = "int8", device=None):
    """Exhaustive device check of the quantisation kernels' fast quotient against the IEEE
    division → ``(mismatches, pairs_checked)``; mismatches must be 0."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    counters = torch.zeros(2, dtype=torch.int64, device=dev)
    kind = {"int8": _lib.QUANT_INT8, "fp8": _lib.QUANT_E4M3}[out_dtype]
    with _dev(dev):
        check(LIB.arke_b200_selftest_quant_division(_DT[dtype], kind, counters.data_ptr(),
                                                    torch.cuda.current_stream(dev).cuda_stream))
    c = counters.cpu()
    return int(c[0]), int(c[1])


def kernel_status(device=None) -> int:
    """Read-and-clear the device's bounded-wait status word (0 = no wait expired)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with _dev(dev):
        return int(LIB.arke_b200_kernel_status(torch.cuda.current_stream(dev).cuda_stream))
