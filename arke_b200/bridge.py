"""torch bridge: the hot-path ops as ``torch.library`` custom ops with fake (meta) kernels,
following the reference's bridge (arke/integration/torch_bridge.py:140-181) but without its eager
fallback — the op body always runs the sm_100a kernel.

    register_ops()                      # idempotent
    q, s   = torch.ops.arke.quantize_per_token(x)
    y      = torch.ops.arke.w8a8_gemm(q, s, w, sw)
    yq, s2 = torch.ops.arke.swiglu_fp8(x2)
    o, lse = torch.ops.arke.gqa_fwd(q, k, v, True)
    y      = torch.ops.arke.rope(x4, cos, sin)
    q, k, v = torch.ops.arke.qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D)
    tok, m = torch.ops.arke.fused_linear_ce(h, w_lm, labels, -100)
"""
from __future__ import annotations

import torch

_REGISTERED = False


def register_ops() -> bool:
    """Registers ``arke::rmsnorm``, ``arke::rmsnorm_quant``, ``arke::quantize_per_token``, ``arke::w8a8_gemm``, ``arke::swiglu_fp8``,
    ``arke::gqa_fwd``, ``arke::rope``, ``arke::qkv_rope_split`` and ``arke::fused_linear_ce``; returns True when (already) registered."""
    global _REGISTERED
    if _REGISTERED:
        return True
    from . import ops

    @torch.library.custom_op("arke::quantize_per_token", mutates_args=())
    def quantize_per_token(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.quantize_per_token(x)

    @quantize_per_token.register_fake
    def _(x):
        return x.new_empty(x.shape, dtype=torch.int8), x.new_empty(x.shape[:-1], dtype=torch.float32)

    @torch.library.custom_op("arke::rmsnorm", mutates_args=())
    def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return ops.rmsnorm(x, w, eps=eps)

    @rmsnorm.register_fake
    def _(x, w, eps):
        return torch.empty_like(x)

    @torch.library.custom_op("arke::rmsnorm_quant", mutates_args=())
    def rmsnorm_quant(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.rmsnorm(x, w, eps=eps, residual=residual, quantize="int8", return_y=False)

    @rmsnorm_quant.register_fake
    def _(x, residual, w, eps):
        return x.new_empty(x.shape, dtype=torch.int8), x.new_empty(x.shape[:-1], dtype=torch.float32)

    @torch.library.custom_op("arke::w8a8_gemm", mutates_args=())
    def w8a8_gemm(xq: torch.Tensor, sx: torch.Tensor, w: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
        return ops.w8a8_gemm(xq, sx, w, sw)

    @w8a8_gemm.register_fake
    def _(xq, sx, w, sw):
        return xq.new_empty((xq.shape[0], w.shape[1]), dtype=torch.bfloat16)

    @torch.library.custom_op("arke::swiglu_fp8", mutates_args=())
    def swiglu_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.swiglu_fp8(x)

    @swiglu_fp8.register_fake
    def _(x):
        return (x.new_empty((*x.shape[:-1], x.shape[-1] // 2), dtype=torch.float8_e4m3fn),
                x.new_empty(x.shape[:-1], dtype=torch.float32))

    @torch.library.custom_op("arke::gqa_fwd", mutates_args=())
    def gqa_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.gqa_fwd(q, k, v, causal=causal)

    @gqa_fwd.register_fake
    def _(q, k, v, causal):
        return torch.empty_like(q), q.new_empty(q.shape[:-1], dtype=torch.float32)

    @torch.library.custom_op("arke::rope", mutates_args=())
    def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        return ops.rope(x, cos, sin)

    @rope.register_fake
    def _(x, cos, sin):
        return torch.empty_like(x, memory_format=torch.contiguous_format)

    @torch.library.custom_op("arke::qkv_rope_split", mutates_args=())
    def qkv_rope_split(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, S: int, Hq: int, Hkv: int,
                       D: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return ops.qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D)

    @qkv_rope_split.register_fake
    def _(qkv, cos, sin, B, S, Hq, Hkv, D):
        return (qkv.new_empty((B, Hq, S, D)), qkv.new_empty((B, Hkv, S, D)), qkv.new_empty((B, Hkv, S, D)))

    @torch.library.custom_op("arke::fused_linear_ce", mutates_args=())
    def fused_linear_ce(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                        ignore_index: int) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.fused_linear_ce(x, w, labels, ignore_index=ignore_index)

    @fused_linear_ce.register_fake
    def _(x, w, labels, ignore_index):
        return x.new_empty((x.shape[0],), dtype=torch.float32), x.new_empty((), dtype=torch.float32)

    _REGISTERED = True
    return True
