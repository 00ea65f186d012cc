"""``torch.autograd`` binding of fused linear + cross-entropy: a loss a training step can call
``backward()`` on, with both directions on the sm_100a kernels.

    from arke_b200.autograd import fused_linear_cross_entropy
    loss = fused_linear_cross_entropy(hidden, lm_head_weight, labels)     # fp32 scalar (mean)
    loss.backward()                                                       # hidden.grad, weight.grad

Forward = ``ref_fused_linear_cross_entropy`` (arke/ir/ops/reference_impls.py:211-213); the backward
is its derivative (the reference has none).  The logits are never stored in fp32: the forward keeps
only the per-row logsumexp, the backward recomputes the logit tiles and holds their gradient in
16 bits.
"""
from __future__ import annotations

import torch


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, labels, ignore_index):
        from . import ops
        part = ops.fused_linear_ce(x, w, labels, ignore_index=ignore_index, want_partials=True)   # (max, sumexp, target)
        lse = part[:, 0] + torch.log(part[:, 1])
        valid = labels != ignore_index
        loss_tok = torch.where(valid, lse - part[:, 2], torch.zeros_like(lse))
        mean = loss_tok.sum() / valid.sum()      # all labels ignored -> 0/0 = NaN, like F.cross_entropy and ops.fused_linear_ce
        ctx.save_for_backward(x, w, labels, lse)
        ctx.ignore_index = ignore_index
        return mean

    @staticmethod
    def backward(ctx, grad_out):
        from . import ops
        x, w, labels, lse = ctx.saved_tensors
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not (need_dx or need_dw):
            return None, None, None, None
        # grad_out stays on the device: the kernel that forms grad / n_valid reads it there
        dx, dw = ops.fused_linear_ce_backward(x, w, labels, lse=lse, grad=grad_out, ignore_index=ctx.ignore_index,
                                              want_dx=need_dx, want_dw=need_dw)
        return dx, dw, None, None


def fused_linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy of ``x @ w.T`` against ``labels`` (``x [M,D]``, ``w [V,D]`` bf16 / f16 on
    a B200, ``labels [M]`` int64), differentiable with respect to ``x`` and ``w``."""
    return _FusedLinearCE.apply(x, w, labels, ignore_index)
