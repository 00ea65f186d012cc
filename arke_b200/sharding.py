"""Multi-GPU execution of the hot path: one process per GPU, ``torch.distributed``.

Every op shards along independent units with **no data-path communication**:

  quantize / SwiGLU / W8A8-FP8 GEMM   rows of X (tokens); weights replicated
  GQA attention                        (batch x KV-head-group) units; the sequence is never split
  fused linear + CE                    tokens (no communication), or the **vocabulary**: rank r
                                       holds W[v0:v1], sees all tokens, emits per-row
                                       (max, sum exp, target logit) and the ranks exchange that
                                       [M,3] fp32 block (98 KB at 8192 tokens) in ONE collective.

The partition helpers are pure Python; the collective is ``all_gather_into_tensor`` (NCCL on
GPUs, gloo in the CPU tests) followed by the ``ce_combine`` kernel.  The backward of the
vocabulary-sharded form has one more exchange: every rank owns its rows of dW outright, and the
ranks' contributions to dX (each ``G[:, v0:v1] @ W[v0:v1]``) are summed with one all-reduce.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [begin, end) of ``n`` units for ``rank`` (first ``n % world`` ranks get
    one extra unit)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Token shard of a [M, ...] tensor (a view)."""
    b, e = shard_bounds(x.shape[0], world, rank)
    return x[b:e]


def attention_units(B: int, Hq: int, Hkv: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) over the B*Hkv (batch, KV-group) units; a unit is the ``Hq//Hkv`` query heads
    that share one KV head, so K/V of a unit are read by one GPU only."""
    return shard_bounds(B * Hkv, world, rank)


def shard_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, world: int, rank: int):
    """Slices of q/k/v ([B,H,S,D]) for this rank's units, reshaped to batch 1 so one kernel launch
    covers them: q -> [1, units*group, S, D], k/v -> [1, units, S, D]."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    grp = Hq // Hkv
    b, e = attention_units(B, Hq, Hkv, world, rank)
    qf = q.reshape(B * Hkv, grp, S, D)[b:e].reshape(1, (e - b) * grp, S, D)
    kf = k.reshape(B * Hkv, 1, k.shape[2], D)[b:e].reshape(1, e - b, k.shape[2], D)
    vf = v.reshape(B * Hkv, 1, v.shape[2], D)[b:e].reshape(1, e - b, v.shape[2], D)
    return qf, kf, vf


def combine_partials_reference(partials: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Pure-torch merge of [G,M,3] shard partials → ``(loss_tok, mean)``; host-side twin of the
    ``ce_combine`` kernel used by the CPU (gloo) tests of the collective plumbing."""
    m, s, t = partials[..., 0], partials[..., 1], partials[..., 2]
    mx = m.max(dim=0).values
    ssum = (s * torch.exp(m - mx[None, :])).sum(dim=0)
    tok = torch.log(ssum) + mx - t.sum(dim=0)
    keep = labels != ignore_index
    tok = torch.where(keep, tok, torch.zeros_like(tok))
    return tok, tok.sum() / keep.sum()


def vocab_sharded_ce(x: torch.Tensor, w_shard: torch.Tensor, labels: torch.Tensor, vocab_offset: int,
                     ignore_index: int = -100, group=None,
                     partial_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None):
    """Fused linear + CE with the vocabulary sharded over the process group.

    Every rank passes all tokens ``x`` [M,D], its slice ``w_shard`` [V_r,D] whose first row is the
    global index ``vocab_offset``, and the global ``labels``.  One ``all_gather_into_tensor`` of
    the [M,3] partials, then the combine.  ``partial_fn`` / ``combine_fn`` default to the CUDA
    kernels; the CPU tests inject host implementations to exercise the exchange with gloo.
    Returns ``(loss_tok [M], mean)`` identical on every rank.
    """
    import torch.distributed as dist
    if partial_fn is None or combine_fn is None:
        from . import ops
        partial_fn = partial_fn or (lambda xx, ww, ll, off: ops.fused_linear_ce(
            xx, ww, ll, ignore_index=ignore_index, vocab_offset=off, want_partials=True))
        combine_fn = combine_fn or (lambda pp, ll: ops.ce_combine(pp, ll, ignore_index=ignore_index))
    part = partial_fn(x, w_shard, labels, vocab_offset).contiguous()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return combine_fn(part.unsqueeze(0), labels)
    # rank-major concatenation along dim 0 (the layout every backend's all-gather accepts)
    gathered = torch.empty((world * part.shape[0], *part.shape[1:]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(gathered, part, group=group)
    return combine_fn(gathered.view(world, *part.shape), labels)


def lse_from_partials(partials: torch.Tensor) -> torch.Tensor:
    """Per-row natural-log logsumexp over the whole vocabulary from gathered shard partials
    ``[G,M,3]`` (or one slice's ``[M,3]``): what the backward needs from the forward."""
    if partials.dim() == 2:
        partials = partials.unsqueeze(0)
    m, s = partials[..., 0], partials[..., 1]
    mx = m.max(dim=0).values
    return mx + torch.log((s * torch.exp(m - mx[None, :])).sum(dim=0))


def vocab_sharded_ce_backward(x: torch.Tensor, w_shard: torch.Tensor, labels: torch.Tensor, vocab_offset: int,
                              lse: torch.Tensor, grad: float = 1.0, ignore_index: int = -100, group=None,
                              backward_fn: Optional[Callable] = None):
    """Backward of :func:`vocab_sharded_ce`: returns ``(dx [M,D] fp32, identical on every rank,
    dw_shard [V_r,D])``.  ``lse`` is the global per-row logsumexp (:func:`lse_from_partials` of the
    gathered partials).  ``backward_fn(x, w_shard, labels, lse, vocab_offset) -> (dx_part, dw)``
    defaults to the CUDA kernels; the CPU tests inject a host implementation."""
    import torch.distributed as dist
    if backward_fn is None:
        from . import ops
        backward_fn = lambda xx, ww, ll, ls, off: ops.fused_linear_ce_backward(  # noqa: E731
            xx, ww, ll, lse=ls, grad=grad, ignore_index=ignore_index, vocab_offset=off)
    dx_part, dw = backward_fn(x, w_shard, labels, lse, vocab_offset)
    dx = dx_part.float().contiguous()            # summed in fp32: 16-bit partial sums would lose bits
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group)
    return dx, dw
