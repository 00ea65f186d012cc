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
        # each rank's share of dX leaves the kernel in fp32 (the accumulators, unrounded)
        backward_fn = lambda xx, ww, ll, ls, off: ops.fused_linear_ce_backward(  # noqa: E731
            xx, ww, ll, lse=ls, grad=grad, ignore_index=ignore_index, vocab_offset=off, dx_dtype=torch.float32)
    dx_part, dw = backward_fn(x, w_shard, labels, lse, vocab_offset)
    dx = dx_part.float().contiguous()            # summed in fp32 (a no-op cast for the CUDA kernels' share)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group)
    return dx, dw


# ---------------------------------------------------------------------------------------------
# failure detection (host side)
# ---------------------------------------------------------------------------------------------
class PeerLostError(RuntimeError):
    """A rank of the group did not reach the step in time.  ``missing`` lists the ranks."""

    def __init__(self, step: int, missing, timeout_s: float):
        super().__init__(f"step {step}: rank(s) {sorted(missing)} did not check in within {timeout_s:.1f} s; "
                         "no collective was launched")
        self.step, self.missing, self.timeout_s = step, sorted(missing), timeout_s


class StepLiveness:
    """Host-side heartbeat for a sharded step: learn that a peer is gone BEFORE launching kernels
    and the collective that would wait for it.

    Every rank calls :meth:`check_in` at the start of step ``k``: it posts ``live/<k>/<rank>`` in the
    process group's key-value store and waits, with a timeout, for the keys of all other ranks.  A
    rank that raised, exited or never joined leaves its key unset and the survivors get a
    :class:`PeerLostError` in bounded time with nothing in flight on the device — the same role the
    per-measurement watchdog plays in the reference's benchmark loop
    (benchmarks/watchdog.py:79-136: a typed timeout instead of a hang, the loop stays alive).
    A rank leaves only between steps (nothing of its own in flight).  If a peer dies after the
    check-in, the process group's own timeout ends the collective with an error; create the group
    with a short ``timeout=`` for that.
    """

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "arke_b200/live"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.prefix = float(timeout_s), prefix

    @classmethod
    def from_default_group(cls, timeout_s: float = 5.0) -> "StepLiveness":
        import torch.distributed as dist
        from torch.distributed import distributed_c10d as c10d
        return cls(c10d._get_default_store(), dist.get_rank(), dist.get_world_size(), timeout_s)

    def _key(self, step: int, rank: int) -> str:
        return f"{self.prefix}/{step}/{rank}"

    def check_in(self, step: int) -> None:
        import datetime
        import time
        self.store.set(self._key(step, self.rank), "1")
        others = [r for r in range(self.world) if r != self.rank]
        deadline = time.monotonic() + self.timeout_s
        missing = list(others)
        while missing:
            left = deadline - time.monotonic()
            if left <= 0:
                raise PeerLostError(step, missing, self.timeout_s)
            try:
                self.store.wait([self._key(step, r) for r in missing], datetime.timedelta(seconds=max(left, 0.05)))
                missing = []
            except Exception:
                # which ones are still absent? (the wait reports only that some key is missing)
                missing = [r for r in missing if not self._has(step, r)]
                if missing and time.monotonic() >= deadline:
                    raise PeerLostError(step, missing, self.timeout_s) from None

    def _has(self, step: int, rank: int) -> bool:
        try:
            return bool(self.store.check([self._key(step, rank)]))
        except Exception:
            return False
