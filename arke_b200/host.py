"""Host-buffer entry point for the W8A8 linear layer: ``quantize_per_token → W8A8 GEMM`` on
activations that live in (pinned) host memory, result returned to (pinned) host memory.

The token rows are cut into chunks and three CUDA streams overlap the host→device copy of chunk
i+1, the kernels of chunk i and the device→host copy of chunk i-1, so a step costs about
``max(H2D, kernels, D2H)`` instead of their sum; across calls the next step's H2D also overlaps
the previous step's D2H.  Device staging buffers are allocated once per ``HostW8A8Linear``.
"""
from __future__ import annotations

import torch

from . import ops


class HostW8A8Linear:
    """``y_host = dequant(quantize(x_host) @ W)`` with W (int8 [K,N]) and its per-channel scales
    resident on the device."""

    def __init__(self, w: torch.Tensor, sw: torch.Tensor, max_rows: int, chunks: int = 4,
                 x_dtype: torch.dtype = torch.bfloat16, out_dtype: torch.dtype = torch.bfloat16):
        if not w.is_cuda or w.dtype != torch.int8 or w.dim() != 2:
            raise ValueError("w must be an int8 [K,N] CUDA tensor")
        self.w, self.sw = w, sw
        self.K, self.N = w.shape
        self.dev = w.device
        self.chunks = max(1, int(chunks))
        self.rows = (max_rows + self.chunks - 1) // self.chunks
        self.out_dtype = out_dtype
        nbuf = 2  # double-buffered staging per chunk slot
        self.x_d = [torch.empty(self.rows, self.K, dtype=x_dtype, device=self.dev) for _ in range(nbuf)]
        self.q_d = [torch.empty(self.rows, self.K, dtype=torch.int8, device=self.dev) for _ in range(nbuf)]
        self.s_d = [torch.empty(self.rows, dtype=torch.float32, device=self.dev) for _ in range(nbuf)]
        self.y_d = [torch.empty(self.rows, self.N, dtype=out_dtype, device=self.dev) for _ in range(nbuf)]
        self.s_h2d, self.s_cmp, self.s_d2h = (torch.cuda.Stream(self.dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(nbuf)]     # x chunk landed on the device
        self.ev_out = [torch.cuda.Event() for _ in range(nbuf)]    # y chunk computed
        self.ev_free_x = [torch.cuda.Event() for _ in range(nbuf)]  # kernels finished reading x_d
        self.ev_free_y = [torch.cuda.Event() for _ in range(nbuf)]  # d2h finished reading y_d
        self._slot = 0
        self._primed = [False] * nbuf

    def __call__(self, x_host: torch.Tensor, y_host: torch.Tensor, wait: bool = True) -> torch.cuda.Event:
        """Enqueue one step; returns an event that fires when ``y_host`` is complete.  ``x_host``
        [M,K] and ``y_host`` [M,N] should be pinned for the copies to be asynchronous.  With
        ``wait`` (default) the caller's current stream also waits for that event, so later work on
        it sees ``y_host``; a caller that streams many steps passes ``wait=False`` and synchronises
        on the returned event itself, which lets the next step's copies and kernels start while
        this step's result is still on its way to the host."""
        M = x_host.shape[0]
        if x_host.shape[1] != self.K or y_host.shape != (M, self.N) or M > self.rows * self.chunks:
            raise ValueError("shape mismatch with the configured pipeline")
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_h2d, self.s_cmp, self.s_d2h):
            s.wait_stream(cur)
        r0 = 0
        while r0 < M:
            r1 = min(M, r0 + self.rows)
            n = r1 - r0
            b = self._slot
            self._slot ^= 1
            with torch.cuda.stream(self.s_h2d):
                if self._primed[b]:
                    self.s_h2d.wait_event(self.ev_free_x[b])
                self.x_d[b][:n].copy_(x_host[r0:r1], non_blocking=True)
                self.ev_in[b].record(self.s_h2d)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[b])
                if self._primed[b]:
                    self.s_cmp.wait_event(self.ev_free_y[b])
                ops.quantize_per_token(self.x_d[b][:n], out=(self.q_d[b][:n], self.s_d[b][:n]))
                self.ev_free_x[b].record(self.s_cmp)
                ops.w8a8_gemm(self.q_d[b][:n], self.s_d[b][:n], self.w, self.sw, out=self.y_d[b][:n])
                self.ev_out[b].record(self.s_cmp)
            with torch.cuda.stream(self.s_d2h):
                self.s_d2h.wait_event(self.ev_out[b])
                y_host[r0:r1].copy_(self.y_d[b][:n], non_blocking=True)
                self.ev_free_y[b].record(self.s_d2h)
            self._primed[b] = True
            r0 = r1
        done = torch.cuda.Event()
        done.record(self.s_d2h)
        if wait:
            cur.wait_event(done)
        return done
