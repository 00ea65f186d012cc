"""Seeded input generators shared by ``make_golden.py`` (which runs the reference on them) and
by the tests (which regenerate the same inputs and compare against the stored outputs).  Inputs
are rebuilt from the seed with a CPU ``torch.Generator``; each fixture also stores a checksum of
the input bits so that a drift of the generator is detected rather than silently mis-compared."""
from __future__ import annotations

import numpy as np
import torch

DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16}

QUANT_CASES = {"a": (16, 64), "b": (7, 769), "c": (5, 4097), "d": (16, 4096), "e": (3, 14336)}
QUANT_BENCH_CASES = {"a": (16, 64), "b": (9, 515), "d": (8, 4096)}
SILU_CASES = {"a": (8, 64), "b": (5, 1030), "c": (8, 4096), "d": (2, 28672)}
GQA_CASES = {"a": (1, 4, 2, 64, 64), "b": (1, 4, 2, 200, 128), "c": (1, 2, 1, 384, 128), "d": (2, 2, 2, 130, 64)}
RMS_CASES = {"a": (8, 64), "b": (5, 1000), "c": (6, 4096)}
ROPE_CASES = {"a": (1, 2, 16, 64), "b": (2, 3, 37, 128), "c": (1, 2, 70, 128), "d": (2, 4, 9, 32)}   # B, H, S, D
FLCE_CASES = {"a": (32, 64, 1000), "b": (130, 256, 5003), "c": (256, 128, 2048)}

TIES = [[127.0, 0.5, 1.5, 2.5, -0.5, 126.5, -126.5, -3.5, 3.5, 63.5, 64.5, -64.5, 0.0, 1.0, -1.0, -127.0],
        [-127.0, 0.5, 1.5, 2.5, -0.5, 126.5, -126.5, -3.5, 3.5, 63.5, 64.5, -64.5, 0.0, 1.0, -1.0, 100.0]]


def _seed(kind: str, name: str, tag: str) -> int:
    return (sum(ord(c) * (i + 1) for i, c in enumerate(kind + ":" + name + ":" + tag)) * 2654435761) % (2**31)


def checksum(*tensors: torch.Tensor) -> np.int64:
    tot = 0
    for t in tensors:
        b = t.contiguous().view(torch.uint8).numpy().astype(np.int64)
        tot = (tot * 1000003 + int((b * (np.arange(b.size, dtype=np.int64).reshape(b.shape) % 251 + 1)).sum())) % (2**61 - 1)
    return np.int64(tot)


def quant_input(name: str, tag: str, cases=QUANT_CASES, kind="quant") -> torch.Tensor:
    M, N = cases[name]
    g = torch.Generator().manual_seed(_seed(kind, name, tag))
    x = torch.randn(M, N, generator=g).to(DTYPES[tag])
    idx = torch.randperm(N, generator=g)[: max(1, N // 100)]
    x[:, idx] = (x[:, idx].float() * 20).to(DTYPES[tag])
    return x


def silu_input(name: str, tag: str) -> torch.Tensor:
    M, N2 = SILU_CASES[name]
    g = torch.Generator().manual_seed(_seed("silu", name, tag))
    return torch.randn(M, N2, generator=g).to(DTYPES[tag])


def gqa_inputs(name: str, tag: str):
    B, Hq, Hkv, S, D = GQA_CASES[name]
    g = torch.Generator().manual_seed(_seed("gqa", name, tag))
    dt = DTYPES[tag]
    q = torch.randn(B, Hq, S, D, generator=g).to(dt)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dt)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dt)
    return q, k, v


def flce_inputs(name: str, tag: str):
    M, D, V = FLCE_CASES[name]
    g = torch.Generator().manual_seed(_seed("flce", name, tag))
    dt = DTYPES[tag]
    x = torch.randn(M, D, generator=g).to(dt)
    w = (torch.randn(V, D, generator=g) * 0.05).to(dt)
    labels = torch.randint(0, V, (M,), generator=g, dtype=torch.int64)
    labels[torch.randperm(M, generator=g)[: max(1, M // 10)]] = -100
    return x, w, labels


def rms_inputs(name: str, tag: str):
    M, N = RMS_CASES[name]
    g = torch.Generator().manual_seed(_seed("rms", name, tag))
    dt = DTYPES[tag]
    x = torch.randn(M, N, generator=g).to(dt)
    res = torch.randn(M, N, generator=g).to(dt)
    w = (1.0 + 0.1 * torch.randn(N, generator=g)).to(dt)
    return x, res, w


def rope_inputs(name: str, tag: str):
    B, H, S, D = ROPE_CASES[name]
    g = torch.Generator().manual_seed(_seed("rope", name, tag))
    dt = torch.float32 if tag == "f32" else DTYPES[tag]
    x = torch.randn(B, H, S, D, generator=g).to(dt)
    # real rotary tables: angle = position * base^(-2i/D)
    inv = 10000.0 ** (-torch.arange(0, D // 2, dtype=torch.float32) * 2.0 / D)
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
    return x, torch.cos(ang).to(dt), torch.sin(ang).to(dt)


def matmul_fp32_inputs():
    g = torch.Generator().manual_seed(0)
    return torch.randn(1024, 1024, generator=g), torch.randn(1024, 1024, generator=g)
