"""GPU parity: GQA flash-attention forward (tcgen05) vs the reference interpreter's golden
outputs and the float64 oracle (which also pins the logsumexp).  O within rtol = atol = 2e-2
(bf16) and 1e-3 for fp16 — the reference's own gate for fp16 attention
(benchmarks/bench_l1.py:134-141); LSE within 1e-3."""
import pytest
import torch

import cases
from conftest import from_bits, load_golden
from oracle import ops as oracle

pytestmark = pytest.mark.gpu


def _ops():
    from arke_b200 import ops
    return ops


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.GQA_CASES))
def test_gqa_golden(name, tag, causal):
    g = load_golden("gqa.npz")
    q, k, v = cases.gqa_inputs(name, tag)
    ref = from_bits(g[f"{name}_{tag}_o_{'causal' if causal else 'full'}_bits"], cases.DTYPES[tag])
    o, lse = _ops().gqa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    assert _ops().kernel_status() == 0
    tol = 2e-2 if tag == "bf16" else 1e-3
    assert torch.allclose(o.cpu().float(), ref.float(), rtol=tol, atol=tol)
    o64, lse64 = oracle.gqa_attention_f64(q, k, v, causal)
    assert torch.allclose(lse.cpu().double(), lse64, rtol=1e-3, atol=1e-3)
    assert (o.cpu().double() - o64).abs().max().item() < (1.5e-2 if tag == "bf16" else 2e-3)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(1, 8, 2, 1024, 128), (2, 4, 4, 513, 128), (1, 4, 1, 2048, 64), (1, 2, 2, 100, 128), (1, 32, 8, 640, 128)])
def test_gqa_vs_f64_oracle(shape, causal):
    B, Hq, Hkv, S, D = shape
    q, k, v = oracle.make_attention_inputs(B, Hq, Hkv, S, D, seed=S)
    o, lse = _ops().gqa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    assert _ops().kernel_status() == 0
    o64, lse64 = oracle.gqa_attention_f64(q, k, v, causal)
    assert torch.allclose(o.cpu().double(), o64, rtol=2e-2, atol=2e-2)
    assert torch.allclose(lse.cpu().double(), lse64, rtol=1e-3, atol=1e-3)


def test_gqa_different_kv_length_non_causal_and_3d_inputs():
    q, k, v = oracle.make_attention_inputs(1, 4, 2, 300, 128, seed=8, Skv=777)
    o, lse = _ops().gqa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=False)
    o64, lse64 = oracle.gqa_attention_f64(q, k, v, False)
    assert torch.allclose(o.cpu().double(), o64, rtol=2e-2, atol=2e-2)
    assert torch.allclose(lse.cpu().double(), lse64, rtol=1e-3, atol=1e-3)
    o3 = _ops().gqa_fwd(q[0].cuda(), k[0].cuda(), v[0].cuda(), causal=False, return_lse=False)
    assert o3.shape == (4, 300, 128) and torch.equal(o3, o[0])


def test_gqa_large_scores_trigger_rescale_path():
    # growing score magnitudes along the sequence force the running maximum to move by > 2^8
    B, Hq, Hkv, S, D = 1, 2, 1, 1024, 128
    q, k, v = oracle.make_attention_inputs(B, Hq, Hkv, S, D, seed=3)
    ramp = torch.linspace(0.2, 6.0, S)[None, None, :, None]
    k = (k.float() * ramp).bfloat16()
    for causal in (False, True):
        o, lse = _ops().gqa_fwd(q.cuda(), k.cuda(), v.cuda(), causal=causal)
        o64, lse64 = oracle.gqa_attention_f64(q, k, v, causal)
        assert torch.allclose(o.cpu().double(), o64, rtol=2e-2, atol=2e-2)
        assert torch.allclose(lse.cpu().double(), lse64, rtol=1e-3, atol=1e-3)


def test_gqa_config_shape_sampled_rows_and_determinism():
    # benchmark configuration: B4 Hq32 Hkv8 S8192 D128 causal; sampled (b, h, rows) vs float64
    B, Hq, Hkv, S, D = 4, 32, 8, 8192, 128
    q, k, v = oracle.make_attention_inputs(B, Hq, Hkv, S, D, seed=4)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o, lse = _ops().gqa_fwd(qd, kd, vd, causal=True)
    o2, lse2 = _ops().gqa_fwd(qd, kd, vd, causal=True)
    assert _ops().kernel_status() == 0
    assert torch.equal(o, o2) and torch.equal(lse, lse2)   # run-to-run identical
    rows = torch.tensor([0, 1, 127, 128, 129, 255, 256, 1000, 4095, 4096, 8191])
    for (b, h) in [(0, 0), (1, 5), (3, 31), (2, 18)]:
        kh = h // (Hq // Hkv)
        qs = q[b, h, rows].double()
        s = (qs @ k[b, kh].double().T) / (D ** 0.5)
        mask = torch.arange(S)[None, :] > rows[:, None]
        s = s.masked_fill(mask, float("-inf"))
        lse_ref = torch.logsumexp(s, -1)
        o_ref = torch.softmax(s, -1) @ v[b, kh].double()
        assert torch.allclose(o[b, h, rows].cpu().double(), o_ref, rtol=2e-2, atol=2e-2)
        assert torch.allclose(lse[b, h, rows].cpu().double(), lse_ref, rtol=1e-3, atol=1e-3)


def test_gqa_rejects_bad_shapes():
    from arke_b200 import _lib
    q = torch.zeros(1, 3, 16, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.UnsupportedError):
        _ops().gqa_fwd(q, k, k)
    q = torch.zeros(1, 2, 16, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.UnsupportedError):
        _ops().gqa_fwd(q, q, q)
    with pytest.raises(_lib.UnsupportedError):
        _ops().gqa_fwd(q.float(), q.float(), q.float())


@pytest.mark.parametrize("shape", [(1, 8, 2, 4096, 128), (1, 4, 4, 8192, 64)])
def test_gqa_fp16_long_sequence_within_the_reference_gate(shape):
    """fp16 causal GQA at long sequences against fp16 SDPA at rtol = atol = 1e-3, the tolerance the
    reference's benchmark gate applies to fp16 flash_attention / grouped_query_attention
    (benchmarks/bench_l1.py:134-141) — the 16-bit P and the polynomial exponentials must not
    accumulate beyond it over 32-64 key tiles."""
    B, Hq, Hkv, S, D = shape
    q, k, v = oracle.make_attention_inputs(B, Hq, Hkv, S, D, seed=S + D, dtype=torch.float16)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o = _ops().gqa_fwd(qc, kc, vc, causal=True, return_lse=False)
    assert _ops().kernel_status() == 0
    rep = Hq // Hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        qc, kc.repeat_interleave(rep, 1), vc.repeat_interleave(rep, 1), is_causal=True)
    assert torch.allclose(o.float(), ref.float(), rtol=1e-3, atol=1e-3), (o.float() - ref.float()).abs().max().item()
    # and against exact arithmetic on sampled heads (SDPA itself rounds P to 16 bits)
    o64, _ = oracle.gqa_attention_f64(q[:, :rep], k[:, :1], v[:, :1], True)
    assert torch.allclose(o[:, :rep].cpu().double(), o64, rtol=1e-3, atol=1e-3)
