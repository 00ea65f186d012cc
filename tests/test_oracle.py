"""CPU: the oracle restatements against the golden vectors produced by the real reference."""
import numpy as np
import pytest
import torch

import cases
from conftest import from_bits, load_golden
from oracle import ops as oracle


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.QUANT_CASES))
def test_quantize_interp_matches_reference(name, tag):
    g = load_golden("quantize_interp.npz")
    x = cases.quant_input(name, tag)
    assert cases.checksum(x) == g[f"{name}_{tag}_in"], "seeded input drifted from the fixture"
    q, scale = oracle.quantize_per_token_interp(x)
    assert np.array_equal(q.numpy(), g[f"{name}_{tag}_q"])  # bit-exact
    assert torch.equal(scale, x.float().abs().amax(-1) / 127.0)


def test_quantize_rounding_ties_half_to_even():
    g = load_golden("quantize_interp.npz")
    ties = torch.tensor(cases.TIES)
    q, scale = oracle.quantize_per_token_interp(ties)
    assert torch.equal(scale, torch.ones(2))
    assert np.array_equal(q.numpy(), g["ties_q"])
    # hand-computed: 0.5->0 1.5->2 2.5->2 -0.5->0 126.5->126 -126.5->-126 -3.5->-4 3.5->4 63.5->64 64.5->64 -64.5->-64
    assert q[0].tolist() == [127, 0, 2, 2, 0, 126, -126, -4, 4, 64, 64, -64, 0, 1, -1, -127]


def test_quantize_zero_row_defined_as_zero():
    x = torch.zeros(2, 32)
    x[1, 3] = 2.0
    q, scale = oracle.quantize_per_token_interp(x)
    assert scale[0] == 0 and torch.all(q[0] == 0) and q[1, 3] == 127


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.QUANT_BENCH_CASES))
def test_quantize_bench_l1_matches_reference(name, tag):
    g = load_golden("quantize_bench_l1.npz")
    x = cases.quant_input(name, tag, cases.QUANT_BENCH_CASES, "quantb")
    assert cases.checksum(x) == g[f"{name}_{tag}_in"]
    q, sc = oracle.quantize_per_token_bench_l1(x)
    assert np.array_equal(q.numpy(), g[f"{name}_{tag}_q"])
    assert torch.equal(sc, from_bits(g[f"{name}_{tag}_scales_bits"], cases.DTYPES[tag]))


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.SILU_CASES))
def test_silu_and_mul_matches_reference(name, tag):
    g = load_golden("silu_and_mul.npz")
    x = cases.silu_input(name, tag)
    assert cases.checksum(x) == g[f"{name}_{tag}_in"]
    y = oracle.silu_and_mul(x)
    assert torch.equal(y, from_bits(g[f"{name}_{tag}_y_bits"], cases.DTYPES[tag]))


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.GQA_CASES))
def test_gqa_matches_reference(name, tag):
    g = load_golden("gqa.npz")
    q, k, v = cases.gqa_inputs(name, tag)
    assert cases.checksum(q, k, v) == g[f"{name}_{tag}_in"]
    for causal, key in ((True, "causal"), (False, "full")):
        ref = from_bits(g[f"{name}_{tag}_o_{key}_bits"], cases.DTYPES[tag])
        o = oracle.gqa_attention(q, k, v, causal)
        assert torch.equal(o, ref)
        # the float64 restatement (which also yields LSE) agrees with the reference output
        o64, lse = oracle.gqa_attention_f64(q, k, v, causal)
        assert torch.allclose(o64.float(), ref.float(), rtol=2e-2, atol=2e-2)
        assert torch.isfinite(lse).all()


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.FLCE_CASES))
def test_flce_matches_reference(name, tag):
    g = load_golden("flce.npz")
    x, w, labels = cases.flce_inputs(name, tag)
    assert cases.checksum(x, w, labels) == g[f"{name}_{tag}_in"]
    tok, mean = oracle.fused_linear_ce(x, w, labels)
    assert abs(mean.item() - float(g[f"{name}_{tag}_mean"])) <= 1e-6
    keep = labels != -100
    assert torch.all(tok[~keep] == 0)
    assert abs((tok.sum() / keep.sum()).item() - mean.item()) <= 1e-4


def test_flce_vocab_shard_combine_equals_unsharded():
    x, w, labels = cases.flce_inputs("b", "bf16")
    tok, mean = oracle.fused_linear_ce(x, w, labels)
    V = w.shape[0]
    for G in (2, 4, 7):
        bounds = [V * i // G for i in range(G + 1)]
        parts = torch.stack([oracle.ce_partials(x, w[bounds[i]:bounds[i + 1]], labels, bounds[i]) for i in range(G)])
        tok2, mean2 = oracle.ce_combine(parts, labels)
        assert torch.allclose(tok2, tok, rtol=1e-5, atol=1e-5)
        assert abs(mean2.item() - mean.item()) < 1e-5


def test_matmul_fp32_pipeline_golden():
    g = load_golden("matmul_fp32_1024.npz")
    A, B = cases.matmul_fp32_inputs()
    assert cases.checksum(A, B) == g["c_in"]
    C = A @ B  # the interpreter's ref_matmul is torch.matmul on the fp32 inputs
    assert np.allclose(C[::64, ::64].numpy(), g["c_sample"], rtol=1e-4, atol=1e-3)
    assert abs(C.double().abs().sum().item() - float(g["c_abs_sum"])) / float(g["c_abs_sum"]) < 1e-6


def test_int8_gemm_acc_exact_small():
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-128, 128, (37, 200), generator=g, dtype=torch.int32)
    w = torch.randint(-127, 128, (200, 53), generator=g, dtype=torch.int32)
    ref = (a.long() @ w.long()).to(torch.int32)
    assert torch.equal(oracle.int8_gemm_acc(a.to(torch.int8), w.to(torch.int8)), ref)
    if hasattr(torch, "_int_mm"):
        a2 = torch.randint(-128, 128, (64, 256), generator=g, dtype=torch.int32).to(torch.int8)
        w2 = torch.randint(-127, 128, (256, 64), generator=g, dtype=torch.int32).to(torch.int8)
        assert torch.equal(torch._int_mm(a2, w2), oracle.int8_gemm_acc(a2, w2))


def test_fp8_quantize_known_values():
    # e4m3 round-to-nearest-even with saturation at 448
    x = torch.tensor([[448.0, 449.0, 463.9, 464.0, 500.0, -500.0, 0.0, 1.0]])
    q, s = oracle.quantize_per_token_fp8(x)
    assert abs(s.item() - 500.0 / 448.0) < 1e-6
    deq = q.float() * s
    assert torch.isfinite(deq).all() and deq[0, 4] == 500.0 and deq[0, 5] == -500.0


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.RMS_CASES))
def test_rmsnorm_matches_reference(name, tag):
    g = load_golden("rmsnorm.npz")
    x, res, w = cases.rms_inputs(name, tag)
    assert cases.checksum(x, res, w) == g[f"{name}_{tag}_in"]
    # the interpreter promotes 16-bit inputs to fp32 for rmsnorm: its output is fp32
    assert torch.equal(oracle.rmsnorm(x.float(), w.float()), torch.from_numpy(g[f"{name}_{tag}_y"]))
    assert torch.equal(oracle.rmsnorm(x.float(), w.float(), residual=res.float()), torch.from_numpy(g[f"{name}_{tag}_yres"]))


@pytest.mark.parametrize("tag", list(cases.DTYPES) + ["f32"])
@pytest.mark.parametrize("name", list(cases.ROPE_CASES))
def test_rope_matches_reference_bit_for_bit(name, tag):
    g = load_golden("rope.npz")
    x, cos, sin = cases.rope_inputs(name, tag)
    assert cases.checksum(x, cos, sin) == g[f"{name}_{tag}_in"]
    y = oracle.rope(x, cos, sin)
    want = torch.from_numpy(g[f"{name}_f32_y"]) if tag == "f32" else from_bits(g[f"{name}_{tag}_y_bits"], cases.DTYPES[tag])
    assert y.dtype == x.dtype and torch.equal(y, want.view(y.shape))


def test_qkv_rope_split_is_rope_on_the_head_views():
    B, S, Hq, Hkv, D = 2, 5, 4, 2, 32
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    cos, sin = oracle.make_rope_tables(S, D)
    q, k, v = oracle.qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D)
    assert q.shape == (B, Hq, S, D) and k.shape == (B, Hkv, S, D) and v.shape == (B, Hkv, S, D)
    row = qkv[1 * S + 3]                                            # token (b=1, s=3)
    assert torch.equal(v[1, 1, 3], row[(Hq + Hkv + 1) * D:(Hq + Hkv + 2) * D])
    assert torch.equal(k[1, 0, 3], oracle.rope(row[Hq * D:(Hq + 1) * D].view(1, 1, 1, D), cos[3:4], sin[3:4]).view(D))
    assert torch.equal(q[1, 2, 3], oracle.rope(row[2 * D:3 * D].view(1, 1, 1, D), cos[3:4], sin[3:4]).view(D))
