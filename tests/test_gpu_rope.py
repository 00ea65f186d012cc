"""GPU parity: rotary embedding, the packed-QKV split and the QKV-projection -> rope -> attention
path through the C ABI, against the reference's golden vectors and the CPU oracle.  rope and the
split only round products and sums of their inputs, so they are compared bit for bit."""
import pytest
import torch

import cases
from conftest import from_bits, load_golden
from oracle import ops as oracle

pytestmark = pytest.mark.gpu
DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _ops():
    from arke_b200 import ops
    return ops


@pytest.mark.parametrize("tag", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("name", list(cases.ROPE_CASES))
def test_rope_golden_bit_exact(name, tag):
    g = load_golden("rope.npz")
    x, cos, sin = cases.rope_inputs(name, tag)
    y = _ops().rope(x.cuda(), cos.cuda(), sin.cuda()).cpu()
    want = torch.from_numpy(g[f"{name}_f32_y"]) if tag == "f32" else from_bits(g[f"{name}_{tag}_y_bits"], DT[tag])
    assert y.dtype == x.dtype and torch.equal(y, want.view(y.shape))


@pytest.mark.parametrize("shape", [(2, 3, 50, 128), (1, 5, 33, 64), (3, 2, 17, 24), (1, 1, 9, 6), (2, 2, 129, 256), (1, 2, 7, 2)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_rope_vs_oracle_bit_exact_incl_scalar_path(shape, dt):
    B, H, S, D = shape            # D/2 not a multiple of the 16-byte vector takes the per-element kernel
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(B, H, S, D, generator=g).to(dt)
    cos, sin = oracle.make_rope_tables(S, D, dtype=dt)
    y = _ops().rope(x.cuda(), cos.cuda(), sin.cuda()).cpu()
    assert torch.equal(y, oracle.rope(x, cos, sin))
    # arbitrary (non-rotation) tables too, as the façade's generators produce (uniform in [-1, 1])
    c2 = (torch.rand(S, D // 2, generator=g) * 2 - 1).to(dt)
    s2 = (torch.rand(S, D // 2, generator=g) * 2 - 1).to(dt)
    assert torch.equal(_ops().rope(x.cuda(), c2.cuda(), s2.cuda()).cpu(), oracle.rope(x, c2, s2))


def test_rope_3d_input_and_view_input():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(6, 40, 64, generator=g).half()                  # the benchmark driver's [B*H, S, D]
    cos, sin = oracle.make_rope_tables(40, 64, dtype=torch.float16)
    assert torch.equal(_ops().rope(x.cuda(), cos.cuda(), sin.cuda()).cpu(), oracle.rope(x, cos, sin))
    xt = torch.randn(40, 6, 64, generator=g).half().transpose(0, 1)  # non-contiguous view
    assert torch.equal(_ops().rope(xt.cuda(), cos.cuda(), sin.cuda()).cpu(), oracle.rope(xt, cos, sin))


@pytest.mark.parametrize("cfg", [(2, 37, 4, 2, 64, 0), (1, 130, 8, 2, 128, 0), (2, 16, 3, 1, 32, 64), (1, 9, 2, 2, 24, 0), (1, 5, 2, 1, 6, 3)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_qkv_rope_split_vs_oracle_bit_exact(cfg, dt):
    B, S, Hq, Hkv, D, pad = cfg    # pad > 0: the projection output is a column slice of a wider buffer
    W = (Hq + 2 * Hkv) * D
    g = torch.Generator().manual_seed(sum(cfg))
    buf = torch.randn(B * S, W + pad, generator=g).to(dt)
    qkv = buf[:, :W]
    cos, sin = oracle.make_rope_tables(S, D, dtype=dt)
    q, k, v = _ops().qkv_rope_split(buf.cuda()[:, :W], cos.cuda(), sin.cuda(), B, S, Hq, Hkv, D)   # keeps the row stride
    qo, ko, vo = oracle.qkv_rope_split(qkv.contiguous(), cos, sin, B, S, Hq, Hkv, D)
    assert torch.equal(q.cpu(), qo) and torch.equal(k.cpu(), ko) and torch.equal(v.cpu(), vo)


def test_qkv_rope_attention_matches_the_unfused_reference_chain():
    B, S, Hq, Hkv, D, hidden = 2, 200, 8, 2, 128, 256
    g = torch.Generator().manual_seed(21)
    x = (torch.randn(B * S, hidden, generator=g) * 0.5).bfloat16()
    w = (torch.randn(hidden, (Hq + 2 * Hkv) * D, generator=g) * hidden ** -0.5).bfloat16()
    cos, sin = oracle.make_rope_tables(S, D)
    o = _ops().qkv_rope_attention(x.cuda(), w.cuda(), cos.cuda(), sin.cuda(), B, S, Hq, Hkv, D, causal=True).cpu()
    qkv = oracle.matmul(x, w)
    qo, ko, vo = oracle.qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D)
    ref = oracle.gqa_attention(qo, ko, vo, causal=True)
    assert o.shape == (B, Hq, S, D)
    assert torch.allclose(o.float(), ref.float(), rtol=2e-2, atol=2e-2)   # the reference's attention tolerance


def test_rope_empty_and_rejections():
    from arke_b200 import _lib
    ops = _ops()
    cos, sin = oracle.make_rope_tables(0, 64)
    assert ops.rope(torch.empty(2, 2, 0, 64, dtype=torch.bfloat16, device="cuda"), cos.cuda(), sin.cuda()).shape == (2, 2, 0, 64)
    x = torch.randn(1, 2, 8, 64, device="cuda").bfloat16()
    cos, sin = (t.cuda() for t in oracle.make_rope_tables(8, 64))
    with pytest.raises(_lib.UnsupportedError):
        ops.rope(x, cos.float(), sin.float())                           # table dtype differs
    with pytest.raises(_lib.UnsupportedError):
        ops.rope(x, cos[:4], sin[:4])                                   # table length differs
    with pytest.raises(_lib.UnsupportedError):
        ops.rope(torch.randn(1, 2, 8, 63, device="cuda").bfloat16(), cos, sin)   # odd head_dim
    with pytest.raises(_lib.UnsupportedError):
        ops.qkv_rope_split(torch.randn(8, 100, device="cuda").bfloat16(), cos, sin, 1, 8, 2, 1, 64)   # width mismatch
    assert ops.kernel_status() == 0


def test_qkv_rope_split_full_size_properties():
    """BASELINE attention shape (B4, S8192, Hq32, Hkv8, D128): V is a pure copy, sampled tokens are
    bit-identical to the oracle, and rotating by (cos, -sin) afterwards restores Q within rounding."""
    B, S, Hq, Hkv, D = 4, 8192, 32, 8, 128
    W = (Hq + 2 * Hkv) * D
    g = torch.Generator(device="cuda").manual_seed(9)
    qkv = torch.randn(B * S, W, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    cos, sin = (t.cuda() for t in oracle.make_rope_tables(S, D))
    q, k, v = _ops().qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D)
    t = qkv.view(B, S, Hq + 2 * Hkv, D)
    assert torch.equal(v, t[:, :, Hq + Hkv:].permute(0, 2, 1, 3))
    toks = [(0, 0), (0, 1), (1, 4095), (2, 8191), (3, 777), (3, 8191)]
    for b, s in toks:
        row = qkv[b * S + s].cpu().view(1, 1, Hq + 2 * Hkv, D).permute(0, 2, 1, 3)   # [1, Htot, 1, D]
        c1, s1 = cos[s:s + 1].cpu(), sin[s:s + 1].cpu()
        assert torch.equal(q[b, :, s].cpu(), oracle.rope(row[:, :Hq], c1, s1).view(Hq, D))
        assert torch.equal(k[b, :, s].cpu(), oracle.rope(row[:, Hq:Hq + Hkv], c1, s1).view(Hkv, D))
    back = _ops().rope(q, cos, -sin)
    orig = t[:, :, :Hq].permute(0, 2, 1, 3).float()
    err = (back.float() - orig).abs().max().item()
    assert err < 0.15, err            # three bf16 roundings of values up to ~5: a few 2^-7 relative steps
    assert _ops().kernel_status() == 0
