"""GPU parity: quantize_per_token and silu_and_mul(+FP8) through the C ABI vs the CPU oracle and
the reference's golden vectors.  Integer outputs are compared bit-exactly."""
import numpy as np
import pytest
import torch

import cases
from conftest import from_bits, load_golden
from oracle import ops as oracle

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _ops():
    from arke_b200 import ops
    return ops


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.QUANT_CASES))
def test_quantize_int8_golden_bit_exact(name, tag):
    g = load_golden("quantize_interp.npz")
    x = cases.quant_input(name, tag)
    q, s = _ops().quantize_per_token(x.cuda())
    assert np.array_equal(q.cpu().numpy(), g[f"{name}_{tag}_q"])
    assert torch.equal(s.cpu(), x.float().abs().amax(-1) / 127.0)


def test_quantize_ties_and_zero_rows():
    g = load_golden("quantize_interp.npz")
    ties = torch.tensor(cases.TIES)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        q, s = _ops().quantize_per_token(ties.to(dt).cuda())
        assert np.array_equal(q.cpu().numpy(), g["ties_q"]), dt
        assert torch.equal(s.cpu(), torch.ones(2))
    z = torch.zeros(3, 4096, dtype=torch.bfloat16)
    z[1, 5] = 3.0
    q, s = _ops().quantize_per_token(z.cuda())
    assert s[0] == 0 and torch.all(q[0] == 0) and q[1, 5] == 127 and torch.all(q[2] == 0)


@pytest.mark.parametrize("shape", [(127, 769), (333, 4097), (1, 16), (257, 4096), (64, 14336), (40, 32768), (3, 40000), (2048, 4096)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_quantize_int8_vs_oracle_bit_exact(shape, dt):
    x = oracle.make_quant_input(*shape, seed=shape[0] + shape[1], dtype=dt)
    q, s = _ops().quantize_per_token(x.cuda())
    qo, so = oracle.quantize_per_token_interp(x)
    assert torch.equal(q.cpu(), qo)
    assert torch.equal(s.cpu(), so)


def test_quantize_near_tie_stress_bit_exact():
    # rows built so that many quotients x/scale sit within a few ulps of k + 0.5
    g = torch.Generator().manual_seed(7)
    M, N = 64, 4096
    amax = (torch.rand(M, generator=g) * 50 + 1).bfloat16().float()
    k = torch.randint(-126, 126, (M, N), generator=g).float() + 0.5
    x = (k * (amax[:, None] / 127.0)).bfloat16()
    x[:, 0] = amax.bfloat16()
    q, s = _ops().quantize_per_token(x.cuda())
    qo, so = oracle.quantize_per_token_interp(x)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)


def test_quantize_strided_rows_and_empty():
    ops = _ops()
    x = oracle.make_quant_input(32, 8192, seed=5).cuda()
    view = x[:, :4096]  # row stride 8192, still 16-byte aligned
    q, s = ops.quantize_per_token(view)
    qo, so = oracle.quantize_per_token_interp(view.cpu())
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    q, s = ops.quantize_per_token(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 64) and s.shape == (0,)
    x3 = oracle.make_quant_input(24, 256, seed=6).reshape(2, 12, 256).cuda()
    q, s = ops.quantize_per_token(x3)
    assert q.shape == (2, 12, 256) and s.shape == (2, 12)


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.QUANT_BENCH_CASES))
def test_quantize_bench_l1_formula_golden(name, tag):
    g = load_golden("quantize_bench_l1.npz")
    x = cases.quant_input(name, tag, cases.QUANT_BENCH_CASES, "quantb")
    q, s = _ops().quantize_per_token(x.cuda(), formula="bench_l1")
    assert np.array_equal(q.cpu().numpy(), g[f"{name}_{tag}_q"])
    ref_s = from_bits(g[f"{name}_{tag}_scales_bits"], cases.DTYPES[tag]).float()
    assert torch.equal(s.cpu(), ref_s)


@pytest.mark.parametrize("shape", [(64, 4096), (33, 1000), (16, 14336)])
def test_quantize_fp8_vs_oracle(shape):
    x = oracle.make_quant_input(*shape, seed=9)
    q, s = _ops().quantize_per_token(x.cuda(), out_dtype="fp8")
    qo, so = oracle.quantize_per_token_fp8(x)
    assert torch.equal(s.cpu(), so)
    deq, deqo = q.cpu().float() * so[:, None], qo.float() * so[:, None]
    assert torch.allclose(deq, deqo, rtol=2e-2, atol=2e-2)  # stated tolerance for dequantised FP8
    match = (q.cpu().view(torch.uint8) == qo.view(torch.uint8)).float().mean().item()
    assert match > 0.9999, f"e4m3 byte match rate {match}"


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.SILU_CASES))
def test_silu_and_mul_golden(name, tag):
    g = load_golden("silu_and_mul.npz")
    x = cases.silu_input(name, tag)
    ref = from_bits(g[f"{name}_{tag}_y_bits"], cases.DTYPES[tag])
    y = _ops().silu_and_mul(x.cuda()).cpu()
    # tolerance: 2e-2 rtol/atol stated for bf16 outputs; in practice at most one ulp of the dtype
    assert torch.allclose(y.float(), ref.float(), rtol=2e-2, atol=2e-2)
    ulp_off = (y.view(torch.int16).int() - ref.view(torch.int16).int()).abs()
    assert ulp_off.max().item() <= 2  # two roundings (silu, product), approx exp/rcp: a few dtype ulps
    assert (ulp_off == 0).float().mean().item() > 0.99


@pytest.mark.parametrize("shape", [(128, 28672), (37, 1030), (5, 34), (64, 8192), (8, 65536 + 32)])
def test_swiglu_fp8_vs_oracle(shape):
    x = oracle.make_swiglu_input(*shape, seed=shape[1])
    ops = _ops()
    y, yq, s = ops.silu_and_mul(x.cuda(), quantize_fp8=True, return_y=True)
    yq2, s2 = ops.swiglu_fp8(x.cuda())
    assert torch.equal(yq.view(torch.uint8), yq2.view(torch.uint8)) and torch.equal(s, s2)
    yo, yqo, so = oracle.swiglu_fp8(x)
    assert torch.allclose(y.cpu().float(), yo.float(), rtol=2e-2, atol=2e-2)
    # fused == two-step: the quantisation must act on the rounded Y the kernel itself produced
    yq_two, s_two = oracle.quantize_per_token_fp8(y.cpu())
    assert torch.equal(s.cpu(), s_two)
    m2 = (yq.cpu().view(torch.uint8) == yq_two.view(torch.uint8)).float().mean().item()
    assert m2 > 0.9999, f"fused vs two-step e4m3 match rate {m2}"
    deq, deqo = yq.cpu().float() * s.cpu()[:, None], yqo.float() * so[:, None]
    assert torch.allclose(deq, deqo, rtol=2e-2, atol=2e-2)
    assert torch.allclose(s.cpu(), so, rtol=1e-2, atol=0)


def test_silu_and_mul_rejects_odd_width_and_fp32_works():
    from arke_b200 import _lib
    ops = _ops()
    with pytest.raises(_lib.UnsupportedError):
        ops.silu_and_mul(torch.randn(4, 33, device="cuda").bfloat16())
    x = torch.randn(9, 70)
    y = ops.silu_and_mul(x.cuda()).cpu()
    assert torch.allclose(y, oracle.silu_and_mul(x), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("out_dtype", ["int8", "fp8"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_fast_quotient_equals_ieee_division_exhaustively(dt, out_dtype):
    # every finite 16-bit x against every positive 16-bit row maximum amax >= |x| (about 1e9 pairs)
    bad, n = _ops().selftest_quant_division(dt, out_dtype)
    assert n > 2e8
    assert bad == 0, f"{bad} of {n} quotients differ from the IEEE division"


def test_quantize_rows_full_of_exact_ties_bit_exact_and_not_slow():
    # x = +-amax/2 gives x/scale = +-63.5 exactly: every such element is a rounding tie
    M, N = 2048, 4096
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, N, generator=g).bfloat16()
    amax = x.abs().amax(-1, keepdim=True)
    half = (amax.float() / 2).bfloat16()
    mask = torch.rand(M, N, generator=g) < 0.25
    x = torch.where(mask, half * torch.where(torch.rand(M, N, generator=g) < 0.5, 1.0, -1.0).bfloat16(), x)
    q, s = _ops().quantize_per_token(x.cuda())
    qo, so = oracle.quantize_per_token_interp(x)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    assert (qo.abs() == 64).float().mean() > 0.1      # the ties are really there (63.5 -> 64)


def test_quantize_extreme_magnitude_rows_take_the_division_path():
    # rows whose maximum is far outside the usual range (bf16 spans 2^-126 .. 2^127)
    rows = []
    for mag in (1e-38, 3e-30, 1e-19, 1.0, 1e19, 1e30, 3e38):
        g = torch.Generator().manual_seed(int(abs(hash(mag)) % 1000))
        rows.append((torch.randn(4096, generator=g) * mag / 4).clamp(-3.3e38, 3.3e38))
    x = torch.stack(rows).bfloat16()
    q, s = _ops().quantize_per_token(x.cuda())
    qo, so = oracle.quantize_per_token_interp(x)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(q.cpu(), qo)


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.RMS_CASES))
def test_rmsnorm_golden(name, tag):
    g = load_golden("rmsnorm.npz")
    x, res, w = cases.rms_inputs(name, tag)
    dt = cases.DTYPES[tag]
    for key, r in (("y", None), ("yres", res)):
        ref32 = torch.from_numpy(g[f"{name}_{tag}_{key}"])          # interpreter output (fp32)
        y = _ops().rmsnorm(x.cuda(), w.cuda(), residual=r.cuda() if r is not None else None).cpu()
        assert y.dtype == dt
        assert torch.allclose(y.float(), ref32, rtol=1e-2, atol=1e-2)   # the V1 rule of the reference
        ref = ref32.to(dt)                                             # correctly rounded 16-bit result
        ulp = (y.view(torch.int16).int() - ref.view(torch.int16).int()).abs()
        assert ulp.max().item() <= 1 and (ulp == 0).float().mean().item() > 0.98


@pytest.mark.parametrize("quant", ["int8", "fp8"])
@pytest.mark.parametrize("shape", [(256, 4096), (33, 1000), (7, 130), (64, 8192), (16, 12288)])
def test_rmsnorm_fused_quantize_equals_two_step(shape, quant):
    M, N = shape
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, N, generator=g).bfloat16()
    res = torch.randn(M, N, generator=g).bfloat16()
    w = (1.0 + 0.1 * torch.randn(N, generator=g)).bfloat16()
    ops = _ops()
    y, q, s = ops.rmsnorm(x.cuda(), w.cuda(), residual=res.cuda(), quantize=quant)
    q2, s2 = ops.rmsnorm(x.cuda(), w.cuda(), residual=res.cuda(), quantize=quant, return_y=False)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    assert torch.allclose(y.cpu().float(), oracle.rmsnorm(x, w, residual=res).float(), rtol=2e-2, atol=2e-2)
    # fused == quantize_per_token of the kernel's own y, bit for bit (oracle quantiser on that y)
    if quant == "int8":
        qo, so = oracle.quantize_per_token_interp(y.cpu())
        assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    else:
        qo, so = oracle.quantize_per_token_fp8(y.cpu())
        assert torch.equal(s.cpu(), so)
        assert torch.allclose(q.cpu().float() * so[:, None], qo.float() * so[:, None], rtol=2e-2, atol=2e-2)
        assert (q.cpu().view(torch.uint8) == qo.view(torch.uint8)).float().mean() > 0.9999
    assert torch.allclose(ops.rmsnorm(x.float().cuda(), w.float().cuda()).cpu(), oracle.rmsnorm(x.float(), w.float()), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 4096), (33, 1000), (5, 17), (2048, 14336)])
def test_dequantize_per_channel_vs_reference_formula(shape, out_dtype):
    M, N = shape
    g = torch.Generator().manual_seed(M + N)
    x = torch.randint(-127, 128, (M, N), generator=g, dtype=torch.int32).to(torch.int8)
    scale = torch.rand(N, generator=g) * 0.99 + 0.01
    zp = torch.randint(-10, 11, (N,), generator=g, dtype=torch.int32).to(torch.int8)
    y = _ops().dequantize_per_channel(x.cuda(), scale.cuda(), zp.cuda(), out_dtype=out_dtype).cpu()
    ref = ((x.float() - zp.float()) * scale)          # ref_dequantize_per_channel
    assert torch.equal(y, ref.to(out_dtype))
    y0 = _ops().dequantize_per_channel(x.cuda(), scale.cuda(), None).cpu()
    assert torch.equal(y0, x.float() * scale)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(300, 4096), (64, 14336), (17, 256)])
def test_quantize_bench_l1_formula_fast_path_vs_oracle(shape, dt):
    """The register-resident kernel also serves the benchmark driver's formula
    (benchmarks/bench_l1.py:443-448); bit-exact with its restatement, all-zero and outlier rows
    included."""
    x = oracle.make_quant_input(*shape, seed=shape[0]).to(dt)
    x[3] = 0
    x[5, 7] = 60000.0 if dt == torch.float16 else 3e38
    q, s = _ops().quantize_per_token(x.cuda(), formula="bench_l1")
    qo, so = oracle.quantize_per_token_bench_l1(x)
    assert torch.equal(q.cpu(), qo)
    assert torch.equal(s.cpu(), so.float())
