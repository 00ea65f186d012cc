"""GPU parity: W8A8 / FP8 GEMM and the dense 16-bit GEMM (tcgen05) vs the CPU oracle.
int32 accumulators are compared bit-exactly; bf16 outputs within rtol = atol = 2e-2."""
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _ops():
    from arke_b200 import ops
    return ops


def _rand_i8(shape, g, lo=-128, hi=128):
    return torch.randint(lo, hi, shape, generator=g, dtype=torch.int32).to(torch.int8)


def _status_ok():
    assert _ops().kernel_status() == 0, "a bounded device-side wait expired"


@pytest.mark.parametrize("layout", ["kn", "nk"])
def test_w8a8_one_tile_known_answer(layout):
    # 128 x 128 x 64 with operands whose product is known in closed form:
    # A[i,k] = (i % 7) - 3, W[k,j] = (j % 5) - 2  ->  acc[i,j] = 64 * A_i * W_j
    M, N, K = 128, 128, 64
    a = ((torch.arange(M) % 7) - 3).to(torch.int8)[:, None].expand(M, K).contiguous()
    wcol = ((torch.arange(N) % 5) - 2).to(torch.int8)
    w = wcol[None, :].expand(K, N).contiguous()
    wd = w if layout == "kn" else w.t().contiguous()
    acc = _ops().quant_gemm(a.cuda(), None, wd.cuda(), None, out_dtype=None, w_layout=layout, return_acc=True)
    _status_ok()
    expect = (64 * a[:, :1].int() * wcol[None, :].int())
    assert torch.equal(acc.cpu(), expect)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 512, 1024), (200, 304, 176), (1000, 1040, 4096), (77, 128, 64), (130, 4000, 528)])
def test_w8a8_acc_bit_exact_and_dequant(shape, layout):
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 7 + N)
    a = _rand_i8((M, K), g)
    w = _rand_i8((K, N), g, -127, 128)
    sa = torch.rand(M, generator=g) * 0.05 + 0.001
    sw = torch.rand(N, generator=g) * 0.019 + 0.001
    wd = w if layout == "kn" else w.t().contiguous()
    y, acc = _ops().w8a8_gemm(a.cuda(), sa.cuda(), wd.cuda(), sw.cuda(), w_layout=layout, return_acc=True)
    _status_ok()
    yo, acco = oracle.w8a8_gemm(a, sa, w, sw)
    assert torch.equal(acc.cpu(), acco)                       # int32 accumulators bit-exact
    assert torch.allclose(y.cpu().float(), yo.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(y.cpu(), yo)                           # same fp32 expression, same rounding


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_w8a8_other_output_dtypes_and_no_scales(out_dtype):
    g = torch.Generator().manual_seed(5)
    a, w = _rand_i8((192, 256), g), _rand_i8((256, 320), g)
    sa = torch.rand(192, generator=g) * 1e-2
    y = _ops().w8a8_gemm(a.cuda(), sa.cuda(), w.cuda(), None, out_dtype=out_dtype)
    _status_ok()
    ref = oracle.dequant_epilogue(oracle.int8_gemm_acc(a, w), sa, None, out_dtype)
    assert torch.equal(y.cpu(), ref)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("shape", [(128, 256, 128), (300, 528, 1024), (1024, 1024, 2048)])
def test_fp8_gemm_vs_oracle(shape, layout):
    M, N, K = shape
    g = torch.Generator().manual_seed(N)
    a = (torch.randn(M, K, generator=g) * 2).to(FP8)
    w = (torch.randn(K, N, generator=g) * 2).to(FP8)
    sa = torch.rand(M, generator=g) * 0.05 + 0.001
    sw = torch.rand(N, generator=g) * 0.019 + 0.001
    wd = w if layout == "kn" else w.t().contiguous()
    y, acc = _ops().fp8_gemm(a.cuda(), sa.cuda(), wd.cuda(), sw.cuda(), w_layout=layout, return_acc=True)
    _status_ok()
    yo, acco = oracle.fp8_gemm(a, sa, w, sw)
    assert torch.allclose(acc.cpu(), acco, rtol=1e-3, atol=1e-2)   # fp32 accumulation order differs
    assert torch.allclose(y.cpu().float(), yo.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 384, 512), (1000, 1000, 1000 - 8), (520, 2048, 4096)])
def test_matmul_16bit_vs_oracle(shape, dt, layout):
    M, N, K = shape
    g = torch.Generator().manual_seed(K)
    a = torch.randn(M, K, generator=g).to(dt)
    b = torch.randn(K, N, generator=g).to(dt)
    bd = b if layout == "kn" else b.t().contiguous()
    c = _ops().matmul(a.cuda(), bd.cuda(), b_layout=layout)
    _status_ok()
    ref = oracle.matmul(a, b)
    # bench_l1 tolerance for matmul is 1e-2 on fp16; outputs here are O(sqrt(K)), rounded to 16 bit
    assert torch.allclose(c.cpu().float(), ref, rtol=2e-2, atol=2e-2 * (K ** 0.5))
    rel = (c.cpu().float() - ref).norm() / ref.norm()
    assert rel < 4e-3


def test_w8a8_linearity_at_full_config_size():
    # size-independent property at the benchmark shape (8192 x 14336 x 4096):
    # acc(A, W1 + W2) == acc(A, W1) + acc(A, W2), and a sampled block equals the oracle
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    M, N, K = 8192, 14336, 4096
    a = _rand_i8((M, K), g).cuda()
    w1 = _rand_i8((K, N), g, -63, 64).cuda()
    w2 = _rand_i8((K, N), g, -63, 64).cuda()
    acc1 = ops.quant_gemm(a, None, w1, None, out_dtype=None, return_acc=True)
    acc2 = ops.quant_gemm(a, None, w2, None, out_dtype=None, return_acc=True)
    acc12 = ops.quant_gemm(a, None, (w1 + w2), None, out_dtype=None, return_acc=True)
    _status_ok()
    assert torch.equal(acc12, acc1 + acc2)
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191])
    cols = slice(14336 - 300, 14336)
    ref = oracle.int8_gemm_acc(a[rows].cpu(), w1[:, cols].cpu())
    assert torch.equal(acc1[rows][:, cols].cpu(), ref)


def test_gemm_rejects_misaligned_strides():
    from arke_b200 import _lib
    a = torch.zeros(16, 24, dtype=torch.int8, device="cuda")   # 24-byte rows: not a multiple of 16
    w = torch.zeros(24, 32, dtype=torch.int8, device="cuda")
    with pytest.raises(_lib.UnsupportedError):
        _ops().w8a8_gemm(a, None, w, None)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("shape", [(128, 128, 32), (256, 384, 512), (1000, 1000, 1000), (1024, 1024, 1024)])
def test_matmul_fp32_as_tf32(shape, layout):
    M, N, K = shape
    g = torch.Generator().manual_seed(K + 1)
    a, b = torch.randn(M, K, generator=g), torch.randn(K, N, generator=g)
    bd = b if layout == "kn" else b.t().contiguous()
    c = _ops().matmul(a.cuda(), bd.cuda(), b_layout=layout)
    _status_ok()
    ref = a.double() @ b.double()
    assert c.dtype == torch.float32
    # the reference's V1 rule: allclose(rtol = atol = 1e-2) (arke/agent/tools.py:510-517); TF32 keeps
    # 10 significand bits, so the error of a length-K dot product is ~1e-3 * sqrt(K) absolute
    assert torch.allclose(c.cpu().double(), ref, rtol=1e-2, atol=1e-3 * (K ** 0.5) * 4)
    assert ((c.cpu().double() - ref).norm() / ref.norm()).item() < 2e-3


@pytest.mark.parametrize("shape", [(300, 528, 192), (1024, 1280, 256), (129, 2048, 4096)])
def test_tile_option_selects_the_kernel_without_changing_results(shape):
    """``gemm_tile_m`` (what a strategy's tile decision maps to) forces the one-CTA or the CTA-pair
    kernel on any shape; integer accumulators must be identical and bf16 results bit-identical."""
    from arke_b200 import ops
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
    w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8).cuda()
    ref = oracle.int8_gemm_acc(xq.cpu(), w.cpu())
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().cuda()
    b = (torch.randn(K, N, generator=g) * 0.5).bfloat16().cuda()
    outs = []
    for tm in (128, 256):
        with ops.options(gemm_tile_m=tm, gemm_band_mb=8):
            acc = ops.quant_gemm(xq, None, w, None, out_dtype=None, return_acc=True)
            outs.append(ops.matmul(a, b))
        assert torch.equal(acc.cpu(), ref), tm
    assert torch.equal(outs[0], outs[1])
    assert ops.kernel_status() == 0


def test_dynamic_and_round_robin_tile_assignment_agree_and_counters_are_cleared():
    """The CTA pairs take their tiles from a device counter (default) or round robin
    (``gemm_static_sched=1``): the results must be bit-identical, every tile must be computed
    exactly once whatever the order, and repeated launches (the last pair to leave zeroes the
    counters; there are 64 counter slots) must keep working."""
    from arke_b200 import ops
    g = torch.Generator().manual_seed(5)
    # many more tiles than CTA pairs, ragged edges, a long-K case and the transposed-A form
    for (M, N, K) in [(4096, 6144, 512), (2504, 9008, 384), (1024, 1536, 8192)]:
        a = (torch.randn(M, K, generator=g) * 0.5).bfloat16().cuda()
        b = (torch.randn(K, N, generator=g) * 0.5).bfloat16().cuda()
        xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
        w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8).cuda()
        at = a.t().contiguous()
        with ops.options(gemm_static_sched=1, gemm_tile_m=256):
            ref, ref_tn = ops.matmul(a, b), ops.matmul_tn(at, b)
            ref_acc = ops.quant_gemm(xq, None, w, None, out_dtype=None, return_acc=True)
        with ops.options(gemm_tile_m=256):
            for _ in range(70 if K == 512 else 3):           # more launches than counter slots
                out = ops.matmul(a, b)
            assert torch.equal(out, ref) and torch.equal(ops.matmul_tn(at, b), ref_tn)
            assert torch.equal(ops.quant_gemm(xq, None, w, None, out_dtype=None, return_acc=True), ref_acc)
        assert ops.kernel_status() == 0
    ref64 = (a.double().cpu() @ b.double().cpu())
    assert ((ref.cpu().double() - ref64).norm() / ref64.norm()).item() < 5e-3


def test_narrow_units_of_the_last_wave_do_not_change_a_bit():
    """The CTA-pair GEMM cuts the tiles of its last, partly filled wave into 2 or 4 narrower units
    along N (MMAs with N = 128 / 64 that read a column range of the staged B tile).  Every output
    element must be the one the whole-tile launch (``gemm_no_split=1``) produces, bit for bit, for
    every operand kind, both B layouts, the transposed-A form and ragged edges; int8 must also be
    the exact integer product."""
    from arke_b200 import ops
    g = torch.Generator().manual_seed(11)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    pairs = sms // 2
    cases = [(8192, 14336, 4096),   # the headline shape: 1792 tiles, 16 in the last wave -> 4 units each
             (1024, 14336, 4096),   # its 1024-row shard: 224 tiles, 2 left over
             (1024, 4864, 1024),    # 76 tiles
             (1100, 4880, 1008),    # ragged M / N / K: 100 tiles, 26 left over -> 2 units each
             (1024, 2048, 512),     # a single wave of 32 tiles -> 2 units each, round-robin assignment
             (1280, 2320, 272)]     # ragged single wave (50 tiles: left whole)
    for (M, N, K) in cases:
        tiles = ((M + 255) // 256) * ((N + 255) // 256)
        xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
        w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8).cuda()
        sx = (torch.rand(M, generator=g) * 0.02 + 0.001).cuda()
        sw = (torch.rand(N, generator=g) * 0.02 + 0.001).cuda()
        wt = w.t().contiguous()
        big = M * N > 1400 * 5000
        outs = {}
        for split in (0, 1):
            with ops.options(gemm_no_split=1 - split, gemm_tile_m=256):
                r = {}
                r["i8_kn"] = ops.w8a8_gemm(xq, sx, w, sw, return_acc=True)
                r["i8_nk"] = ops.w8a8_gemm(xq, sx, wt, sw, w_layout="nk", return_acc=True)
                if not big:
                    a16 = (xq.float() / 64).bfloat16()
                    b16 = (w.float() / 64).bfloat16()
                    r["bf16_kn"] = (ops.matmul(a16, b16),)
                    r["bf16_nk"] = (ops.matmul(a16, b16.t().contiguous(), b_layout="nk"),)
                    if M % 8 == 0:
                        r["f16_tn"] = (ops.matmul_tn(a16.half().t().contiguous(), b16.half()),)
                    a8 = (xq.float() / 32).to(torch.float8_e4m3fn)
                    b8 = (w.float() / 32).to(torch.float8_e4m3fn)
                    r["fp8_kn"] = ops.fp8_gemm(a8, sx, b8, sw, return_acc=True)
                    if K % 4 == 0:
                        r["tf32_nk"] = (ops.matmul(xq.float(), wt.float(), b_layout="nk"),)
                outs[split] = r
        for key, whole in outs[0].items():
            for t0, t1 in zip(whole, outs[1][key]):
                assert torch.equal(t0, t1), (M, N, K, key, tiles % pairs)
        if not big:
            ref = xq.cpu().int() @ w.cpu().int()
            assert torch.equal(outs[1]["i8_kn"][1].cpu(), ref) and torch.equal(outs[1]["i8_nk"][1].cpu(), ref)
        assert ops.kernel_status() == 0

