"""GPU: failure detection without faulting the GPU — typed host-side rejections, empty inputs, the
bounded-wait status word, and run-to-run determinism (the reference's staged gate repeats a run
three times and requires identical results, arke/agent/verification.py:182-191)."""
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu


def _ops():
    from arke_b200 import ops
    return ops


def test_expired_wait_sets_status_word_and_context_stays_usable():
    from arke_b200 import _lib
    ops = _ops()
    assert ops.kernel_status() == 0
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.LIB.arke_b200_selftest_wait_timeout(2_000_000, stream))   # ~1 ms of SM cycles
    torch.cuda.synchronize()
    assert ops.kernel_status() != 0          # the expiry was recorded ...
    assert ops.kernel_status() == 0          # ... and reading it cleared it
    x = oracle.make_quant_input(64, 512, seed=1)
    q, s = ops.quantize_per_token(x.cuda())  # the context is still healthy
    assert torch.equal(q.cpu(), oracle.quantize_per_token_interp(x)[0])
    with pytest.raises(_lib.ArkeB200Error):
        _lib.check(_lib.LIB.arke_b200_selftest_wait_timeout(0, stream))


def test_empty_inputs_are_no_ops():
    ops = _ops()
    dev = "cuda"
    assert ops.silu_and_mul(torch.empty(0, 64, dtype=torch.bfloat16, device=dev)).shape == (0, 32)
    y = ops.w8a8_gemm(torch.empty(0, 64, dtype=torch.int8, device=dev), None,
                      torch.zeros(64, 32, dtype=torch.int8, device=dev), None)
    assert y.shape == (0, 32)
    o, lse = ops.gqa_fwd(torch.empty(0, 4, 16, 128, dtype=torch.bfloat16, device=dev),
                         torch.empty(0, 2, 16, 128, dtype=torch.bfloat16, device=dev),
                         torch.empty(0, 2, 16, 128, dtype=torch.bfloat16, device=dev))
    assert o.shape == (0, 4, 16, 128) and lse.shape == (0, 4, 16)
    assert ops.rmsnorm(torch.empty(0, 64, dtype=torch.bfloat16, device=dev), torch.ones(64, dtype=torch.bfloat16, device=dev)).shape == (0, 64)
    assert ops.kernel_status() == 0


def test_host_side_rejections_are_typed():
    from arke_b200 import _lib
    ops = _ops()
    dev = "cuda"
    with pytest.raises(_lib.UnsupportedError):          # int64 activations
        ops.quantize_per_token(torch.zeros(4, 64, dtype=torch.int64, device=dev))
    with pytest.raises(_lib.UnsupportedError):          # mixed operand dtypes
        ops.quant_gemm(torch.zeros(16, 64, dtype=torch.int8, device=dev), None,
                       torch.zeros(64, 32, dtype=torch.float8_e4m3fn, device=dev), None)
    with pytest.raises(_lib.UnsupportedError):          # inner dimensions differ
        ops.w8a8_gemm(torch.zeros(16, 64, dtype=torch.int8, device=dev), None,
                      torch.zeros(48, 32, dtype=torch.int8, device=dev), None)
    with pytest.raises(_lib.UnsupportedError):          # hidden size not a multiple of 8
        x, w, l = oracle.make_flce_inputs(8, 36, 64, seed=1)
        ops.fused_linear_ce(x.cuda(), w.cuda(), l.cuda())
    with pytest.raises(_lib.ArkeB200Error):             # tensors on different devices / CPU
        ops.matmul(torch.zeros(8, 8, dtype=torch.bfloat16), torch.zeros(8, 8, dtype=torch.bfloat16, device=dev))


def test_three_runs_bit_identical():
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-128, 128, (1536, 1024), generator=g, dtype=torch.int32).to(torch.int8).cuda()
    w = torch.randint(-127, 128, (1024, 2048), generator=g, dtype=torch.int32).to(torch.int8).cuda()
    sa, sw = torch.rand(1536, generator=g).cuda(), torch.rand(2048, generator=g).cuda()
    ys = [ops.w8a8_gemm(a, sa, w, sw) for _ in range(3)]
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2])
    x, wl, lab = oracle.make_flce_inputs(1024, 512, 20000, seed=4)
    xd, wd, ld = x.cuda(), wl.cuda(), lab.cuda()
    rs = [ops.fused_linear_ce(xd, wd, ld) for _ in range(3)]
    assert all(torch.equal(rs[0][0], r[0]) and torch.equal(rs[0][1], r[1]) for r in rs[1:])
    xs = oracle.make_swiglu_input(256, 8192, seed=5).cuda()
    zs = [ops.swiglu_fp8(xs) for _ in range(3)]
    assert all(torch.equal(zs[0][0].view(torch.uint8), z[0].view(torch.uint8)) and torch.equal(zs[0][1], z[1]) for z in zs[1:])
    assert ops.kernel_status() == 0
