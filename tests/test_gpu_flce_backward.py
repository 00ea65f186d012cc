"""GPU: backward of fused linear + cross-entropy and the transposed-A GEMM it uses, vs the CPU
oracle (autograd of the reference's forward expression).  The logits gradient is held in 16 bits,
so gradients are compared with the tolerance the reference uses for this op's forward (1e-2),
relative to the gradient's magnitude."""
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu


def _ops():
    from arke_b200 import ops
    return ops


def _close(got: torch.Tensor, ref: torch.Tensor, tol: float = 1e-2):
    got, ref = got.float().cpu(), ref.float()
    scale = ref.abs().max().item() + 1e-30
    err = (got - ref).abs().max().item()
    fro = ((got - ref).norm() / (ref.norm() + 1e-30)).item()
    assert err <= tol * scale and fro <= tol, (err / scale, fro)


@pytest.mark.parametrize("shape", [(64, 200, 128, 64), (304, 520, 192, 256), (1024, 1280, 256, 512), (136, 2048, 4096, 64)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b_layout", ["kn", "nk"])
def test_matmul_tn_vs_oracle(shape, dt, b_layout):
    M, N, K, _ = shape
    g = torch.Generator().manual_seed(M + N + K)
    a_t = (torch.randn(K, M, generator=g) * 0.5).to(dt)
    b = (torch.randn(K, N, generator=g) * 0.5).to(dt)
    ref = a_t.float().T @ b.float()
    bb = b if b_layout == "kn" else b.T.contiguous()
    for tm in (128, 256):
        with _ops().options(gemm_tile_m=tm):
            c = _ops().matmul_tn(a_t.cuda(), bb.cuda(), b_layout=b_layout, out_dtype=torch.float32)
        assert torch.allclose(c.cpu(), ref, rtol=1e-3, atol=1e-2 * ref.abs().max().item()), tm
    # a row-strided A (a column slice of a wider buffer) is taken as is
    wide = torch.zeros(K, M + 24, dtype=dt)
    wide[:, :M] = a_t
    c2 = _ops().matmul_tn(wide.cuda()[:, :M], bb.cuda(), b_layout=b_layout, out_dtype=torch.float32)
    assert torch.allclose(c2.cpu(), ref, rtol=1e-3, atol=1e-2 * ref.abs().max().item())
    assert _ops().kernel_status() == 0


@pytest.mark.parametrize("cfg", [(32, 64, 1000), (130, 256, 5003), (256, 128, 2048), (1100, 512, 3000)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_flce_backward_vs_autograd_of_the_reference_forward(cfg, dt):
    M, D, V = cfg
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=M + V, dtype=dt, ignore_frac=0.1)
    dxo, dwo = oracle.fused_linear_ce_backward(x, w, labels)
    for tm in (128, 256):
        with _ops().options(gemm_tile_m=tm):
            dx, dw = _ops().fused_linear_ce_backward(x.cuda(), w.cuda(), labels.cuda())
        assert dx.dtype == dt and dw.dtype == dt and dx.shape == x.shape and dw.shape == w.shape
        _close(dx, dxo)
        _close(dw, dwo)
    ign = (labels == -100)
    assert ign.any() and torch.all(dx.cpu()[ign] == 0)          # ignored rows get exactly zero
    assert _ops().kernel_status() == 0


def test_flce_backward_grad_scale_skips_and_all_ignored():
    x, w, labels = oracle.make_flce_inputs(200, 128, 1500, seed=3)
    dxo, dwo = oracle.fused_linear_ce_backward(x, w, labels)
    dx, dw = _ops().fused_linear_ce_backward(x.cuda(), w.cuda(), labels.cuda(), grad=0.25, want_dw=False)
    assert dw is None
    _close(dx, dxo * 0.25)
    dx, dw = _ops().fused_linear_ce_backward(x.cuda(), w.cuda(), labels.cuda(), want_dx=False)
    assert dx is None
    _close(dw, dwo)
    all_ign = torch.full_like(labels, -100)
    dx, dw = _ops().fused_linear_ce_backward(x.cuda(), w.cuda(), all_ign.cuda())
    assert torch.all(dx == 0) and torch.all(dw == 0)


def test_flce_backward_vocab_slices_sum_to_the_whole():
    """Each vocabulary slice, given the global lse, yields its rows of dW and its share of dX."""
    M, D, V = 256, 128, 4096
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=8)
    xc, wc, lc = x.cuda(), w.cuda(), labels.cuda()
    part = _ops().fused_linear_ce(xc, wc, lc, want_partials=True)
    lse = part[:, 0] + torch.log(part[:, 1])
    dx_full, dw_full = _ops().fused_linear_ce_backward(xc, wc, lc, lse=lse)
    dx_sum = torch.zeros(M, D, device="cuda")
    for r in range(4):
        v0, v1 = r * V // 4, (r + 1) * V // 4
        dx_r, dw_r = _ops().fused_linear_ce_backward(xc, wc[v0:v1].contiguous(), lc, lse=lse, vocab_offset=v0)
        dx_sum += dx_r.float()
        assert torch.equal(dw_r, dw_full[v0:v1])                 # same tiles, same arithmetic
    _close(dx_sum, dx_full.float().cpu())
    dxo, _ = oracle.fused_linear_ce_backward(x, w, labels)
    _close(dx_sum, dxo)


def test_flce_backward_rejections():
    from arke_b200 import _lib
    x, w, labels = (t.cuda() for t in oracle.make_flce_inputs(64, 64, 500, seed=1))
    with pytest.raises(_lib.UnsupportedError):
        _ops().fused_linear_ce_backward(x.float(), w.float(), labels)
    with pytest.raises(_lib.UnsupportedError):
        _ops().fused_linear_ce_backward(x, w, labels.float())
    with pytest.raises(_lib.ArkeB200Error):
        _ops().fused_linear_ce_backward(x, w, labels, workspace=torch.empty(1024, dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        _ops().fused_linear_ce_backward(x, w, labels, vocab_offset=100)
    assert _ops().kernel_status() == 0


def test_autograd_function_matches_torch_autograd():
    from arke_b200.autograd import fused_linear_cross_entropy
    x, w, labels = oracle.make_flce_inputs(300, 256, 3000, seed=12, ignore_frac=0.05)
    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    loss = fused_linear_cross_entropy(xg, wg, labels.cuda())
    (loss * 2.0).backward()                                       # upstream gradient 2.0
    assert abs(loss.item() - oracle.fused_linear_ce(x, w, labels)[1].item()) <= 1e-3
    dxo, dwo = oracle.fused_linear_ce_backward(x, w, labels)
    _close(xg.grad, dxo * 2.0)
    _close(wg.grad, dwo * 2.0)
    # only one input requires a gradient: the other GEMM is skipped
    xg2 = x.cuda().requires_grad_(True)
    fused_linear_cross_entropy(xg2, w.cuda(), labels.cuda()).backward()
    _close(xg2.grad, dxo)


def test_f16_backward_keeps_the_softmax_tail_with_many_tokens():
    """n_valid = 4096 and a near-uniform softmax over 16384 classes: p ~ 6e-5 per class.  Scaled by
    1 / n_valid before the 16-bit rounding (1.5e-8) every off-target entry of the logits gradient
    would flush to zero in f16 and dX would keep only its one-hot term; the gradient is stored
    unscaled instead and the off-target part must match the oracle."""
    M, D, V = 4096, 128, 16384
    g = torch.Generator().manual_seed(77)
    x = torch.randn(M, D, generator=g).half()
    w = (torch.randn(V, D, generator=g) * 0.02).half()          # logits ~ N(0, 0.23): near-uniform softmax
    labels = torch.randint(0, V, (M,), generator=g)
    # dX is taken in fp32: at 1e-7 the off-target part is below what an f16 OUTPUT can hold
    # (smallest subnormal 6e-8), which is the caller's choice of dtype, not the kernel's arithmetic
    dx, dw = _ops().fused_linear_ce_backward(x.cuda(), w.cuda(), labels.cuda(), dx_dtype=torch.float32)
    dxo, dwo = oracle.fused_linear_ce_backward(x, w, labels)
    # off-target part of dX:  dX + w[label] / n  =  (1/n) sum_j p_j w_j
    onehot = w.float()[labels] / M
    off_ref = dxo + onehot
    off_got = dx.float().cpu() + onehot
    assert off_ref.abs().max().item() > 0
    rel = ((off_got - off_ref).norm() / off_ref.norm()).item()
    assert rel < 0.05, rel                                       # all-zero tail would give rel = 1
    _close(dx, dxo)
    _close(dw, dwo)
    assert _ops().kernel_status() == 0


def test_backward_fp32_dx_and_device_scalar_grad():
    x, w, labels = oracle.make_flce_inputs(300, 128, 2500, seed=21)
    xc, wc, lc = x.cuda(), w.cuda(), labels.cuda()
    dxo, dwo = oracle.fused_linear_ce_backward(x, w, labels)
    dx32, dw = _ops().fused_linear_ce_backward(xc, wc, lc, dx_dtype=torch.float32)
    assert dx32.dtype == torch.float32 and dw.dtype == x.dtype
    _close(dx32, dxo)
    dx16, _ = _ops().fused_linear_ce_backward(xc, wc, lc, want_dw=False)
    assert torch.equal(dx32.to(x.dtype), dx16)                   # same accumulators, rounded once
    gdev = torch.tensor(0.5, device="cuda")
    dxg, dwg = _ops().fused_linear_ce_backward(xc, wc, lc, grad=gdev)
    dxh, dwh = _ops().fused_linear_ce_backward(xc, wc, lc, grad=0.5)
    assert torch.equal(dxg, dxh) and torch.equal(dwg, dwh)
    from arke_b200 import _lib
    with pytest.raises(_lib.UnsupportedError):
        _ops().fused_linear_ce_backward(xc, wc, lc, dx_dtype=torch.float64)


def test_autograd_all_ignored_is_nan_like_the_reference():
    from arke_b200.autograd import fused_linear_cross_entropy
    x, w, labels = oracle.make_flce_inputs(64, 64, 500, seed=2)
    ign = torch.full_like(labels, -100)
    loss = fused_linear_cross_entropy(x.cuda(), w.cuda(), ign.cuda())
    assert torch.isnan(loss) and torch.isnan(oracle.fused_linear_ce(x, w, ign)[1])
    assert torch.isnan(_ops().fused_linear_ce(x.cuda(), w.cuda(), ign.cuda())[1])
