"""GPU parity: fused linear + cross-entropy (tcgen05 GEMM with online-softmax epilogue) vs the
reference interpreter's golden means and the CPU oracle.  fp32 losses: |diff| <= 1e-3."""
import pytest
import torch

import cases
from conftest import load_golden
from oracle import ops as oracle

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _ops():
    from arke_b200 import ops
    return ops


@pytest.mark.parametrize("tag", list(cases.DTYPES))
@pytest.mark.parametrize("name", list(cases.FLCE_CASES))
def test_flce_golden_mean_and_oracle_per_token(name, tag):
    g = load_golden("flce.npz")
    x, w, labels = cases.flce_inputs(name, tag)
    tok, mean = _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.cuda())
    assert _ops().kernel_status() == 0
    assert abs(mean.item() - float(g[f"{name}_{tag}_mean"])) <= TOL
    tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
    assert torch.allclose(tok.cpu(), tok_o, rtol=TOL, atol=TOL)
    assert torch.all(tok.cpu()[labels == -100] == 0)


@pytest.mark.parametrize("shape", [(128, 64, 256), (1, 64, 7), (300, 512, 3000), (1024, 1024, 32000), (257, 136, 10007)])
def test_flce_ragged_shapes_vs_oracle(shape):
    M, D, V = shape
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=M + V, ignore_frac=0.05)
    tok, mean = _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.cuda())
    assert _ops().kernel_status() == 0
    tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
    assert torch.allclose(tok.cpu(), tok_o, rtol=TOL, atol=TOL)
    assert abs(mean.item() - mean_o.item()) <= TOL


def test_flce_large_logits_are_stable():
    # logits of magnitude ~ +-60: the online softmax must not overflow
    M, D, V = 256, 256, 4096
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=3)
    w = (w.float() * 12).bfloat16()
    tok, mean = _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.cuda())
    tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
    assert torch.isfinite(tok).all()
    assert torch.allclose(tok.cpu(), tok_o, rtol=TOL, atol=2e-3)


def test_flce_all_ignored_gives_nan_mean_like_torch():
    x, w, labels = oracle.make_flce_inputs(64, 64, 512, seed=1)
    labels[:] = -100
    tok, mean = _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.cuda())
    assert torch.all(tok == 0) and torch.isnan(mean)
    assert torch.isnan(oracle.fused_linear_ce(x, w, labels)[1])


@pytest.mark.parametrize("G", [2, 4, 8])
def test_flce_vocab_shard_partials_combine(G):
    M, D, V = 512, 256, 16032 * 2
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=G)
    ops = _ops()
    xd, ld = x.cuda(), labels.cuda()
    bounds = [V * i // G for i in range(G + 1)]
    parts = torch.stack([ops.fused_linear_ce(xd, w[bounds[i]:bounds[i + 1]].cuda(), ld, vocab_offset=bounds[i], want_partials=True)
                         for i in range(G)])
    tok, mean = ops.ce_combine(parts, ld)
    tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
    assert torch.allclose(tok.cpu(), tok_o, rtol=TOL, atol=TOL)
    assert abs(mean.item() - mean_o.item()) <= TOL
    # and the partials themselves match the oracle's shard partials
    po = oracle.ce_partials(x, w[bounds[1]:bounds[2]], labels, bounds[1])
    assert torch.allclose(parts[1].cpu()[:, 0], po[:, 0], rtol=1e-3, atol=1e-3)
    assert torch.allclose(parts[1].cpu()[:, 2], po[:, 2], rtol=1e-3, atol=1e-3)


def test_flce_full_vocab_size_sampled_rows():
    # the benchmark's vocabulary (128256) and hidden size (4096) on 256 tokens; every row checked
    M, D, V = 256, 4096, 128256
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=5)
    tok, mean = _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.cuda())
    assert _ops().kernel_status() == 0
    tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
    assert torch.allclose(tok.cpu(), tok_o, rtol=TOL, atol=TOL)
    assert abs(mean.item() - mean_o.item()) <= TOL


def test_flce_rejects_float_labels_and_small_workspace():
    from arke_b200 import _lib
    x, w, labels = oracle.make_flce_inputs(64, 64, 512, seed=1)
    with pytest.raises(_lib.UnsupportedError):
        _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.float().cuda())
    with pytest.raises(_lib.ArkeB200Error):
        _ops().fused_linear_ce(x.cuda(), w.cuda(), labels.cuda(), workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))


def test_flce_out_of_range_label_on_a_whole_vocabulary_call():
    """``F.cross_entropy`` (the reference's definition) raises for a label outside [0, V); a call
    that covers the whole vocabulary gives that row NaN and records status code 6, instead of a
    plausible-looking ``lse - 0``.  A vocabulary-slice call cannot know and keeps "not in my slice"."""
    x, w, labels = oracle.make_flce_inputs(96, 64, 700, seed=4, ignore_frac=0.0)
    bad = labels.clone()
    bad[5], bad[40] = 700, -3
    with pytest.raises((IndexError, RuntimeError)):
        oracle.fused_linear_ce(x, w, bad)
    ops = _ops()
    assert ops.kernel_status() == 0
    tok, mean = ops.fused_linear_ce(x.cuda(), w.cuda(), bad.cuda())
    assert ops.kernel_status() == 6 and ops.kernel_status() == 0          # reported once, then cleared
    tok = tok.cpu()
    assert torch.isnan(tok[5]) and torch.isnan(tok[40]) and torch.isnan(mean)
    good = torch.ones(96, dtype=torch.bool)
    good[5] = good[40] = False
    tok_o, _ = oracle.fused_linear_ce(x, w, labels)
    assert torch.allclose(tok[good], tok_o[good], rtol=TOL, atol=TOL)
    # slice call: the same labels are simply "held by another slice"
    part = ops.fused_linear_ce(x.cuda(), w.cuda(), bad.cuda(), want_partials=True)
    assert ops.kernel_status() == 0 and part[5, 2].item() == 0.0
