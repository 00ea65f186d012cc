"""GPU parity at the full BASELINE sizes through size-independent properties and sampled rows
(the CPU oracle cannot run these sizes in seconds): quantize round trip / idempotence, SwiGLU+FP8
fused == two-step on sampled rows, fused linear+CE sampled rows and shard-combine invariance."""
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu


def _ops():
    from arke_b200 import ops
    return ops


def test_quantize_config2_round_trip_idempotence_and_sampled_rows():
    ops = _ops()
    x = oracle.make_quant_input(8192, 4096, seed=1)
    xd = x.cuda()
    q, s = ops.quantize_per_token(xd)
    # sampled rows bit-exact against the oracle
    rows = torch.tensor([0, 1, 2, 127, 128, 4095, 4096, 8190, 8191])
    qo, so = oracle.quantize_per_token_interp(x[rows])
    assert torch.equal(q[rows].cpu(), qo) and torch.equal(s[rows].cpu(), so)
    # every row: scale = amax/127, |x - q*scale| <= scale/2 (+1 ulp of the product), extreme hits +-127
    assert torch.equal(s.cpu(), x.float().abs().amax(-1) / 127.0)   # CPU division (IEEE), as the reference
    err = (xd.float() - q.float() * s[:, None]).abs()
    assert bool((err <= s[:, None] * 0.5 * (1 + 1e-4) + 1e-12).all())   # half a step, plus fp32 rounding of q*s and x/s
    assert bool((q.abs().amax(-1) == 127).all())
    # idempotence: the dequantised tensor quantises to the same codes with the same scale
    deq = (q.float() * s[:, None])
    q2, s2 = ops.quantize_per_token(deq)
    assert torch.equal(q2, q)
    assert torch.allclose(s2, s, rtol=1e-6, atol=0)


def test_swiglu_config3_sampled_rows_and_fused_equals_two_step():
    ops = _ops()
    M, N2 = 16384, 28672
    x = oracle.make_swiglu_input(M, N2, seed=3)
    xd = x.cuda()
    yq, s = ops.swiglu_fp8(xd)
    rows = torch.tensor([0, 1, 255, 256, 8191, 8192, 16382, 16383])
    yo, yqo, so = oracle.swiglu_fp8(x[rows])
    deq, deqo = yq[rows].cpu().float() * s[rows].cpu()[:, None], yqo.float() * so[:, None]
    assert torch.allclose(deq, deqo, rtol=2e-2, atol=2e-2)
    assert torch.allclose(s[rows].cpu(), so, rtol=1e-2, atol=0)
    # whole tensor: fused fp8 output == quantising the kernel's own bf16 y (two-step), and
    # row-shard invariance (token sharding cannot change any row)
    y = ops.silu_and_mul(xd)
    yq2, s2 = ops.quantize_per_token(y, out_dtype="fp8")
    assert torch.equal(s2, s)
    assert (yq2.view(torch.uint8) == yq.view(torch.uint8)).float().mean().item() > 0.99999
    half = ops.swiglu_fp8(xd[M // 2:])
    assert torch.equal(half[0].view(torch.uint8), yq[M // 2:].view(torch.uint8)) and torch.equal(half[1], s[M // 2:])


def test_flce_config5_sampled_rows_and_shard_invariance():
    ops = _ops()
    M, D, V = 8192, 4096, 128256
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=5)
    xd, wd, ld = x.cuda(), w.cuda(), labels.cuda()
    tok, mean = ops.fused_linear_ce(xd, wd, ld)
    assert ops.kernel_status() == 0
    keep = ld != -100
    assert int((~keep).sum()) == 82 and bool((tok[~keep] == 0).all())
    assert abs((tok.sum() / keep.sum()).item() - mean.item()) <= 1e-4
    # sampled token rows against the oracle (fp32 logits materialised for those rows only)
    rows = torch.tensor([0, 1, 127, 128, 129, 4095, 4096, 8000, 8191])
    tok_o, _ = oracle.fused_linear_ce(x[rows], w, labels[rows])
    assert torch.allclose(tok[rows].cpu(), tok_o, rtol=1e-3, atol=1e-3)
    # vocabulary sharded 8 ways and recombined == unsharded (what the 8-GPU run computes)
    G = 8
    bounds = [V * i // G for i in range(G + 1)]
    parts = torch.stack([ops.fused_linear_ce(xd, wd[bounds[i]:bounds[i + 1]], ld, vocab_offset=bounds[i], want_partials=True)
                         for i in range(G)])
    tok8, mean8 = ops.ce_combine(parts, ld)
    assert torch.allclose(tok8, tok, rtol=1e-4, atol=1e-4)
    assert abs(mean8.item() - mean.item()) <= 1e-4


def test_flce_backward_config5_properties_and_sampled_rows():
    """Config 5 backward (M 8192, D 4096, V 128256): ignored rows get zero gradient, the columns of
    dW sum to ~0 (every row of the logits gradient sums to zero), and sampled rows of dX / dW match
    a CPU restatement built from the kernel's own logsumexp."""
    ops = _ops()
    M, D, V = 8192, 4096, 128256
    x, w, labels = oracle.make_flce_inputs(M, D, V, seed=5)
    xd, wd, ld = x.cuda(), w.cuda(), labels.cuda()
    part = ops.fused_linear_ce(xd, wd, ld, want_partials=True)
    lse = part[:, 0] + torch.log(part[:, 1])
    dx, dw = ops.fused_linear_ce_backward(xd, wd, ld, lse=lse)
    assert ops.kernel_status() == 0
    keep = labels != -100
    n = int(keep.sum())
    assert n < M and bool((dx[(~keep).cuda()] == 0).all())
    # checksum of checksums: sum_v dW[v, :] = sum_i (sum_v G[i, v]) x_i = 0 up to the 16-bit rounding of G
    col = dw.float().sum(0)
    assert col.abs().max().item() <= 2e-2 * dw.float().abs().sum(0).max().item()
    lse_c = lse.cpu()
    # sampled token rows of dX: G_i = (softmax(x_i W^T) - onehot) / n, dX_i = G_i W
    wf = w.float()
    for i in [0, 1, 4095, 8191] + [int(torch.nonzero(~keep)[0])]:
        logits = wf @ x[i].float()
        g = torch.exp(logits - lse_c[i])
        if labels[i] != -100:
            g[labels[i]] -= 1.0
            g /= n
        else:
            g.zero_()
        ref = g @ wf
        got = dx[i].float().cpu()
        assert (got - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-12, i
    # sampled vocabulary rows of dW: dW_v = sum_i G[i, v] x_i
    xf = x.float()
    for v in [0, 255, 256, 64127, 128255, int(labels[keep][0])]:
        g = torch.exp(xf @ wf[v] - lse_c)
        g[labels == v] -= 1.0
        g = torch.where(keep, g / n, torch.zeros_like(g))
        ref = g @ xf
        got = dw[v].float().cpu()
        assert (got - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-12, v
