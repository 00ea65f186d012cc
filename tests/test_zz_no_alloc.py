"""GPU: the allocation-free fused linear + cross-entropy entry point.

Some hosts cannot give the library a workspace: their memory pool already owns all device
memory, or they must not allocate at the point where the loss is computed.  For them
``arke_b200_fused_linear_ce_static`` keeps its scratch in an 8 MiB array built into the library.
This test calls it through the C ABI twice in a row (different inputs, so stale scratch from the
first call would show) and checks both results against the workspace-based entry point, with the
tolerance used for every fp32 loss in this suite (1e-3).  It is collected last on purpose and
passes both on its own in a fresh process and after the other tests.
"""
import pytest
import torch

from oracle import ops as oracle

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _call_static(ops, x, w, labels):
    loss = torch.full((x.shape[0],), float("nan"), dtype=torch.float32, device="cuda")
    mean = torch.full((), float("nan"), dtype=torch.float32, device="cuda")
    ops.fused_linear_ce_static(x, w, labels, loss, mean)
    return loss, mean


def test_static_entry_matches_workspace_entry_twice_in_a_row():
    from arke_b200 import ops
    results = []
    for seed, (M, D, V) in ((11, (512, 256, 32000)), (12, (300, 512, 5003))):
        x, w, labels = oracle.make_flce_inputs(M, D, V, seed=seed, ignore_frac=0.05)
        xd, wd, ld = x.cuda(), w.cuda(), labels.cuda()
        assert ops.fused_linear_ce_workspace_bytes(M, V, D) <= ops.STATIC_SCRATCH_BYTES
        loss_s, mean_s = _call_static(ops, xd, wd, ld)
        loss_w, mean_w = ops.fused_linear_ce(xd, wd, ld)
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        assert torch.allclose(loss_s, loss_w, rtol=TOL, atol=TOL)
        assert abs(mean_s.item() - mean_w.item()) <= TOL
        assert torch.all(loss_s[ld == -100] == 0)
        # and against the CPU oracle, like the workspace-based tests
        tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
        assert torch.allclose(loss_s.cpu(), tok_o, rtol=TOL, atol=TOL)
        assert abs(mean_s.item() - mean_o.item()) <= TOL
        results.append(mean_s.item())
    assert results[0] != results[1]


def test_static_entry_rejects_problems_beyond_its_scratch():
    from arke_b200 import ops, _lib
    M, D, V = 8192, 64, 128256          # needs ~33 MB of scratch: beyond the built-in 8 MiB
    assert ops.fused_linear_ce_workspace_bytes(M, V, D) > ops.STATIC_SCRATCH_BYTES
    x = torch.zeros(M, D, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(V, D, dtype=torch.bfloat16, device="cuda")
    labels = torch.zeros(M, dtype=torch.int64, device="cuda")
    loss = torch.empty(M, dtype=torch.float32, device="cuda")
    mean = torch.empty((), dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.ArkeB200Error) as ei:
        ops.fused_linear_ce_static(x, w, labels, loss, mean)
    assert ei.value.code == -6 and "8388608" in str(ei.value)
