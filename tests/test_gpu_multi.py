"""GPU (needs >= 2 devices, skipped otherwise): the vocabulary-sharded fused linear + CE over NCCL
equals the unsharded result, and the token-sharded ops need no communication."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARKE_ROOT"])
from arke_b200 import ops
from arke_b200.sharding import lse_from_partials, shard_bounds, shard_rows, vocab_sharded_ce, vocab_sharded_ce_backward
from oracle import ops as oracle
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
x, w, labels = oracle.make_flce_inputs(512, 256, 8192 + 24, seed=9, ignore_frac=0.05)
b, e = shard_bounds(w.shape[0], world, rank)
tok, mean = vocab_sharded_ce(x.cuda(), w[b:e].cuda(), labels.cuda(), b)
tok_o, mean_o = oracle.fused_linear_ce(x, w, labels)
assert torch.allclose(tok.cpu(), tok_o, rtol=1e-3, atol=1e-3), "sharded per-token loss mismatch"
assert abs(mean.item() - mean_o.item()) <= 1e-3
# backward of the sharded form: global lse from the gathered partials, own rows of dW, all-reduced dX
part = ops.fused_linear_ce(x.cuda(), w[b:e].cuda(), labels.cuda(), vocab_offset=b, want_partials=True)
gathered = torch.empty((world * part.shape[0], 3), dtype=part.dtype, device="cuda")
dist.all_gather_into_tensor(gathered, part.contiguous())
lse = lse_from_partials(gathered.view(world, -1, 3))
dx, dw = vocab_sharded_ce_backward(x.cuda(), w[b:e].cuda(), labels.cuda(), b, lse)
dx_o, dw_o = oracle.fused_linear_ce_backward(x, w, labels)
def close(got, ref):
    got, ref = got.float().cpu(), ref.float()
    return (got - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() and ((got - ref).norm() / ref.norm()).item() <= 1e-2
assert close(dx, dx_o), "sharded dX mismatch"
assert close(dw, dw_o[b:e]), "sharded dW mismatch"
# token sharding: each rank quantises its rows; concatenation equals the unsharded oracle
xq = oracle.make_quant_input(1000, 512, seed=3)
q, s = ops.quantize_per_token(shard_rows(xq, world, rank).cuda())
qo, so = oracle.quantize_per_token_interp(xq)
rb, re_ = shard_bounds(1000, world, rank)
assert torch.equal(q.cpu(), qo[rb:re_]) and torch.equal(s.cpu(), so[rb:re_])
assert ops.kernel_status() == 0
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_vocab_sharded_ce_two_gpus_nccl(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, ARKE_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
