"""GPU: the checked build (``-DARKE_B200_CHECKED``) of the kernel library.

Every kernel of that build re-derives, right before a global access, that the element index it
computed lies inside the tensor, and otherwise records status code 7 and skips the access — the
stand-in for an address sanitizer on hosts where none can run.  Here the ragged and strided shapes
of every op run against that build in a child process (``ARKE_B200_SO`` selects the library):
the status word must stay 0 and the results must equal the default build's bit for bit.  The
self-test shows that the check does fire (on an index one past an extent, without a memory access).
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
CHECKED = ROOT / "arke_b200" / "libarke_b200_checked.so"

CHILD = r"""
import hashlib, json, os, sys, torch
sys.path.insert(0, os.environ["ARKE_ROOT"])
from arke_b200 import ops, _lib
from oracle import ops as oracle
out = {"version": _lib.version()}
def h(*ts):
    m = hashlib.sha256()
    for t in ts:
        m.update(t.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes())
    return m.hexdigest()
g = torch.Generator().manual_seed(0)
def rnd(*shape, dtype=torch.bfloat16):
    return torch.randn(*shape, generator=g).to(dtype).cuda()
# row kernels: fast path, ragged generic path, strided rows, fp16, fused outputs
for (M, N) in [(37, 4096), (5, 769), (130, 1040), (1, 16)]:
    x = rnd(M, N)
    out[f"quant_{M}x{N}"] = h(*ops.quantize_per_token(x))
    out[f"quant_fp8_{M}x{N}"] = h(*[t.view(torch.uint8) if t.dtype != torch.float32 else t for t in ops.quantize_per_token(x, out_dtype="fp8")])
    out[f"quant_l1_{M}x{N}"] = h(*ops.quantize_per_token(x.half(), formula="bench_l1"))
    w = rnd(N)
    out[f"rms_{M}x{N}"] = h(ops.rmsnorm(x, w))
    y, q, s = ops.rmsnorm(x, w, residual=rnd(M, N), quantize="int8")
    out[f"rmsq_{M}x{N}"] = h(y, q, s)
    if N % 2 == 0:
        y, yq, sc = ops.silu_and_mul(x, quantize_fp8=True, return_y=True)
        out[f"silu_{M}x{N}"] = h(y, yq.view(torch.uint8), sc)
wide = rnd(33, 2048 + 64)
out["quant_strided"] = h(*ops.quantize_per_token(wide[:, :2048]))
out["dequant"] = h(ops.dequantize_per_channel(torch.randint(-128, 127, (45, 333), generator=g, dtype=torch.int8).cuda(), rnd(333, dtype=torch.float32).abs() + 0.1, None))
# rope and the packed QKV split
cos, sin = (t.cuda() for t in oracle.make_rope_tables(50, 64))
out["rope"] = h(ops.rope(rnd(2, 3, 50, 64), cos, sin))
out["qkv_split"] = h(*ops.qkv_rope_split(rnd(2 * 50, (4 + 2 * 2) * 64), cos, sin, 2, 50, 4, 2, 64))
# GEMMs: ragged M / N / K, both tile forms, int8 accumulators, fp32 (TF32), transposed A
for (M, N, K) in [(129, 272, 192), (300, 528, 1040), (1030, 1296, 256)]:
    xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
    wq = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8).cuda()
    sa, sw = rnd(M, dtype=torch.float32).abs(), rnd(N, dtype=torch.float32).abs()
    for tm in (128, 256):
        with ops.options(gemm_tile_m=tm):
            yq, acc = ops.quant_gemm(xq, sa, wq, sw, return_acc=True)
            out[f"w8a8_{M}x{N}x{K}_{tm}"] = h(yq, acc)
            out[f"mm_{M}x{N}x{K}_{tm}"] = h(ops.matmul(rnd(M, K), rnd(K, N)))
out["mm_tn"] = h(ops.matmul_tn(rnd(256, 136), rnd(256, 200), out_dtype=torch.float32))
out["mm_f32"] = h(ops.matmul(rnd(70, 96, dtype=torch.float32), rnd(96, 50, dtype=torch.float32).t().contiguous(), b_layout="nk"))
# attention: ragged sequence, different key length, both head sizes
for (B, Hq, Hkv, S, Skv, D, causal) in [(1, 4, 2, 300, 300, 128, True), (2, 2, 1, 77, 513, 64, False)]:
    q, k, v = (t.cuda() for t in oracle.make_attention_inputs(B, Hq, Hkv, S, D, seed=S, Skv=Skv))
    out[f"gqa_{S}_{Skv}_{D}"] = h(*ops.gqa_fwd(q, k, v, causal=causal))
# fused linear + CE forward / backward, ragged vocabulary
x, w, lab = (t.cuda() for t in oracle.make_flce_inputs(130, 64, 1003, seed=3, ignore_frac=0.1))
out["flce"] = h(*ops.fused_linear_ce(x, w, lab))
out["flce_partials"] = h(ops.fused_linear_ce(x, w[:512].contiguous(), lab, vocab_offset=0, want_partials=True))
out["flce_bwd"] = h(*ops.fused_linear_ce_backward(x, w, lab))
torch.cuda.synchronize()
out["status"] = ops.kernel_status()
rc = _lib.LIB.arke_b200_selftest_bounds_check(None)
torch.cuda.synchronize()
out["selftest_rc"] = rc
out["status_after_selftest"] = ops.kernel_status()
out["status_cleared"] = ops.kernel_status()
print("RESULT " + json.dumps(out))
"""


def _run(lib: Path | None) -> dict:
    env = dict(os.environ, ARKE_ROOT=str(ROOT))
    if lib is not None:
        env["ARKE_B200_SO"] = str(lib)
    else:
        env.pop("ARKE_B200_SO", None)
    p = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_checked_build_reports_nothing_on_ragged_shapes_and_changes_no_result():
    if not CHECKED.exists():
        pytest.skip("checked library not built (python -m arke_b200.build --flag=-DARKE_B200_CHECKED --out ...)")
    checked, default = _run(CHECKED), _run(None)
    assert "checked build" in checked["version"] and "checked build" not in default["version"]
    assert checked["status"] == 0 and default["status"] == 0
    skip = {"version", "status", "selftest_rc", "status_after_selftest", "status_cleared"}
    diff = [k for k in default if k not in skip and default[k] != checked[k]]
    assert not diff, diff
    assert len([k for k in default if k not in skip]) >= 40
    # the check fires when an index is one past the extent (no memory access in that self-test)
    assert checked["selftest_rc"] == 0 and checked["status_after_selftest"] == 7 and checked["status_cleared"] == 0
    assert default["selftest_rc"] != 0 and default["status_after_selftest"] == 0
