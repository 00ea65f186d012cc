#!/usr/bin/env python
"""Benchmark of the B200 hot path: one JSON line per run.

Headline workload (``--workload w8a8``, the Llama-3-8B MLP up-projection of BASELINE.json
configs[1]): one *step* = per-token INT8 quantisation of X bf16 [8192,4096] followed by the W8A8
GEMM against W int8 [4096,14336] with int32 accumulation and dequantisation to bf16.
``value`` = GEMM operations (2*M*N*K) per second of whole-step time, summed over all GPUs (each
GPU runs the full per-GPU workload on its own tokens: weak scaling, no communication).

The JSON line also carries
  roofline      the dominant kernel (the tcgen05 GEMM) timed with CUDA events inside the timed region
  e2e           the same step driven through the plugin API from pinned HOST buffers
                (H2D of X, D2H of Y inside the timed region)
  cpu_baseline  the CPU oracle (restatement of the reference path) on a bounded sample, N=1 only
  per_op        the other hot-path ops (quantize, SwiGLU+FP8, FP8 GEMM, GQA attention, fused
                linear+CE) each with its own roofline fraction
  clocks        nvidia-smi SM clock / throttle reasons sampled during the timed region

``--impl reference`` times the reference's CPU path for the same workload (the oracle port; the
reference itself is pure Python/PyTorch-eager and is not present on the GPU box).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = {
    "w8a8": dict(M=8192, K=4096, N=14336),
    "swiglu": dict(M=16384, N2=28672),
    "gqa": dict(B=4, Hq=32, Hkv=8, S=8192, D=128),
    "flce": dict(M=8192, D=4096, V=128256),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch at the full sizes, from the ncu capture
# summarised in profiles/dram_traffic_full_size.md (outputs still resident in L2 at kernel end are
# not counted by the write counter, so traffic can be below the algorithmic bytes)
TRAFFIC = {"w8a8_gemm": 299999744, "fp8_gemm": 302069248, "fused_linear_ce": 4246542592,
           "rmsnorm_residual_quant_int8": 145927680,
           "gqa_fwd_causal": 638203904, "quantize_per_token": 70791936, "swiglu_fp8": 1143861760,
           "qkv_rope_split": 759137792,
           # three launches: logits gradient 6.56 GB, dX 24.12 GB, dW 21.38 GB (operand re-reads)
           "fused_linear_ce_backward": 52054000000}
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0, "int8_tops": 4500.0, "fp8_tflops": 4500.0}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------
# clock sampling
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples ``nvidia-smi`` (SM clock, throttle reasons) every 200 ms while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.tmp = None

    def start(self):
        try:
            self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            self.tmp.flush()
            rows = [r.split(",") for r in Path(self.tmp.name).read_text().strip().splitlines() if r.strip()]
            os.unlink(self.tmp.name)
        except Exception:
            return out
        clocks, reasons, mx = [], set(), None
        for r in rows:
            r = [c.strip() for c in r]
            if len(r) < 9:
                continue
            try:
                clocks.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            out.update(sm_mhz=statistics.median(clocks), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(clocks))
        return out


# ---------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def time_loop(fn, steps, warmup, stream=None):
    """Untimed warm-up then ``steps`` calls bracketed by CUDA events; returns total ms."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def graph_time(fn, iters, warmup=3):
    """Average device time (ms) of ``fn`` replayed ``iters`` times inside one CUDA graph, so that
    microsecond-scale kernels are not limited by the host's launch rate."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def roofline(bound, achieved, peak_meas, peak_nominal, unit, traffic=None, src="measured", note=None):
    r = {"bound": bound, "achieved": round(achieved, 1), "peak": peak_meas, "unit": unit,
         "frac": round(achieved / peak_meas, 4), "frac_of_nominal": round(achieved / peak_nominal, 4),
         "peak_nominal": peak_nominal, "peak_source": src, "traffic": traffic}
    if note:
        r["note"] = note
    return r


# ---------------------------------------------------------------------------------------------
# CPU baseline / reference arm (oracle port of the reference path on host cores)
# ---------------------------------------------------------------------------------------------
def cpu_w8a8_sample(rows: int, reps: int = 1):
    """Times the CPU oracle (quantize_per_token + int8 GEMM + dequantisation) on ``rows`` tokens of
    the w8a8 workload; returns (TOPS, seconds per rep, cores)."""
    from oracle import ops as oracle
    c = CFG["w8a8"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = oracle.make_quant_input(rows, c["K"], seed=1)
    w, sw = oracle.make_w8a8_weights(c["K"], c["N"], seed=2)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        q, s = oracle.quantize_per_token_interp(x)
        y, acc = oracle.w8a8_gemm(q, s, w, sw)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    ops = 2.0 * rows * c["N"] * c["K"]
    return ops / best / 1e12, best, cores


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    c = CFG["w8a8"]
    rows = args.ref_rows
    times = []
    from oracle import ops as oracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = oracle.make_quant_input(rows, c["K"], seed=1)
    w, sw = oracle.make_w8a8_weights(c["K"], c["N"], seed=2)

    def step():
        q, s = oracle.quantize_per_token_interp(x)
        oracle.w8a8_gemm(q, s, w, sw)

    for _ in range(args.warmup):
        step()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    per = sum(times) / len(times)
    tops = 2.0 * rows * c["N"] * c["K"] / per / 1e12
    line = {
        "impl": "reference", "metric": "w8a8_gemm_tops", "value": round(tops, 5), "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per * 1e3 * (c["M"] / rows), 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "w8a8: quantize_per_token bf16[8192x4096] + int8 GEMM x [4096x14336] -> bf16",
                   "sample": f"{rows} of {c['M']} tokens per step; ms_per_step extrapolated to the full batch"},
        "cpu_baseline": {"value": round(tops, 5), "unit": "TOPS", "cores": cores, "kind": "port",
                         "sample": f"{rows} tokens x full W per step, torch CPU ({torch.get_num_threads()} threads), "
                                   "oracle restatement of ref_quantize_per_token + exact int GEMM + dequant"},
        "e2e": {"value": round(tops, 5), "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# per-op measurements (N = 1): each returns a dict with its own roofline
# ---------------------------------------------------------------------------------------------
SMALL = {
    "w8a8": dict(M=2048, K=4096, N=14336),
    "swiglu": dict(M=2048, N2=28672),
    "gqa": dict(B=1, Hq=8, Hkv=2, S=4096, D=128),
    "flce": dict(M=2048, D=4096, V=32064),
}
DEV = "cuda"


def _hbm(peaks, nbytes, ms):
    return roofline("hbm", nbytes / ms / 1e6, peaks["hbm_gbs"], NOMINAL["hbm_gbs"], "GB/s", src=peaks["source"])


def op_quantize(ops, oracle, peaks, cfg, iters, small):
    """config 2a: four rotating inputs (268 MB > 126 MB L2); timed as one CUDA graph of 40 launches."""
    c = cfg["w8a8"]
    xs = [oracle.make_quant_input(c["M"], c["K"], seed=1).to(DEV)]
    xs += [xs[0].clone() for _ in range(3)]
    q = torch.empty(c["M"], c["K"], dtype=torch.int8, device=DEV)
    s = torch.empty(c["M"], dtype=torch.float32, device=DEV)
    k = [0]

    def fq():
        k[0] = (k[0] + 1) & 3
        ops.quantize_per_token(xs[k[0]], out=(q, s))

    ms = time_loop(fq, 4, 3) / 4 if small else graph_time(fq, 40)
    nbytes = c["M"] * c["K"] * 3 + c["M"] * 4
    return {"quantize_per_token": {"us": round(ms * 1e3, 2), "bytes": nbytes, "roofline": _hbm(peaks, nbytes, ms)}}


def op_rmsnorm(ops, oracle, peaks, cfg, iters, small):
    """rmsnorm_residual fused with the per-token INT8 quantisation that feeds the W8A8 GEMM
    (8192 x 4096 bf16; reads X and the residual, writes only q + scales); four rotating inputs."""
    c = cfg["w8a8"]
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(c["M"], c["K"], generator=g).to(torch.bfloat16).to(DEV) for _ in range(2)]
    xs += [xs[0].clone(), xs[1].clone()]
    res = [x.clone() for x in xs]
    w = torch.ones(c["K"], dtype=torch.bfloat16, device=DEV)
    k = [0]

    def f():
        k[0] = (k[0] + 1) & 3
        ops.rmsnorm(xs[k[0]], w, residual=res[k[0]], quantize="int8", return_y=False)

    ms = time_loop(f, 4, 3) / 4 if small else graph_time(f, 40)   # one CUDA graph of 40 launches
    nbytes = c["M"] * c["K"] * 5 + c["M"] * 4 + c["K"] * 2
    return {"rmsnorm_residual_quant_int8": {"us": round(ms * 1e3, 2), "bytes": nbytes, "roofline": _hbm(peaks, nbytes, ms)}}


def op_rope(ops, oracle, peaks, cfg, iters, small):
    """Packed-QKV split + rotary embedding at the attention configuration (config 4): the
    projection output [B*S, (Hq+2Hkv)*D] is read once (403 MB > L2) and Q, K, V written once."""
    c = cfg["gqa"]
    B, S, Hq, Hkv, D = c["B"], c["S"], c["Hq"], c["Hkv"], c["D"]
    W = (Hq + 2 * Hkv) * D
    g = torch.Generator(device=DEV).manual_seed(7)
    qkv = torch.randn(B * S, W, generator=g, device=DEV, dtype=torch.float32).bfloat16()
    cos, sin = (t.to(DEV) for t in oracle.make_rope_tables(S, D))
    ms = time_loop(lambda: ops.qkv_rope_split(qkv, cos, sin, B, S, Hq, Hkv, D), iters, 3) / iters
    nbytes = 2 * B * S * W * 2 + 2 * S * (D // 2) * 2
    return {"qkv_rope_split": {"us": round(ms * 1e3, 2), "bytes": nbytes, "roofline": _hbm(peaks, nbytes, ms)}}


def op_swiglu(ops, oracle, peaks, cfg, iters, small):
    """config 3 (input 940 MB > L2): fp8-only output, and the variant that also writes bf16 Y."""
    c3 = cfg["swiglu"]
    x3 = oracle.make_swiglu_input(c3["M"], c3["N2"], seed=3).to(DEV)
    n = c3["N2"] // 2
    ms = time_loop(lambda: ops.swiglu_fp8(x3), iters, 3) / iters
    nb = c3["M"] * c3["N2"] * 2 + c3["M"] * n + c3["M"] * 4
    out = {"swiglu_fp8": {"us": round(ms * 1e3, 1), "bytes": nb, "variant": "fp8 + scales only (no bf16 Y)",
                          "roofline": _hbm(peaks, nb, ms)}}
    if not small:
        ms = time_loop(lambda: ops.silu_and_mul(x3, quantize_fp8=True, return_y=True), iters, 3) / iters
        nb2 = nb + c3["M"] * n * 2
        out["swiglu_fp8_with_y"] = {"us": round(ms * 1e3, 1), "bytes": nb2, "roofline": _hbm(peaks, nb2, ms)}
    return out


def op_fp8_gemm(ops, oracle, peaks, cfg, iters, small):
    c = cfg["w8a8"]
    g = torch.Generator().manual_seed(2)
    a8 = torch.randn(c["M"], c["K"], generator=g).to(torch.float8_e4m3fn).to(DEV)
    w8 = torch.randn(c["K"], c["N"], generator=g).to(torch.float8_e4m3fn).to(DEV)
    sa = torch.rand(c["M"], generator=g).to(DEV)
    swv = torch.rand(c["N"], generator=g).to(DEV)
    y = torch.empty(c["M"], c["N"], dtype=torch.bfloat16, device=DEV)
    ms = time_loop(lambda: ops.fp8_gemm(a8, sa, w8, swv, out=y), iters, 3) / iters
    fl = 2.0 * c["M"] * c["N"] * c["K"]
    return {"fp8_gemm": {"us": round(ms * 1e3, 1), "flop": fl,
                         "roofline": roofline("tensor", fl / ms / 1e9, 2 * peaks["bf16_tflops"], NOMINAL["fp8_tflops"], "TFLOP/s",
                                              src=peaks["source"], note="peak = 2 x measured bf16 cuBLAS burst (no measured fp8 peak)")}}


def op_w8a8_gemm(ops, oracle, peaks, cfg, iters, small):
    c = cfg["w8a8"]
    x = oracle.make_quant_input(c["M"], c["K"], seed=1).to(DEV)
    q, sx = ops.quantize_per_token(x)
    w, sw = oracle.make_w8a8_weights(c["K"], c["N"], seed=2)
    w, sw = w.to(DEV), sw.to(DEV)
    y = torch.empty(c["M"], c["N"], dtype=torch.bfloat16, device=DEV)
    ms = time_loop(lambda: ops.w8a8_gemm(q, sx, w, sw, out=y), iters, 3) / iters
    fl = 2.0 * c["M"] * c["N"] * c["K"]
    return {"w8a8_gemm": {"us": round(ms * 1e3, 1), "flop": fl,
                          "roofline": roofline("tensor", fl / ms / 1e9, 2 * peaks["bf16_tflops"], NOMINAL["int8_tops"], "TOP/s",
                                               src=peaks["source"], note="peak = 2 x measured bf16 cuBLAS burst (no measured int8 peak)")}}


def op_gqa(ops, oracle, peaks, cfg, iters, small):
    c4 = cfg["gqa"]
    qq, kk, vv = oracle.make_attention_inputs(c4["B"], c4["Hq"], c4["Hkv"], c4["S"], c4["D"], seed=4)
    qq, kk, vv = qq.to(DEV), kk.to(DEV), vv.to(DEV)
    ms = time_loop(lambda: ops.gqa_fwd(qq, kk, vv, causal=True), iters, 3) / iters
    fl = 2.0 * c4["B"] * c4["Hq"] * c4["S"] * c4["S"] * c4["D"]
    return {"gqa_fwd_causal": {"us": round(ms * 1e3, 1), "flop": fl,
                               "roofline": roofline("tensor", fl / ms / 1e9, peaks["bf16_tflops"], NOMINAL["bf16_tflops"], "TFLOP/s",
                                                    src=peaks["source"])}}


def op_flce(ops, oracle, peaks, cfg, iters, small):
    c5 = cfg["flce"]
    x5, w5, l5 = oracle.make_flce_inputs(c5["M"], c5["D"], c5["V"], seed=5)
    x5, w5, l5 = x5.to(DEV), w5.to(DEV), l5.to(DEV)
    ws = torch.empty(ops.fused_linear_ce_workspace_bytes(c5["M"], c5["V"], c5["D"]), dtype=torch.uint8, device=DEV)
    n5 = max(2, iters // 2)
    ms = time_loop(lambda: ops.fused_linear_ce(x5, w5, l5, workspace=ws), n5, 2) / n5
    fl = 2.0 * c5["M"] * c5["V"] * c5["D"]
    return {"fused_linear_ce": {"us": round(ms * 1e3, 1), "flop": fl,
                                "roofline": roofline("tensor", fl / ms / 1e9, peaks["bf16_tflops_sustained"], NOMINAL["bf16_tflops"],
                                                     "TFLOP/s", src=peaks["source"], note="peak = sustained cuBLAS bf16 (multi-ms kernel)")}}


def op_flce_bwd(ops, oracle, peaks, cfg, iters, small):
    """Backward of config 5: logits gradient (recomputed logits, 16-bit G in a 2.1 GB workspace),
    dX = G W and dW = G^T X — three GEMM-sized launches, 3 x 2*M*V*D flop."""
    c5 = cfg["flce"]
    x5, w5, l5 = oracle.make_flce_inputs(c5["M"], c5["D"], c5["V"], seed=5)
    x5, w5, l5 = x5.to(DEV), w5.to(DEV), l5.to(DEV)
    part = ops.fused_linear_ce(x5, w5, l5, want_partials=True)
    lse = part[:, 0] + torch.log(part[:, 1])
    ws = torch.empty(ops.fused_linear_ce_backward_workspace_bytes(c5["M"], c5["V"]), dtype=torch.uint8, device=DEV)
    n5 = max(2, iters // 2)
    ms = time_loop(lambda: ops.fused_linear_ce_backward(x5, w5, l5, lse=lse, workspace=ws), n5, 2) / n5
    fl = 6.0 * c5["M"] * c5["V"] * c5["D"]
    return {"fused_linear_ce_backward": {"us": round(ms * 1e3, 1), "flop": fl,
                                         "roofline": roofline("tensor", fl / ms / 1e9, peaks["bf16_tflops_sustained"], NOMINAL["bf16_tflops"],
                                                              "TFLOP/s", src=peaks["source"],
                                                              note="three launches (logits gradient, dX, dW); peak = sustained cuBLAS bf16")}}


OPS = {"quantize": op_quantize, "rmsnorm": op_rmsnorm, "rope": op_rope, "swiglu": op_swiglu, "fp8": op_fp8_gemm, "w8a8": op_w8a8_gemm, "gqa": op_gqa, "flce": op_flce, "flce_bwd": op_flce_bwd}


def per_op_measurements(ops, oracle, peaks, quick: bool, only=None, small=False):
    """Each hot-path op at its BASELINE configuration (or at the reduced ``SMALL`` shapes used for
    profiler captures); ``only`` restricts the run to one op."""
    out = {}
    iters = 3 if small else (5 if quick else 10)
    cfg = dict(CFG)
    if small:
        cfg.update(SMALL)
    for name, fn in OPS.items():
        if only is not None and name != only:
            continue
        if only is None and name == "w8a8":
            continue  # the headline step already reports it
        out.update(fn(ops, oracle, peaks, cfg, iters, small))
        torch.cuda.empty_cache()
    if not small:
        for k, v in out.items():
            if k in TRAFFIC:
                v["roofline"]["traffic"] = TRAFFIC[k]
    return out


def run_single_op(args):
    """``--only OP [--small]``: one op, one JSON line; the entry point used for profiler captures."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the B200 path has no CPU fallback)")
    torch.cuda.set_device(0)
    from arke_b200 import ops
    from oracle import ops as oracle
    res = per_op_measurements(ops, oracle, measured_peaks(), True, only=args.only, small=args.small)
    if ops.kernel_status() != 0:
        raise SystemExit("bench.py: a device-side wait expired")
    print(json.dumps({"only": args.only, "small": bool(args.small), "per_op": res}))


# ---------------------------------------------------------------------------------------------
# main arm
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the B200 path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from arke_b200 import ops
    from oracle import ops as oracle  # input generators + the CPU-baseline leg only
    peaks = measured_peaks()

    c = CFG["w8a8"]
    M, K, N = c["M"], c["K"], c["N"]
    NBUF = 4
    x0 = oracle.make_quant_input(M, K, seed=1 + rank)
    xs = [x0.to(dev)] + [None] * (NBUF - 1)
    for i in range(1, NBUF):
        xs[i] = xs[0].clone()
    w_cpu, sw_cpu = oracle.make_w8a8_weights(K, N, seed=2)
    w, sw = w_cpu.to(dev), sw_cpu.to(dev)
    q = torch.empty(M, K, dtype=torch.int8, device=dev)
    sx = torch.empty(M, dtype=torch.float32, device=dev)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    step_i = [0]
    gemm_events = []

    def step(record=False):
        step_i[0] = (step_i[0] + 1) % NBUF
        ops.quantize_per_token(xs[step_i[0]], out=(q, sx))
        if record:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            ops.w8a8_gemm(q, sx, w, sw, out=y)
            b.record()
            gemm_events.append((a, b))
        else:
            ops.w8a8_gemm(q, sx, w, sw, out=y)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if use_dist:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if use_dist:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    # The same K steps once more with an event pair around every GEMM launch: the kernel's own
    # duration for the roofline.  Kept out of the timed region above because an event record
    # between the two kernels of a step removes their programmatic-dependent-launch overlap.
    for _ in range(args.steps):
        step(record=True)
    torch.cuda.synchronize()
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events) / len(gemm_events)
    # keep the GPU busy a little longer so that nvidia-smi gets samples under load for short runs
    if rank == 0:
        t_end = time.time() + max(0.0, 1.0 - ms_total / 1e3)
        while time.time() < t_end:
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    status = ops.kernel_status()
    if status != 0:
        raise SystemExit(f"bench.py: a device-side wait expired (kernel status {status})")
    if use_dist:
        tt = torch.tensor([ms_total, gemm_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total, gemm_ms = float(tt[0]), float(tt[1])
    ms_step = ms_total / args.steps
    gemm_ops = 2.0 * M * N * K
    value = gemm_ops * world / (ms_step * 1e-3) / 1e12

    if use_dist:
        dist.barrier()
    # ---- e2e: host buffers through the public API, copies inside the timed region ----
    from arke_b200.host import HostW8A8Linear
    xh = x0.pin_memory()
    yh = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    host_linear = HostW8A8Linear(w, sw, max_rows=M, chunks=8)

    # H2D of X, quantize, GEMM, D2H of Y — chunked and overlapped on 3 streams.  Steps are streamed
    # (wait=False): the next step's copies may start while this step's result is still going to
    # the host; the closing event is recorded after the current stream has waited for the last
    # step's completion event, so the timed region covers every copy.
    n_e2e = max(3, min(args.steps, 10))
    for _ in range(2):
        host_linear(xh, yh).synchronize()
    torch.cuda.synchronize()
    cur = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    done = None
    for _ in range(n_e2e):
        done = host_linear(xh, yh, wait=False)
    cur.wait_event(done)
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    if use_dist:
        tt = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_e2e = float(tt[0])
    e2e_val = gemm_ops * world / (ms_e2e * 1e-3) / 1e12

    # ---- N > 1: fused linear + CE with the vocabulary sharded over the ranks (the one op with a
    # collective: all-gather of the [M,3] per-row partials over NCCL, then the combine kernel) ----
    sharded = None
    if use_dist:
        from arke_b200.sharding import shard_bounds, vocab_sharded_ce
        c5 = CFG["flce"]
        v0, v1 = shard_bounds(c5["V"], world, rank)
        x5, w5, l5 = oracle.make_flce_inputs(c5["M"], c5["D"], v1 - v0, seed=5)   # this rank's W slice
        l5 = torch.randint(0, c5["V"], (c5["M"],), generator=torch.Generator().manual_seed(55), dtype=torch.int64)
        x5, w5, l5 = x5.to(dev), w5.to(dev), l5.to(dev)
        dist.broadcast(x5, 0)            # every rank sees the same tokens
        ws = torch.empty(ops.fused_linear_ce_workspace_bytes(c5["M"], v1 - v0, c5["D"]), dtype=torch.uint8, device=dev)
        part_fn = lambda xx, ww, ll, off: ops.fused_linear_ce(xx, ww, ll, vocab_offset=off, want_partials=True, workspace=ws)  # noqa: E731
        run5 = lambda: vocab_sharded_ce(x5, w5, l5, v0, partial_fn=part_fn)  # noqa: E731
        dist.barrier()
        n5 = 5
        ms5 = time_loop(run5, n5, 2) / n5
        tt = torch.tensor([ms5], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms5 = float(tt[0])
        fl5 = 2.0 * c5["M"] * c5["V"] * c5["D"]
        sharded = {"us": round(ms5 * 1e3, 1), "flop": fl5, "tflops_all_gpus": round(fl5 / ms5 / 1e9, 1),
                   "vocab_per_gpu": v1 - v0, "collective": "all_gather_into_tensor [M,3] fp32 (98 KB per rank) + ce_combine",
                   "scaling": "strong (total vocabulary fixed)"}

    if rank != 0:
        if use_dist:
            dist.barrier()
            dist.destroy_process_group()
        return

    line = {
        "metric": "w8a8_gemm_tops", "value": round(value, 1), "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": "w8a8: quantize_per_token bf16[8192x4096] (1% outlier channels x20) + int8 GEMM x W[4096x14336] "
                               "(int32 accumulate) -> bf16, per GPU",
                   "l2": f"{NBUF} rotating input sets (268 MB) + 235 MB output per step exceed the 126 MB L2",
                   "w_layout": "[K,N] row-major as given (MN-major UMMA operand, no re-layout)",
                   "sharding": "tokens (rows of X) per GPU, W replicated, no collective"},
        "gpu_launches": 2 * args.steps,
        "roofline": roofline("tensor", gemm_ops / (gemm_ms * 1e-3) / 1e12, 2 * peaks["bf16_tflops"], NOMINAL["int8_tops"], "TOP/s",
                             src=peaks["source"],
                             note="kernel gemm_pair_tcgen05_kernel<i8> (two-CTA tcgen05); peak = 2 x measured bf16 cuBLAS burst (no measured int8 peak); "
                                  "achieved = 2*M*N*K / mean CUDA-event time of the GEMM launch over a repeat of the timed steps "
                                  "(events between the kernels would break the dependent-launch overlap of the timed region itself)"),
        "e2e": {"value": round(e2e_val, 1), "unit": "TOPS", "h2d_bytes_per_step": M * K * 2 * world,
                "d2h_bytes_per_step": M * N * 2 * world, "ms_per_step": round(ms_e2e, 3)},
        "clocks": clocks,
    }
    line["roofline"]["kernel_us"] = round(gemm_ms * 1e3, 1)
    line["roofline"]["traffic"] = TRAFFIC["w8a8_gemm"]
    if world == 1 and not args.no_cpu_baseline:
        cpu_rows, cpu_reps = M, 4
        tops, secs, cores = cpu_w8a8_sample(cpu_rows, reps=cpu_reps)
        line["cpu_baseline"] = {"value": round(tops, 5), "unit": "TOPS", "cores": cores, "kind": "port",
                                "sample": f"{cpu_rows} of {M} tokens x full W, best of {cpu_reps} passes of {secs:.2f} s, "
                                          "torch CPU oracle (quantize + exact int GEMM + dequant)"}
    if world == 1 and not args.no_per_op:
        line["per_op"] = per_op_measurements(ops, oracle, peaks, args.quick)
    if sharded is not None:
        line["per_op"] = {"fused_linear_ce_vocab_sharded": sharded}
    print(json.dumps(line))
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--ref-rows", type=int, default=4096, help="tokens per CPU step of --impl reference (bounded sample)")
    ap.add_argument("--no-per-op", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", choices=list(OPS), default=None, help="measure one op only (one JSON line)")
    ap.add_argument("--small", action="store_true", help="with --only: reduced shapes for profiler captures")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_single_op(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
