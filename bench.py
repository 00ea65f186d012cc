#!/usr/bin/env python
"""Benchmark of the B200 hot path: one JSON line per run.

Headline workload (``--workload w8a8``, the Llama-3-8B MLP up-projection of BASELINE.json
configs[1]): one *step* = per-token INT8 quantisation of X bf16 [8192,4096] followed by the W8A8
GEMM against W int8 [4096,14336] with int32 accumulation and dequantisation to bf16.
``value`` = GEMM operations (2*M*N*K) per second of whole-step time, summed over all GPUs (each
GPU runs the full per-GPU workload on its own tokens: weak scaling, no communication).

The JSON line also carries
  roofline      the dominant kernel (the tcgen05 GEMM) timed with CUDA events, against the INT8 GEMM
                rate of the vendor library measured in the same run on the same GPU; ``sustained``
                inside it repeats the measurement in a loop of about two seconds (power-capped clocks)
  e2e           the same step driven through the plugin API from pinned HOST buffers
                (H2D of X, D2H of Y inside the timed region)
  cpu_baseline  the CPU path (reference interpreter for the quantisation when the reference package
                is staged, oracle restatement for the integer GEMM) on the full batch, N=1 only
  per_op        the other hot-path ops (quantize, SwiGLU+FP8, FP8 GEMM, GQA attention, fused
                linear+CE) each with its own roofline fraction; at N > 1 the strong-scaling
                shards of the communication-free ops and the vocabulary-sharded loss with a
                parity check of the multi-rank result
  clocks        SM clock / throttle reasons sampled through NVML inside the timed region

``--impl reference`` times the reference's CPU path for the same workload on the host cores.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch at the full sizes, from one ncu
# capture per kernel (outputs still resident in L2 at kernel end are not counted by the write
# counter, so traffic can be below the algorithmic bytes).  TRAFFIC_CAPTURED names the capture
# each figure comes from; a kernel whose source changed after that date needs a new capture.
TRAFFIC = {"w8a8_gemm": 299999744, "fp8_gemm": 302069248, "fused_linear_ce": 2211112704,
           "rmsnorm_residual_quant_int8": 145927680,
           "gqa_fwd_causal": 638203904, "quantize_per_token": 70791936, "swiglu_fp8": 1143861760,
           "qkv_rope_split": 759137792,
           # three launches: logits gradient 4.37 GB, dX 21.20 GB (long K: the pairs lose their k alignment), dW 6.82 GB
           "fused_linear_ce_backward": 32387460864}
TRAFFIC_CAPTURED = {k: "ncu capture of 2026-11-25 (profiles/, full-size launch)" for k in TRAFFIC}
for _k in ("fused_linear_ce", "fused_linear_ce_backward"):
    TRAFFIC_CAPTURED[_k] = "ncu capture of 2026-11-25 with the dynamic tile scheduler (profiles/dynamic_tile_scheduler_traffic.md)"
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0, "int8_tops": 4500.0, "fp8_tflops": 4500.0}
NBUF = 4   # rotating input sets of the headline step


def bench_config():
    """The `config` object of the JSON line — the same for both arms (same workload, same sizes)."""
    return {"workload": "w8a8: quantize_per_token bf16[8192x4096] (1% outlier channels x20) + int8 GEMM x W[4096x14336] "
                        "(int32 accumulate) -> bf16, per GPU",
            "l2": f"{NBUF} rotating input sets (268 MB) + 235 MB output per step exceed the 126 MB L2",
            "w_layout": "[K,N] row-major as given (MN-major UMMA operand, no re-layout)",
            "sharding": "tokens (rows of X) per GPU, W replicated, no collective"}


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
    """Reads the SM clock, the power draw and the clock-event (throttle) reasons of one GPU through
    NVML from a background thread, about once per millisecond, with a host timestamp per sample.
    ``window(t0, t1)`` summarises the samples taken between two ``time.perf_counter()`` stamps, so
    even a timed region of a few milliseconds gets its own clock record.  Reading only: no setting
    of the GPU is touched.  Falls back to ``nvidia-smi -lms 200`` when NVML cannot be loaded."""
    R_SW_POWER_CAP, R_HW_SLOWDOWN, R_SW_THERMAL, R_HW_THERMAL = 0x4, 0x8, 0x20, 0x40
    SMI_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                  "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, cuda_index: int):
        self.cuda_index = cuda_index
        self.samples = []          # (t, sm_mhz, reasons_bitmask, power_w)
        self.sm_max = None
        self.source = None
        self._stop = False
        self._thread = None
        self._smi = None
        self._smi_tmp = None
        self._t_start = None

    def start(self):
        import threading
        self._t_start = time.perf_counter()
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.cuda_index).uuid)
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.cuda_index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
            reasons_fn(h)

            def loop():
                while not self._stop:
                    try:
                        t = time.perf_counter()
                        clk = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        rs = int(reasons_fn(h))
                        pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                        self.samples.append((t, clk, rs, pw))
                    except Exception:
                        pass
                    time.sleep(0.001)

            sys.setswitchinterval(0.0005)      # let the sampler run while the main thread launches
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            self.source = "nvml"
            return
        except Exception:
            self.source = None
        try:
            self._smi_tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self._smi = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.SMI_FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.cuda_index)], stdout=self._smi_tmp, stderr=subprocess.DEVNULL)
            self.source = "nvidia-smi"
        except Exception:
            self._smi = None

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._smi is not None:
            try:
                self._smi.terminate()
                self._smi.wait(timeout=5)
                self._smi_tmp.flush()
                rows = [r.split(",") for r in Path(self._smi_tmp.name).read_text().strip().splitlines() if r.strip()]
                os.unlink(self._smi_tmp.name)
                # nvidia-smi gives no timestamps: spread the rows evenly over the sampling time
                t1 = time.perf_counter()
                for i, r in enumerate(rows):
                    r = [c.strip() for c in r]
                    if len(r) < 9:
                        continue
                    bits = 0
                    for bit, val in zip((self.R_HW_SLOWDOWN, self.R_HW_THERMAL, self.R_SW_THERMAL, self.R_SW_POWER_CAP), r[5:9]):
                        if val.lower().startswith("active"):
                            bits |= bit
                    try:
                        self.sm_max = float(r[2])
                        self.samples.append((self._t_start + (t1 - self._t_start) * (i + 0.5) / len(rows), float(r[1]), bits,
                                             float(r[3])))
                    except ValueError:
                        pass
            except Exception:
                pass

    def window(self, t0: float, t1: float, what: str):
        """Median SM clock, maximum power and the union of throttle reasons of the samples taken
        in [t0, t1] (host clock)."""
        rows = [r for r in self.samples if t0 <= r[0] <= t1]
        out = {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": len(rows),
               "window": what, "window_ms": round((t1 - t0) * 1e3, 2), "source": self.source}
        if rows:
            bits = 0
            for r in rows:
                bits |= r[2]
            names = [(self.R_HW_SLOWDOWN, "hw_slowdown"), (self.R_HW_THERMAL, "hw_thermal_slowdown"),
                     (self.R_SW_THERMAL, "sw_thermal_slowdown"), (self.R_SW_POWER_CAP, "sw_power_cap")]
            out.update(sm_mhz=statistics.median(r[1] for r in rows), reasons=sorted(n for b, n in names if bits & b),
                       power_w_max=round(max(r[3] for r in rows), 1))
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


def sustained_loop(fn, est_ms: float, seconds: float, sampler, what: str):
    """``fn`` back to back for about ``seconds`` (one CUDA-event pair around the whole loop) with the
    clock samples of exactly that loop: the rate a power-capped part holds, and ``ms x MHz``, the
    clock-normalised duration that tells a clock (power) effect from a kernel effect."""
    n = max(8, int(seconds * 1e3 / max(est_ms, 1e-3)))
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1) / n
    out = {"ms": round(ms, 5), "launches": n, "loop_s": round(t1 - t0, 2)}
    if sampler is not None:
        w = sampler.window(t0 + 0.25 * (t1 - t0), t1, what)     # the first quarter is the ramp to the power cap
        out.update(sm_mhz_median=w["sm_mhz"], power_w_max=w.get("power_w_max"), reasons=w["reasons"],
                   clock_samples=w["samples"])
        if w["sm_mhz"]:
            out["ms_x_mhz"] = round(ms * w["sm_mhz"], 2)
    return out


def burst_time(fn, steps: int = 20, warmup: int = 5, idle_s: float = 0.5):
    """The protocol of the headline region applied to any callable: the GPU idles, ``warmup``
    launches, then ``steps`` launches inside one event pair.  Returns ms per launch."""
    torch.cuda.synchronize()
    time.sleep(idle_s)
    return time_loop(fn, steps, warmup) / steps


def library_peaks(dev, sampler, seconds: float = 2.0):
    """Tensor-core rates of the vendor library on THIS GPU in THIS run: the denominators of the
    INT8 / FP8 rooflines.  ``torch._int_mm`` (cuBLASLt INT8, int32 accumulate) and
    ``torch._scaled_mm`` (cuBLASLt FP8 e4m3) on 8192^3, as a burst (same protocol as the headline
    region) and in a loop of ``seconds`` with the clocks of that loop.  A kind the library refuses
    is reported as None and the caller falls back to 2 x the measured bf16 rate."""
    n = 8192
    ops_ = 2.0 * n * n * n
    out = {}
    g = torch.Generator(device=dev).manual_seed(11)
    try:
        a = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8, generator=g)
        b = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8, generator=g).t()   # column-major B
        f = lambda: torch._int_mm(a, b)  # noqa: E731
        ms = burst_time(f)
        sus = sustained_loop(f, ms, seconds, sampler, "torch._int_mm 8192^3 loop")
        out["int8"] = {"burst_tops": round(ops_ / ms / 1e9, 1), "sustained_tops": round(ops_ / sus["ms"] / 1e9, 1),
                       "sustained": sus, "how": "torch._int_mm 8192^3 (cuBLASLt), burst = 20 launches after idle + 5 warm-up"}
        del a, b
    except Exception as exc:
        out["int8"] = None
        out["int8_error"] = str(exc).splitlines()[0][:200]
    try:
        a = torch.randn(n, n, device=dev, generator=g).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev, generator=g).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
        ms = burst_time(f)
        sus = sustained_loop(f, ms, seconds, sampler, "torch._scaled_mm 8192^3 loop")
        out["fp8"] = {"burst_tflops": round(ops_ / ms / 1e9, 1), "sustained_tflops": round(ops_ / sus["ms"] / 1e9, 1),
                      "sustained": sus, "how": "torch._scaled_mm e4m3 8192^3 -> bf16 (cuBLASLt), same protocol"}
        del a, b
    except Exception as exc:
        out["fp8"] = None
        out["fp8_error"] = str(exc).splitlines()[0][:200]
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------
# CPU baseline / reference arm (oracle port of the reference path on host cores)
# ---------------------------------------------------------------------------------------------
def _cpu_step_fn(rows: int):
    """One CPU step of the headline workload on ``rows`` tokens -> (callable, description).

    The quantisation half runs the reference's own ``INTERPRETER.execute("quantize_per_token",
    {"X": X.float()})`` (arke/ir/ops/interpreter.py:42-141 -> reference_impls.py:215-218) when the
    reference package is staged beside the oracle, else its restatement; the reference has no
    quantised GEMM at all, so the int8 GEMM + dequantisation half is the oracle restatement
    (exact integer accumulation in float64, fp32 epilogue) in both cases."""
    import oracle as oracle_pkg
    from oracle import ops as oracle
    c = CFG["w8a8"]
    x = oracle.make_quant_input(rows, c["K"], seed=1)
    w, sw = oracle.make_w8a8_weights(c["K"], c["N"], seed=2)
    interp = None
    if oracle_pkg.use_reference() is not None:
        try:
            from arke.ir.ops.interpreter import INTERPRETER
            interp = INTERPRETER
        except Exception:
            interp = None
    if interp is not None:
        def step():
            xf = x.float()
            q = interp.execute("quantize_per_token", {"X": xf})
            q = q[0] if isinstance(q, tuple) else q
            sx = xf.abs().amax(dim=-1) / 127.0
            return oracle.w8a8_gemm(q, sx, w, sw)
        how = ("quantize = the reference's INTERPRETER.execute('quantize_per_token') on X.float(); int8 GEMM + dequant = "
               "oracle restatement (the reference has no quantised GEMM)")
    else:
        def step():
            q, sx = oracle.quantize_per_token_interp(x)
            return oracle.w8a8_gemm(q, sx, w, sw)
        how = "oracle restatement of ref_quantize_per_token + exact int GEMM + dequant (reference package not staged)"
    return step, how


def cpu_w8a8_sample(rows: int, reps: int = 1):
    """Times the CPU path on ``rows`` tokens of the w8a8 workload; returns (TOPS, seconds per
    pass, cores, description)."""
    c = CFG["w8a8"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    step, how = _cpu_step_fn(rows)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    ops = 2.0 * rows * c["N"] * c["K"]
    return ops / best / 1e12, best, cores, how


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    c = CFG["w8a8"]
    rows = args.ref_rows
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    step, how = _cpu_step_fn(rows)
    times = []
    for _ in range(args.warmup):
        step()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    per = sum(times) / len(times)
    tops = 2.0 * rows * c["N"] * c["K"] / per / 1e12
    full = rows == c["M"]
    line = {
        "impl": "reference", "metric": "w8a8_gemm_tops", "value": round(tops, 5), "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(per * 1e3 * (c["M"] / rows), 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": bench_config(),
        "cpu_baseline": {"value": round(tops, 5), "unit": "TOPS", "cores": cores, "kind": "port",
                         "sample": ("the full batch of 8192 tokens x full W per step" if full else
                                    f"{rows} of {c['M']} tokens x full W per step (ms_per_step extrapolated to the full batch)")
                                   + f", torch CPU ({torch.get_num_threads()} threads); {how}"},
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


def op_quantize(ops, oracle, peaks, cfg, iters, small, ctx):
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

    ms = time_loop(fq, 4, 3) / 4 if (small or ctx.get("eager")) else graph_time(fq, 40)
    nbytes = c["M"] * c["K"] * 3 + c["M"] * 4
    r = _hbm(peaks, nbytes, ms)
    r["note"] = ("achieved counts the algorithmic bytes; the 33.5 MB of q written by one launch stay in the 126 MB L2 "
                 "(the GEMM that follows reads them there), so the DRAM counters see about 70 % of them")
    r["achieved_dram_gbs"] = round(TRAFFIC["quantize_per_token"] / ms / 1e6, 1) if not small else None
    return {"quantize_per_token": {"us": round(ms * 1e3, 2), "bytes": nbytes, "roofline": r}}


def op_rmsnorm(ops, oracle, peaks, cfg, iters, small, ctx):
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

    ms = time_loop(f, 4, 3) / 4 if (small or ctx.get("eager")) else graph_time(f, 40)   # one CUDA graph of 40 launches
    nbytes = c["M"] * c["K"] * 5 + c["M"] * 4 + c["K"] * 2
    return {"rmsnorm_residual_quant_int8": {"us": round(ms * 1e3, 2), "bytes": nbytes, "roofline": _hbm(peaks, nbytes, ms)}}


def op_rope(ops, oracle, peaks, cfg, iters, small, ctx):
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


def op_swiglu(ops, oracle, peaks, cfg, iters, small, ctx):
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


def op_fp8_gemm(ops, oracle, peaks, cfg, iters, small, ctx):
    c = cfg["w8a8"]
    g = torch.Generator().manual_seed(2)
    a8 = torch.randn(c["M"], c["K"], generator=g).to(torch.float8_e4m3fn).to(DEV)
    w8 = torch.randn(c["K"], c["N"], generator=g).to(torch.float8_e4m3fn).to(DEV)
    sa = torch.rand(c["M"], generator=g).to(DEV)
    swv = torch.rand(c["N"], generator=g).to(DEV)
    y = torch.empty(c["M"], c["N"], dtype=torch.bfloat16, device=DEV)
    f = lambda: ops.fp8_gemm(a8, sa, w8, swv, out=y)  # noqa: E731
    ms = time_loop(f, iters, 3) / iters
    fl = 2.0 * c["M"] * c["N"] * c["K"]
    sus = None
    if not small and ctx.get("sampler") is not None:
        sus = sustained_loop(f, ms, ctx["sustain_s"], ctx["sampler"], "fp8 GEMM loop")
        sus["achieved"] = round(fl / sus["ms"] / 1e9, 1)
    return {"fp8_gemm": {"us": round(ms * 1e3, 1), "flop": fl,
                         "roofline": _tensor_roofline("fp8", fl / ms / 1e9, sus, (ctx.get("lib") or {}).get("fp8"), peaks,
                                                      "kernel gemm_pair_tcgen05_kernel<f8f6f4>; same main loop as the INT8 GEMM")}}


def op_w8a8_gemm(ops, oracle, peaks, cfg, iters, small, ctx):
    c = cfg["w8a8"]
    x = oracle.make_quant_input(c["M"], c["K"], seed=1).to(DEV)
    q, sx = ops.quantize_per_token(x)
    w, sw = oracle.make_w8a8_weights(c["K"], c["N"], seed=2)
    w, sw = w.to(DEV), sw.to(DEV)
    y = torch.empty(c["M"], c["N"], dtype=torch.bfloat16, device=DEV)
    ms = time_loop(lambda: ops.w8a8_gemm(q, sx, w, sw, out=y), iters, 3) / iters
    fl = 2.0 * c["M"] * c["N"] * c["K"]
    return {"w8a8_gemm": {"us": round(ms * 1e3, 1), "flop": fl,
                          "roofline": _tensor_roofline("int8", fl / ms / 1e9, None, (ctx.get("lib") or {}).get("int8"), peaks,
                                                       "kernel gemm_pair_tcgen05_kernel<i8>")}}


def op_gqa(ops, oracle, peaks, cfg, iters, small, ctx):
    c4 = cfg["gqa"]
    qq, kk, vv = oracle.make_attention_inputs(c4["B"], c4["Hq"], c4["Hkv"], c4["S"], c4["D"], seed=4)
    qq, kk, vv = qq.to(DEV), kk.to(DEV), vv.to(DEV)
    f = lambda: ops.gqa_fwd(qq, kk, vv, causal=True)  # noqa: E731
    ms = time_loop(f, iters, 3) / iters
    fl = 2.0 * c4["B"] * c4["Hq"] * c4["S"] * c4["S"] * c4["D"]
    res = {"us": round(ms * 1e3, 1), "flop": fl,
           "roofline": roofline("tensor", fl / ms / 1e9, peaks["bf16_tflops"], NOMINAL["bf16_tflops"], "TFLOP/s",
                                src=peaks["source"], note="peak = cuBLAS bf16 burst (the timed window is a few ms)")}
    if not small:
        # context only: the vendor library's attention (torch SDPA) on the same inputs, same loop
        try:
            import torch.nn.functional as F
            g = lambda: F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, enable_gqa=True)  # noqa: E731
            res["library_us"] = round(time_loop(g, iters, 3) / iters * 1e3, 1)
            res["library"] = "torch.nn.functional.scaled_dot_product_attention(enable_gqa=True), backend chosen by torch"
        except Exception as exc:
            res["library_us"] = None
            res["library"] = f"torch SDPA unavailable: {str(exc).splitlines()[0][:120]}"
        if ctx.get("sampler") is not None:
            sus = sustained_loop(f, ms, ctx["sustain_s"], ctx["sampler"], "gqa loop")
            res["roofline"]["sustained"] = {
                "achieved": round(fl / sus["ms"] / 1e9, 1), "peak": peaks["bf16_tflops_sustained"],
                "frac": round(fl / sus["ms"] / 1e9 / peaks["bf16_tflops_sustained"], 4), "kernel_us": round(sus["ms"] * 1e3, 1),
                "sm_mhz_median": sus.get("sm_mhz_median"), "ms_x_mhz": sus.get("ms_x_mhz"), "power_w_max": sus.get("power_w_max")}
    return {"gqa_fwd_causal": res}


def op_flce(ops, oracle, peaks, cfg, iters, small, ctx):
    c5 = cfg["flce"]
    x5, w5, l5 = oracle.make_flce_inputs(c5["M"], c5["D"], c5["V"], seed=5)
    x5, w5, l5 = x5.to(DEV), w5.to(DEV), l5.to(DEV)
    ws = torch.empty(ops.fused_linear_ce_workspace_bytes(c5["M"], c5["V"], c5["D"]), dtype=torch.uint8, device=DEV)
    n5 = max(2, iters // 2)
    ms = time_loop(lambda: ops.fused_linear_ce(x5, w5, l5, workspace=ws), n5, 2) / n5
    fl = 2.0 * c5["M"] * c5["V"] * c5["D"]
    res = {"us": round(ms * 1e3, 1), "flop": fl,
           "roofline": roofline("tensor", fl / ms / 1e9, peaks["bf16_tflops"], NOMINAL["bf16_tflops"],
                                "TFLOP/s", src=peaks["source"], note="peak = cuBLAS bf16 burst: the timed window is tens of ms, far below a second")}
    if not small and ctx.get("sampler") is not None:
        sus = sustained_loop(lambda: ops.fused_linear_ce(x5, w5, l5, workspace=ws), ms, ctx["sustain_s"], ctx["sampler"], "flce loop")
        res["roofline"]["sustained"] = {
            "achieved": round(fl / sus["ms"] / 1e9, 1), "peak": peaks["bf16_tflops_sustained"],
            "frac": round(fl / sus["ms"] / 1e9 / peaks["bf16_tflops_sustained"], 4), "kernel_us": round(sus["ms"] * 1e3, 1),
            "sm_mhz_median": sus.get("sm_mhz_median"), "ms_x_mhz": sus.get("ms_x_mhz"), "power_w_max": sus.get("power_w_max")}
    return {"fused_linear_ce": res}


def op_flce_bwd(ops, oracle, peaks, cfg, iters, small, ctx):
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
                                         "roofline": roofline("tensor", fl / ms / 1e9, peaks["bf16_tflops"], NOMINAL["bf16_tflops"],
                                                              "TFLOP/s", src=peaks["source"],
                                                              note="three launches (logits gradient, dX, dW); peak = cuBLAS bf16 burst (window of tens of ms)")}}


OPS = {"quantize": op_quantize, "rmsnorm": op_rmsnorm, "rope": op_rope, "swiglu": op_swiglu, "fp8": op_fp8_gemm, "w8a8": op_w8a8_gemm, "gqa": op_gqa, "flce": op_flce, "flce_bwd": op_flce_bwd}


def per_op_measurements(ops, oracle, peaks, quick: bool, only=None, small=False, lib=None, sampler=None, sustain_s=2.0,
                        eager=False):
    """Each hot-path op at its BASELINE configuration (or at the reduced ``SMALL`` shapes used for
    profiler captures); ``only`` restricts the run to one op.  Every window here is far shorter than
    a second, so fractions are against the burst peaks; the tensor-core ops add a ``sustained``
    entry (a loop of seconds, against the sustained peaks) when a clock sampler is given."""
    out = {}
    ctx = {"lib": lib, "sampler": sampler, "sustain_s": sustain_s, "eager": eager}
    iters = 3 if small else (5 if quick else 10)
    cfg = dict(CFG)
    if small:
        cfg.update(SMALL)
    for name, fn in OPS.items():
        if only is not None and name != only:
            continue
        if only is None and name == "w8a8":
            continue  # the headline step already reports it
        out.update(fn(ops, oracle, peaks, cfg, iters, small, ctx))
        torch.cuda.empty_cache()
    if not small:
        for k, v in out.items():
            if k in TRAFFIC:
                v["roofline"]["traffic"] = TRAFFIC[k]
                v["roofline"]["traffic_captured"] = TRAFFIC_CAPTURED[k]
    return out


def run_single_op(args):
    """``--only OP [--small]``: one op, one JSON line; the entry point used for profiler captures."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the B200 path has no CPU fallback)")
    torch.cuda.set_device(0)
    from arke_b200 import ops
    from oracle import ops as oracle
    opts = {}
    for item in args.option or []:
        k, _, v = item.partition("=")
        opts[k] = int(v)
    with ops.options(**opts):
        res = per_op_measurements(ops, oracle, measured_peaks(), True, only=args.only, small=args.small, eager=args.eager)
    if ops.kernel_status() != 0:
        raise SystemExit("bench.py: a device-side wait expired")
    print(json.dumps({"only": args.only, "small": bool(args.small), "per_op": res}))


# ---------------------------------------------------------------------------------------------
# main arm
# ---------------------------------------------------------------------------------------------
def multi_gpu_legs(ops, oracle, dev, rank, world, max_over_ranks, barrier):
    """The N > 1 part of the run; returns the ``per_op`` object of the JSON line.

    parity   the vocabulary-sharded loss and its backward on a small fixed problem, compared with
             the single-rank kernels (every rank) and with the CPU oracle (rank 0)
    sharded  fused linear + CE at the BASELINE size with the vocabulary split over the ranks: the
             one op with a collective (all-gather of the [M,3] partials, then the combine kernel)
    strong   the communication-free ops: each rank times its shard of the FIXED BASELINE problem
             (token rows / (batch x KV-group) units) and, beside it, the whole problem on one GPU;
             speed-up = T(1 GPU, whole problem) / max over ranks T(shard)
    """
    import torch.distributed as dist
    from arke_b200.sharding import (lse_from_partials, shard_attention, shard_bounds, vocab_sharded_ce,
                                    vocab_sharded_ce_backward)
    out = {}

    # ---------------- parity ----------------
    Mp, Dp, Vp = 512, 256, 8216
    xp, wp, lp = oracle.make_flce_inputs(Mp, Dp, Vp, seed=17, ignore_frac=0.05)     # identical on every rank (seeded)
    xd, wd, ld = xp.to(dev), wp.to(dev), lp.to(dev)
    v0, v1 = shard_bounds(Vp, world, rank)
    wsh = wd[v0:v1].contiguous()
    part = ops.fused_linear_ce(xd, wsh, ld, vocab_offset=v0, want_partials=True).contiguous()
    gathered = torch.empty((world * Mp, 3), dtype=part.dtype, device=dev)
    dist.all_gather_into_tensor(gathered, part)
    tok_s, mean_s = ops.ce_combine(gathered.view(world, Mp, 3), ld)
    lse = lse_from_partials(gathered.view(world, Mp, 3))
    dx_s, dw_s = vocab_sharded_ce_backward(xd, wsh, ld, v0, lse)
    tok_1, mean_1 = ops.fused_linear_ce(xd, wd, ld)
    dx_1, dw_1 = ops.fused_linear_ce_backward(xd, wd, ld, dx_dtype=torch.float32)
    loss_abs = float((tok_s - tok_1).abs().max())
    mean_abs = abs(float(mean_s) - float(mean_1))
    dx_rel = float((dx_s - dx_1).norm() / dx_1.norm())
    dw_rel = float((dw_s.float() - dw_1[v0:v1].float()).norm() / dw_1[v0:v1].float().norm())
    loss_abs, mean_abs, dx_rel, dw_rel = max_over_ranks(loss_abs, mean_abs, dx_rel, dw_rel)
    parity = {"problem": f"M={Mp} D={Dp} V={Vp} bf16, 5% ignored labels, vocabulary split over {world} ranks",
              "loss_max_abs": loss_abs, "mean_abs": mean_abs, "dx_rel": dx_rel, "dw_rel": dw_rel,
              "versus": "the single-rank kernels on the same inputs (max over ranks)"}
    ok = loss_abs <= 1e-3 and mean_abs <= 1e-3 and dx_rel <= 1e-2 and dw_rel <= 1e-2
    if rank == 0:
        tok_o, mean_o = oracle.fused_linear_ce(xp, wp, lp)
        dxo, _ = oracle.fused_linear_ce_backward(xp, wp, lp)
        parity["loss_vs_oracle_max_abs"] = float((tok_s.cpu() - tok_o).abs().max())
        parity["dx_vs_oracle_rel"] = float((dx_s.cpu() - dxo).norm() / dxo.norm())
        ok = ok and parity["loss_vs_oracle_max_abs"] <= 1e-3 and parity["dx_vs_oracle_rel"] <= 1e-2
    parity["tolerances"] = "loss 1e-3 abs, gradients 1e-2 relative (16-bit logits gradient)"
    parity["ok"] = bool(ok)
    del xd, wd, ld, wsh, dx_s, dw_s, dx_1, dw_1

    # ---------------- vocabulary-sharded fused linear + CE at the BASELINE size ----------------
    c5 = CFG["flce"]
    v0, v1 = shard_bounds(c5["V"], world, rank)
    x5, w5, l5 = oracle.make_flce_inputs(c5["M"], c5["D"], v1 - v0, seed=5)   # this rank's W slice
    l5 = torch.randint(0, c5["V"], (c5["M"],), generator=torch.Generator().manual_seed(55), dtype=torch.int64)
    x5, w5, l5 = x5.to(dev), w5.to(dev), l5.to(dev)
    dist.broadcast(x5, 0)            # every rank sees the same tokens
    ws = torch.empty(ops.fused_linear_ce_workspace_bytes(c5["M"], v1 - v0, c5["D"]), dtype=torch.uint8, device=dev)
    part_fn = lambda xx, ww, ll, off: ops.fused_linear_ce(xx, ww, ll, vocab_offset=off, want_partials=True, workspace=ws)  # noqa: E731
    run5 = lambda: vocab_sharded_ce(x5, w5, l5, v0, partial_fn=part_fn)  # noqa: E731
    barrier()
    n5 = 5
    ms5 = time_loop(run5, n5, 2) / n5
    (ms5,) = max_over_ranks(ms5)
    fl5 = 2.0 * c5["M"] * c5["V"] * c5["D"]
    out["fused_linear_ce_vocab_sharded"] = {
        "us": round(ms5 * 1e3, 1), "flop": fl5, "tflops_all_gpus": round(fl5 / ms5 / 1e9, 1),
        "vocab_per_gpu": v1 - v0, "collective": "all_gather_into_tensor [M,3] fp32 (98 KB per rank) + ce_combine",
        "scaling": "strong (total vocabulary fixed)", "parity": parity}
    del x5, w5, l5, ws
    torch.cuda.empty_cache()

    def strong(name, t_full_ms, t_shard_ms, units, note):
        t_full, t_shard = max_over_ranks(t_full_ms, t_shard_ms)
        out[name] = {"strong": {"us_max_over_ranks": round(t_shard * 1e3, 2), "us_one_gpu_whole_problem": round(t_full * 1e3, 2),
                                "speedup_vs_n1": round(t_full / t_shard, 2), "units_per_rank": units, "note": note}}

    # ---------------- quantize, and quantize + W8A8 GEMM: token rows ----------------
    c = CFG["w8a8"]
    M, K, N = c["M"], c["K"], c["N"]
    xs = [oracle.make_quant_input(M, K, seed=1).to(dev)]
    xs += [xs[0].clone() for _ in range(NBUF - 1)]                       # 268 MB of inputs in rotation
    w, sw = (t.to(dev) for t in oracle.make_w8a8_weights(K, N, seed=2))
    bounds = [shard_bounds(M, world, r) for r in range(world)]
    rows = bounds[rank][1] - bounds[rank][0]
    q = torch.empty(M, K, dtype=torch.int8, device=dev)
    sx = torch.empty(M, dtype=torch.float32, device=dev)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    k = [0]

    def shard_view(t):       # a different row shard of a different buffer every launch: bytes come from HBM
        k[0] += 1
        b, e = bounds[(rank + k[0]) % world]
        return xs[k[0] % NBUF][b:e], b, e

    def fq_shard():
        xv, b, e = shard_view(None)
        ops.quantize_per_token(xv, out=(q[b:e], sx[b:e]))

    def fq_full():
        k[0] += 1
        ops.quantize_per_token(xs[k[0] % NBUF], out=(q, sx))

    def fs_shard():
        xv, b, e = shard_view(None)
        ops.quantize_per_token(xv, out=(q[b:e], sx[b:e]))
        ops.w8a8_gemm(q[b:e], sx[b:e], w, sw, out=y[b:e])

    def fs_full():
        k[0] += 1
        ops.quantize_per_token(xs[k[0] % NBUF], out=(q, sx))
        ops.w8a8_gemm(q, sx, w, sw, out=y)

    barrier()
    t_full = graph_time(fq_full, 40)
    barrier()
    t_shard = graph_time(fq_shard, 40)
    strong("quantize_per_token", t_full, t_shard, rows, "rows of X per rank; one CUDA graph of 40 launches, 4 rotating inputs")
    barrier()
    t_full = graph_time(fs_full, 20)
    barrier()
    t_shard = graph_time(fs_shard, 20)
    strong("w8a8_step", t_full, t_shard, rows, "quantize + W8A8 GEMM on the rank's rows, W replicated; one CUDA graph of 20 steps")
    del xs, q, sx, y, w, sw
    torch.cuda.empty_cache()

    # ---------------- packed SwiGLU + FP8: token rows ----------------
    c3 = CFG["swiglu"]
    x3 = oracle.make_swiglu_input(c3["M"], c3["N2"], seed=3).to(dev)
    b3 = [shard_bounds(c3["M"], world, r) for r in range(world)]

    def f3_shard():
        k[0] += 1
        b, e = b3[(rank + k[0]) % world]
        ops.swiglu_fp8(x3[b:e])

    barrier()
    t_full = time_loop(lambda: ops.swiglu_fp8(x3), 10, 3) / 10
    barrier()
    t_shard = graph_time(f3_shard, 2 * world)
    strong("swiglu_fp8", t_full, t_shard, b3[rank][1] - b3[rank][0],
           "rows per rank, a different row shard of the 940 MB input every launch; one CUDA graph")
    del x3
    torch.cuda.empty_cache()

    # ---------------- causal GQA forward: (batch x KV-group) units ----------------
    c4 = CFG["gqa"]
    qq, kk, vv = (t.to(dev) for t in oracle.make_attention_inputs(c4["B"], c4["Hq"], c4["Hkv"], c4["S"], c4["D"], seed=4))
    shards = [shard_attention(qq, kk, vv, world, r) for r in range(world)]

    def f4_shard():
        k[0] += 1
        qs, ks, vs = shards[(rank + k[0]) % world]
        ops.gqa_fwd(qs, ks, vs, causal=True)

    barrier()
    t_full = time_loop(lambda: ops.gqa_fwd(qq, kk, vv, causal=True), 5, 2) / 5
    barrier()
    t_shard = time_loop(f4_shard, 2 * world, 3) / (2 * world)
    strong("gqa_fwd_causal", t_full, t_shard, shards[rank][1].shape[1],
           "(batch x KV-group) units per rank, the sequence is never split; a different unit shard every launch")
    del qq, kk, vv, shards
    torch.cuda.empty_cache()
    if ops.kernel_status() != 0:
        raise SystemExit("bench.py: a device-side wait expired in the multi-GPU legs")
    return out


def _tensor_roofline(kind, achieved_burst, sus, lib, peaks, note):
    """Roofline object of a tensor-core kernel against the vendor library's rate for the same
    operand kind measured in this run (``lib`` = library_peaks()[kind] or None), with the nominal
    peak and the 2 x bf16 proxy beside it; ``sus`` = sustained_loop() of the same kernel."""
    unit = "TOP/s" if kind == "int8" else "TFLOP/s"
    nominal = NOMINAL["int8_tops" if kind == "int8" else "fp8_tflops"]
    key = "tops" if kind == "int8" else "tflops"
    if lib:
        peak, src = lib[f"burst_{key}"], f"measured in this run: {lib['how']}"
    else:
        peak, src = 2 * peaks["bf16_tflops"], f"2 x {peaks['source']} bf16 cuBLAS burst (the library refused a {kind} GEMM here)"
    r = roofline("tensor", achieved_burst, peak, nominal, unit, src=src, note=note)
    r["frac_of_2x_bf16_burst"] = round(achieved_burst / (2 * peaks["bf16_tflops"]), 4)
    if sus is not None:
        sp = lib[f"sustained_{key}"] if lib else 2 * peaks["bf16_tflops_sustained"]
        r["sustained"] = {"achieved": sus["achieved"], "peak": sp, "frac": round(sus["achieved"] / sp, 4),
                          "frac_of_nominal": round(sus["achieved"] / nominal, 4),
                          "frac_of_2x_bf16_sustained": round(sus["achieved"] / (2 * peaks["bf16_tflops_sustained"]), 4),
                          "kernel_us": round(sus["ms"] * 1e3, 1), "sm_mhz_median": sus.get("sm_mhz_median"),
                          "ms_x_mhz": sus.get("ms_x_mhz"), "power_w_max": sus.get("power_w_max"),
                          "reasons": sus.get("reasons"), "loop_s": sus["loop_s"], "launches": sus["launches"]}
        if lib and lib["sustained"].get("ms_x_mhz"):
            r["sustained"]["library_ms_x_mhz"] = lib["sustained"]["ms_x_mhz"]
            r["sustained"]["library_sm_mhz_median"] = lib["sustained"].get("sm_mhz_median")
    return r


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the B200 path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        # stdout carries the one JSON line: NCCL's version banner (printed when the communicator
        # is made, if the environment asks for NCCL_DEBUG=VERSION) is sent to stderr instead
        sys.stdout.flush()
        saved_fd = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_fd, 1)
            os.close(saved_fd)
    from arke_b200 import ops
    from oracle import ops as oracle  # input generators, the CPU-baseline leg and the N > 1 parity check only
    peaks = measured_peaks()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler is not None:
        sampler.start()

    def barrier():
        if use_dist:
            dist.barrier()

    def max_over_ranks(*vals):
        if not use_dist:
            return [float(v) for v in vals]
        tt = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return [float(v) for v in tt]

    c = CFG["w8a8"]
    M, K, N = c["M"], c["K"], c["N"]
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

    # ---- the timed region: W warm-up steps, then exactly K steps between two events ----
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.window(t0, t1, f"the {args.steps} timed steps") if sampler is not None else None
    # The same K steps once more with an event pair around every GEMM launch: the kernel's own
    # duration for the roofline.  Kept out of the timed region above because an event record
    # between the two kernels of a step removes their programmatic-dependent-launch overlap.
    for _ in range(args.steps):
        step(record=True)
    torch.cuda.synchronize()
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events) / len(gemm_events)
    status = ops.kernel_status()
    if status != 0:
        raise SystemExit(f"bench.py: a device-side wait expired (kernel status {status})")
    ms_total, gemm_ms = max_over_ranks(ms_total, gemm_ms)
    ms_step = ms_total / args.steps
    gemm_ops = 2.0 * M * N * K
    value = gemm_ops * world / (ms_step * 1e-3) / 1e12

    # ---- sustained leg: the same step, and the GEMM alone, looped for seconds (power-capped clocks) ----
    barrier()
    sus_step = sustained_loop(step, ms_step, args.sustain_s, sampler, "whole-step loop")
    barrier()
    sus_gemm = sustained_loop(lambda: ops.w8a8_gemm(q, sx, w, sw, out=y), gemm_ms, args.sustain_s, sampler, "GEMM-only loop")
    sus_step_ms, sus_gemm_ms = max_over_ranks(sus_step["ms"], sus_gemm["ms"])
    sus_gemm["ms"] = sus_gemm_ms
    sus_gemm["achieved"] = round(gemm_ops / sus_gemm_ms / 1e9, 1)
    if sus_gemm.get("sm_mhz_median"):
        sus_gemm["ms_x_mhz"] = round(sus_gemm_ms * sus_gemm["sm_mhz_median"], 2)

    # ---- the vendor library's INT8 / FP8 GEMM rate on this GPU, in this run (roofline denominators) ----
    barrier()
    lib = library_peaks(dev, sampler, args.sustain_s) if not args.no_library_peaks else {"int8": None, "fp8": None}
    barrier()

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
    barrier()
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
    # the PCIe floor beside it: the bare copies of one step (235 MB D2H with 67 MB H2D the other
    # way, no kernels), all ranks at once — what the host side of the links delivers to N GPUs
    y_dev_full = y
    s2 = torch.cuda.Stream(dev)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        with torch.cuda.stream(s2):
            xs[0].copy_(xh, non_blocking=True)
        yh.copy_(y_dev_full, non_blocking=True)
    cur.wait_stream(s2)
    e1.record()
    torch.cuda.synchronize()
    ms_copy = e0.elapsed_time(e1) / 3
    ms_e2e, ms_copy = max_over_ranks(ms_e2e, ms_copy)
    e2e_val = gemm_ops * world / (ms_e2e * 1e-3) / 1e12
    xs[0].copy_(xs[1])

    # ---- N > 1: (1) parity of the multi-rank result, (2) fused linear + CE with the vocabulary
    # sharded over the ranks (the one op with a collective), (3) strong scaling of the
    # communication-free ops: each rank times its shard of the FIXED BASELINE problem ----
    multi = None
    if use_dist:
        multi = multi_gpu_legs(ops, oracle, dev, rank, world, max_over_ranks, barrier)

    if rank != 0:
        if use_dist:
            dist.barrier()
            dist.destroy_process_group()
        return

    line = {
        "metric": "w8a8_gemm_tops", "value": round(value, 1), "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": bench_config(),
        "gpu_launches": 2 * args.steps,
        "roofline": _tensor_roofline(
            "int8", gemm_ops / (gemm_ms * 1e-3) / 1e12, sus_gemm, lib.get("int8"), peaks,
            "kernel gemm_pair_tcgen05_kernel<i8> (two-CTA tcgen05); achieved = 2*M*N*K / mean CUDA-event time of the GEMM launch "
            "over a repeat of the timed steps (events between the kernels would break the dependent-launch overlap of the timed "
            "region itself); `sustained` = the same launch looped for seconds under the power cap"),
        "sustained": {"ms_per_step": round(sus_step_ms, 4), "value": round(gemm_ops * world / (sus_step_ms * 1e-3) / 1e12, 1),
                      "unit": "TOPS", "sm_mhz_median": sus_step.get("sm_mhz_median"), "power_w_max": sus_step.get("power_w_max"),
                      "reasons": sus_step.get("reasons"), "loop_s": sus_step["loop_s"], "steps": sus_step["launches"],
                      "note": "the timed steps repeated back to back for seconds: the rate under the 1 kW power cap"},
        "library_peaks": lib,
        "e2e": {"value": round(e2e_val, 1), "unit": "TOPS", "h2d_bytes_per_step": M * K * 2 * world,
                "d2h_bytes_per_step": M * N * 2 * world, "ms_per_step": round(ms_e2e, 3),
                "bare_copies_ms_per_step": round(ms_copy, 3),
                "bare_copies_gbs_all_ranks": round((M * K * 2 + M * N * 2) * world / ms_copy / 1e6, 1),
                "note": "bare_copies = the step's H2D + D2H alone (no kernels) on all ranks at once: the PCIe/host floor of e2e"},
        "clocks": clocks,
    }
    line["roofline"]["kernel_us"] = round(gemm_ms * 1e3, 1)
    line["roofline"]["traffic"] = TRAFFIC["w8a8_gemm"]
    line["roofline"]["traffic_captured"] = TRAFFIC_CAPTURED["w8a8_gemm"]
    if world == 1 and not args.no_cpu_baseline:
        cpu_rows, cpu_reps = M, 4
        tops, secs, cores, how = cpu_w8a8_sample(cpu_rows, reps=cpu_reps)
        line["cpu_baseline"] = {"value": round(tops, 5), "unit": "TOPS", "cores": cores, "kind": "port",
                                "sample": f"{cpu_rows} of {M} tokens x full W, best of {cpu_reps} passes of {secs:.2f} s; {how}"}
    if world == 1 and not args.no_per_op:
        line["per_op"] = per_op_measurements(ops, oracle, peaks, args.quick, lib=lib, sampler=sampler, sustain_s=args.sustain_s)
    if multi is not None:
        line["per_op"] = multi
    sampler.stop()
    print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()
    if multi is not None and not multi["fused_linear_ce_vocab_sharded"]["parity"]["ok"]:
        raise SystemExit("bench.py: the multi-rank result differs from the single-rank kernels (see per_op ... parity)")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--ref-rows", type=int, default=8192, help="tokens per CPU step of --impl reference (default: the full batch)")
    ap.add_argument("--no-per-op", action="store_true")
    ap.add_argument("--no-library-peaks", action="store_true", help="skip the vendor-library INT8/FP8 GEMM measurement")
    ap.add_argument("--sustain-s", type=float, default=2.0, help="length of each sustained (power-capped) loop in seconds")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--only", choices=list(OPS), default=None, help="measure one op only (one JSON line)")
    ap.add_argument("--small", action="store_true", help="with --only: reduced shapes for profiler captures")
    ap.add_argument("--option", action="append", metavar="NAME=VALUE",
                    help="with --only: a library tuning option for the run, e.g. gemm_static_sched=1")
    ap.add_argument("--eager", action="store_true", help="with --only: plain launches instead of a CUDA graph (profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_single_op(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
