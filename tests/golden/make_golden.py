"""Generates ``tests/golden/*.npz`` by running the real reference (blueyi/arke) in this container.

Usage (the reference checkout is read-only, so no bytecode is written):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/arke [fixture ...]

(with fixture names, e.g. ``rope``, only those files are rewritten).

Inputs come from the seeded generators in ``cases.py``; the fixtures store only the outputs of
the reference — its semantic-IR interpreter (``arke.ir.ops.interpreter.INTERPRETER``),
``ArkePipeline.execute`` for the FP32 GEMM example, and the eager baseline runner for the
benchmark driver's quantize golden — plus a checksum of the input bits.  16-bit float tensors are
stored as int16 bit patterns (``*_bits``).
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype in (torch.bfloat16, torch.float16)
    return t.contiguous().view(torch.int16).numpy()


def rope_fixture(INTERPRETER) -> None:
    # rope: the interpreter evaluates x1*cos - x2*sin / x2*cos + x1*sin in the input dtype
    out = {}
    for name in cases.ROPE_CASES:
        for tag in list(cases.DTYPES) + ["f32"]:
            x, cos, sin = cases.rope_inputs(name, tag)
            y = INTERPRETER.execute("rope", {"X": x, "cos": cos, "sin": sin})
            assert y.dtype == x.dtype and y.shape == x.shape
            out[f"{name}_{tag}_y" + ("" if tag == "f32" else "_bits")] = y.numpy() if tag == "f32" else bits(y)
            out[f"{name}_{tag}_in"] = cases.checksum(x, cos, sin)
    np.savez_compressed(HERE / "rope.npz", **out)


def main(ref_root: str, only=()) -> None:
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from arke.ir.ops.interpreter import INTERPRETER  # type: ignore

    torch.set_num_threads(4)
    if only:
        if "rope" in only:
            rope_fixture(INTERPRETER)
        rest = [o for o in only if o != "rope"]
        if rest:
            raise SystemExit(f"partial regeneration is implemented for: rope (asked: {rest})")
        return

    # quantize_per_token: interpreter evaluated on X.float() (as the V1 hook does)
    out = {}
    for name in cases.QUANT_CASES:
        for tag in cases.DTYPES:
            x = cases.quant_input(name, tag)
            out[f"{name}_{tag}_q"] = INTERPRETER.execute("quantize_per_token", {"X": x.float()}).numpy()
            out[f"{name}_{tag}_in"] = cases.checksum(x)
    ties = torch.tensor(cases.TIES)
    out["ties_q"] = INTERPRETER.execute("quantize_per_token", {"X": ties}).numpy()
    np.savez_compressed(HERE / "quantize_interp.npz", **out)

    # the benchmark driver's quantize golden (same code in benchmarks/bench_l1.py:443-448 and the
    # eager baseline runner, benchmarks/baselines/pytorch_eager.py:178-183)
    from benchmarks.baselines.pytorch_eager import PyTorchEagerRunner  # type: ignore
    eager = PyTorchEagerRunner()
    out = {}
    for name in cases.QUANT_BENCH_CASES:
        for tag in cases.DTYPES:
            x = cases.quant_input(name, tag, cases.QUANT_BENCH_CASES, "quantb")
            q, sc = eager.run_with_inputs("quantize_per_token", x)
            out[f"{name}_{tag}_q"] = q.numpy()
            out[f"{name}_{tag}_scales_bits"] = bits(sc)
            out[f"{name}_{tag}_in"] = cases.checksum(x)
    np.savez_compressed(HERE / "quantize_bench_l1.npz", **out)

    out = {}
    for name in cases.SILU_CASES:
        for tag in cases.DTYPES:
            x = cases.silu_input(name, tag)
            y = INTERPRETER.execute("silu_and_mul", {"X": x})
            assert y.dtype == x.dtype
            out[f"{name}_{tag}_y_bits"] = bits(y)
            out[f"{name}_{tag}_in"] = cases.checksum(x)
    np.savez_compressed(HERE / "silu_and_mul.npz", **out)

    out = {}
    for name in cases.GQA_CASES:
        for tag in cases.DTYPES:
            q, k, v = cases.gqa_inputs(name, tag)
            for causal in (True, False):
                o = INTERPRETER.execute("grouped_query_attention", {"Q": q, "K": k, "V": v}, {"is_causal": causal})
                out[f"{name}_{tag}_o_{'causal' if causal else 'full'}_bits"] = bits(o)
            out[f"{name}_{tag}_in"] = cases.checksum(q, k, v)
    np.savez_compressed(HERE / "gqa.npz", **out)

    out = {}
    for name in cases.FLCE_CASES:
        for tag in cases.DTYPES:
            x, w, labels = cases.flce_inputs(name, tag)
            loss = INTERPRETER.execute("fused_linear_cross_entropy", {"X": x, "W": w, "labels": labels})
            out[f"{name}_{tag}_mean"] = np.float32(loss.item())
            out[f"{name}_{tag}_in"] = cases.checksum(x, w, labels)
    np.savez_compressed(HERE / "flce.npz", **out)

    out = {}
    for name in cases.RMS_CASES:
        for tag in cases.DTYPES:
            x, res, w = cases.rms_inputs(name, tag)
            # the interpreter promotes 16-bit inputs to fp32 for these ops (dtype_map in the catalog),
            # so its result is the fp32 value of the formula on the 16-bit inputs
            y = INTERPRETER.execute("rmsnorm", {"X": x, "W": w})
            yr = INTERPRETER.execute("rmsnorm_residual", {"X": x, "residual": res, "W": w})
            assert y.dtype == torch.float32 and yr.dtype == torch.float32
            out[f"{name}_{tag}_y"] = y.numpy()
            out[f"{name}_{tag}_yres"] = yr.numpy()
            out[f"{name}_{tag}_in"] = cases.checksum(x, res, w)
    np.savez_compressed(HERE / "rmsnorm.npz", **out)

    rope_fixture(INTERPRETER)

    # FP32 GEMM 1024^3 through the .ak pipeline (the semantic-IR interpreter path)
    from arke.compiler.pipeline import ArkePipeline  # type: ignore
    pipe = ArkePipeline()
    compiled = pipe.compile_file(str(Path(ref_root) / "examples/operators/01_matmul.ak"))
    A, B = cases.matmul_fp32_inputs()
    res = pipe.execute(compiled, {"A": A, "B": B})
    C = res if isinstance(res, torch.Tensor) else (list(res.values())[0] if isinstance(res, dict) else res[0])
    np.savez_compressed(HERE / "matmul_fp32_1024.npz", c_sample=C[::64, ::64].contiguous().numpy(),
                        c_sum=np.float64(C.double().sum().item()),
                        c_abs_sum=np.float64(C.double().abs().sum().item()), c_in=cases.checksum(A, B))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("ARKE_REFERENCE_DIR"):
        sys.exit("usage: make_golden.py <reference checkout> [fixture ...]   (or set ARKE_REFERENCE_DIR)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["ARKE_REFERENCE_DIR"], tuple(sys.argv[2:]))
