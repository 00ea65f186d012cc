"""GPU: the reference's OWN drivers, unmodified, pointed at the installed B200 backend.

``oracle/make_ref.py`` stages the reference's Python package beside the oracle; these tests put it
on ``sys.path``, call ``arke_b200.install.install()`` — the one call a maintainer adds — and then
run the drivers the way the reference's users do:

  * ``benchmarks.bench_l1.run_op`` (benchmarks/bench_l1.py:797-1184): timing through
    ``runner.get_fn`` and the correctness gate ``runner.run_with_inputs`` vs the golden of the
    ladder at ``_correctness_tolerances`` (:134-141) on registry shapes;
  * ``arke run --backend b200`` = ``arke.cli._cmd_run`` -> ``arke.agent.backends.run_backend``
    (arke/agent/backends.py:57-108, 226-288);
  * the façade tools ``compile_and_profile`` (arke/agent/tools.py:435-727: V1 comparison with the
    interpreter, V2 kernel-only timing) and ``verify_correctness`` (:1043-1190) on CUDA;
  * ``arke.agent.verification.staged_correctness_gate`` (:130-215);
  * the fusion harness rows of ``benchmarks.bench_l2``: fused linear + CE at the real vocabulary
    (:921-1043), ``silu_and_mul`` (:780-918).

What is asserted is the reference's own verdict (``correctness_status``, ``allclose``,
``correct``), not a restated tolerance.  With ``ARKE_B200_DRIVER_REPORT=<path>`` the rows are
also written to a JSON file.
"""
from __future__ import annotations

import json
import os
from types import SimpleNamespace

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

_ROWS: list[dict] = []

# op -> registry shape tags (benchmarks/shape_registry.py); two or more per op, one of them ragged
L1_CASES = {
    "quantize_per_token": ["llama3-int8-512", "non-align-1", "extreme-long-batch"],
    "silu_and_mul": ["llama3-8b", "gpt2-sm"],
    "matmul": ["square-1k", "llama-ffn", "non-align-5"],
    "flash_attention": ["llama2-7b-512", "llama2-7b-2k", "gpt2-sm-1k"],
    "grouped_query_attention": ["llama3-8b-512", "llama3-8b-2k", "llama3-batch4"],
    "fused_linear_cross_entropy": ["gpt2-seq128", "llama3-seq512"],
    "rmsnorm": ["llama-7b", "non-align-1"],
    "rmsnorm_residual": ["llama-7b", "llama-long"],
    "rope": ["llama2-512", "llama3-kv-512"],
}

# Baselines kept beside the system under test: the ones the golden ladder can pick for these ops
# (benchmarks/golden_ladder.py:84-118).  The torch.compile-based runners are left out: they spend
# minutes compiling and are never a golden for these ops.
_KEEP = {"B200ArkeRunner", "CuBLASRunner", "FlashAttnRunner", "LigerRunner", "PyTorchEagerRunner"}


@pytest.fixture(scope="module")
def ref():
    if oracle.use_reference() is None:
        pytest.skip("reference package not staged: run `python oracle/make_ref.py --src <checkout>`")
    import benchmarks.bench_l1 as l1        # registers the reference's runners, ArkeRunner included
    import benchmarks.bench_l2 as l2
    from benchmarks.baselines import base
    from arke_b200.install import install
    report = install()
    assert report["backend"] and report["agent_backends"] and report["runner"], report
    saved = list(base._REGISTRY)
    base._REGISTRY[:] = [c for c in saved if c.__name__ in _KEEP]
    yield SimpleNamespace(l1=l1, l2=l2, base=base, report=report)
    base._REGISTRY[:] = saved


def test_install_makes_the_b200_runner_the_one_named_arke(ref):
    import benchmarks.baselines.arke_runner as ar
    from arke_b200.runner import B200ArkeRunner
    assert ar.ArkeRunner is B200ArkeRunner                      # what bench_l2 imports by name
    arke = [r for r in ref.base.get_all_runners() if r.name == "Arke"]
    assert len(arke) == 1 and isinstance(arke[0], B200ArkeRunner) and arke[0].priority == 5
    assert "sm_100a" in arke[0].source


@pytest.mark.parametrize("op", sorted(L1_CASES))
def test_bench_l1_run_op(ref, op):
    results = ref.l1.run_op(op, warmup=3, reps=10, shape_tags=L1_CASES[op])
    arke = [r for r in results if r.baseline == "Arke"]
    assert sorted(r.shape_tag for r in arke) == sorted(L1_CASES[op]), [(r.shape_tag, r.baseline) for r in results]
    for r in arke:
        row = {"driver": "bench_l1.run_op", "op": op, "shape": r.shape_tag, "status": r.status,
               "latency_us": r.latency_us, "correctness_status": r.correctness_status, "allclose": r.allclose,
               "max_abs_diff": r.max_abs_diff, "rtol": r.rtol, "atol": r.atol, "golden": r.golden_runner,
               "reason": r.correctness_reason or r.reason}
        _ROWS.append(row)
        assert r.status == "ok", row
        assert r.correctness_status == "ok" and r.allclose is True, row
        assert r.latency_us > 0 and r.latency_us != float("inf"), row


ARKE_RUN = [
    ("matmul", "512,768,1024", True),
    ("rmsnorm", "512,4096", True),
    ("quantize_per_token", "512,4096", True),
    ("silu_and_mul", "256,8192", True),
    ("flash_attention", "1,8,512,128", True),
    ("grouped_query_attention", "2,8,256,64", True),
]


@pytest.mark.parametrize("op,shape,ok", ARKE_RUN)
def test_arke_run_backend_b200(ref, op, shape, ok, capsys):
    """``arke run --kernel <op> --shape ... --backend b200 --json`` (arke/cli.py:217-243)."""
    from arke import cli
    args = cli._build_parser().parse_args(["run", "--kernel", op, "--shape", shape, "--backend", "b200", "--json"])
    rc = cli._cmd_run(args)
    out = json.loads(capsys.readouterr().out)
    _ROWS.append({"driver": "arke run --backend b200", "op": op, "shape": shape, "success": out["success"],
                  "mode": out["mode"], "message": out["message"]})
    assert (rc == 0) is ok and out["success"] is ok, out
    assert out["backend"] == "b200" and out["mode"] == "registry"
    for alias in ("sm_100a", "nvidia_blackwell"):
        from arke.backend.protocol import get_default_registry
        assert get_default_registry().get(alias).name == "b200"


def test_run_backend_reports_float_labels_as_a_run_error(ref):
    """The registry driver feeds ``torch.randn`` fp32 for every input, labels included
    (arke/agent/backends.py:272-276): that is a typed error here, never a silent cast."""
    from arke.agent.backends import run_backend
    res = run_backend("b200", op_name="fused_linear_cross_entropy",
                      shapes={"X": [64, 128], "W": [1000, 128], "labels": [64]})
    assert res.success is False and "run error" in res.message and "labels" in res.message


FACADE = [
    ("quantize_per_token", {"X": [128, 4096]}),
    ("quantize_per_token", {}),                                   # the tool's default [4, 8]
    ("silu_and_mul", {"X": [64, 2048]}),
    ("rmsnorm", {}),                                              # default X [4, 128], W [128]
    ("rmsnorm_residual", {"X": [64, 4096], "residual": [64, 4096], "W": [4096]}),
    ("matmul", {}),                                               # default A [64, 32], B [32, 128]
    ("matmul", {"A": [256, 512], "B": [512, 384]}),
    ("flash_attention", {"Q": [1, 4, 256, 64], "K": [1, 4, 256, 64], "V": [1, 4, 256, 64]}),
    ("grouped_query_attention", {"Q": [1, 8, 256, 128], "K": [1, 2, 256, 128], "V": [1, 2, 256, 128]}),
    ("fused_linear_cross_entropy", {}),                           # default X [8, 64], W [100, 64], labels [8]
    ("fused_linear_cross_entropy", {"X": [256, 512], "W": [8000, 512], "labels": [256]}),
]


@pytest.mark.parametrize("op,shapes", FACADE)
def test_facade_compile_and_profile_on_cuda(ref, op, shapes):
    """V1 (interpreter comparison) and V2 (kernel-only timing through prepare / run_fast /
    benchmark_cached) of the parent tool, with the B200 backend in the backend slot."""
    from arke_b200.facade import tool_classes
    tool = tool_classes()["compile_and_profile"]()
    res = tool.execute({"op_name": op, "shapes": shapes})
    data = res.data or {}
    _ROWS.append({"driver": "facade compile_and_profile", "op": op, "shapes": shapes, "success": res.success,
                  "error": getattr(res, "error", None), **{k: data.get(k) for k in (
                      "correct", "max_diff", "latency_ms", "baseline_ratio", "vs_default", "backend",
                      "num_real_kernels", "num_fallback")}, "warnings": list(getattr(res, "warnings", []) or [])})
    assert res.success, res.error
    assert data["backend"] == "b200" and data["num_real_kernels"] == 1 and data["num_fallback"] == 0
    assert data["correct"] is True, data
    assert not res.warnings, res.warnings                         # no "validation skipped" / "profiling skipped"
    assert data["latency_ms"] and data["latency_ms"] > 0 and data["vs_default"] == 1.0


def test_facade_strategy_reaches_the_kernel_and_noop_is_detected(ref):
    """With a bound environment the parent hands the decision log to ``lower(graph, strategy=…)``
    (tools.py:477-481) and compares the two kernels' ``cubin`` keys (:578-581)."""
    from arke.agent.env import ArkeEnv
    from arke.ir.strategy import Decision
    from arke_b200.facade import tool_classes
    shapes = {"A": [1024, 512], "B": [512, 1024]}
    env = ArkeEnv.from_op("matmul", shapes)
    tool = tool_classes()["compile_and_profile"](env)
    # L3 warp-grid decision (arke/ir/strategy.py:49-53): block rows = WM * WTM * 16 = 128 -> one-CTA tiles
    env.state.apply_decision(Decision(kind="wmma_tile", params={"WM": 2, "WN": 2, "WTM": 4, "WTN": 4}, level=3))
    res = tool.execute({"op_name": "matmul", "shapes": shapes})
    assert res.success, res.error
    assert res.data["correct"] is True and res.data["strategy_decisions"] == 1
    assert res.data["strategy_noop"] is False and res.data["default_latency_ms"] > 0
    assert res.data["compiles_used"] == 1
    _ROWS.append({"driver": "facade compile_and_profile (strategy)", "op": "matmul", "shapes": shapes,
                  **{k: res.data.get(k) for k in ("correct", "latency_ms", "default_latency_ms", "vs_default",
                                                   "strategy_noop", "meas_spread")}})


VERIFY = [
    ("quantize_per_token", {"X": [128, 1024]}),
    ("silu_and_mul", {"X": [64, 1024]}),
    ("rmsnorm", {"X": [64, 1024], "W": [1024]}),
    ("matmul", {"A": [128, 256], "B": [256, 128]}),
    ("grouped_query_attention", {"Q": [1, 8, 128, 64], "K": [1, 2, 128, 64], "V": [1, 2, 128, 64]}),
    ("fused_linear_cross_entropy", {"X": [64, 256], "W": [1000, 256], "labels": [64]}),
]


@pytest.mark.parametrize("op,shapes", VERIFY)
def test_facade_verify_correctness_on_cuda(ref, op, shapes):
    from arke.agent.env import ArkeEnv
    from arke_b200.facade import tool_classes
    env = ArkeEnv.from_op(op, shapes)
    tool = tool_classes()["verify_correctness"](env)
    res = tool.execute({})
    _ROWS.append({"driver": "facade verify_correctness", "op": op, "shapes": shapes, "success": res.success,
                  "error": getattr(res, "error", None), **(res.data or {})})
    assert res.success, res.error
    assert res.data["correct"] is True and res.data["validation_tier"] == "V1_b200" and res.data["backend"] == "b200"
    assert res.data["compiles_used"] == 1


def test_tool_registry_gets_the_b200_tools(ref):
    from arke.agent.env import ArkeEnv
    from arke.agent.tools import ToolRegistry
    from arke_b200.facade import install_tools
    env = ArkeEnv.from_op("silu_and_mul", {"X": [32, 512]})
    reg = ToolRegistry.with_env(env)
    assert install_tools(reg, env) == ["compile_and_profile", "verify_correctness"]
    res = reg.get("compile_and_profile").execute({"op_name": "silu_and_mul", "shapes": {"X": [32, 512]}})
    assert res.success and res.data["backend"] == "b200" and res.data["correct"] is True
    res = reg.get("verify_correctness").execute({})
    assert res.success and res.data["validation_tier"] == "V1_b200"


@pytest.mark.parametrize("op", ["quantize_per_token", "silu_and_mul", "grouped_query_attention"])
def test_staged_correctness_gate(ref, op):
    """The five-stage firewall (smoke, shape sweep, stability, determinism, edge) with the B200
    backend as the candidate and the interpreter as the reference."""
    from arke.agent.verification import GateStage, staged_correctness_gate
    from arke.backend.protocol import get_default_registry
    from arke.ir.graph import IRGraph
    from arke.ir.ops.interpreter import INTERPRETER
    be = get_default_registry().get("b200")

    def shapes_for(stage, i):
        if op == "grouped_query_attention":
            s = {GateStage.SMOKE: 128, GateStage.EDGE: 77}.get(stage, 64 + 48 * i)
            return {"Q": [1, 8, s, 64], "K": [1, 2, s, 64], "V": [1, 2, s, 64]}
        rows = {GateStage.SMOKE: 32, GateStage.EDGE: 1}.get(stage, 8 + 37 * i)
        cols = {GateStage.SMOKE: 1024, GateStage.EDGE: 1026}.get(stage, 256 + 128 * i)
        return {"X": [rows, cols]}

    def make_inputs(stage, i):
        g = torch.Generator().manual_seed(1000 * int(stage.value if hasattr(stage, "value") else stage) + i)
        scale = 30.0 if stage == GateStage.STABILITY else 1.0
        return {k: (torch.randn(v, generator=g) * scale).half().cuda() for k, v in shapes_for(stage, i).items()}

    kernels = {}

    def run_candidate(inputs):
        key = tuple((k, tuple(v.shape)) for k, v in inputs.items())
        if key not in kernels:
            graph = IRGraph.single_node(op, {k: list(v.shape) for k, v in inputs.items()}, dtype="float16",
                                        output_name="output")
            kernels[key] = be.compile(be.lower(graph))
            assert kernels[key].success, kernels[key].error
        return be.run(kernels[key], inputs)["output"]

    def run_reference(inputs):
        return INTERPRETER.execute(op, {k: v.float().cpu() for k, v in inputs.items()})

    def allclose(cand, refv):
        c = cand.float().cpu()
        if refv.is_floating_point():
            return bool(torch.allclose(c, refv.float(), rtol=1e-2, atol=1e-2)), float((c - refv.float()).abs().max())
        return bool(torch.equal(c.long(), refv.long())), float((c.long() - refv.long()).abs().max())

    report = staged_correctness_gate(
        run_candidate=run_candidate, run_reference=run_reference, make_inputs=make_inputs, allclose=allclose,
        is_finite=lambda t: bool(torch.isfinite(t.float()).all()), equal=lambda a, b: bool(torch.equal(a, b)),
        shape_sweep_count=6)
    _ROWS.append({"driver": "staged_correctness_gate", "op": op, "all_passed": report.all_passed,
                  "stages": [(s.stage.name, s.passed, s.max_diff) for s in report.stages]})
    assert report.all_passed, report.summary()
    assert len(report.stages) == 5


def test_bench_l2_fused_linear_ce_at_the_real_vocabulary(ref):
    """``_run_fused_linear_ce_op`` is the only reference driver that runs fused linear + CE at
    V = 128256 (the llama3 tag); it scores the row whose approach is "arke" against the
    interpreter at 1e-2 (benchmarks/bench_l2.py:921-1043, 413-419)."""
    shapes = [s for s in ref.l1._get_shapes("fused_linear_cross_entropy") if s.tag in ("llama3-seq512", "gpt2-seq128")]
    assert len(shapes) == 2
    results = ref.l2._run_fused_linear_ce_op("linear_ce", shapes, 2, 5)
    rows = {(r.shape_tag, r.approach): r for r in results}
    for tag, vocab in (("llama3-seq512", 128256), ("gpt2-seq128", 50257)):
        r = rows[(tag, "arke")]
        _ROWS.append({"driver": "bench_l2 linear_ce", "op": "fused_linear_cross_entropy", "shape": f"{tag} V={r.N}",
                      "status": r.status, "latency_us": r.latency_us, "correctness_status": r.correctness_status,
                      "allclose": r.allclose, "max_abs_diff": r.max_abs_diff,
                      "separate_us": rows[(tag, "separate")].latency_us,
                      "liger_us": rows[(tag, "liger")].latency_us if (tag, "liger") in rows else None})
        assert r.N == vocab and r.status == "ok", vars(r)
        assert r.correctness_status == "ok" and r.allclose is True, vars(r)
        assert "sm_100a" in r.source


def test_bench_l2_silu_and_mul_row(ref):
    shapes = [s for s in ref.l1._get_shapes("silu_and_mul") if s.tag in ("llama3-8b", "gpt2-sm")]
    results = ref.l2._run_gated_fused_op("silu_and_mul", shapes, 2, 5)
    rows = {(r.shape_tag, r.approach): r for r in results}
    for tag in ("llama3-8b", "gpt2-sm"):
        r = rows[(tag, "arke")]
        _ROWS.append({"driver": "bench_l2 silu_and_mul", "op": "silu_and_mul", "shape": tag, "status": r.status,
                      "latency_us": r.latency_us, "correctness_status": r.correctness_status, "allclose": r.allclose,
                      "max_abs_diff": r.max_abs_diff, "separate_us": rows[(tag, "separate")].latency_us,
                      "liger_us": rows[(tag, "liger")].latency_us if (tag, "liger") in rows else None})
        assert r.status == "ok" and r.correctness_status == "ok" and r.allclose is True, vars(r)


def test_zz_write_driver_report():
    """Not a check: stores the rows collected above where ``ARKE_B200_DRIVER_REPORT`` points."""
    path = os.environ.get("ARKE_B200_DRIVER_REPORT")
    if path and _ROWS:
        with open(path, "w") as fh:
            json.dump(_ROWS, fh, indent=1, default=str)
