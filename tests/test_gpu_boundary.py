"""GPU: the reference-facing plugin layer (backend seam, benchmark runner, torch bridge) drives the
CUDA kernels and applies the reference's own V1 comparison rule: float outputs
``allclose(rtol=atol=1e-2)``, integer outputs ``torch.equal`` (arke/agent/tools.py:510-517)."""
from dataclasses import dataclass, field

import pytest
import torch

import oracle as oracle_pkg
from oracle import ops as oracle

pytestmark = pytest.mark.gpu


@dataclass
class Node:
    id: str
    op: str
    inputs: dict
    outputs: list
    attrs: dict = field(default_factory=dict)


@dataclass
class Graph:
    nodes: list
    graph_inputs: list
    graph_outputs: list


def graph(op, inputs, attrs=None, outputs=("output",)):
    return Graph([Node("output", op, dict(inputs), list(outputs), dict(attrs or {}))], list(inputs.values()), list(outputs))


_VERBOSE_DTYPE = {torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32"}


def real_graph(op, tensors, attrs=None):
    """The graph the reference's own entry points hand to ``lower()``: ``IRGraph.single_node``
    (arke/ir/graph.py:447-534), available when the reference package is staged beside the oracle."""
    if oracle_pkg.ref_path() is None:
        return None
    from arke.ir.graph import IRGraph
    first = next(iter(tensors.values()))
    g = IRGraph.single_node(op, {k: list(t.shape) for k, t in tensors.items()},
                            dtype=_VERBOSE_DTYPE.get(first.dtype, "float32"), output_name="output")
    if attrs:
        g.nodes[0].attrs.update(attrs)
    return g


def run(op, tensors, attrs=None, outputs=("output",)):
    from arke_b200.backend import B200Backend
    be = B200Backend()
    g = real_graph(op, tensors, attrs) if tuple(outputs) == ("output",) else None
    if g is not None:
        names = {k: g.nodes[0].inputs[k] for k in tensors}       # schema name -> graph value name
    else:
        names = {k: f"v_{k}" for k in tensors}
        g = graph(op, names, attrs, outputs)
    k = be.compile(be.lower(g))
    assert k.success, k.error
    return be, k, be.run(k, {names[n]: t.cuda() for n, t in tensors.items()})


def test_the_graphs_in_this_file_are_the_reference_ones_when_it_is_staged():
    g = real_graph("quantize_per_token", {"X": torch.zeros(4, 8)})
    if g is None:
        pytest.skip("reference package not staged")
    from arke.ir.graph import IRGraph
    assert isinstance(g, IRGraph) and len(g.nodes) == 1 and g.graph_outputs == ["output"]


def test_v1_rule_quantize_fp16_is_bit_exact_like_the_hook():
    torch.manual_seed(42)
    x = torch.randn(128, 4096).half()
    _, _, out = run("quantize_per_token", {"X": x})
    ref = oracle.quantize_per_token_interp(x)[0]          # interpreter on X.float().cpu()
    assert torch.equal(out["output"].cpu().long(), ref.long())
    _, _, out2 = run("quantize_per_token", {"X": x}, outputs=("q", "scale"))
    assert set(out2) == {"q", "scale"} and torch.equal(out2["q"].cpu(), ref)


def test_v1_rule_float_ops():
    torch.manual_seed(42)
    x = torch.randn(64, 2048).half()
    _, _, out = run("silu_and_mul", {"X": x})
    assert torch.allclose(out["output"].cpu().float(), oracle.silu_and_mul(x.float()), rtol=1e-2, atol=1e-2)
    q, k, v = oracle.make_attention_inputs(1, 8, 2, 256, 128, seed=1, dtype=torch.float16)
    # V1 passes no attrs to the interpreter: the default must be non-causal
    _, _, out = run("grouped_query_attention", {"Q": q, "K": k, "V": v})
    assert torch.allclose(out["output"].cpu().float(), oracle.gqa_attention(q.float(), k.float(), v.float(), False), rtol=1e-2, atol=1e-2)
    for key in ("is_causal", "causal"):
        _, _, out = run("grouped_query_attention", {"Q": q, "K": k, "V": v}, {key: True})
        assert torch.allclose(out["output"].cpu().float(), oracle.gqa_attention(q.float(), k.float(), v.float(), True), rtol=1e-2, atol=1e-2)
    _, _, out = run("flash_attention", {"Q": q, "K": q, "V": q}, {"is_causal": True})
    assert torch.allclose(out["output"].cpu().float(), oracle.gqa_attention(q.float(), q.float(), q.float(), True), rtol=1e-2, atol=1e-2)
    xh, wh, lab = oracle.make_flce_inputs(128, 256, 5000, seed=2, dtype=torch.float16)
    _, _, out = run("fused_linear_cross_entropy", {"X": xh, "W": wh, "labels": lab})
    assert out["output"].dim() == 0
    assert abs(out["output"].item() - oracle.fused_linear_ce(xh, wh, lab)[1].item()) <= 1e-2
    a, b = torch.randn(128, 256).half(), torch.randn(256, 192).half()
    _, _, out = run("matmul", {"A": a, "B": b})
    assert torch.allclose(out["output"].cpu().float(), a.float() @ b.float(), rtol=1e-2, atol=1e-1)


def test_typed_rejections_are_runtime_errors_not_fallbacks():
    from arke_b200.backend import B200Backend
    be = B200Backend()
    k = be.compile(be.lower(graph("matmul", {"A": "a", "B": "b"})))
    a32, b32 = torch.randn(64, 64, device="cuda"), torch.randn(64, 64, device="cuda")
    out = be.run(k, {"a": a32, "b": b32})   # `arke run` feeds fp32 randn for every input: TF32 path
    assert torch.allclose(out["output"], a32 @ b32, rtol=1e-2, atol=5e-2)
    with pytest.raises(RuntimeError):       # mixed dtypes are rejected
        be.run(k, {"a": a32, "b": b32.half()})
    k = be.compile(be.lower(graph("fused_linear_cross_entropy", {"X": "x", "W": "w", "labels": "l"})))
    with pytest.raises(RuntimeError):       # float labels, as the registry driver would pass
        be.run(k, {"x": torch.randn(8, 64, device="cuda").half(), "w": torch.randn(32, 64, device="cuda").half(),
                   "l": torch.randn(8, device="cuda")})


def test_fine_grained_benchmark_api():
    x = torch.randn(256, 4096).half()
    be, k, _ = run("quantize_per_token", {"X": x})
    h = be.prepare(k)
    key = next(iter(k.metadata["plan"].input_map.values()))
    out = be.run_fast(h, {key: x.cuda()})
    assert out["output"].dtype == torch.int8
    ms = be.benchmark_cached(h, iters=20, warmup=5)
    assert 0 < ms < 5
    assert 0 < be.benchmark(k, {key: x.cuda()}, iters=10, warmup=2) < 5
    be.release(h)
    with pytest.raises(RuntimeError):
        be.benchmark_cached(h)


def test_runner_mirrors_bench_l1_goldens():
    from arke_b200.runner import B200ArkeRunner
    r = B200ArkeRunner()
    assert r.available
    x = torch.randn(64, 4096, device="cuda").half()
    q, scales = r.run_with_inputs("quantize_per_token", x)
    qo, so = oracle.quantize_per_token_bench_l1(x.cpu())
    assert torch.equal(q.cpu(), qo) and torch.equal(scales.cpu(), so)      # 2-tuple (q, amax) like the golden
    q3 = torch.randn(8, 256, 128, device="cuda").half()                     # 3-D [B*H, S, D] as the driver passes
    k3 = torch.randn(2, 256, 128, device="cuda").half()
    o = r.run_with_inputs("grouped_query_attention", q3, k3, k3)
    ref = torch.nn.functional.scaled_dot_product_attention(q3, k3.repeat_interleave(4, 0), k3.repeat_interleave(4, 0), is_causal=True)
    assert isinstance(o, torch.Tensor) and torch.allclose(o.float(), ref.float(), rtol=1e-3, atol=1e-3)
    for op, (M, N, K) in {"quantize_per_token": (512, 4096, 0), "silu_and_mul": (128, 28672, 0), "matmul": (256, 512, 128),
                          "flash_attention": (8, 512, 128), "grouped_query_attention": (32, 256, 128),
                          "fused_linear_cross_entropy": (256, 4096, 128)}.items():
        fn = r.get_fn(op, M, N, K)
        assert fn is not None, (op, r.last_unsupported_reason)
        assert isinstance(fn(), torch.Tensor)
    assert r.get_fn("layernorm", 8, 8) is None


def test_torch_bridge_ops_and_fake_kernels():
    from arke_b200.bridge import register_ops
    assert register_ops() and register_ops()
    x = oracle.make_quant_input(64, 512, seed=3).cuda()
    q, s = torch.ops.arke.quantize_per_token(x)
    qo, so = oracle.quantize_per_token_interp(x.cpu())
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    w, sw = oracle.make_w8a8_weights(512, 256, seed=4)
    y = torch.ops.arke.w8a8_gemm(q, s, w.cuda(), sw.cuda())
    assert torch.equal(y.cpu(), oracle.w8a8_gemm(qo, so, w, sw)[0])
    with torch._subclasses.fake_tensor.FakeTensorMode():
        xf = torch.empty(64, 512, dtype=torch.bfloat16, device="cuda")
        qf, sf = torch.ops.arke.quantize_per_token(xf)
        assert qf.shape == (64, 512) and qf.dtype == torch.int8 and sf.shape == (64,)


def test_host_pipeline_matches_device_path():
    from arke_b200 import ops
    from arke_b200.host import HostW8A8Linear
    M, K, N = 1000, 512, 768
    x = oracle.make_quant_input(M, K, seed=8)
    w, sw = oracle.make_w8a8_weights(K, N, seed=9)
    lin = HostW8A8Linear(w.cuda(), sw.cuda(), max_rows=M, chunks=3)
    xh, yh = x.pin_memory(), torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    for _ in range(3):                      # repeated steps reuse the staging buffers
        yh.zero_()
        lin(xh, yh).synchronize()
        q, s = oracle.quantize_per_token_interp(x)
        assert torch.equal(yh, oracle.w8a8_gemm(q, s, w, sw)[0])


def test_backend_serves_rmsnorm_ops():
    torch.manual_seed(42)
    x, res = torch.randn(64, 4096).half(), torch.randn(64, 4096).half()
    w = torch.ones(4096).half()
    _, _, out = run("rmsnorm", {"X": x, "W": w})
    assert torch.allclose(out["output"].cpu().float(), oracle.rmsnorm(x.float(), w.float()), rtol=1e-2, atol=1e-2)
    _, _, out = run("rmsnorm_residual", {"X": x, "residual": res, "W": w})
    assert torch.allclose(out["output"].cpu().float(), oracle.rmsnorm(x.float(), w.float(), residual=res.float()), rtol=1e-2, atol=1e-2)


def test_registry_driver_sequence_with_fp32_inputs():
    # what `arke run --backend b200` does (arke/agent/backends.py:226-288): single-node graph, fp32
    # randn for every input, lower -> compile -> run; success means "no exception"
    torch.manual_seed(0)
    cases_ = {
        "quantize_per_token": {"X": [64, 512]},
        "silu_and_mul": {"X": [64, 1024]},
        "rmsnorm": {"X": [64, 512], "W": [512]},
        "matmul": {"A": [128, 64], "B": [64, 96]},
        "flash_attention": {"Q": [1, 4, 256, 128], "K": [1, 4, 256, 128], "V": [1, 4, 256, 128]},
        "grouped_query_attention": {"Q": [1, 8, 128, 128], "K": [1, 2, 128, 128], "V": [1, 2, 128, 128]},
    }
    for op, shapes in cases_.items():
        tensors = {k: torch.randn(*shp) for k, shp in shapes.items()}
        _, _, out = run(op, tensors)
        assert isinstance(out, dict) and len(out) >= 1
        assert all(torch.isfinite(v.float()).all() for v in out.values()), op
    o = run("flash_attention", {k: torch.randn(1, 4, 256, 128) for k in ("Q", "K", "V")})[2]["output"]
    assert o.dtype == torch.float32


def test_rope_through_backend_runner_and_bridge():
    # backend: the façade's V1 rule compares with the interpreter on .float().cpu() at 1e-2
    torch.manual_seed(42)
    x = torch.randn(1, 2, 16, 32).half()
    cos = torch.empty(16, 16).uniform_(-1, 1).half()
    sin = torch.empty(16, 16).uniform_(-1, 1).half()
    _, _, out = run("rope", {"X": x, "cos": cos, "sin": sin})
    assert torch.allclose(out["output"].cpu().float(), oracle.rope(x.float(), cos.float(), sin.float()), rtol=1e-2, atol=1e-2)
    assert torch.equal(out["output"].cpu(), oracle.rope(x, cos, sin))        # and bit-exact in fp16
    # runner: X only, 3-D, tables synthesised like the benchmark driver's golden (fp32 angles)
    from arke_b200.runner import B200ArkeRunner
    r = B200ArkeRunner()
    x3 = torch.randn(6, 300, 128, device="cuda").half()
    y = r.run_with_inputs("rope", x3)
    # (the golden evaluates the trigonometric functions on the tensor's device: benchmarks/bench_l1.py:480-486)
    inv = 1.0 / (10000 ** (torch.arange(0, 128, 2, dtype=torch.float32, device="cuda") / 128))
    fr = torch.einsum("i,j->ij", torch.arange(300, dtype=torch.float32, device="cuda"), inv)
    emb = torch.cat([fr, fr], -1)
    xc = x3.cpu()
    rot = torch.cat([-xc[..., 64:], xc[..., :64]], -1)
    gold = xc * torch.cos(emb).unsqueeze(0).half().cpu() + rot * torch.sin(emb).unsqueeze(0).half().cpu()
    assert torch.allclose(y.cpu().float(), gold.float(), rtol=1e-3, atol=1e-3)  # the driver's fp16 tolerance
    assert torch.equal(y.cpu(), gold)
    assert r.run_with_inputs("rope", torch.randn(2, 8, 65, device="cuda").half()) is None and "even" in r.last_unsupported_reason
    fn = r.get_fn("rope", 64, 256, 128)
    assert fn is not None and fn().shape[-1] == 128
    # bridge
    from arke_b200.bridge import register_ops
    register_ops()
    c4, s4 = oracle.make_rope_tables(16, 32, dtype=torch.float16)
    assert torch.equal(torch.ops.arke.rope(x.cuda(), c4.cuda(), s4.cuda()).cpu(), oracle.rope(x, c4, s4))
    with torch._subclasses.fake_tensor.FakeTensorMode():
        qf, kf, vf = torch.ops.arke.qkv_rope_split(torch.empty(32, 256, dtype=torch.bfloat16, device="cuda"),
                                                   torch.empty(16, 16, dtype=torch.bfloat16, device="cuda"),
                                                   torch.empty(16, 16, dtype=torch.bfloat16, device="cuda"), 2, 16, 4, 2, 32)
        assert qf.shape == (2, 4, 16, 32) and kf.shape == vf.shape == (2, 2, 16, 32)


def test_strategy_reaches_the_kernel_choice_and_keeps_results():
    from dataclasses import dataclass, field as dfield
    from arke_b200.backend import B200Backend

    @dataclass
    class Decision:
        kind: str
        params: dict = dfield(default_factory=dict)
        level: int = 1

    be = B200Backend()
    g = graph("matmul", {"A": "a", "B": "b"})
    a = torch.randn(512, 256, device="cuda").half()
    b = torch.randn(256, 384, device="cuda").half()
    outs = {}
    for name, strat in {"default": None, "pair": [Decision("tile", {"BM": 256})], "one_cta": [Decision("wmma_tile", {"WM": 2, "WTM": 4}, 3)]}.items():
        k = be.compile(be.lower(g, strategy=strat) if strat is not None else be.lower(g))
        assert k.success
        outs[name] = be.run(k, {"a": a, "b": b})["output"]
        h = be.prepare(k)
        be.run_fast(h, {"a": a, "b": b})
        assert be.benchmark_cached(h, iters=5, warmup=2) > 0
    assert torch.equal(outs["default"], outs["pair"]) and torch.equal(outs["default"], outs["one_cta"])
    from arke_b200 import _lib
    assert _lib.LIB.arke_b200_get_option(b"gemm_tile_m") == 0      # options do not leak out of run()


def test_cross_attention_backend_and_runner():
    """`cross_attention` (arke/ir/ops/reference_impls.py:256-257): never causal, key length differs
    from the query length; the benchmark driver passes 3-D [B*H, S, D] tensors."""
    torch.manual_seed(42)
    q = torch.randn(1, 4, 96, 128).half()
    k = torch.randn(1, 4, 333, 128).half()
    v = torch.randn(1, 4, 333, 128).half()
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=False)
    _, _, out = run("cross_attention", {"Q": q, "K": k, "V": v}, {"is_causal": True})   # the attr must not make it causal
    assert torch.allclose(out["output"].cpu().float(), ref, rtol=1e-2, atol=1e-2)
    from arke_b200.runner import B200ArkeRunner
    r = B200ArkeRunner()
    o = r.run_with_inputs("cross_attention", q[0].cuda(), k[0].cuda(), v[0].cuda())
    assert o.shape == (4, 96, 128) and torch.allclose(o.cpu().float(), ref[0], rtol=1e-3, atol=1e-3)
    fn = r.get_fn("cross_attention", 8, 256, 128)
    assert fn is not None and fn().shape == (8, 256, 128)
