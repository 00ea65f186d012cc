"""``B200Backend`` — the reference's backend seam implemented on the sm_100a kernel library.

Mirrors the ``ArkeBackend`` protocol (arke/backend/protocol.py:94-137): ``lower`` turns a
single-node ``IRGraph`` into a ``BackendArtifact`` describing the C-ABI call, ``compile`` resolves
the symbol in the ahead-of-time-built library (nothing is JIT-compiled), ``run`` feeds torch CUDA
tensors through :mod:`arke_b200.ops` on the caller's stream and returns a dict keyed by the graph
outputs.  Error conventions are the reference's: ``lower`` raises ``ValueError`` for an op it does
not serve (arke/backend/cuda_c_backend.py:482-486), ``compile`` returns ``CompiledKernel.fail``
instead of raising (:518-550), ``run`` raises ``RuntimeError`` on a failed kernel (:565-566).
There is no interpreter, eager or CPU fallback anywhere in this class.

The fine-grained benchmark API that the V2 hook duck-types (arke/agent/tools.py:549-553,646-650;
shape taken from arke/backend/llvm_backend.py:491-710) is provided as ``prepare / run_fast /
benchmark_cached / release / benchmark`` with CUDA-event, kernel-only timing.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional

try:  # the reference's own artifact types, when Arke is importable
    from arke.backend.protocol import BackendArtifact, BackendCapabilities, CompiledKernel  # type: ignore
except Exception:  # field-compatible mirrors (arke/backend/protocol.py:36-92)

    @dataclass
    class BackendArtifact:  # type: ignore[no-redef]
        source_code: str
        backend_name: str
        op_name: str = ""
        metadata: dict = field(default_factory=dict)

    @dataclass
    class CompiledKernel:  # type: ignore[no-redef]
        success: bool
        compiled_fn: Any = None
        binary_path: Optional[str] = None
        error: Optional[str] = None
        backend_name: str = ""
        metadata: dict = field(default_factory=dict)

        @classmethod
        def ok(cls, fn=None, backend_name: str = "", **meta):
            return cls(success=True, compiled_fn=fn, backend_name=backend_name, metadata=meta)

        @classmethod
        def fail(cls, error: str):
            return cls(success=False, error=error)

    @dataclass
    class BackendCapabilities:  # type: ignore[no-redef]
        backend_name: str
        hardware: Any
        supported_ops: frozenset = frozenset()
        tensor_core: bool = False
        async_copy: bool = False
        max_pipeline_stages: int = 1
        supported_dtypes: tuple = ("f16", "f32")

        def supports_op(self, op_name: str) -> bool:
            return op_name in self.supported_ops


from .hardware import nvidia_sm100_b200

# catalog op name -> (schema input names in order, C-ABI symbol, number of outputs)
OP_TABLE = {
    "quantize_per_token": (("X",), "arke_b200_quantize_per_token", 2),
    "silu_and_mul": (("X",), "arke_b200_silu_and_mul", 1),
    "rmsnorm": (("X", "W"), "arke_b200_rmsnorm", 1),
    "rmsnorm_residual": (("X", "residual", "W"), "arke_b200_rmsnorm", 1),
    "dequantize_per_channel": (("X_int8", "scale", "zero_point"), "arke_b200_dequantize_per_channel", 1),
    "matmul": (("A", "B"), "arke_b200_matmul", 1),
    "rope": (("X", "cos", "sin"), "arke_b200_rope", 1),
    "flash_attention": (("Q", "K", "V"), "arke_b200_gqa_fwd", 1),
    "grouped_query_attention": (("Q", "K", "V"), "arke_b200_gqa_fwd", 1),
    "cross_attention": (("Q", "K", "V"), "arke_b200_gqa_fwd", 1),
    "fused_linear_cross_entropy": (("X", "W", "labels"), "arke_b200_fused_linear_ce", 1),
}


# Ops whose kernels have a tile choice a strategy can reach.
_TILED_OPS = ("matmul", "fused_linear_cross_entropy")


def strategy_to_options(op: str, strategy) -> dict:
    """Map the agent loop's decisions to the library's tuning options.

    The reference's strategy-aware backends read a ``StrategyIR`` or a bare decision list
    (arke/backend/cuda_c_backend.py:489-498, arke/backend/llvm_backend.py:238-262).  The kinds that
    have a counterpart in the hand-written kernels:

      * L1 ``tile`` with ``BM`` (arke/backend/cuda_c_matmul_templates.py:41-50) and L3 ``wmma_tile``
        with ``WM``/``WTM`` (arke/ir/strategy.py:368-396; block rows = WM * WTM * 16): a block of
        256 rows or more selects the CTA-pair kernel (256 x 256 tiles, ``cta_group::2``), a smaller
        one the one-CTA kernel (128 x 256 tiles) -> ``gemm_tile_m``;
      * ``l2_band_mb`` in a ``tile`` decision's params -> ``gemm_band_mb``.

    Later decisions override earlier ones.  Everything else (``pipeline_stages``, ``block_threads``,
    ``unroll``, ``vectorize`` ...) is fixed at compile time in these kernels and is left out, which
    the artifact reports as ``strategy_noop`` when nothing applied.
    """
    if op not in _TILED_OPS or strategy is None:
        return {}
    decisions = getattr(strategy, "decisions", strategy)
    if not isinstance(decisions, (list, tuple)):
        return {}
    out: dict = {}
    for d in decisions:
        kind = getattr(d, "kind", None) if not isinstance(d, dict) else d.get("kind")
        params = (getattr(d, "params", None) if not isinstance(d, dict) else d.get("params")) or {}
        rows = None
        if kind == "tile" and "BM" in params:
            rows = int(params["BM"])
        elif kind == "wmma_tile" and "WM" in params:
            rows = int(params["WM"]) * int(params.get("WTM", 1)) * 16
        if rows is not None and rows > 0:
            out["gemm_tile_m"] = 256 if rows >= 256 else 128
        if kind == "tile" and "l2_band_mb" in params:
            out["gemm_band_mb"] = max(1, min(4096, int(params["l2_band_mb"])))
    return out


@dataclass
class OpPlan:
    """What ``lower`` decided for the graph's single node."""
    op: str
    symbol: str
    schema_inputs: tuple            # schema names in call order
    input_map: dict                 # schema name -> graph input value name
    outputs: list                   # node output value names
    graph_outputs: list
    attrs: dict = field(default_factory=dict)
    use_interpreter: bool = False   # always False: consumers check this key (arke_runner.py:254-314)
    options: dict = field(default_factory=dict)   # tuning options derived from a strategy


@dataclass
class _Prepared:
    """Handle returned by ``prepare``: the kernel closure plus the inputs of the last ``run_fast``."""
    fn: Callable[[dict], Any]
    plan: OpPlan
    inputs: Optional[dict] = None


class B200Backend:
    """Backend ``"b200"`` for the reference's ``BackendRegistry``."""

    name = "b200"

    def __init__(self, chip: str = "sm_100a"):
        self.chip = chip
        self.hardware = nvidia_sm100_b200()

    # ---------------------------------------------------------------- protocol
    def supports_op(self, op_name: str) -> bool:
        return op_name in OP_TABLE

    def capabilities(self, hw=None) -> BackendCapabilities:
        return BackendCapabilities(
            backend_name=self.name, hardware=hw or self.hardware, supported_ops=frozenset(OP_TABLE),
            tensor_core=True, async_copy=True, max_pipeline_stages=6,
            supported_dtypes=("f16", "bf16", "f32", "i8", "e4m3"))

    def lower(self, graph, hw=None, strategy=None) -> BackendArtifact:
        nodes = list(getattr(graph, "nodes", []))
        if len(nodes) != 1:
            raise ValueError(f"B200Backend lowers single-node graphs only (got {len(nodes)} nodes)")
        node = nodes[0]
        if node.op not in OP_TABLE:
            raise ValueError(f"B200Backend does not support op {node.op!r}; supported: {sorted(OP_TABLE)}")
        schema_inputs, symbol, _ = OP_TABLE[node.op]
        input_map = dict(node.inputs)
        missing = [s for s in schema_inputs if s not in input_map]
        if missing:
            # tolerate callers that key node.inputs positionally by their own names
            names = list(node.inputs.values())
            if len(names) == len(schema_inputs):
                input_map = dict(zip(schema_inputs, names))
            else:
                raise ValueError(f"{node.op}: graph node lacks inputs {missing}")
        plan = OpPlan(op=node.op, symbol=symbol, schema_inputs=schema_inputs, input_map=input_map,
                      outputs=list(node.outputs), graph_outputs=list(getattr(graph, "graph_outputs", []) or node.outputs),
                      attrs=dict(getattr(node, "attrs", {}) or {}))
        src = (f"// arke_b200: {node.op} -> extern \"C\" {symbol}(...) in libarke_b200.so (sm_100a, AOT)\n"
               f"// inputs: {input_map}  attrs: {plan.attrs}\n")
        meta = {"num_real_kernels": 1, "num_fallback": 0, "plan": plan,
                "plans": [{"use_interpreter": False, "node": node, "input_order": list(schema_inputs),
                           "wrapper": None}],
                "chip": self.chip}
        if strategy is not None:
            plan.options = strategy_to_options(node.op, strategy)
            meta["strategy_options"] = dict(plan.options)
            meta["strategy_noop"] = not plan.options
        return BackendArtifact(source_code=src, backend_name=self.name, op_name=node.op, metadata=meta)

    def compile(self, artifact: BackendArtifact) -> CompiledKernel:
        try:
            plan: OpPlan = artifact.metadata["plan"]
            from . import _lib
            getattr(_lib.LIB, plan.symbol)  # AttributeError if the library lacks the entry point
            fn = _make_runner(plan)
            if plan.options:
                from . import ops as _ops
                inner, opts = fn, dict(plan.options)

                def fn(inputs, _inner=inner, _opts=opts):   # noqa: F811 - the tuned variant of the closure
                    with _ops.options(**_opts):
                        return _inner(inputs)
        except Exception as exc:  # the reference's compile() never raises
            return CompiledKernel.fail(f"arke_b200 compile failed: {exc}")
        # "cubin" is what the façade compares to tell whether a strategy changed the kernel
        # (arke/agent/tools.py:578-581): the entry point plus the options that select its variant
        variant = "".join(f";{k}={v}" for k, v in sorted(plan.options.items()))
        k = CompiledKernel.ok(fn, backend_name=self.name, num_real_kernels=1, num_fallback=0,
                              plan=plan, cubin=f"{plan.symbol}@{_lib.version()}{variant}")
        k.binary_path = str(_lib.lib_path())
        return k

    def run(self, kernel: CompiledKernel, inputs: dict) -> dict:
        if not getattr(kernel, "success", False) or kernel.compiled_fn is None:
            raise RuntimeError(f"Cannot run failed kernel: {getattr(kernel, 'error', None)}")
        plan: OpPlan = kernel.metadata["plan"]
        try:
            result = kernel.compiled_fn(inputs)
        except (ValueError, TypeError, KeyError) as exc:
            raise RuntimeError(f"arke_b200 {plan.op}: {exc}") from exc
        return _bind_outputs(plan, result)

    # --------------------------------------------- fine-grained benchmark API (V2 hook)
    def prepare(self, compiled: CompiledKernel) -> _Prepared:
        if not getattr(compiled, "success", False):
            raise RuntimeError(f"Cannot prepare failed kernel: {compiled.error}")
        return _Prepared(fn=compiled.compiled_fn, plan=compiled.metadata["plan"])

    def run_fast(self, handle: _Prepared, inputs: dict) -> dict:
        handle.inputs = inputs
        return _bind_outputs(handle.plan, handle.fn(inputs))

    def benchmark_cached(self, handle: _Prepared, iters: int = 100, warmup: int = 30) -> float:
        """Mean kernel-only latency in ms (CUDA events) on the inputs of the last ``run_fast``."""
        if handle.inputs is None:
            raise RuntimeError("benchmark_cached: call run_fast(handle, inputs) first")
        return _event_time(lambda: handle.fn(handle.inputs), iters, warmup)

    def benchmark(self, compiled: CompiledKernel, inputs: dict, iters: int = 100, warmup: int = 30) -> float:
        if not getattr(compiled, "success", False):
            raise RuntimeError(f"Cannot benchmark failed kernel: {compiled.error}")
        return _event_time(lambda: compiled.compiled_fn(inputs), iters, warmup)

    def release(self, handle: _Prepared) -> None:
        handle.inputs = None


# -------------------------------------------------------------------------------------------
def _event_time(fn: Callable[[], Any], iters: int, warmup: int) -> float:
    import torch
    for _ in range(max(0, warmup)):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(max(1, iters)):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / max(1, iters)


def _bind_outputs(plan: OpPlan, result) -> dict:
    """Tuple results bind to successive node outputs; a single-output graph gets element 0 under
    its output name (``"output"`` for graphs from ``IRGraph.single_node``)."""
    names = plan.graph_outputs or plan.outputs or ["output"]
    if isinstance(result, tuple):
        if len(names) >= len(result):
            return {n: r for n, r in zip(names, result)}
        out = {names[0]: result[0]}
        for i, r in enumerate(result[1:], start=1):
            out[plan.outputs[i] if i < len(plan.outputs) else f"{names[0]}_{i}"] = r
        return out
    return {names[0]: result}


def _as_tensor(v, what: str):
    import torch
    if isinstance(v, torch.Tensor):
        return v
    try:
        import numpy as np
        if isinstance(v, np.ndarray):
            raise TypeError(f"{what}: numpy input given; arke_b200 takes CUDA torch tensors (no host round trip)")
    except ImportError:
        pass
    raise TypeError(f"{what}: expected a torch.Tensor, got {type(v).__name__}")


def _make_runner(plan: OpPlan) -> Callable[[dict], Any]:
    """Closure that pulls the op's tensors out of the inputs dict (keyed by graph value names or by
    schema names) and calls the kernel.  Runtime tensors are trusted, not graph metadata: graphs
    from ``IRGraph.single_node`` stamp one dtype on every input and leave output shapes empty."""
    from . import ops

    def fetch(inputs: dict, schema_name: str):
        key = plan.input_map.get(schema_name, schema_name)
        if key in inputs:
            return _as_tensor(inputs[key], f"{plan.op}.{schema_name}")
        if schema_name in inputs:
            return _as_tensor(inputs[schema_name], f"{plan.op}.{schema_name}")
        raise KeyError(f"missing input {key!r} (schema name {schema_name!r})")

    attrs = plan.attrs
    op = plan.op

    if op == "quantize_per_token":
        def run(inputs):
            x = fetch(inputs, "X")
            q, scale = ops.quantize_per_token(x, out_dtype=attrs.get("quant_dtype", "int8"),
                                              formula=attrs.get("formula", "interp"))
            return (q, scale) if len(plan.outputs) > 1 or attrs.get("return_scale") else q
        return run
    if op == "silu_and_mul":
        def run(inputs):
            x = fetch(inputs, "X")
            if attrs.get("quant_dtype") == "fp8" or attrs.get("out_dtype") == "fp8":
                return ops.swiglu_fp8(x)
            return ops.silu_and_mul(x)
        return run
    if op in ("rmsnorm", "rmsnorm_residual"):
        def run(inputs):
            x, w = fetch(inputs, "X"), fetch(inputs, "W")
            res = fetch(inputs, "residual") if op == "rmsnorm_residual" else None
            quant = attrs.get("quant_dtype")
            return ops.rmsnorm(x, w.to(x.dtype), eps=float(attrs.get("eps", 1e-6)), residual=res, quantize=quant)
        return run
    if op == "dequantize_per_channel":
        def run(inputs):
            import torch
            x, sc = fetch(inputs, "X_int8"), fetch(inputs, "scale")
            try:
                zp = fetch(inputs, "zero_point")
            except KeyError:
                zp = None
            if x.dtype != torch.int8:          # drivers that stamp one float dtype on every input
                x = x.round().clamp(-128, 127).to(torch.int8)
            return ops.dequantize_per_channel(x, sc, zp)
        return run
    if op == "rope":
        def run(inputs):
            x, cos, sin = fetch(inputs, "X"), fetch(inputs, "cos"), fetch(inputs, "sin")
            S, half = x.shape[-2], x.shape[-1] // 2
            # drivers that give every input the default [4, 8] shape cannot mean a rotary table
            if tuple(cos.shape) != (S, half) or tuple(sin.shape) != (S, half):
                raise ValueError(f"rope: cos and sin must be [S, D/2] = [{S}, {half}], got {tuple(cos.shape)} and {tuple(sin.shape)}")
            return ops.rope(x, cos.to(x.dtype), sin.to(x.dtype))
        return run
    if op == "matmul":
        def run(inputs):
            import torch
            a, b = fetch(inputs, "A"), fetch(inputs, "B")
            if a.dtype in (torch.int8, ops.FP8):
                return ops.quant_gemm(a, None, b, None, out_dtype=None, return_acc=True)
            return ops.matmul(a, b)
        return run
    # The registry driver behind `arke run` feeds fp32 tensors for every input
    # (arke/agent/backends.py:272-276).  The tensor-core kernels of these two ops take 16-bit
    # operands, so fp32 inputs are rounded to bf16 here and the result is returned as fp32; this
    # stays inside the reference's 1e-2 comparison rule.
    import torch

    def to16(t):
        return t.to(torch.bfloat16) if t.dtype == torch.float32 else t

    if op in ("flash_attention", "grouped_query_attention", "cross_attention"):
        def run(inputs):
            q, k, v = fetch(inputs, "Q"), fetch(inputs, "K"), fetch(inputs, "V")
            was32 = q.dtype == torch.float32
            q, k, v = to16(q), to16(k), to16(v)
            # cross_attention is never causal (arke/ir/ops/reference_impls.py:256-257)
            causal = op != "cross_attention" and bool(attrs.get("is_causal", attrs.get("causal", False)))
            if attrs.get("return_lse"):
                o, lse = ops.gqa_fwd(q, k, v, causal=causal, softmax_scale=attrs.get("scale"))
                return (o.float() if was32 else o), lse
            o = ops.gqa_fwd(q, k, v, causal=causal, softmax_scale=attrs.get("scale"), return_lse=False)
            return o.float() if was32 else o
        return run
    if op == "fused_linear_cross_entropy":
        def run(inputs):
            x, w, labels = fetch(inputs, "X"), fetch(inputs, "W"), fetch(inputs, "labels")
            if labels.dtype in (torch.int32, torch.int16, torch.uint8, torch.int8):
                labels = labels.long()
            tok, mean = ops.fused_linear_ce(to16(x), to16(w), labels, ignore_index=int(attrs.get("ignore_index", -100)))
            return tok if attrs.get("reduction") == "none" else mean
        return run
    raise ValueError(f"no runner for op {op!r}")
