"""Façade tools of the agent loop, bound to the B200 backend.

The reference's ``compile_and_profile`` and ``verify_correctness`` tools construct their backend
inside ``execute`` / ``_validate_real`` from a fixed list (arke/agent/tools.py:346-382 picks
``CudaCBackend`` / ``LLVMBackend`` / ``TritonBackend`` / ``MockBackend``; :1054,1097 always builds
``TritonBackend``).  The two subclasses here keep every other line of those methods — input
generation, the interpreter comparison (V1: ``allclose(1e-2, 1e-2)`` for floating results,
``torch.equal`` for integer ones, tools.py:505-517), the kernel-only timing discipline (V2,
tools.py:549-690), budget accounting — and replace only the backend construction:

  * ``B200CompileAndProfileTool`` runs the parent with ``backend="llvm"`` while the name
    ``LLVMBackend`` of ``arke.backend.llvm_backend`` is bound to a factory of ``B200Backend``.
    That slot is the one the parent hands the accumulated decisions to
    (``lower(graph, strategy=…)``, tools.py:477-481) and the one it times through
    ``prepare`` / ``run_fast`` / ``benchmark_cached`` (tools.py:549-553), both of which
    ``B200Backend`` implements.  The result's ``backend`` is reported as ``"b200"``.
  * ``B200VerifyCorrectnessTool`` runs the parent's ``_validate_real`` while ``TritonBackend`` of
    ``arke.backend.triton_backend`` is bound to the same factory, and reports
    ``validation_tier="V1_b200"``.

Both keep the tool names ``"compile_and_profile"`` / ``"verify_correctness"``, so
``ToolRegistry.register`` (tools.py:1361-1362) replaces the stock tools in place.  The classes
are created on demand because the reference package is not a dependency of this one.
"""
from __future__ import annotations

import contextlib
import importlib
import threading
from typing import Any

_swap_lock = threading.RLock()


@contextlib.contextmanager
def _bound(module_name: str, attr: str, value: Any):
    """Temporarily bind ``module.attr`` to ``value`` (serialised: the tools are not concurrent-safe,
    tools.py:314-318, 1031-1035)."""
    mod = importlib.import_module(module_name)
    with _swap_lock:
        had = hasattr(mod, attr)
        old = getattr(mod, attr, None)
        setattr(mod, attr, value)
        try:
            yield
        finally:
            if had:
                setattr(mod, attr, old)
            else:
                delattr(mod, attr)


def _b200_factory(*_args: Any, **_kwargs: Any):
    """Stands in for ``LLVMBackend(chip=…)`` / ``TritonBackend(device=…)``."""
    from .backend import B200Backend
    return B200Backend()


def _relabel(result: Any, **fields: Any) -> Any:
    data = getattr(result, "data", None)
    if isinstance(data, dict):
        for k, v in fields.items():
            if k in data:
                data[k] = v
    return result


_tool_classes: dict[str, type] = {}


def tool_classes() -> dict[str, type]:
    """``{"compile_and_profile": B200CompileAndProfileTool, "verify_correctness":
    B200VerifyCorrectnessTool}`` — built on first use from the installed reference's base classes."""
    if _tool_classes:
        return _tool_classes
    from arke.agent.tools import CompileAndProfileTool, VerifyCorrectnessTool  # type: ignore

    class B200CompileAndProfileTool(CompileAndProfileTool):  # type: ignore[misc, valid-type]
        """``compile_and_profile`` on the B200 backend (same parameters and result keys)."""

        @property
        def description(self) -> str:
            return ("Compile an operator from IR graph through the pass pipeline and the B200 "
                    "(sm_100a) backend, validate it against the reference implementation and time it")

        def execute(self, params: dict[str, Any]):
            import torch
            if not torch.cuda.is_available() or params.get("force_mock") is True:
                return super().execute(params)         # the parent's mock tier, unchanged
            routed = dict(params)
            routed["backend"] = "llvm"                 # the strategy-aware, fine-grained-timing slot
            with _bound("arke.backend.llvm_backend", "LLVMBackend", _b200_factory):
                result = super().execute(routed)
            err = getattr(result, "error", None)
            if isinstance(err, str) and "Backend llvm" in err:
                result.error = err.replace("Backend llvm", "Backend b200")
            return _relabel(result, backend="b200")

    class B200VerifyCorrectnessTool(VerifyCorrectnessTool):  # type: ignore[misc, valid-type]
        """``verify_correctness`` on the B200 backend (same parameters and result keys)."""

        def _validate_real(self, seed: int, rtol: float, atol: float):
            with _bound("arke.backend.triton_backend", "TritonBackend", _b200_factory):
                return super()._validate_real(seed, rtol, atol)

        def execute(self, params: dict[str, Any]):
            result = super().execute(params)
            data = getattr(result, "data", None)
            if isinstance(data, dict) and data.get("validation_tier") == "V1_triton":
                data["validation_tier"] = "V1_b200"
                data["backend"] = "b200"
            return result

    _tool_classes["compile_and_profile"] = B200CompileAndProfileTool
    _tool_classes["verify_correctness"] = B200VerifyCorrectnessTool
    return _tool_classes


def install_tools(registry: Any, env: Any = None) -> list[str]:
    """Replace the stock tools of a ``ToolRegistry`` by their B200 versions.  ``env`` is the bound
    ``ArkeEnv``; without one only ``compile_and_profile`` is replaced (``verify_correctness`` needs
    an environment, tools.py:795-803)."""
    classes = tool_classes()
    replaced = []
    if env is None:
        old = registry.get("compile_and_profile") if "compile_and_profile" in registry else None
        env = getattr(old, "_env", None)
    registry.register(classes["compile_and_profile"](env))
    replaced.append("compile_and_profile")
    if env is not None:
        registry.register(classes["verify_correctness"](env))
        replaced.append("verify_correctness")
    return replaced
