"""``HardwareModel`` instance for one B200 (sm_100a), in the reference's own structure
(arke/backend/hardware.py:105-203: MemoryLevel / SyncDomain / ComputeUnit / AlignmentConstraints).

When the reference package is importable its dataclasses are used, so the instance is accepted
wherever Arke expects a ``HardwareModel``; otherwise field-compatible local dataclasses are used.
"""
from __future__ import annotations

from dataclasses import dataclass, field

try:  # the reference's own types, when Arke is on the path
    from arke.backend.hardware import (AlignmentConstraints, ComputeUnit, HardwareModel,  # type: ignore
                                       MemoryLevel, SyncDomain)
except Exception:  # pragma: no cover - exercised on machines without the reference checkout

    @dataclass(frozen=True)
    class MemoryLevel:
        name: str
        scope: str
        size_bytes: int = 0
        bandwidth_gbps: float = 0.0
        latency_cycles: int = 0

    @dataclass(frozen=True)
    class SyncDomain:
        name: str
        width: int = 0
        barrier_free: bool = False

    @dataclass(frozen=True)
    class ComputeUnit:
        kind: str
        count: int = 0
        supported_dtypes: tuple = ()
        peak_tflops: float = 0.0

    @dataclass(frozen=True)
    class AlignmentConstraints:
        warp_size: int = 32
        mma_tile: tuple = ()
        vector_width: int = 4
        shared_bank_bytes: int = 4

    @dataclass(frozen=True)
    class HardwareModel:
        name: str
        compute_capability: tuple
        num_sms: int
        max_threads_per_block: int
        max_threads_per_sm: int
        memory_levels: tuple
        sync_domains: tuple
        compute_units: tuple
        alignment: AlignmentConstraints = field(default_factory=AlignmentConstraints)

        def memory_level(self, name):
            return next((m for m in self.memory_levels if m.name == name), None)

        def shared_memory_bytes(self):
            m = self.memory_level("shared")
            return m.size_bytes if m else 0

        def has_tensor_core(self):
            return any(cu.kind == "tensor_core" for cu in self.compute_units)

        def tensor_core(self):
            return next((cu for cu in self.compute_units if cu.kind == "tensor_core"), None)

        @property
        def warp_size(self):
            return self.alignment.warp_size


def _make(cls, positional, **kw):
    """Construct a reference dataclass whatever its positional field names are."""
    try:
        return cls(*positional, **kw)
    except TypeError:
        return cls(*positional)


def nvidia_sm100_b200(name: str = "nvidia_blackwell") -> "HardwareModel":
    """One B200: 148 SMs (2 dies), 227 KB shared memory per CTA, 256 KB tensor memory per SM,
    126 MB L2, 180 GB HBM3e at ~7.7 TB/s, 5th-gen tensor cores (tcgen05, UMMA 128x256x16 bf16)."""
    return HardwareModel(
        name=name,
        compute_capability=(10, 0),
        num_sms=148,
        max_threads_per_block=1024,
        max_threads_per_sm=2048,
        memory_levels=(
            _make(MemoryLevel, ("register", "thread"), size_bytes=256 * 1024, bandwidth_gbps=0.0, latency_cycles=1),
            _make(MemoryLevel, ("tensor_memory", "block"), size_bytes=256 * 1024, bandwidth_gbps=0.0, latency_cycles=20),
            _make(MemoryLevel, ("shared", "block"), size_bytes=227 * 1024, bandwidth_gbps=0.0, latency_cycles=30),
            _make(MemoryLevel, ("l2", "device"), size_bytes=126 * 1024 * 1024, bandwidth_gbps=0.0, latency_cycles=300),
            _make(MemoryLevel, ("global", "device"), size_bytes=180 * 1024 ** 3, bandwidth_gbps=7700.0, latency_cycles=800),
        ),
        sync_domains=(
            _make(SyncDomain, ("warp",), width=32, barrier_free=True),
            _make(SyncDomain, ("block",), width=1024, barrier_free=False),
            _make(SyncDomain, ("cluster",), width=8, barrier_free=False),
            _make(SyncDomain, ("device",), width=0, barrier_free=False),
        ),
        compute_units=(
            _make(ComputeUnit, ("simt",), count=128, supported_dtypes=("f16", "bf16", "f32", "i32"), peak_tflops=75.0),
            _make(ComputeUnit, ("tensor_core",), count=4,
                  supported_dtypes=("f16", "bf16", "tf32", "e4m3", "e5m2", "i8"), peak_tflops=2250.0),
        ),
        alignment=AlignmentConstraints(warp_size=32, mma_tile=(128, 256, 16), vector_width=8, shared_bank_bytes=4),
    )
