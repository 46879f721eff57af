"""Device-memory checkpoints: what the caching allocator holds at named points of a run, and what each phase added.

    from telefuser_b200.utils.memory_snapshot import record_memory_snapshot, set_memory_baseline, get_memory_analysis

    set_memory_baseline()                    # after the weights are resident
    record_memory_snapshot("text_encoded")
    record_memory_snapshot("denoised")
    record_memory_snapshot("decoded")
    print(get_memory_analysis())

A snapshot holds the allocator's four counters in MiB: live tensor bytes (`allocated`), bytes the allocator has taken
from the driver (`reserved`: what `nvidia-smi` shows, minus the context), and the peaks of both since the last reset.
`reserved - allocated` is the pool overhead (cached blocks and fragmentation). The analysis lists every checkpoint with
its growth over the baseline and over the previous checkpoint and names the phase with the highest peak, which is the
number that decides whether a configuration fits. On machines without CUDA every counter reads zero.
Role: telefuser/utils/memory_snapshot.py of the reference (snapshot, checkpoint registry, analysis).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Callable

import torch

MIB = float(1 << 20)


@dataclass(frozen=True)
class MemorySnapshot:
    allocated_mb: float = 0.0
    reserved_mb: float = 0.0
    peak_allocated_mb: float = 0.0
    peak_reserved_mb: float = 0.0

    @property
    def pool_overhead_mb(self) -> float:
        return max(0.0, self.reserved_mb - self.allocated_mb)

    @property
    def pool_overhead_pct(self) -> float:
        return 100.0 * self.pool_overhead_mb / self.reserved_mb if self.reserved_mb > 0 else 0.0

    def to_dict(self) -> dict:
        return {**{k: round(v, 2) for k, v in asdict(self).items()}, "pool_overhead_mb": round(self.pool_overhead_mb, 2)}

    def __sub__(self, other: "MemorySnapshot") -> "MemorySnapshot":
        return MemorySnapshot(*(a - b for a, b in zip(asdict(self).values(), asdict(other).values())))


def _read_cuda(device) -> tuple[float, float, float, float]:
    if not torch.cuda.is_available():
        return 0.0, 0.0, 0.0, 0.0
    return (torch.cuda.memory_allocated(device), torch.cuda.memory_reserved(device), torch.cuda.max_memory_allocated(device),
            torch.cuda.max_memory_reserved(device))  # fmt: skip


def capture_memory_snapshot(device=None, reader: Callable | None = None) -> MemorySnapshot:
    """The allocator's counters on `device` (default: the current one) in MiB; `reader` replaces the CUDA queries in tests."""
    a, r, pa, pr = (reader or _read_cuda)(device)
    return MemorySnapshot(a / MIB, r / MIB, pa / MIB, pr / MIB)


def reset_peak_memory_stats(device=None) -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats(device)


class MemoryCheckpoints:
    """Ordered, named snapshots of one run plus an optional baseline."""

    def __init__(self, reader: Callable | None = None) -> None:
        self._reader = reader
        self.baseline: MemorySnapshot | None = None
        self.points: dict[str, MemorySnapshot] = {}

    def set_baseline(self, device=None) -> MemorySnapshot:
        self.baseline = capture_memory_snapshot(device, self._reader)
        return self.baseline

    def record(self, name: str, device=None) -> MemorySnapshot:
        snap = capture_memory_snapshot(device, self._reader)
        if name in self.points:  # a phase that runs more than once keeps its worst reading
            old = self.points[name]
            snap = MemorySnapshot(max(old.allocated_mb, snap.allocated_mb), max(old.reserved_mb, snap.reserved_mb),
                                  max(old.peak_allocated_mb, snap.peak_allocated_mb), max(old.peak_reserved_mb, snap.peak_reserved_mb))  # fmt: skip
        self.points[name] = snap
        return snap

    def analysis(self) -> dict:
        base = self.baseline or MemorySnapshot()
        rows, prev = [], base
        for name, snap in self.points.items():
            rows.append({"checkpoint": name, **snap.to_dict(), "allocated_over_baseline_mb": round(snap.allocated_mb - base.allocated_mb, 2),
                         "allocated_over_previous_mb": round(snap.allocated_mb - prev.allocated_mb, 2),
                         "peak_over_baseline_mb": round(snap.peak_allocated_mb - base.allocated_mb, 2)})  # fmt: skip
            prev = snap
        top = max(rows, key=lambda r: r["peak_allocated_mb"], default=None)
        return {"baseline": base.to_dict(), "checkpoints": rows, "highest_peak_checkpoint": top["checkpoint"] if top else None,
                "highest_peak_allocated_mb": top["peak_allocated_mb"] if top else 0.0,
                "highest_peak_reserved_mb": max((r["peak_reserved_mb"] for r in rows), default=0.0)}  # fmt: skip

    def summary(self) -> str:
        a = self.analysis()
        lines = [f"baseline: {a['baseline']['allocated_mb']:.1f} MiB allocated, {a['baseline']['reserved_mb']:.1f} MiB reserved"]
        for r in a["checkpoints"]:
            lines.append(f"{r['checkpoint']:<24} alloc {r['allocated_mb']:>10.1f}  (+{r['allocated_over_previous_mb']:.1f})  "
                         f"peak {r['peak_allocated_mb']:>10.1f}  reserved {r['reserved_mb']:>10.1f}  pool {r['pool_overhead_mb']:.1f} MiB")  # fmt: skip
        if a["highest_peak_checkpoint"]:
            lines.append(f"highest peak: {a['highest_peak_allocated_mb']:.1f} MiB at {a['highest_peak_checkpoint']!r}")
        return "\n".join(lines)


_DEFAULT = MemoryCheckpoints()


def reset_memory_registry() -> None:
    global _DEFAULT
    _DEFAULT = MemoryCheckpoints()


def set_memory_baseline(device=None) -> MemorySnapshot:
    return _DEFAULT.set_baseline(device)


def record_memory_snapshot(name: str, device=None) -> MemorySnapshot:
    return _DEFAULT.record(name, device)


def get_memory_snapshots() -> dict[str, MemorySnapshot]:
    return dict(_DEFAULT.points)


def get_memory_analysis() -> dict:
    return _DEFAULT.analysis()


def print_memory_analysis() -> None:
    from telefuser_b200.utils.logging import logger

    logger.info("device memory by checkpoint\n" + _DEFAULT.summary())
