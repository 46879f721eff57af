"""Packing of a module's tensors into one flat buffer, used by weight sharding and layer offload.

Tensors that already share a storage (for instance q/k/v weights re-homed as row slices of one fused
buffer) are packed as one unit and keep their relative offsets, so zero-copy fused views survive a
re-bind. After `bind(slot)` every packed tensor is a permanent view into `slot`; whoever owns the
slot decides when its contents are valid.
"""

from __future__ import annotations

import torch
from torch import nn

ALIGN = 128  # elements; keeps every unit 256-byte aligned for bf16 (TMA needs 16 bytes)


def _extent(t: torch.Tensor) -> int:
    if t.numel() == 0:
        return 0
    return 1 + sum((s - 1) * st for s, st in zip(t.shape, t.stride()))


class PackedBlock:
    def __init__(self, block: nn.Module, min_numel: int = 1 << 12, matrices_only: bool = True) -> None:
        self.block = block
        tensors = list(block.named_parameters()) + list(block.named_buffers())
        groups: dict[tuple, list] = {}
        for _name, t in tensors:
            groups.setdefault((t.dtype, t.untyped_storage().data_ptr()), []).append(t)
        self.entries: list[tuple] = []  # (tensor, flat offset, shape, stride)
        dtypes = set()
        off = 0
        for (dt, _ptr), members in groups.items():
            lo = min(t.storage_offset() for t in members)
            hi = max(t.storage_offset() + _extent(t) for t in members)
            if hi - lo < min_numel or (matrices_only and not any(t.dim() == 2 for t in members)):
                continue  # biases, norm weights, modulation tables stay where they are
            dtypes.add(dt)
            for t in members:
                self.entries.append((t, off + t.storage_offset() - lo, tuple(t.shape), tuple(t.stride())))
            off += -(-(hi - lo) // ALIGN) * ALIGN
        if len(dtypes) > 1:
            raise ValueError(f"the packed tensors of a block must share one dtype, found {sorted(map(str, dtypes))}")
        self.dtype = dtypes.pop() if dtypes else torch.float32
        self.numel = off
        self.device = tensors[0][1].device if tensors else torch.device("cpu")

    def pack_into(self, flat: torch.Tensor) -> None:
        for t, o, shape, stride in self.entries:
            torch.as_strided(flat, shape, stride, o).copy_(t.data)

    def bind(self, slot: torch.Tensor) -> None:
        for t, o, shape, stride in self.entries:
            t.data = torch.as_strided(slot, shape, stride, o)

    def nbytes(self) -> int:
        return self.numel * torch.empty((), dtype=self.dtype).element_size()
