"""Sequential (synchronous) CPU offload and whole-model moves.

`enable_sequential_cpu_offload(model, device, vram_limit_gb)` keeps weights in pinned host memory and
brings one unit at a time to the device around its forward: a unit is a child of one of the model's
block lists, or any other direct child with parameters. After its forward a unit goes back to the
host unless the device still has more than `vram_limit_gb` free, in which case it is kept (state
KEEP) and never moves again; with 180 GB of HBM most models end up fully resident after one pass.
The host copy is made once and reused (weights are read-only at inference), so "offload" is only a
pointer swap back to the pinned tensor.
Role parity: telefuser/offload/sequential_offload.py:34-318 (offload / onload / keep states,
vram_limit), offload/model_offload.py:14-35.
"""

from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

OFFLOADED, ONLOADED, KEEP = 0, 1, 2


def move_tensors_to_pinned_cpu(tensors: Iterable[torch.Tensor]) -> None:
    pin = torch.cuda.is_available()
    for t in tensors:
        if t.device.type != "cpu" or (pin and not t.data.is_pinned()):
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=pin)
            host.copy_(t.data)
            t.data = host


def move_tensors_to_device(tensors: Iterable[torch.Tensor], device, non_blocking: bool = True) -> None:
    for t in tensors:
        if t.device != torch.device(device):
            t.data = t.data.to(device, non_blocking=non_blocking)


class OffloadUnit:
    def __init__(self, module: nn.Module, device, vram_limit_bytes: int | None) -> None:
        self.module, self.device, self.limit = module, torch.device(device), vram_limit_bytes
        self.tensors = list(module.parameters()) + list(module.buffers())
        move_tensors_to_pinned_cpu(self.tensors)
        self.host = [t.data for t in self.tensors]
        self.state = OFFLOADED
        module.register_forward_pre_hook(self._pre)
        module.register_forward_hook(self._post)

    def free_vram(self) -> int:
        if self.device.type != "cuda":
            return 0
        return torch.cuda.mem_get_info(self.device)[0]

    def onload(self) -> None:
        if self.state == OFFLOADED:
            for t, h in zip(self.tensors, self.host):
                t.data = h.to(self.device, non_blocking=True)
            self.state = ONLOADED

    def offload(self) -> None:
        if self.state == ONLOADED:
            for t, h in zip(self.tensors, self.host):
                t.data = h
            self.state = OFFLOADED

    def keep(self) -> None:
        self.onload()
        self.state = KEEP

    def _pre(self, _m, _args) -> None:
        self.onload()

    def _post(self, _m, _args, _out) -> None:
        if self.state != ONLOADED:
            return
        if self.limit is not None and self.free_vram() > self.limit:
            self.state = KEEP
        else:
            if self.device.type == "cuda":
                torch.cuda.current_stream(self.device).synchronize()  # readers done before the storage is dropped
            self.offload()


def enable_sequential_cpu_offload(model: nn.Module, device, vram_limit_gb: float | None = None,
                                  module_names: list[str] | None = None) -> list[OffloadUnit]:  # fmt: skip
    limit = None if vram_limit_gb is None else int(vram_limit_gb * (1 << 30))
    units: list[OffloadUnit] = []
    block_lists = module_names or list(getattr(model, "layer_name_list", []) or [])
    seen: set[int] = set()
    for name in block_lists:
        for blk in model.get_submodule(name):
            units.append(OffloadUnit(blk, device, limit))
            seen.update(id(m) for m in blk.modules())
        seen.add(id(model.get_submodule(name)))
    if not units:  # no block list declared: every direct child with parameters is a unit
        for child in model.children():
            if any(True for _ in child.parameters()):
                units.append(OffloadUnit(child, device, limit))
                seen.update(id(m) for m in child.modules())
    # embeddings, heads and the model's own parameters are small and are read by the model's own
    # forward without going through a child's forward: they stay on the device
    rest = [t for m in model.modules() if id(m) not in seen
            for t in list(m.parameters(recurse=False)) + list(m.buffers(recurse=False))]  # fmt: skip
    move_tensors_to_device(rest, device)
    model._offload_units = units
    return units
