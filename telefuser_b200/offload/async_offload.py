"""Layer-wise asynchronous weight offload: a ring of GPU slots fed from pinned host memory.

The last `offload_ratio` of the blocks live in pinned host buffers (one consolidated buffer per
block, so a block moves with ONE `cudaMemcpyAsync`); `prefetch_size + 1` device slots rotate over
them. `before_layer(i)` makes the compute stream wait for block i's copy and queues the copies of the
next `prefetch_size` offloaded blocks on the copy stream (each waits for its slot's last reader);
`after_layer(i)` marks the slot free. Blocks that stay resident are untouched. Parameters are
permanent views into their slot, so fused-weight views stay valid. A 14B block is ~0.7 GB: at the
measured ~55 GB/s of a PCIe 5 x16 host link that is ~13 ms, hidden behind a block's compute at 720p.
Role parity: telefuser/offload/async_offload.py:18-427 (`AsyncOffloadManager` with
before_layer / after_layer hooks, prefetch and pinned staging).
"""

from __future__ import annotations

import torch
from torch import nn

from telefuser_b200.utils.packing import PackedBlock


class AsyncOffloadManager:
    def __init__(self, blocks, enabled: bool = True, offload_ratio: float = 1.0, prefetch_size: int = 1,
                 device=None, pin_cpu_memory: bool = True, min_numel: int = 1 << 12) -> None:  # fmt: skip
        self.blocks = list(blocks)
        self.enabled = enabled
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.cuda = self.device.type == "cuda"
        n = len(self.blocks)
        n_off = min(n, max(0, round(n * offload_ratio))) if enabled else 0
        self.first_offloaded = n - n_off
        self.prefetch = max(1, prefetch_size)
        self.host: dict[int, torch.Tensor] = {}
        self.packs: dict[int, PackedBlock] = {}
        self.slot_of: dict[int, int] = {}
        self.slots: list[torch.Tensor] = []
        self.ready: list = []
        self.free: list = []
        self.resident: list[int] = []
        self.copies = 0
        if n_off == 0:
            return
        from telefuser_b200.parallel.fsdp import _prepare_fused

        size, dtype = 0, None
        for i in range(self.first_offloaded, n):
            blk = self.blocks[i]
            _prepare_fused(blk)
            pack = PackedBlock(blk, min_numel)
            host = torch.empty(pack.numel, dtype=pack.dtype, pin_memory=pin_cpu_memory and torch.cuda.is_available())
            pack.pack_into(host)
            self.packs[i], self.host[i] = pack, host
            size, dtype = max(size, pack.numel), pack.dtype
        n_slots = min(n_off, self.prefetch + 1)
        self.slots = [torch.empty(size, dtype=dtype, device=self.device) for _ in range(n_slots)]
        self.ready, self.free, self.resident = [None] * n_slots, [None] * n_slots, [-1] * n_slots
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        for j, i in enumerate(range(self.first_offloaded, n)):
            self.slot_of[i] = j % n_slots
            self.packs[i].bind(self.slots[j % n_slots])
        # everything that is not packed (biases, norms) and the resident blocks go to the device once
        for blk in self.blocks:
            for t in list(blk.parameters()) + list(blk.buffers()):
                if t.device != self.device and not any(t is e[0] for p in self.packs.values() for e in p.entries):
                    t.data = t.data.to(self.device)

    def offloaded_bytes(self) -> int:
        return sum(h.numel() * h.element_size() for h in self.host.values())

    def _load(self, i: int) -> None:
        s = self.slot_of[i]
        if self.resident[s] == i:
            return
        dst = self.slots[s][: self.packs[i].numel]
        if self.cuda:
            if self.free[s] is not None:
                self.stream.wait_event(self.free[s])
            with torch.cuda.stream(self.stream):
                dst.copy_(self.host[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.ready[s] = ev
        else:
            dst.copy_(self.host[i])
        self.resident[s] = i
        self.copies += 1

    def before_layer(self, i: int) -> None:
        if i < self.first_offloaded or not self.host:
            return
        self._load(i)
        if self.cuda and self.ready[self.slot_of[i]] is not None:
            torch.cuda.current_stream().wait_event(self.ready[self.slot_of[i]])
        n = len(self.blocks)
        n_off = n - self.first_offloaded
        for k in range(1, min(self.prefetch, len(self.slots) - 1) + 1):
            j = self.first_offloaded + (i - self.first_offloaded + k) % n_off  # wraps to the next forward's first block
            if self.slot_of[j] != self.slot_of[i]:
                self._load(j)

    def after_layer(self, i: int) -> None:
        if i < self.first_offloaded or not self.host or not self.cuda:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.free[self.slot_of[i]] = ev


def attach_layer_hooks(manager: AsyncOffloadManager) -> None:
    """For models whose block loop does not call before_layer / after_layer itself."""
    for i, blk in enumerate(manager.blocks):
        blk.register_forward_pre_hook(lambda _m, _a, i=i: manager.before_layer(i))
        blk.register_forward_hook(lambda _m, _a, _o, i=i: manager.after_layer(i))
