"""Weight sharding for inference (ZeRO-3 style): every rank keeps 1/P of each block's weights and
the full block is rebuilt just in time by an all-gather that overlaps the previous block's compute.

Layout: a wrapped block's parameters are packed into one flat buffer (tensors that already share a
storage, such as fused QKV weights, stay adjacent and keep their relative offsets), padded to a
multiple of P x 128 elements and split evenly. Two gather slots per dtype rotate over the blocks:
block i lives in slot i % 2, so the all-gather of block i+1 (side stream) runs while block i
computes; parameters are permanent views of their slot, therefore cached fused views stay valid.
NVSwitch makes the all-gather cost independent of P, so the unit is a whole block (hundreds of MB).
Role parity: telefuser/distributed/fsdp.py (`shard_model` with FSDP1/FSDP2 wrapping of the named
ModuleList children and forward prefetch).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from telefuser_b200.utils.packing import ALIGN, PackedBlock

MIN_SHARD_NUMEL = 1 << 12


def _prepare_fused(module: nn.Module) -> None:
    for m in module.modules():
        for name in dir(type(m)):
            if name.startswith("fused_") and callable(getattr(m, name)):
                getattr(m, name)()


class _Unit:
    """One wrapped block: packing plan + the local shard."""

    def __init__(self, block: nn.Module, rank: int, world: int, min_shard_numel: int = MIN_SHARD_NUMEL) -> None:
        self.block = block
        self.pack = PackedBlock(block, min_shard_numel)
        self.dtype = self.pack.dtype
        chunk = -(-self.pack.numel // (world * ALIGN)) * ALIGN
        self.numel, self.chunk = chunk * world, chunk
        flat = torch.zeros(self.numel, dtype=self.dtype, device=self.pack.device)
        self.pack.pack_into(flat)
        self.shard = flat[rank * chunk : (rank + 1) * chunk].clone()
        del flat

    def bind(self, slot: torch.Tensor) -> None:
        self.pack.bind(slot)


class ShardedBlocks:
    def __init__(self, blocks: list[nn.Module], group=None, prefetch: bool = True,
                 min_shard_numel: int = MIN_SHARD_NUMEL) -> None:  # fmt: skip
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.units = [_Unit(b, self.rank, self.world, min_shard_numel) for b in blocks]
        size = max(u.numel for u in self.units)
        dev, dtype = self.units[0].shard.device, self.units[0].dtype
        self.slots = [torch.empty(size, dtype=dtype, device=dev) for _ in range(2)]
        self.cuda = dev.type == "cuda"
        self.stream = torch.cuda.Stream(dev) if self.cuda else None
        self.ready: list = [None, None]  # event per slot: gather finished
        self.free: list = [None, None]  # event per slot: last consumer finished
        self.resident = [-1, -1]
        self.prefetch = prefetch
        for i, u in enumerate(self.units):
            u.bind(self.slots[i % 2])
            u.block.register_forward_pre_hook(self._pre(i))
            u.block.register_forward_hook(self._post(i))

    def bytes_per_rank(self) -> int:
        return sum(u.shard.numel() * u.shard.element_size() for u in self.units)

    def _gather(self, i: int) -> None:
        s = i % 2
        if self.resident[s] == i:
            return
        u = self.units[i]
        out = self.slots[s][: u.numel]
        if self.cuda:
            if self.free[s] is not None:
                self.stream.wait_event(self.free[s])
            with torch.cuda.stream(self.stream):
                self._all_gather(out, u.shard)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.ready[s] = ev
        else:
            self._all_gather(out, u.shard)
        self.resident[s] = i

    def _all_gather(self, out: torch.Tensor, shard: torch.Tensor) -> None:
        if self.world == 1:
            out.copy_(shard)
        else:
            dist.all_gather_into_tensor(out, shard, group=self.group)

    def _pre(self, i: int):
        def hook(_m, _inputs):
            self._gather(i)
            if self.cuda and self.ready[i % 2] is not None:
                torch.cuda.current_stream().wait_event(self.ready[i % 2])
            if self.prefetch and len(self.units) > 1:
                self._gather((i + 1) % len(self.units))

        return hook

    def _post(self, i: int):
        def hook(_m, _inputs, _output):
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
                self.free[i % 2] = ev

        return hook


def shard_model(model: nn.Module, device=None, wrap_module_names: list[str] | None = None, group=None,
                prefetch: bool = True, min_shard_numel: int = MIN_SHARD_NUMEL) -> nn.Module:  # fmt: skip
    """Shards the children of the named ModuleLists over `group`; everything else stays replicated."""
    if device is not None:
        model.to(device)
    names = wrap_module_names or (model.get_fsdp_module_names() if hasattr(model, "get_fsdp_module_names") else [])
    blocks: list[nn.Module] = []
    for n in names:
        sub = model.get_submodule(n)
        blocks.extend(list(sub) if isinstance(sub, (nn.ModuleList, nn.Sequential)) else [sub])
    if not blocks:
        raise ValueError("no module to shard")
    for b in blocks:
        _prepare_fused(b)
    model._sharded_blocks = ShardedBlocks(blocks, group, prefetch, min_shard_numel)
    model.fsdp = True
    return model
