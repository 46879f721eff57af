"""Tensor parallelism by in-place weight sharding.

The model code calls `ops.linear(x, module.weight, module.bias)` with the weights it finds on its
sub-modules, so TP does not swap modules: it slices their parameters in place and marks where partial
sums must be reduced.

Plan: `{module-path pattern (fnmatch, `*` = one or more path parts): style}` with styles
* `colwise`  - keep rows `[rank*out/P, (rank+1)*out/P)` of `weight` (and `bias`): output features split
* `rowwise`  - keep the matching columns of `weight`; `bias` stays on TP rank 0 only (zero elsewhere),
               so that the sum over ranks adds it once
* `heads`    - divide `num_heads` of the module by P and record `head_start` (for per-head tables)
* `allreduce`- all-reduce (sum) the module's output over the TP group after its forward
* `group`    - only set `module.tp_group` / `tp_rank` / `tp_size` (the module reduces where it needs to)
Role parity: telefuser/distributed/tp_parallelize.py (`parallelize_module` over a plan); the
reference applies torch DTensor styles, here the sharding is explicit.
"""

from __future__ import annotations

import fnmatch

import torch
import torch.distributed as dist
from torch import nn


def _tp_info(mesh_or_group):
    if mesh_or_group is None:
        return None, 0, 1
    if hasattr(mesh_or_group, "group") and hasattr(mesh_or_group, "coord"):
        return mesh_or_group.group("tp"), mesh_or_group.coord("tp"), mesh_or_group.size("tp")
    g = mesh_or_group
    return g, dist.get_rank(g), dist.get_world_size(g)


def shard_dim(t: torch.Tensor, dim: int, rank: int, size: int) -> torch.Tensor:
    n = t.shape[dim]
    if n % size:
        raise ValueError(f"dimension {dim} of size {n} is not divisible by the TP degree {size}")
    return t.narrow(dim, rank * (n // size), n // size).clone()  # own storage: the full tensor can be freed


def _reshard_param(module: nn.Module, name: str, new: torch.Tensor) -> None:
    old = getattr(module, name)
    setattr(module, name, nn.Parameter(new, requires_grad=False) if isinstance(old, nn.Parameter) else new)


def apply_colwise(module: nn.Module, rank: int, size: int) -> None:
    _reshard_param(module, "weight", shard_dim(module.weight.data, 0, rank, size))
    if getattr(module, "bias", None) is not None:
        _reshard_param(module, "bias", shard_dim(module.bias.data, 0, rank, size))
    if hasattr(module, "out_features"):
        module.out_features //= size


def apply_rowwise(module: nn.Module, rank: int, size: int) -> None:
    _reshard_param(module, "weight", shard_dim(module.weight.data, 1, rank, size))
    if getattr(module, "bias", None) is not None and rank != 0:
        _reshard_param(module, "bias", torch.zeros_like(module.bias.data))
    if hasattr(module, "in_features"):
        module.in_features //= size


def apply_heads(module: nn.Module, rank: int, size: int) -> None:
    h = module.num_heads
    if h % size:
        raise ValueError(f"{h} heads are not divisible by the TP degree {size}")
    module.num_heads = h // size
    module.head_start = rank * (h // size)


def all_reduce_sum(t: torch.Tensor, group) -> torch.Tensor:
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(t, group=group)
    return t


def _allreduce_hook(group):
    def hook(_module, _inputs, output):
        if isinstance(output, tuple):
            return (all_reduce_sum(output[0].contiguous(), group), *output[1:])
        return all_reduce_sum(output.contiguous(), group)

    return hook


def _match(pattern: str, name: str) -> bool:
    return fnmatch.fnmatchcase(name, pattern)


def parallelize_module(module: nn.Module, mesh_or_group, plan: dict[str, str | list[str]]) -> nn.Module:
    group, rank, size = _tp_info(mesh_or_group)
    if size <= 1 or not plan:
        return module
    applied = 0
    for name, sub in module.named_modules():
        for pattern, styles in plan.items():
            if not _match(pattern, name):
                continue
            for style in [styles] if isinstance(styles, str) else styles:
                if style == "colwise":
                    apply_colwise(sub, rank, size)
                elif style == "rowwise":
                    apply_rowwise(sub, rank, size)
                elif style == "heads":
                    apply_heads(sub, rank, size)
                elif style == "allreduce":
                    sub.register_forward_hook(_allreduce_hook(group))
                elif style == "group":
                    pass
                else:
                    raise ValueError(f"unknown TP style {style!r} for {name}")
                sub.tp_group, sub.tp_rank, sub.tp_size = group, rank, size
                applied += 1
    if applied == 0:
        raise ValueError("the TP plan matched no module")
    module.tp_group, module.tp_rank, module.tp_size = group, rank, size
    return module
