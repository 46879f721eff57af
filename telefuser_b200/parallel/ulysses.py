"""Ulysses sequence parallelism: sequence-sharded <-> head-sharded all-to-all.

``scatter_heads``: [B, S/P, H, D] -> [B, S, H/P, D]   (before attention)
``gather_heads`` : [B, S, H/P, D] -> [B, S/P, H, D]   (after attention)

This module is the collective-library path (NCCL on GPUs, gloo in CPU tests)
and the correctness baseline for the fused peer-memory kernels. Semantics match
the reference's ``telefuser/distributed/ulysses_comm.py:38-124``; async variants
return a handle whose ``wait()`` yields the tensor so q/k/v exchanges overlap
with the remaining projections.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .mesh import get_mesh


class _Done:
    def __init__(self, t):
        self._t = t

    def wait(self):
        return self._t


class _PendingA2A:
    def __init__(self, work, out, finish):
        self._work, self._out, self._finish = work, out, finish

    def wait(self):
        if self._work is not None:
            self._work.wait()
            self._work = None
        return self._finish(self._out)


def _a2a(send: torch.Tensor, group, async_op: bool):
    out = torch.empty_like(send)
    work = dist.all_to_all_single(out, send, group=group, async_op=async_op)
    return out, work


def scatter_heads(x: torch.Tensor, group=None, async_op: bool = False):
    """[B, S_local, H, D] -> [B, S_local * P, H / P, D]; token order = rank-major."""
    mesh = get_mesh()
    group = group if group is not None else mesh.group("ulysses")
    P = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    if P == 1:
        return _Done(x) if async_op else x
    B, S, H, D = x.shape
    if H % P:
        raise ValueError(f"num_heads {H} not divisible by ulysses degree {P}")
    send = x.reshape(B, S, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()  # [P, B, S, H/P, D]
    out, work = _a2a(send, group, async_op)

    def finish(o):
        return o.permute(1, 0, 2, 3, 4).reshape(B, P * S, H // P, D)

    if async_op:
        return _PendingA2A(work, out, finish)
    return finish(out)


def gather_heads(x: torch.Tensor, group=None, async_op: bool = False):
    """[B, S, H_local, D] -> [B, S / P, H_local * P, D] (inverse of `scatter_heads`)."""
    mesh = get_mesh()
    group = group if group is not None else mesh.group("ulysses")
    P = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    if P == 1:
        return _Done(x) if async_op else x
    B, S, Hl, D = x.shape
    if S % P:
        raise ValueError(f"sequence {S} not divisible by ulysses degree {P}")
    send = x.reshape(B, P, S // P, Hl, D).permute(1, 0, 2, 3, 4).contiguous()  # [P, B, S/P, Hl, D]
    out, work = _a2a(send, group, async_op)

    def finish(o):
        return o.permute(1, 2, 0, 3, 4).reshape(B, S // P, P * Hl, D)

    if async_op:
        return _PendingA2A(work, out, finish)
    return finish(out)


# Names used by pipeline code written against the reference.
ulysses_scatter_heads = scatter_heads
ulysses_gather_heads = gather_heads


def all_to_all_split_cat(x: torch.Tensor, split_dim: int, cat_dim: int, group=None) -> torch.Tensor:
    """Generic list all-to-all: split on `split_dim`, concatenate what arrives on `cat_dim`."""
    mesh = get_mesh()
    group = group if group is not None else mesh.group("ulysses")
    P = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    if P == 1:
        return x
    parts = [t.contiguous() for t in x.chunk(P, dim=split_dim)]
    recv = [torch.empty_like(parts[0]) for _ in range(P)]
    dist.all_to_all(recv, parts, group=group)
    return torch.cat(recv, dim=cat_dim)
