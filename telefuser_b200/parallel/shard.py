"""Sharding helpers: token-stream split / gather for sequence parallelism and
branch split / gather for classifier-free-guidance parallelism.

Behavioural counterpart of the reference's
``telefuser/distributed/parallel_shard.py:97-250``; tensors are returned
(functional style) rather than resized in place.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .mesh import ParallelMesh, get_mesh


def _sp(mesh: ParallelMesh | None):
    mesh = mesh or get_mesh()
    return mesh, mesh.size("sp"), mesh.coord("sp"), mesh.group("sp")


def padded_len(n: int, parts: int) -> int:
    return (n + parts - 1) // parts * parts


def sequence_parallel_shard(tensors, seq_dims, mesh: ParallelMesh | None = None):
    """Returns this rank's slice of each tensor along its sequence dim (zero-padded to a multiple of P).

    Tensors whose sequence extent is 1 (broadcast modulation) are returned unchanged.
    """
    mesh, P, r, _ = _sp(mesh)
    if P == 1:
        return list(tensors)
    out = []
    for t, d in zip(tensors, seq_dims):
        n = t.shape[d]
        if n == 1:
            out.append(t)
            continue
        total = padded_len(n, P)
        if total != n:
            pad_shape = list(t.shape)
            pad_shape[d] = total - n
            t = torch.cat([t, t.new_zeros(pad_shape)], dim=d)
        out.append(t.narrow(d, r * (total // P), total // P).contiguous())
    return out


def sequence_parallel_unshard(tensors, seq_dims, seq_lens, mesh: ParallelMesh | None = None):
    """All-gathers each tensor along its sequence dim and trims the padding to `seq_lens`."""
    mesh, P, _, group = _sp(mesh)
    if P == 1:
        return list(tensors)
    out = []
    for t, d, n in zip(tensors, seq_dims, seq_lens):
        t = t.contiguous()
        if mesh.fused and t.is_cuda and d == 1 and t.dim() == 3 and t.shape[0] == 1 and (t.shape[2] * t.element_size()) % 16 == 0:
            # every rank stores its rows straight into all ranks' full buffer over NVLink (no gather list, no cat)
            from .symm import all_gather_rows_fused, get_workspace

            rows, width = t.shape[1], t.shape[2]
            ws = get_workspace(group, P * rows * width * t.element_size() + 4096, tag="sp_unshard")
            full = all_gather_rows_fused(t[0], ws, name=f"sp_unshard_{width}")
            out.append(full[:n].clone().unsqueeze(0))
            continue
        parts = [torch.empty_like(t) for _ in range(P)]
        dist.all_gather(parts, t, group=group)
        out.append(torch.cat(parts, dim=d).narrow(d, 0, n))
    return out


def cfg_parallel_shard(cond_items, uncond_items, mesh: ParallelMesh | None = None):
    """Picks the branch this rank computes: cfg rank 0 -> conditional, rank 1 -> unconditional."""
    mesh = mesh or get_mesh()
    if mesh.size("cfg") == 1:
        return None
    return cond_items if mesh.coord("cfg") == 0 else uncond_items


def cfg_parallel_unshard(pred: torch.Tensor, mesh: ParallelMesh | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """All-gathers the per-branch predictions; returns (cond, uncond) on every rank."""
    mesh = mesh or get_mesh()
    P = mesh.size("cfg")
    if P == 1:
        raise RuntimeError("cfg_parallel_unshard called without CFG parallelism")
    pred = pred.contiguous()
    both = torch.empty((P * pred.shape[0], *pred.shape[1:]), dtype=pred.dtype, device=pred.device)
    dist.all_gather_into_tensor(both, pred, group=mesh.group("cfg"))
    both = both.view(P, *pred.shape)
    return both[0], both[1]
