"""Ring attention (context parallel), USP (ring x Ulysses) and the strategy router.

Ring: every rank keeps its query shard and the K,V shards travel round the ring; step r attends to
the shard that started r ranks upstream while the next shard is already in flight (`isend`/`irecv`
into the other half of a double buffer); partial results are merged by log-sum-exp. Non-causal, so
the visiting order does not matter. This is the collective-library path and the oracle for the fused form
(`symm.ring_attention_fused`: one peer-store all-gather of K / V overlapped with the local attention).
USP: all-to-all over the Ulysses group (sequence -> heads) inside each ring group, ring attention
over the ring group, inverse all-to-all.
Role parity: telefuser/distributed/ring.py:61-214, ops/attention/attention_impl.py:319-558.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from telefuser_b200.ops import functional as TF

from . import ulysses
from .mesh import get_attention_strategy, get_mesh


def _group_info(group):
    if group is None or not dist.is_initialized():
        return 0, 1, [0]
    return dist.get_rank(group), dist.get_world_size(group), dist.get_process_group_ranks(group)


def _fused_ok(q, k, fused: bool) -> bool:
    return fused and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and q.shape[0] == 1 and k.shape[0] == 1


def ring_attention(q, k, v, group=None, scale=None, return_lse: bool = False, fused: bool = False):
    """q, k, v: [B, S_local, H, D] shards of one sequence over `group` -> [B, S_local, H, D].
    `fused`: exchange K / V by peer stores overlapped with the local attention instead of NCCL ring steps."""
    rank, P, ranks = _group_info(group)
    if P == 1:
        return TF.attention(q, k, v, scale, return_lse)
    if _fused_ok(q, k, fused):
        from .symm import get_workspace, ring_attention_fused, ring_workspace_bytes

        ws = get_workspace(group, ring_workspace_bytes(k.shape[1], k.shape[2], k.shape[3], P), tag="ring")
        return ring_attention_fused(q, k, v, ws, scale, return_lse)
    nxt, prv = ranks[(rank + 1) % P], ranks[(rank - 1) % P]
    cur = torch.stack([k, v]).contiguous()  # one message per step
    other = torch.empty_like(cur)
    out = lse = None
    for step in range(P):
        works = []
        if step + 1 < P:
            ops = [dist.P2POp(dist.isend, cur, nxt, group), dist.P2POp(dist.irecv, other, prv, group)]
            works = dist.batch_isend_irecv(ops)
        o_i, lse_i = TF.attention(q, cur[0], cur[1], scale, return_lse=True)
        out, lse = (o_i, lse_i) if out is None else TF.merge_attn_states(out, lse, o_i, lse_i)
        for w in works:
            w.wait()
        cur, other = other, cur
    return (out, lse) if return_lse else out


def usp_attention(q, k, v, ulysses_group=None, ring_group=None, scale=None, fused: bool = False):
    """Sequence sharded over ring x Ulysses; heads are exchanged inside the Ulysses group first."""
    hq = ulysses.scatter_heads(q, ulysses_group, async_op=True)
    hk = ulysses.scatter_heads(k, ulysses_group, async_op=True)
    hv = ulysses.scatter_heads(v, ulysses_group, async_op=True)
    o = ring_attention(hq.wait(), hk.wait(), hv.wait(), ring_group, scale, fused=fused)
    return ulysses.gather_heads(o, ulysses_group)


def long_context_attention(q, k, v, scale=None, mesh=None, strategy: str | None = None):
    """Routes to local / Ulysses / ring / USP attention by the mesh's sequence-parallel degrees."""
    mesh = mesh or get_mesh()
    strategy = strategy or get_attention_strategy(mesh)
    if strategy == "local":
        return TF.attention(q, k, v, scale)
    if strategy == "ulysses":
        g = mesh.group("ulysses")
        if mesh.fused and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128:
            from .symm import get_workspace, ulysses_attention_fused

            B, S, H, D = q.shape  # 3 head-sharded slabs + the output buffer, each B*S*H*D elements
            ws = get_workspace(g, 4 * (B * S * H * D * 2 + 256) + 4096)
            return ulysses_attention_fused(q, k, v, ws, scale)
        hq = ulysses.scatter_heads(q, g, async_op=True)
        hk = ulysses.scatter_heads(k, g, async_op=True)
        hv = ulysses.scatter_heads(v, g, async_op=True)
        return ulysses.gather_heads(TF.attention(hq.wait(), hk.wait(), hv.wait(), scale), g)
    if strategy == "ring":
        return ring_attention(q, k, v, mesh.group("ring"), scale, fused=mesh.fused)
    if strategy == "usp":
        return usp_attention(q, k, v, mesh.group("ulysses"), mesh.group("ring"), scale, fused=mesh.fused)
    raise ValueError(f"unknown attention strategy {strategy!r}")
