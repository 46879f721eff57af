"""Tensor-parallel linears whose collective runs inside the GEMM kernel over peer-mapped memory.

* `gemm_reduce_scatter` / `gemm_all_reduce`: row-parallel linear (K sharded). The GEMM epilogue stores each
  partial tile straight into the slab buffer of the rank that owns those rows (NVLink stores overlap the
  tensor-core work tile by tile); after one barrier every owner sums its P slabs in fp32, applies gate and
  residual once, and either keeps its rows (reduce-scatter) or pushes them to every rank (all-reduce).
* `all_gather_gemm`: column-parallel linear on row-sharded activations. A few CTAs of the GEMM launch pull
  the peers' row shards into local memory with bulk copies (each byte crosses NVLink once) while the other
  CTAs multiply the shards that have already landed, starting with the local one.
Without a peer workspace (CPU tensors, gloo groups, fused collectives disabled) the same functions compose
the library collective with a plain linear, which is also the numerical reference in the tests.
Role parity: the tensor-parallel plan of telefuser/models/wan_video_dit.py:1228-1304 (DTensor styles); the
reference leaves the collectives to NCCL.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import native


def _world(group) -> tuple[int, int]:
    if group is None or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _use_peer(x: torch.Tensor, ws) -> bool:
    return ws is not None and x.is_cuda and x.dtype == torch.bfloat16


# ---------------------------------------------------------------------------
# row-parallel: GEMM -> reduce-scatter / all-reduce
# ---------------------------------------------------------------------------
def _rs_reference(x, weight, bias, residual, gate, group, all_reduce: bool):
    rank, P = _world(group)
    y = TF.linear(x, weight, bias).float()
    M = y.shape[0]
    if P > 1:
        dist.all_reduce(y, group=group)
    y = y if all_reduce else y[rank * (M // P) : (rank + 1) * (M // P)]
    if gate is not None:
        g = gate.float().reshape(-1, gate.shape[-1])
        y = y * (g if g.shape[0] in (1, y.shape[0]) else g.repeat_interleave(y.shape[0] // g.shape[0], dim=0))
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def _gemm_rs(x, weight, bias, residual, gate, group, ws, all_reduce: bool, name: str):
    """x [M, K/P]; weight [N, K/P]; residual / gate rows: the full M for all_reduce, this rank's M/P otherwise."""
    rank, P = _world(group)
    M, K = x.shape
    N = weight.shape[0]
    if not _use_peer(x, ws) or P == 1 or M % P or N % 8 or K % 8:
        return _rs_reference(x, weight, bias, residual, gate, group, all_reduce)
    lib = native.load()
    seg = M // P
    slabs = ws.region(f"{name}_slabs", (P, seg, N), torch.bfloat16)
    x2 = x if x.stride(-1) == 1 else x.contiguous()
    w2 = weight if weight.stride(-1) == 1 else weight.contiguous()
    b = None if bias is None else bias.to(torch.bfloat16)
    ws.barrier()  # every rank has finished reducing the previous contents of its slabs
    code = lib.tfb_gemm_bf16_rs(x2.data_ptr(), x2.stride(0), w2.data_ptr(), w2.stride(0), ws.peer_table(f"{name}_slabs"), N,
                                P, rank, seg, N, K, native.ptr(b), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_gemm_bf16_rs")
    ws.barrier()  # all partial tiles have landed
    g2, ldg, rpg, grow0 = None, 0, 1, 0
    if gate is not None:  # gate rows divide the rows that `gate` / `residual` cover (all M, or this rank's M/P)
        g2 = gate.float().reshape(-1, N).contiguous()
        ldg = N
        rpg = max((M if all_reduce else seg) // g2.shape[0], 1)
        grow0 = rank * seg if all_reduce else 0
    res_rows = None
    if residual is not None:
        r2 = residual.reshape(-1, N)
        res_rows = r2[rank * seg : (rank + 1) * seg] if all_reduce else r2
        if res_rows.stride(-1) != 1:
            res_rows = res_rows.contiguous()
    if all_reduce:
        full = ws.region(f"{name}_full", (M, N), torch.bfloat16)
        dsts, n_dst, row0 = ws.peer_table(f"{name}_full"), P, rank * seg
        out = full
    else:
        out = torch.empty(seg, N, device=x.device, dtype=torch.bfloat16)
        dsts, n_dst, row0 = (ctypes.c_void_p * 1)(out.data_ptr()), 1, 0
    code = lib.tfb_slab_reduce(slabs.data_ptr(), P, seg, N, N, None, native.ptr(res_rows),
                               res_rows.stride(0) if res_rows is not None else 0, native.ptr(g2), ldg, rpg, grow0, dsts,
                               n_dst, N, row0, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_slab_reduce")
    if all_reduce:
        ws.barrier()  # every owner's rows have arrived
        out = out.clone()  # the region is reused by the next call
    return out


def gemm_reduce_scatter(x, weight, bias=None, residual=None, gate=None, group=None, ws=None, name: str = "tp_rs"):
    """rows [rank*M/P, +M/P) of `residual + gate * (sum over ranks of x @ weight.T + bias)`.

    `bias` is added to this rank's partial product, so exactly one rank of the group must pass it (the row
    parallel sharding keeps it on rank 0). `residual` / `gate` cover this rank's M/P rows."""
    return _gemm_rs(x, weight, bias, residual, gate, group, ws, False, name)


def gemm_all_reduce(x, weight, bias=None, residual=None, gate=None, group=None, ws=None, name: str = "tp_ar"):
    """The full `residual + gate * (sum over ranks of x @ weight.T + bias)` on every rank."""
    return _gemm_rs(x, weight, bias, residual, gate, group, ws, True, name)


# ---------------------------------------------------------------------------
# column-parallel on row-sharded input: all-gather -> GEMM
# ---------------------------------------------------------------------------
def all_gather_gemm(x_local, weight, bias=None, act=None, group=None, ws=None, n_copiers: int = 8, name: str = "tp_ag"):
    """act(concat over ranks of x_local @ weight.T + bias): x_local [rows, K] (same rows on every rank) -> [rows*P, N]."""
    rank, P = _world(group)
    rows, K = x_local.shape
    N = weight.shape[0]
    if not _use_peer(x_local, ws) or P == 1 or N % 8 or K % 8:
        if P > 1:
            parts = [torch.empty_like(x_local) for _ in range(P)]
            dist.all_gather(parts, x_local.contiguous(), group=group)
            x_full = torch.cat(parts, dim=0)
        else:
            x_full = x_local
        return TF.linear(x_full, weight, bias, act=act)
    lib = native.load()
    shard = ws.region(f"{name}_shard", (rows, K), torch.bfloat16)
    gathered = torch.empty(P * rows, K, device=x_local.device, dtype=torch.bfloat16)
    sync = torch.empty(16, device=x_local.device, dtype=torch.int32)
    out = torch.empty(P * rows, N, device=x_local.device, dtype=torch.bfloat16)
    w2 = weight if weight.stride(-1) == 1 else weight.contiguous()
    b = None if bias is None else bias.to(torch.bfloat16)
    ws.barrier()  # the peers' copiers of the previous call are done with this rank's shard
    shard.copy_(x_local)
    ws.barrier()  # every shard is complete
    code = lib.tfb_gemm_bf16_ag(ws.peer_table(f"{name}_shard"), gathered.data_ptr(), sync.data_ptr(), int(n_copiers),
                                w2.data_ptr(), w2.stride(0), out.data_ptr(), N, P, rank, rows, N, K, native.ptr(b),
                                1 if act == "gelu_tanh" else 0, native.stream_ptr())  # fmt: skip
    if act not in (None, "gelu_tanh"):
        raise ValueError(f"unknown activation {act}")
    native.check(code, "tfb_gemm_bf16_ag")
    return out
