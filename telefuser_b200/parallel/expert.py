"""Expert parallelism: the experts of every MoE layer are split evenly over the ranks of a group.

CUDA path (one node, peer-mapped memory, no all-to-all and no host synchronisation):
  histogram rows pushed to every peer -> barrier -> plan kernel (every rank derives all owners' buffer
  layouts from the same P x E matrix) -> dispatch kernel stores token rows straight into the owners'
  receive buffers -> barrier -> grouped GEMMs + SiLU-mul on the local experts -> barrier -> combine
  kernel loads each token's k expert outputs from the owners' buffers and forms the weighted sum.
CPU / gloo path (the oracle): every rank all-gathers tokens, ids and weights, evaluates the pairs whose
expert it owns for all tokens, and the partial sums are all-reduced.
The reference has no expert parallelism (its MoE layers run replicated or weight-sharded); this is the
`ep` mesh dimension of this framework.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from telefuser_b200.ops import moe as MOE
from telefuser_b200.ops import native

ALIGN = MOE.ALIGN


@dataclass
class ExpertParallelState:
    group: object
    rank: int
    world: int
    num_experts: int  # global

    @property
    def local_experts(self) -> int:
        return self.num_experts // self.world

    @classmethod
    def shard_(cls, experts, group) -> "ExpertParallelState":
        """Keeps this rank's slice of `experts.w1 / w2 / w3` (in place) and returns the EP state."""
        if experts.w1.dtype == torch.float8_e4m3fn:
            raise ValueError("expert parallelism shards bf16 experts; e4m3 experts (quantize_fp8_) run unsharded")
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        E = experts.w1.shape[0]
        if E % world:
            raise ValueError(f"{E} experts are not divisible by the expert-parallel degree {world}")
        n = E // world
        sl = slice(rank * n, (rank + 1) * n)
        w13 = experts.fused_w13()[sl].clone()
        inter = w13.shape[1] // 2
        experts.w1.data, experts.w3.data = w13[:, :inter], w13[:, inter:]
        experts._w13 = w13
        experts.w2.data = experts.w2.data[sl].clone()
        return cls(group, rank, world, E)


def _reference_ep(tokens, indices, weights, w13_local, w2_local, st: ExpertParallelState):
    g, P = st.group, st.world
    T = tokens.shape[0]
    all_t = [torch.empty_like(tokens) for _ in range(P)]
    all_i = [torch.empty_like(indices) for _ in range(P)]
    all_w = [torch.empty_like(weights) for _ in range(P)]
    dist.all_gather(all_t, tokens.contiguous(), group=g)
    dist.all_gather(all_i, indices.contiguous(), group=g)
    dist.all_gather(all_w, weights.contiguous(), group=g)
    tk, ix, ww = torch.cat(all_t), torch.cat(all_i).long(), torch.cat(all_w).float()
    lo = st.rank * st.local_experts
    mine = (ix >= lo) & (ix < lo + st.local_experts)
    part = MOE.experts_forward_reference(tk.float(), torch.where(mine, ix - lo, torch.zeros_like(ix)),
                                         torch.where(mine, ww, torch.zeros_like(ww)), w13_local.float(),
                                         w2_local.float())  # fmt: skip
    dist.all_reduce(part, group=g)
    return part[st.rank * T : (st.rank + 1) * T].to(tokens.dtype)


class _EPWorkspace:
    def __init__(self, st: ExpertParallelState, T: int, K: int, C: int, inter: int, device) -> None:
        from .symm import PeerWorkspace

        E, P = st.num_experts, st.world
        self.rows = -(-(P * T * K + st.local_experts * (ALIGN - 1)) // ALIGN) * ALIGN
        nbytes = 2 * self.rows * C * 2 + P * E * 4 + 4096
        self.ws = PeerWorkspace(st.group, nbytes, device)
        self.counts_all = self.ws.region("ep_counts", (P, E), torch.int32)
        self.x_recv = self.ws.region("ep_x", (self.rows, C), torch.bfloat16)
        self.y_recv = self.ws.region("ep_y", (self.rows, C), torch.bfloat16)
        i32 = dict(device=device, dtype=torch.int32)
        self.dst_base = torch.empty(E, **i32)
        self.tile_expert = torch.empty(self.rows // ALIGN, **i32)
        self.cursor = torch.zeros(E, **i32)
        self.row_map = torch.empty(T * K, **i32)
        self.h13 = torch.empty(self.rows, 2 * inter, device=device, dtype=torch.bfloat16)
        self.h = torch.empty(self.rows, inter, device=device, dtype=torch.bfloat16)
        self.recv_table = self.ws.peer_table("ep_x")
        self.y_table = self.ws.peer_table("ep_y")
        self.count_table = self.ws.peer_table("ep_counts")


_EP_WS: dict = {}


def experts_forward_ep(tokens, indices, weights, w13_local, w2_local, st: ExpertParallelState, residual=None):
    """tokens [T, C] (same T on every rank); indices / weights [T, K] over GLOBAL expert ids."""
    T, C = tokens.shape
    K = indices.shape[1]
    inter = w13_local.shape[1] // 2
    if not (tokens.is_cuda and tokens.dtype == torch.bfloat16 and C % 64 == 0 and inter % 64 == 0):
        out = _reference_ep(tokens, indices, weights, w13_local, w2_local, st)
        return out if residual is None else (out.float() + residual.float()).to(tokens.dtype)
    key = (id(st.group), T, K, C, inter)
    w = _EP_WS.get(key)
    if w is None:
        w = _EP_WS[key] = _EPWorkspace(st, T, K, C, inter, tokens.device)
    lib, sp = native.load(), native.stream_ptr()
    E, P, r = st.num_experts, st.world, st.rank
    ids = indices.to(torch.int32).contiguous()
    wts = weights.float().contiguous()
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    native.check(lib.tfb_peer_push_rows(counts.data_ptr(), E * 4, w.count_table, P, r, 1, E * 4, E * 4, sp),
                 "tfb_peer_push_rows")  # fmt: skip
    w.ws.barrier()
    native.check(lib.tfb_moe_ep_plan(w.counts_all.data_ptr(), P, E, r, ALIGN, w.dst_base.data_ptr(),
                                     w.tile_expert.data_ptr(), w.rows // ALIGN, sp), "tfb_moe_ep_plan")  # fmt: skip
    xc = tokens.contiguous()
    native.check(lib.tfb_moe_ep_dispatch(xc.data_ptr(), C, ids.data_ptr(), w.dst_base.data_ptr(), w.cursor.data_ptr(),
                                         E, P, T, K, w.recv_table, w.row_map.data_ptr(), sp), "tfb_moe_ep_dispatch")  # fmt: skip
    w.ws.barrier()
    El = st.local_experts
    native.check(lib.tfb_gemm_bf16_grouped(w.x_recv.data_ptr(), C, w13_local.data_ptr(), C, w.h13.data_ptr(), 2 * inter,
                                           w.rows, 2 * inter, C, El, w.tile_expert.data_ptr(), 0, sp),
                 "tfb_gemm_bf16_grouped")  # fmt: skip
    native.check(lib.tfb_act_mul(w.h13.data_ptr(), w.h.data_ptr(), w.rows, inter, 0, sp), "tfb_act_mul")
    native.check(lib.tfb_gemm_bf16_grouped(w.h.data_ptr(), inter, w2_local.data_ptr(), inter, w.y_recv.data_ptr(), C,
                                           w.rows, C, inter, El, w.tile_expert.data_ptr(), 0, sp),
                 "tfb_gemm_bf16_grouped")  # fmt: skip
    w.ws.barrier()
    out = torch.empty_like(xc)
    res = None if residual is None else residual.contiguous()
    native.check(lib.tfb_moe_ep_combine(w.y_table, P, C, w.row_map.data_ptr(), wts.data_ptr(), T, K, native.ptr(res),
                                        out.data_ptr(), sp), "tfb_moe_ep_combine")  # fmt: skip
    return out


def release() -> None:
    for w in _EP_WS.values():
        w.ws.close()
    _EP_WS.clear()
