"""Mixture-of-experts ops: router and routed expert FFN.

CUDA path (no host synchronisation, fixed launch sequence, CUDA-graph friendly):
route kernel (scores, group-limited top-k, weights, histogram) -> plan kernel (128-row-aligned
expert segments + per-tile expert table) -> permute kernel -> grouped tcgen05 GEMM (gate|up) ->
SiLU-mul -> grouped GEMM (down) -> weighted combine in fp32. Buffers are sized for the worst case
`T*K + E*127` rows, so nothing depends on the routing outcome on the host.
CPU path: plain PyTorch with the same semantics (the numerics oracle).
Role parity: telefuser/ops/moe.py:9-133 (`route_topk`, `grouped_expert_forward`); the W8A8 expert path
(`quantize_expert_weight_fp8`, `experts_forward_fp8`) is at the end of this file.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native
from .functional import _native, act_mul

ALIGN = 128  # rows; the grouped GEMM's M tile


def route_topk_reference(logits, num_expert_groups=1, top_k_groups=None, top_k=1, correction_bias=None,
                         routing_scale=1.0, use_softmax=False):  # fmt: skip
    T, E = logits.shape
    per_group = E // num_expert_groups
    top_k_groups = num_expert_groups if top_k_groups is None else top_k_groups
    scores = logits.float().softmax(-1) if use_softmax else logits.float().sigmoid()
    sel = scores if correction_bias is None else scores + correction_bias.float().reshape(1, -1)
    if top_k_groups < num_expert_groups:
        grouped = sel.reshape(T, num_expert_groups, per_group)
        gv = grouped.topk(min(2, per_group), dim=-1).values.sum(-1)
        keep = torch.zeros_like(gv, dtype=torch.bool).scatter_(1, gv.topk(top_k_groups, dim=-1).indices, True)
        sel = sel.masked_fill(~keep.unsqueeze(-1).expand(T, num_expert_groups, per_group).reshape(T, E), float("-inf"))
    idx = sel.topk(top_k, dim=-1).indices
    w = scores.gather(-1, idx)
    w = w / w.sum(-1, keepdim=True).clamp_min(torch.finfo(w.dtype).eps)
    return idx, w * routing_scale


def route_topk(logits, num_expert_groups=1, top_k_groups=None, top_k=1, correction_bias=None, routing_scale=1.0,
               use_softmax=False, return_counts=False):  # fmt: skip
    """logits [T, E] -> (indices int [T, K], weights fp32 [T, K]) (+ counts int32 [E] on request)."""
    if logits.ndim != 2:
        raise ValueError("router logits must have shape [tokens, experts]")
    T, E = logits.shape
    if not 1 <= top_k <= E or E % num_expert_groups:
        raise ValueError("invalid top_k / expert grouping")
    top_k_groups = num_expert_groups if top_k_groups is None else top_k_groups
    if not 1 <= top_k_groups <= num_expert_groups:
        raise ValueError("top_k_groups must be within the number of groups")
    if not _native(logits) or E > 1024 or top_k > 32 or num_expert_groups > 32:
        idx, w = route_topk_reference(logits, num_expert_groups, top_k_groups, top_k, correction_bias, routing_scale,
                                      use_softmax)  # fmt: skip
        if return_counts:
            return idx, w, torch.bincount(idx.reshape(-1), minlength=E).to(torch.int32)
        return idx, w
    lg = logits.float().contiguous()
    bias = None if correction_bias is None else correction_bias.float().contiguous()
    ids = torch.empty(T, top_k, device=lg.device, dtype=torch.int32)
    w = torch.empty(T, top_k, device=lg.device, dtype=torch.float32)
    counts = torch.empty(E, device=lg.device, dtype=torch.int32)
    code = native.load().tfb_moe_route(lg.data_ptr(), native.ptr(bias), T, E, num_expert_groups, top_k_groups, top_k,
                                       float(routing_scale), int(use_softmax), ids.data_ptr(), w.data_ptr(),
                                       counts.data_ptr(), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_moe_route")
    return (ids, w, counts) if return_counts else (ids, w)


def experts_forward_reference(x, indices, weights, w13, w2):
    """x [T, C]; w13 [E, 2I, C] (gate rows then up rows); w2 [E, C, I] -> [T, C] (fp32 route reduction)."""
    T, C = x.shape
    out = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    inter = w13.shape[1] // 2
    for e in range(w13.shape[0]):
        tok, slot = (indices == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = F.linear(x[tok], w13[e])
        h = F.silu(h[:, :inter]) * h[:, inter:]
        y = F.linear(h.to(x.dtype), w2[e])
        out.index_add_(0, tok, y.float() * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


class MoEWorkspace:
    """Worst-case sized buffers for one (T, K, E, hidden, inter) shape; reused across calls."""

    def __init__(self, T: int, K: int, E: int, hidden: int, inter: int, device, dtype=torch.bfloat16) -> None:
        self.key = (T, K, E, hidden, inter)
        rows = -(-(T * K + E * (ALIGN - 1)) // ALIGN) * ALIGN
        self.rows = rows
        i32 = dict(device=device, dtype=torch.int32)
        self.offsets = torch.empty(E + 1, **i32)
        self.tile_expert = torch.empty(rows // ALIGN, **i32)
        self.cursor = torch.zeros(E, **i32)
        self.row_map = torch.empty(T * K, **i32)
        self.x_perm = torch.zeros(rows, hidden, device=device, dtype=dtype)
        self.h13 = torch.empty(rows, 2 * inter, device=device, dtype=dtype)
        self.h = torch.empty(rows, inter, device=device, dtype=dtype)
        self.y = torch.empty(rows, hidden, device=device, dtype=dtype)


_WORKSPACES: dict = {}


def experts_forward(x, indices, weights, w13, w2, counts=None, residual=None, workspace: MoEWorkspace | None = None):
    """Routed expert FFN: sum_k weights[t,k] * W2[e](silu(W1[e] x) * W3[e] x) (+ residual)."""
    T, C = x.shape
    E, two_i, _ = w13.shape
    inter = two_i // 2
    K = indices.shape[1]
    ok = (_native(x) and x.dtype == torch.bfloat16 and w13.dtype == torch.bfloat16 and C % 64 == 0 and inter % 64 == 0
          and w13.is_contiguous() and w2.is_contiguous())  # fmt: skip
    if not ok:
        out = experts_forward_reference(x, indices.long(), weights, w13, w2)
        return out if residual is None else (out.float() + residual.float()).to(x.dtype)
    lib = native.load()
    st = native.stream_ptr()
    ws = workspace
    if ws is None:
        key = (T, K, E, C, inter, x.device.index)
        ws = _WORKSPACES.get(key)
        if ws is None:
            ws = _WORKSPACES[key] = MoEWorkspace(T, K, E, C, inter, x.device)
    ids = indices.to(torch.int32).contiguous()
    wts = weights.float().contiguous()
    if counts is None:
        counts = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    xc = x.contiguous()
    native.check(lib.tfb_moe_plan(counts.data_ptr(), E, ALIGN, ws.offsets.data_ptr(), ws.tile_expert.data_ptr(),
                                  ws.rows // ALIGN, st), "tfb_moe_plan")  # fmt: skip
    native.check(lib.tfb_moe_permute(xc.data_ptr(), C, ids.data_ptr(), ws.offsets.data_ptr(), ws.cursor.data_ptr(), E,
                                     T, K, ws.x_perm.data_ptr(), ws.row_map.data_ptr(), st), "tfb_moe_permute")  # fmt: skip
    native.check(lib.tfb_gemm_bf16_grouped(ws.x_perm.data_ptr(), C, w13.data_ptr(), C, ws.h13.data_ptr(), 2 * inter,
                                           ws.rows, 2 * inter, C, E, ws.tile_expert.data_ptr(), 0, st),
                 "tfb_gemm_bf16_grouped")  # fmt: skip
    # gate rows come first in w13, so h13 = [gate | up] per row
    code = lib.tfb_act_mul(ws.h13.data_ptr(), ws.h.data_ptr(), ws.rows, inter, 0, st)
    native.check(code, "tfb_act_mul")
    native.check(lib.tfb_gemm_bf16_grouped(ws.h.data_ptr(), inter, w2.data_ptr(), inter, ws.y.data_ptr(), C, ws.rows,
                                           C, inter, E, ws.tile_expert.data_ptr(), 0, st), "tfb_gemm_bf16_grouped")  # fmt: skip
    out = torch.empty_like(xc)
    res = None if residual is None else residual.contiguous()
    native.check(lib.tfb_moe_combine(ws.y.data_ptr(), C, ws.row_map.data_ptr(), wts.data_ptr(), T, K, native.ptr(res),
                                     out.data_ptr(), st), "tfb_moe_combine")  # fmt: skip
    return out


def quantize_expert_weight_fp8(weight: torch.Tensor):
    """Stacked expert weights [E, out, in] -> (e4m3 [E, out, in], fp32 scale [E, out]) with one scale per output
    channel of each expert (amax / 448). Role parity: telefuser/ops/moe.py:136-146."""
    if weight.ndim != 3:
        raise ValueError(f"expert weights are stacked as [experts, out_features, in_features], got {tuple(weight.shape)}")
    w = weight.float()
    scale = (w.abs().amax(dim=2) / 448.0).clamp_min(1e-12)
    return (w / scale.unsqueeze(2)).clamp(-448, 448).to(torch.float8_e4m3fn), scale


def experts_forward_fp8_reference(x, indices, weights, w13, w13_scale, w2, w2_scale):
    """The W8A8 expert FFN spelled out per expert: rows quantised per token before each GEMM, e4m3 weights with
    per-channel scales, fp32 accumulation and fp32 route reduction."""
    from .functional import linear_fp8

    T, C = x.shape
    out = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    for e in range(w13.shape[0]):
        tok, slot = (indices == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = act_mul(linear_fp8(x[tok], w13[e], w13_scale[e]), "silu")
        y = linear_fp8(h, w2[e], w2_scale[e])
        out.index_add_(0, tok, y.float() * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


def experts_forward_fp8(x, indices, weights, w13, w13_scale, w2, w2_scale, counts=None, residual=None,
                        workspace: MoEWorkspace | None = None):  # fmt: skip
    """Routed expert FFN on e4m3 weights (`quantize_expert_weight_fp8`): w13 [E, 2I, C] gate rows then up rows with
    scale [E, 2I]; w2 [E, C, I] with scale [E, C]. Activations are quantised per token in front of each GEMM.

    CUDA path: the plan / permute / combine kernels of the bf16 path around one W8A8 tensor-core GEMM pair per
    non-empty expert segment; the segment bounds are read back once per call (the per-expert launches need them on
    the host), so unlike the bf16 path this one is not capturable in a CUDA graph.
    Role parity: telefuser/ops/moe.py:148-206 (`fp8_expert_forward`)."""
    from .functional import linear_fp8

    if w13.dtype != torch.float8_e4m3fn or w2.dtype != torch.float8_e4m3fn:
        raise ValueError("expert weights must be quantised (quantize_expert_weight_fp8) before the FP8 forward")
    T, C = x.shape
    E, two_i, _ = w13.shape
    inter = two_i // 2
    K = indices.shape[1]
    ok = _native(x) and x.dtype == torch.bfloat16 and C % 64 == 0 and inter % 64 == 0
    if not ok:
        out = experts_forward_fp8_reference(x, indices.long(), weights, w13, w13_scale, w2, w2_scale)
        return out if residual is None else (out.float() + residual.float()).to(x.dtype)
    lib = native.load()
    st = native.stream_ptr()
    ws = workspace
    if ws is None:
        key = (T, K, E, C, inter, x.device.index)
        ws = _WORKSPACES.get(key)
        if ws is None:
            ws = _WORKSPACES[key] = MoEWorkspace(T, K, E, C, inter, x.device)
    ids = indices.to(torch.int32).contiguous()
    wts = weights.float().contiguous()
    if counts is None:
        counts = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    xc = x.contiguous()
    native.check(lib.tfb_moe_plan(counts.data_ptr(), E, ALIGN, ws.offsets.data_ptr(), ws.tile_expert.data_ptr(),
                                  ws.rows // ALIGN, st), "tfb_moe_plan")  # fmt: skip
    native.check(lib.tfb_moe_permute(xc.data_ptr(), C, ids.data_ptr(), ws.offsets.data_ptr(), ws.cursor.data_ptr(), E,
                                     T, K, ws.x_perm.data_ptr(), ws.row_map.data_ptr(), st), "tfb_moe_permute")  # fmt: skip
    bounds = ws.offsets.tolist()  # 128-row-aligned segment starts, one per expert, plus the end
    w13_scale, w2_scale = w13_scale.to(x.device, torch.float32), w2_scale.to(x.device, torch.float32)
    for e in range(E):
        lo, hi = bounds[e], bounds[e + 1]
        if hi <= lo:
            continue
        h = act_mul(linear_fp8(ws.x_perm[lo:hi], w13[e], w13_scale[e]), "silu")
        ws.y[lo:hi].copy_(linear_fp8(h, w2[e], w2_scale[e]))
    out = torch.empty_like(xc)
    res = None if residual is None else residual.contiguous()
    native.check(lib.tfb_moe_combine(ws.y.data_ptr(), C, ws.row_map.data_ptr(), wts.data_ptr(), T, K, native.ptr(res),
                                     out.data_ptr(), st), "tfb_moe_combine")  # fmt: skip
    return out


__all__ = ["route_topk", "route_topk_reference", "experts_forward", "experts_forward_reference", "MoEWorkspace",
           "act_mul", "quantize_expert_weight_fp8", "experts_forward_fp8", "experts_forward_fp8_reference"]  # fmt: skip
