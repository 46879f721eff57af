"""Windowed top-k block-sparse attention with a temporal KV cache (FlashVSR).

Tokens of a [F, H, W] grid are regrouped into 3-D windows (2 x 8 x 8 = 128 tokens), so that one window is one
key block of the block-sparse attention kernel. A query window may attend to the windows inside a
`local_range` x `local_range` neighbourhood (in window units) of every temporal window group, cached groups
included; among those, a draft attention map over mean-pooled windows picks, per head and per temporal query
group, the `topk` strongest (query window, key window) pairs. The kernel works on pairs of adjacent query
windows (256 rows) and gives each pair the union of its two masks, i.e. it never drops a selected block; the
CPU path evaluates the 128-row masks exactly. Keys and values of the last `kv_len` temporal groups are
returned in window layout as the cache for the next clip.
Role parity: telefuser/ops/attention/local_sparse_attn.py:30-547.
"""

from __future__ import annotations

import math

import torch

from telefuser_b200.ops import sparse_attention as SA

_LOCAL_MASKS: dict = {}


def window_partition(x: torch.Tensor, win) -> torch.Tensor:
    """[B, F, H, W, C] -> [B * windows, wf*wh*ww, C], windows ordered (frame group, row, column)."""
    B, F, H, W, C = x.shape
    wf, wh, ww = win
    if F % wf or H % wh or W % ww:
        raise ValueError(f"grid ({F},{H},{W}) is not divisible by the window ({wf},{wh},{ww})")
    x = x.view(B, F // wf, wf, H // wh, wh, W // ww, ww, C).permute(0, 1, 3, 5, 2, 4, 6, 7)
    return x.reshape(-1, wf * wh * ww, C)


def window_reverse(windows: torch.Tensor, win, orig) -> torch.Tensor:
    F, H, W = orig
    wf, wh, ww = win
    nf, nh, nw = F // wf, H // wh, W // ww
    B = windows.shape[0] // (nf * nh * nw)
    x = windows.view(B, nf, nh, nw, wf, wh, ww, -1).permute(0, 1, 4, 2, 5, 3, 6, 7)
    return x.reshape(B, F, H, W, -1)


def build_local_block_mask(block_h: int, block_w: int, win_h: int = 6, win_w: int = 6, include_self: bool = True,
                           device=None) -> torch.Tensor:  # fmt: skip
    """[bh*bw, bh*bw] bool: window j lies in the win_h x win_w neighbourhood centred (floor) on window i."""
    r = torch.arange(block_h, device=device).repeat_interleave(block_w)
    c = torch.arange(block_w, device=device).repeat(block_h)
    dr = r[None, :] - (r[:, None] - win_h // 2)
    dc = c[None, :] - (c[:, None] - win_w // 2)
    mask = (dr >= 0) & (dr <= win_h - 1) & (dc >= 0) & (dc <= win_w - 1)
    if not include_self:
        mask.fill_diagonal_(False)
    return mask


@torch.no_grad()
def draft_block_mask(q_w, k_w, nheads: int, n_groups: int, topk: int, local_mask: torch.Tensor) -> torch.Tensor:
    """q_w [nQ, 128, C], k_w [nK, 128, C] (window layout) -> [1, heads, nQ, nK] bool."""
    nQ, nK = q_w.shape[0], k_w.shape[0]
    D = q_w.shape[-1] // nheads
    qm = q_w.float().mean(dim=1).view(nQ, nheads, D).permute(1, 0, 2)
    km = k_w.float().mean(dim=1).view(nK, nheads, D).permute(1, 0, 2)
    scores = torch.einsum("hld,hmd->hlm", qm, km) / math.sqrt(D)
    per = local_mask.shape[0]
    allowed = local_mask.to(scores.device).repeat(nQ // per, nK // per)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    amap = torch.softmax(scores, dim=-1).view(nheads * n_groups, -1)  # one row per (head, temporal query group)
    k = min(amap.shape[1] - 1, topk)
    if k <= 0:
        return torch.zeros(1, nheads, nQ, nK, dtype=torch.bool, device=scores.device)
    thresh = torch.topk(amap, k=k + 1, dim=1).values[:, -1:]
    return (amap > thresh).view(1, nheads, nQ, nK)


def local_sparse_attention(q, k, v, B: int, f: int, h: int, w: int, D: int, topk: int, local_range: int, num_heads: int,
                           kv_len: int, pre_cache_k=None, pre_cache_v=None, win=(2, 8, 8)):  # fmt: skip
    """q, k, v: [B, f*h*w, D] (D = heads * head_dim) in grid order -> (out [B, f*h*w, D], cache_k, cache_v)."""
    if B != 1:
        raise ValueError("local sparse attention runs one clip at a time")
    q_w, k_w, v_w = (window_partition(t.view(B, f, h, w, D), win) for t in (q, k, v))
    n_groups = f // win[0]
    per_group = k_w.shape[0] // n_groups
    if pre_cache_k is not None and pre_cache_v is not None:
        k_w = torch.cat([pre_cache_k.to(k_w.device), k_w], dim=0)
        v_w = torch.cat([pre_cache_v.to(v_w.device), v_w], dim=0)
    key = (h // win[1], w // win[2], local_range)
    if key not in _LOCAL_MASKS:
        _LOCAL_MASKS[key] = build_local_block_mask(key[0], key[1], local_range, local_range, include_self=True)
    mask = draft_block_mask(q_w, k_w, num_heads, n_groups, topk, _LOCAL_MASKS[key])
    hd = D // num_heads
    q4 = q_w.reshape(1, -1, num_heads, hd)
    k4 = k_w.reshape(1, -1, num_heads, hd)
    v4 = v_w.reshape(1, -1, num_heads, hd)
    block = q_w.shape[1]
    if q.is_cuda and block == 128 and hd == 128 and q.dtype == torch.bfloat16:
        out = SA.block_sparse_attention(q4, k4, v4, SA.to_kernel_granularity(mask, q4.shape[1], k4.shape[1]))
    else:
        out = _masked_reference(q4, k4, v4, mask, block)
    out = window_reverse(out.reshape(q_w.shape[0], block, D), win, (f, h, w)).reshape(B, f * h * w, D)
    if k_w.shape[0] // per_group > kv_len:
        k_w, v_w = k_w[per_group:], v_w[per_group:]
    return out, k_w, v_w


def _masked_reference(q, k, v, mask, block: int):
    """Exact evaluation of a [1, H, nQ, nK] block mask with `block`-row query and key blocks."""
    full = mask.repeat_interleave(block, dim=2).repeat_interleave(block, dim=3)[:, :, : q.shape[1], : k.shape[1]]
    qh, kh, vh = (t.permute(0, 2, 1, 3).float() for t in (q, k, v))
    s = (qh @ kh.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~full, float("-inf"))
    p = torch.softmax(s, dim=-1).nan_to_num(0.0)
    return (p @ vh).permute(0, 2, 1, 3).to(q.dtype)
