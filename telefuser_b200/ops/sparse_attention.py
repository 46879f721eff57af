"""Block-sparse attention and the builders of its block masks.

Kernel: the dense tcgen05 attention pipeline where every CTA (256 query rows of one head) visits only
the 128-key blocks listed for it. Masks are therefore `[.., ceil(Sq/256), ceil(Skv/128)]` booleans;
`lists_from_mask` turns one into the (index list, count) pair the kernel reads.
Builders:
* `radial_block_mask`: log-sparse spatio-temporal pattern for video tokens laid out frame by frame
  (+ trailing text tokens): frames at temporal distance d keep a diagonal band whose width halves each
  time d doubles, and below a width of 128 only every k-th frame pair is kept; the first frame (attention
  sink) and the text rows / columns stay dense. Block decisions are made from column densities computed
  in closed form (no token-level mask is materialised).
* `topk_block_mask`: data-dependent selection (mean-pooled q.k block scores, top-k key blocks per query
  group), the gating used by block-sparse refiners and by local / draft attention.
* `local_window_block_mask`: 3-D window locality for a (T, H, W) token grid.
Role parity: telefuser/ops/attention/sparse_patterns.py:74-270,480-615, bsa.py:101-196,
local_sparse_attn.py:31-76,129-236.
"""

from __future__ import annotations

import math

import torch

from . import native
from .functional import _native

BQ, BK = 256, 128


# ---------------------------------------------------------------------------
# kernel wrapper
# ---------------------------------------------------------------------------
def lists_from_mask(mask: torch.Tensor):
    """bool [..., nQ, nK] -> (int32 idx [..., nQ, max_blocks], int32 cnt [..., nQ])."""
    m = mask.bool()
    cnt = m.sum(-1).to(torch.int32)
    mx = max(1, int(cnt.max().item()))
    order = torch.argsort((~m).to(torch.int8), dim=-1, stable=True)  # selected blocks first, ascending
    return order[..., :mx].to(torch.int32).contiguous(), cnt.contiguous()


def expand_mask_reference(mask: torch.Tensor, Sq: int, Skv: int) -> torch.Tensor:
    """Block mask [..., nQ, nK] -> token mask [..., Sq, Skv]."""
    return mask.repeat_interleave(BQ, -2)[..., :Sq, :].repeat_interleave(BK, -1)[..., :Skv]


def block_sparse_attention_reference(q, k, v, mask, scale=None):
    B, Sq, H, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    tok = expand_mask_reference(_broadcast_mask(mask, B, H), Sq, k.shape[1])
    s = (q.float().permute(0, 2, 1, 3) @ k.float().permute(0, 2, 3, 1)) * scale
    s = s.masked_fill(~tok, float("-inf"))
    p = torch.softmax(s, dim=-1).nan_to_num(0.0)  # rows without any block: zeros
    return (p @ v.float().permute(0, 2, 1, 3)).permute(0, 2, 1, 3).to(q.dtype)


def _broadcast_mask(mask, B, H):
    m = mask
    while m.dim() < 4:
        m = m.unsqueeze(0)
    return m.expand(B, H, *m.shape[-2:])


def block_sparse_attention(q, k, v, mask=None, lists=None, scale=None):
    """q [B, Sq, H, 128], k/v [B, Skv, H, 128] bf16; mask bool [nQ, nK] / [H, nQ, nK] / [B, H, nQ, nK]
    (nQ = ceil(Sq/256), nK = ceil(Skv/128)) or precomputed `lists = (idx, cnt)` of shape [B, H, nQ, *]."""
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    if not _native(q) or q.dtype != torch.bfloat16 or D != 128:
        if mask is None:
            raise ValueError("the reference path needs the block mask")
        return block_sparse_attention_reference(q, k, v, mask, scale)
    if lists is None:
        lists = lists_from_mask(_broadcast_mask(mask, B, H).to(q.device))
    idx, cnt = lists
    nQ = (Sq + BQ - 1) // BQ
    if idx.shape[:3] != (B, H, nQ) or cnt.shape != (B, H, nQ):
        raise ValueError(f"block lists must have shape [{B}, {H}, {nQ}, *]")
    scale = scale if scale is not None else 1.0 / math.sqrt(D)

    def prep(t):
        S = t.shape[1]
        if t.stride(-1) != 1 or t.stride(2) != D or (B > 1 and t.stride(0) % 8) or t.stride(1) % 8:
            t = t.contiguous()
        return t, t.stride(1), (t.stride(0) if B > 1 else S * t.stride(1))

    (q, ldq, bsq), (k, ldk, bsk), (v, ldv, bsv) = prep(q), prep(k), prep(v)
    out = torch.empty(B, Sq, H, D, device=q.device, dtype=torch.bfloat16)
    idx, cnt = idx.contiguous(), cnt.contiguous()
    code = native.load().tfb_attn_fwd_sparse(q.data_ptr(), ldq, bsq, k.data_ptr(), ldk, bsk, v.data_ptr(), ldv, bsv,
                                             out.data_ptr(), H * D, Sq * H * D, None, B, H, Sq, Skv, scale,
                                             idx.data_ptr(), cnt.data_ptr(), idx.shape[-1], 0, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_attn_fwd_sparse")
    return out


# ---------------------------------------------------------------------------
# mask builders
# ---------------------------------------------------------------------------
def _window_width(dist: int, tokens_per_frame: int, decay_factor: float, block: int) -> float:
    if dist <= 1:
        return float(tokens_per_frame)
    group = dist.bit_length()
    return max(2 ** tokens_per_frame.bit_length() / 2**group * decay_factor, float(block))


def _pair_kept(dist: int, tokens_per_frame: int) -> bool:
    group = dist.bit_length()
    decay = 2 ** tokens_per_frame.bit_length() / 2**group
    if decay >= 128:
        return True
    return dist % int(128 / decay) == 0


def radial_block_mask_128(seq_len: int, video_tokens: int, num_frames: int, decay_factor: float = 0.5,
                          model_type: str = "wan", block: int = 128) -> torch.Tensor:  # fmt: skip
    """bool [seq_len // 128, seq_len // 128] at 128 x 128 granularity (the published pattern)."""
    nb = seq_len // block
    final = torch.zeros(nb, nb, dtype=torch.bool)
    tpf = video_tokens // num_frames
    vb = video_tokens // block
    final[vb:] = True
    final[:, vb:] = True
    rows = torch.arange(tpf)
    n_rb = n_cb = (tpf - 1) // block + 1  # the published pattern keeps ceil(tpf / 128) blocks per frame pair
    for i in range(num_frames):
        r_off = (i * tpf) % block
        # token row range of every row block, clipped to the frame
        r0 = (torch.arange(n_rb) * block - r_off).clamp(0, tpf)
        r1 = ((torch.arange(n_rb) + 1) * block - r_off).clamp(0, tpf)  # exclusive
        for j in range(num_frames):
            dist = abs(i - j)
            if j == 0 and model_type == "wan":
                w = float("inf")
            else:
                # A dropped frame pair still contributes its first and last row block (the published
                # pattern marks them unconditionally), so it is evaluated with an empty band.
                w = _window_width(dist, tpf, decay_factor, block) if _pair_kept(dist, tpf) else -1.0
            c_off = (j * tpf) % block
            # rows r of block R with |c - r| <= w: overlap of [c - w, c + w] with [r0, r1)
            lo = torch.maximum(torch.ceil(rows - w).clamp_min(0)[None, :], r0[:, None].float())
            hi = torch.minimum((torch.floor(rows + w) + 1).clamp_max(tpf)[None, :], r1[:, None].float())
            dens = (hi - lo).clamp_min(0) / block  # [n_rb, tpf] column densities per row block
            pad = torch.zeros(n_rb, c_off + tpf + block)
            pad[:, c_off : c_off + tpf] = dens
            dens = pad[:, : n_cb * block].reshape(n_rb, n_cb, block)
            nonzero = (dens > 0).sum(-1)
            high = (dens > 1 / 3).sum(-1)
            bm = high / (nonzero + 1e-9) > 0.6
            bm[0] = True
            bm[-1] = True
            rs, cs = (i * tpf) // block, (j * tpf) // block
            re, ce = min(nb, rs + n_rb), min(nb, cs + n_cb)
            final[rs:re, cs:ce] |= bm[: re - rs, : ce - cs]
    return final


def to_kernel_granularity(mask128: torch.Tensor, Sq: int, Skv: int) -> torch.Tensor:
    """[.., Sq/128, Skv/128] (floor) -> [.., ceil(Sq/256), ceil(Skv/128)]; ragged tail blocks are kept dense."""
    nQ, nK = (Sq + BQ - 1) // BQ, (Skv + BK - 1) // BK
    full = torch.ones(*mask128.shape[:-2], 2 * nQ, nK, dtype=torch.bool, device=mask128.device)
    r, c = min(mask128.shape[-2], 2 * nQ), min(mask128.shape[-1], nK)
    full[..., :r, :c] = mask128[..., :r, :c]
    return full.view(*mask128.shape[:-2], nQ, 2, nK).any(-2)


class RadialMaskMap:
    """Cache of radial block masks per (sequence length, decay factor)."""

    def __init__(self, video_token_num: int, num_frame: int, model_type: str = "wan") -> None:
        self.video_token_num, self.num_frame, self.model_type = video_token_num, num_frame, model_type
        self._cache: dict = {}

    def query_block_mask(self, seq_len: int, decay_factor: float = 0.5, device="cpu"):
        key = (seq_len, decay_factor)
        hit = self._cache.get(key)
        if hit is None:
            m128 = radial_block_mask_128(seq_len, self.video_token_num, self.num_frame, decay_factor, self.model_type)
            mask = to_kernel_granularity(m128, seq_len, seq_len)
            hit = self._cache[key] = (mask, 1.0 - mask.float().mean().item())
        return hit[0].to(device)

    def sparsity(self, seq_len: int, decay_factor: float = 0.5) -> float:
        self.query_block_mask(seq_len, decay_factor)
        return self._cache[(seq_len, decay_factor)][1]

    def clear(self) -> None:
        self._cache.clear()


def radial_attention(q, k, v, mask_map: RadialMaskMap, decay_factor: float = 0.5, dense: bool = False, scale=None):
    """Radial sparse attention for [B, S, H, D] video(+text) tokens; `dense=True` (warm-up layers / steps) runs
    full attention."""
    from .functional import attention

    if dense:
        return attention(q, k, v, scale)
    mask = mask_map.query_block_mask(q.shape[1], decay_factor, q.device)
    key = ("lists", q.shape[0], q.shape[2], q.shape[1], decay_factor, str(q.device))
    lists = mask_map._cache.get(key)
    if lists is None and q.is_cuda:
        lists = mask_map._cache[key] = lists_from_mask(_broadcast_mask(mask, q.shape[0], q.shape[2]))
    return block_sparse_attention(q, k, v, mask, lists, scale)


def mean_pool_blocks(x: torch.Tensor, block: int) -> torch.Tensor:
    """[B, S, H, D] -> [B, ceil(S/block), H, D] mean over each block (the ragged tail averages what it has)."""
    B, S, H, D = x.shape
    n = (S + block - 1) // block
    pad = n * block - S
    xf = torch.nn.functional.pad(x.float(), (0, 0, 0, 0, 0, pad)).view(B, n, block, H, D)
    cnt = torch.full((n,), float(block), device=x.device)
    if pad:
        cnt[-1] = block - pad
    return xf.sum(2) / cnt.view(1, n, 1, 1)


def topk_block_mask(q, k, sparsity: float = 0.9, keep_first: int = 1, keep_diagonal: bool = True,
                    min_blocks: int = 1) -> torch.Tensor:  # fmt: skip
    """bool [B, H, nQ, nK]: per 256-row query group the key blocks with the largest pooled q.k scores;
    `sparsity` = fraction of key blocks dropped."""
    qc, kc = mean_pool_blocks(q, BQ), mean_pool_blocks(k, BK)
    score = torch.einsum("bqhd,bkhd->bhqk", qc, kc)
    nK = score.shape[-1]
    keep = max(min_blocks, min(nK, int(round(nK * (1.0 - sparsity)))))
    mask = torch.zeros_like(score, dtype=torch.bool).scatter_(-1, score.topk(keep, dim=-1).indices, True)
    if keep_first:
        mask[..., :keep_first] = True
    if keep_diagonal:
        nQ = score.shape[-2]
        qi = torch.arange(nQ, device=q.device)
        for d in (0, 1):
            kb = (qi * 2 + d).clamp_max(nK - 1)
            mask[..., qi, kb] = True
    return mask


def local_window_block_mask(grid: tuple[int, int, int], window: tuple[int, int, int]) -> torch.Tensor:
    """bool [nQ, nK] for tokens in (T, H, W) raster order: a query group attends to every key block that
    holds a token within +-window of one of its tokens along each axis."""
    T, H, W = grid
    wt, wh, ww = window
    n = T * H * W
    idx = torch.arange(n)
    t, h, w = idx // (H * W), (idx // W) % H, idx % W
    nQ, nK = (n + BQ - 1) // BQ, (n + BK - 1) // BK

    def span(coord, size, blk):
        nb = (n + blk - 1) // blk
        pad = nb * blk - n
        c = torch.nn.functional.pad(coord, (0, pad), value=-1).view(nb, blk)
        lo = torch.where(c >= 0, c, torch.full_like(c, size)).min(1).values
        return lo, c.max(1).values

    mask = torch.ones(nQ, nK, dtype=torch.bool)
    for coord, size, win in ((t, T, wt), (h, H, wh), (w, W, ww)):
        qlo, qhi = span(coord, size, BQ)
        klo, khi = span(coord, size, BK)
        mask &= (klo[None, :] <= qhi[:, None] + win) & (khi[None, :] >= qlo[:, None] - win)
    return mask


# ---------------------------------------------------------------------------
# 3-D chunked top-k block-sparse attention (LongCat-Video refinement)
# ---------------------------------------------------------------------------
def to_3d_blocks(x: torch.Tensor, grid, chunk) -> torch.Tensor:
    """[B, T*H*W, heads, D] in grid order -> the same tokens ordered chunk by chunk (chunks of t x h x w tokens)."""
    B, _, Hh, D = x.shape
    (T, H, W), (t, h, w) = grid, chunk
    x = x.view(B, T // t, t, H // h, h, W // w, w, Hh, D).permute(0, 1, 3, 5, 2, 4, 6, 7, 8)
    return x.reshape(B, T * H * W, Hh, D)


def from_3d_blocks(x: torch.Tensor, grid, chunk) -> torch.Tensor:
    B, _, Hh, D = x.shape
    (T, H, W), (t, h, w) = grid, chunk
    x = x.view(B, T // t, H // h, W // w, t, h, w, Hh, D).permute(0, 1, 4, 2, 5, 3, 6, 7, 8)
    return x.reshape(B, T * H * W, Hh, D)


def bsa_3d_attention(q, k, v, latent_shape_q, latent_shape_k=None, sparsity: float = 0.9375, chunk_3d_shape_q=(4, 4, 4),
                     chunk_3d_shape_k=(4, 4, 4)):  # fmt: skip
    """q, k, v: [B, S, H, D] in (T, H, W) order. Tokens are regrouped into 3-D chunks; every query chunk keeps the
    `(1 - sparsity)` fraction of key chunks with the largest mean-pooled q.k score. On GPUs with chunks of 64 or
    128 tokens the kernel's 256 x 128 blocks receive the union of the masks of the chunks they contain."""
    latent_shape_k = latent_shape_k or latent_shape_q
    cq, ck = math.prod(chunk_3d_shape_q), math.prod(chunk_3d_shape_k)
    qb, kb, vb = to_3d_blocks(q, latent_shape_q, chunk_3d_shape_q), to_3d_blocks(k, latent_shape_k, chunk_3d_shape_k), \
        to_3d_blocks(v, latent_shape_k, chunk_3d_shape_k)  # fmt: skip
    qm = mean_pool_blocks(qb, cq).float().permute(0, 2, 1, 3)  # [B, H, nQ, D]
    km = mean_pool_blocks(kb, ck).float().permute(0, 2, 1, 3)
    score = qm @ km.transpose(-1, -2)
    keep = max(1, int((1 - sparsity) * score.shape[-1]))
    mask = torch.zeros_like(score, dtype=torch.bool).scatter_(3, torch.topk(score, keep, dim=-1).indices, True)
    if _native(q) and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and BQ % cq == 0 and BK % ck == 0 \
            and q.shape[1] % BQ == 0 and k.shape[1] % BK == 0:  # fmt: skip
        m = mask.view(*mask.shape[:2], mask.shape[2] // (BQ // cq), BQ // cq, mask.shape[3] // (BK // ck), BK // ck)
        out = block_sparse_attention(qb, kb, vb, m.any(dim=(3, 5)))
    else:
        tok = mask.repeat_interleave(cq, dim=2).repeat_interleave(ck, dim=3)
        s = (qb.float().permute(0, 2, 1, 3) @ kb.float().permute(0, 2, 3, 1)) / math.sqrt(q.shape[-1])
        p = torch.softmax(s.masked_fill(~tok, float("-inf")), dim=-1)
        out = (p @ vb.float().permute(0, 2, 1, 3)).permute(0, 2, 1, 3).to(q.dtype)
    return from_3d_blocks(out, latent_shape_q, chunk_3d_shape_q)
