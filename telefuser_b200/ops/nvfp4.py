"""NVFP4 storage format: e2m1 values with one e4m3 scale per 16 elements and one fp32 scale per tensor.

    x  ~=  e2m1_code * e4m3_block_scale / global_scale

`global_scale = 448 * 6 / amax(tensor)` puts the block scales in the range of e4m3, `block_scale =
e4m3(amax(block) * global_scale / 6)`, and each value is rounded to the nearest of the eight e2m1 magnitudes
{0, 0.5, 1, 1.5, 2, 3, 4, 6} (ties to the even code). Two codes share a byte (even element in the low nibble), 4.5
bits per weight. Scale factors can be kept row-major or in the 128 x 4 tile order that tensor-core GEMMs and the
usual FP4 checkpoints use (`swizzle_block_scales` / `unswizzle_block_scales`).

This module is the format itself and a weight-only linear on top of it: the quantiser, the exact de-quantiser, the
scale layouts, and `quantize_linear_nvfp4_` (the weight is expanded to bf16 into a scratch buffer shared by layers
of the same shape, then multiplied on the bf16 tensor-core GEMM, as the NF4 path does). Everything here is tensor
ops, identical on CPU and GPU. There is no FP4 tensor-core GEMM in the library: a 128 x 192 single-CTA tile would
need more shared-memory read bandwidth than an SM has and would run at the FP8 kernel's rate.
Role: the reference's `scaled_fp4_quant` and NVFP4 checkpoint layout (tf-kernel/tf_kernel/gemm.py:159,
tf-kernel/csrc/gemm/nvfp4_quant_kernels.cu); its FP4 GEMM (`cutlass_scaled_fp4_mm`) has no counterpart here.
"""

from __future__ import annotations

import fnmatch

import torch
from torch import nn

from telefuser_b200.ops import functional as TF

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# decision boundaries between neighbouring magnitudes and what a value exactly on a boundary rounds to (the even code)
_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
_TIE_TO_UPPER = torch.tensor([False, True, False, True, False, True, False])  # 0.25->0, 0.75->1, 1.25->1, 1.75->2, ...
BLOCK = 16
E2M1_MAX, E4M3_MAX = 6.0, 448.0


def e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (sign << 3 | magnitude index) of every element, round-to-nearest-even; saturates at 6."""
    mag = x.abs().float()
    b = _BOUNDS.to(x.device)
    idx = torch.bucketize(mag, b, right=False)  # a value on a boundary lands in the lower bin ...
    on = torch.isclose(mag.unsqueeze(-1), b, rtol=0, atol=0).float()  # ... unless that boundary's even code is the upper one
    up = (on * _TIE_TO_UPPER.to(x.device).float()).sum(-1) > 0
    idx = (idx + up.long()).clamp_max(7)
    return (idx | ((x < 0).long() << 3)).to(torch.uint8)


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor | float | None = None, swizzle: bool = False):
    """x [..., K] with K % 16 == 0 -> (packed uint8 [..., K / 2], block scales e4m3 [..., K / 16] or tiled, global scale
    fp32 [1]). A given `global_scale` (calibrated) is used as is."""
    K = x.shape[-1]
    if K % BLOCK:
        raise ValueError(f"the last dimension ({K}) must be a multiple of {BLOCK}")
    xf = x.detach().float()
    if global_scale is None:
        gs = (E4M3_MAX * E2M1_MAX) / xf.abs().amax().clamp_min(1e-30)
    else:
        gs = torch.as_tensor(global_scale, dtype=torch.float32, device=x.device).reshape(())
    blocks = xf.reshape(*x.shape[:-1], K // BLOCK, BLOCK)
    sf = (blocks.abs().amax(-1) * gs / E2M1_MAX).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    denom = sf.float().unsqueeze(-1)
    scaled = torch.where(denom > 0, blocks * gs / denom.clamp_min(1e-30), torch.zeros_like(blocks))
    codes = e2m1_codes(scaled).reshape(*x.shape[:-1], K)
    packed = (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()
    if swizzle:
        if x.dim() != 2:
            raise ValueError("the tiled scale layout is defined for 2-D operands")
        sf = swizzle_block_scales(sf)
    return packed, sf, gs.reshape(1)


def dequantize_nvfp4(packed: torch.Tensor, sf: torch.Tensor, global_scale: torch.Tensor, dtype=torch.float32,
                     swizzled_rows: int | None = None) -> torch.Tensor:  # fmt: skip
    """Exact inverse of the storage format: [..., K / 2] codes + scales -> [..., K] values. `swizzled_rows`: the scales
    are in tile order and cover that many rows (2-D operands). `global_scale` holds one value, or one per row (the
    fused view of several layers, each quantised with its own tensor scale)."""
    K = packed.shape[-1] * 2
    if swizzled_rows is not None:
        sf = unswizzle_block_scales(sf, swizzled_rows, K // BLOCK)
    lo, hi = packed & 0x0F, packed >> 4
    codes = torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], K).long()
    vals = E2M1_VALUES.to(packed.device)[codes & 7] * torch.where((codes & 8) > 0, -1.0, 1.0)
    vals = vals.reshape(*packed.shape[:-1], K // BLOCK, BLOCK) * sf.float().unsqueeze(-1)
    gs = global_scale.float()
    gs = gs.reshape(()) if gs.numel() == 1 else gs.reshape(*packed.shape[:-1], 1)  # one per tensor, or one per row
    return (vals.reshape(*packed.shape[:-1], K) / gs).to(dtype)


def swizzle_block_scales(sf: torch.Tensor) -> torch.Tensor:
    """[rows, cols] scales -> tiles of 128 rows x 4 columns (512 bytes each), tiles ordered row-tile major; inside a tile
    row r and column c sit at (r % 32) * 16 + (r // 32) * 4 + c. Rows and columns are zero-padded to whole tiles."""
    rows, cols = sf.shape
    rt, ct = -(-rows // 128), -(-cols // 4)
    raw = torch.zeros(rt * 128, ct * 4, dtype=torch.uint8, device=sf.device)
    raw[:rows, :cols] = sf.view(torch.uint8)
    t = raw.view(rt, 4, 32, ct, 4).permute(0, 3, 2, 1, 4)  # [row tile, col tile, r % 32, r // 32, c]
    return t.contiguous().view(rt * ct, 512).view(torch.float8_e4m3fn)


def unswizzle_block_scales(tiled: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    rt, ct = -(-rows // 128), -(-cols // 4)
    t = tiled.view(torch.uint8).view(rt, ct, 32, 4, 4).permute(0, 3, 2, 1, 4)  # [row tile, r // 32, r % 32, col tile, c]
    return t.contiguous().view(rt * 128, ct * 4)[:rows, :cols].contiguous().view(torch.float8_e4m3fn)


# ---------------------------------------------------------------------------------------------------
# weight-only linear
# ---------------------------------------------------------------------------------------------------
_SCRATCH: dict = {}


def _scratch(shape, device, dtype) -> torch.Tensor:
    stream = torch.cuda.current_stream(device).cuda_stream if torch.device(device).type == "cuda" else 0
    key = (tuple(shape), str(device), dtype, stream)
    buf = _SCRATCH.get(key)
    if buf is None:
        buf = _SCRATCH[key] = torch.empty(shape, device=device, dtype=dtype)
    return buf


def expand_nvfp4_weight(weight: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """Packed parameter [N, K / 2] tagged by `quantize_linear_nvfp4_` -> dense [N, K] in a scratch buffer that layers of
    the same shape share (valid until the next expansion of that shape on the same stream)."""
    sf, gs = weight.tfb_nvfp4_sf, weight.tfb_nvfp4_global
    if sf.device != weight.device:  # the module was moved after quantisation
        sf = weight.tfb_nvfp4_sf = sf.to(weight.device)
        gs = weight.tfb_nvfp4_global = gs.to(weight.device)
    out = _scratch((weight.shape[0], weight.shape[1] * 2), weight.device, dtype)
    out.copy_(dequantize_nvfp4(weight.data, sf, gs, dtype))
    return out


class QuantizedLinearNVFP4(nn.Linear):
    """An `nn.Linear` whose weight is stored as NVFP4 (packed codes in `weight`, buffers `weight_scale` e4m3 per 16 input
    channels and `weight_global_scale`); the forward expands it and runs the dense linear."""

    def _sync(self) -> None:
        self.weight.tfb_nvfp4_sf, self.weight.tfb_nvfp4_global = self.weight_scale, self.weight_global_scale

    def _apply(self, fn, recurse=True):
        r = super()._apply(fn, recurse)
        self._sync()
        return r

    def _load_from_state_dict(self, *a, **kw):
        super()._load_from_state_dict(*a, **kw)
        self._sync()

    def forward(self, x):
        return TF.linear(x, self.weight, self.bias)


def quantize_linear_nvfp4_(lin: nn.Linear) -> nn.Linear:
    """In place: the weight becomes packed e2m1 codes [N, K / 2] (uint8) tagged with its scales; buffers are registered
    for checkpoints; the class becomes `QuantizedLinearNVFP4` for plain `nn.Linear` modules."""
    if lin.weight.dtype == torch.uint8:
        return lin
    if lin.in_features % BLOCK:
        raise ValueError(f"in_features {lin.in_features} is not a multiple of {BLOCK}")
    packed, sf, gs = quantize_nvfp4(lin.weight.data)
    lin.weight = nn.Parameter(packed, requires_grad=False)
    for name, t in (("weight_scale", sf), ("weight_global_scale", gs)):
        if name in lin._buffers:
            setattr(lin, name, t)
        else:
            lin.register_buffer(name, t)
    if type(lin) is nn.Linear:
        lin.__class__ = QuantizedLinearNVFP4
    lin.weight.tfb_nvfp4_sf, lin.weight.tfb_nvfp4_global = lin.weight_scale, lin.weight_global_scale
    return lin


def quantize_model_nvfp4_(model: nn.Module, include_names=None, exclude_names=None, min_features: int = 64) -> int:
    """NVFP4 weight storage for every `nn.Linear` whose qualified name passes the patterns; returns the count."""
    n = 0
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear) or min(m.in_features, m.out_features) < min_features or m.in_features % BLOCK:
            continue
        if exclude_names and any(fnmatch.fnmatch(name, p) or p in name for p in exclude_names):
            continue
        if include_names and not any(fnmatch.fnmatch(name, p) or p in name for p in include_names):
            continue
        quantize_linear_nvfp4_(m)
        n += 1
    from telefuser_b200.ops.quant import invalidate_fused_caches

    invalidate_fused_caches(model)
    return n
