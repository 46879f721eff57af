"""Microscaling 4- and 6-bit weight storage (OCP MX element formats): MXFP4 (e2m1) and MXFP6 (e2m3 or e3m2), each with
one power-of-two UE8M0 scale per 32 input elements.

These are checkpoint formats: the offline converter writes them and `dequantize_mx` expands them when a checkpoint is
loaded. Everything here is tensor arithmetic, so it runs the same on CPU and GPU. The block-scaled 8-bit format that the
tensor-core GEMM consumes directly is MXFP8 (`ops/functional.py::quant_mxfp8`).

Role parity: tools/convert/quant.py:87-129 (`QuantWeightMxFP4`, `QuantWeightMxFP6`; there they call a quantiser from a
package that is not part of the project).

Element formats (no infinities, no NaNs; subnormals at the smallest exponent):
    e2m1: bias 1, values 0, 0.5, 1, 1.5, 2, 3, 4, 6                        (largest power of two: 2^2)
    e2m3: bias 1, 32 magnitudes 0 ... 7.5 in steps of 0.125 / 0.25 / 0.5   (2^2)
    e3m2: bias 3, 32 magnitudes 0 ... 28                                     (2^4)
Block scale: 2^(floor(log2(block amax)) - emax_elem), clamped to the UE8M0 range and stored as the biased exponent byte.
Rounding: to nearest, ties to the even code; magnitudes beyond the largest value saturate.
Packing: little-endian bit stream along K: two 4-bit codes per byte, or four 6-bit codes per three bytes.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import torch

MX_BLOCK = 32


@dataclass(frozen=True)
class MXFormat:
    name: str
    exp_bits: int
    man_bits: int
    bias: int

    @property
    def bits(self) -> int:
        return 1 + self.exp_bits + self.man_bits

    @property
    def emax(self) -> int:
        """Exponent of the largest normal value (every code is finite in these formats)."""
        return (1 << self.exp_bits) - 1 - self.bias


MX_FORMATS = {
    "mxfp4": MXFormat("mxfp4", 2, 1, 1),
    "mxfp6_e2m3": MXFormat("mxfp6_e2m3", 2, 3, 1),
    "mxfp6_e3m2": MXFormat("mxfp6_e3m2", 3, 2, 3),
}
MX_FORMATS["mxfp6"] = MX_FORMATS["mxfp6_e3m2"]  # the variant with more range is the default for weights


def mx_format(fmt) -> MXFormat:
    if isinstance(fmt, MXFormat):
        return fmt
    try:
        return MX_FORMATS[str(fmt).lower()]
    except KeyError:
        raise ValueError(f"unknown MX element format {fmt!r}; known: {sorted(MX_FORMATS)}") from None


@lru_cache(maxsize=None)
def _magnitudes(fmt: MXFormat) -> torch.Tensor:
    """Value of every magnitude code (sign bit cleared), ascending."""
    codes = torch.arange(1 << (fmt.exp_bits + fmt.man_bits))
    e, m = codes >> fmt.man_bits, codes & ((1 << fmt.man_bits) - 1)
    frac = m.float() / (1 << fmt.man_bits)
    normal = (1.0 + frac) * torch.exp2((e - fmt.bias).float())
    subnormal = frac * 2.0 ** (1 - fmt.bias)
    return torch.where(e == 0, subnormal, normal)


def mx_code_values(fmt) -> torch.Tensor:
    """fp32 value of every code of the format, indexed by the code (sign in the top bit)."""
    f = mx_format(fmt)
    mag = _magnitudes(f)
    return torch.cat([mag, -mag])


def _encode(x: torch.Tensor, fmt: MXFormat) -> torch.Tensor:
    """fp32 values (already divided by their block scale) -> uint8 codes."""
    mag = _magnitudes(fmt).to(x.device)
    mids = (mag[:-1] + mag[1:]) / 2
    a = x.abs().clamp_max(mag[-1])
    idx = torch.bucketize(a, mids, right=False)  # number of midpoints strictly below |x|: a tie picks the lower code
    tie = (idx < mids.numel()) & (a == mids[idx.clamp_max(mids.numel() - 1)])
    idx = idx + (tie & (idx % 2 == 1)).long()  # ... and moves up when the lower code is odd
    sign = (x < 0) | ((x == 0) & (torch.signbit(x)))
    return (idx | (sign.long() << (fmt.bits - 1))).to(torch.uint8)


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 codes [..., K] of `bits` bits each -> bytes [..., K * bits / 8], little-endian bit order along K."""
    K = codes.shape[-1]
    if bits == 4:
        if K % 2:
            raise ValueError(f"4-bit packing needs an even number of elements per row, got {K}")
        return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()
    if bits == 6:
        if K % 4:
            raise ValueError(f"6-bit packing needs rows of a multiple of 4 elements, got {K}")
        c = codes.reshape(*codes.shape[:-1], K // 4, 4).to(torch.int32)
        word = c[..., 0] | (c[..., 1] << 6) | (c[..., 2] << 12) | (c[..., 3] << 18)
        out = torch.stack([word & 0xFF, (word >> 8) & 0xFF, (word >> 16) & 0xFF], dim=-1).to(torch.uint8)
        return out.reshape(*codes.shape[:-1], K // 4 * 3).contiguous()
    raise ValueError(f"no packing for {bits}-bit codes")


def unpack_codes(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of `pack_codes`."""
    if bits == 4:
        return torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    if bits == 6:
        b = packed.reshape(*packed.shape[:-1], packed.shape[-1] // 3, 3).to(torch.int32)
        word = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16)
        out = torch.stack([(word >> s) & 0x3F for s in (0, 6, 12, 18)], dim=-1).to(torch.uint8)
        return out.reshape(*packed.shape[:-1], packed.shape[-1] // 3 * 4)
    raise ValueError(f"no packing for {bits}-bit codes")


def quantize_mx(x: torch.Tensor, fmt="mxfp4"):
    """x [..., K] (K a multiple of 32) -> (packed codes uint8 [..., K * bits / 8], UE8M0 scales uint8 [..., K / 32])."""
    f = mx_format(fmt)
    K = x.shape[-1]
    if K % MX_BLOCK:
        raise ValueError(f"MX formats scale blocks of {MX_BLOCK} elements along the last axis; {K} is not a multiple")
    blocks = x.float().reshape(*x.shape[:-1], K // MX_BLOCK, MX_BLOCK)
    amax = blocks.abs().amax(-1)
    exp = torch.floor(torch.log2(amax.clamp_min(2.0**-126))) - f.emax
    exp = torch.where(amax > 0, exp, torch.full_like(exp, -127.0)).clamp(-127, 127)
    codes = _encode(blocks * torch.exp2(-exp).unsqueeze(-1), f).reshape(*x.shape[:-1], K)
    return pack_codes(codes, f.bits), (exp + 127).to(torch.uint8)


def dequantize_mx(packed: torch.Tensor, scales: torch.Tensor, fmt="mxfp4", dtype=torch.float32) -> torch.Tensor:
    """Exact expansion of `quantize_mx` output: code value x 2^(scale byte - 127)."""
    f = mx_format(fmt)
    codes = unpack_codes(packed, f.bits)
    vals = mx_code_values(f).to(packed.device)[codes.long()]
    K = vals.shape[-1]
    scale = torch.exp2(scales.float() - 127.0)
    return (vals.reshape(*vals.shape[:-1], K // MX_BLOCK, MX_BLOCK) * scale.unsqueeze(-1)).reshape(*vals.shape[:-1], K).to(dtype)


def bits_per_weight(fmt) -> float:
    """Storage cost including the block scales (4.25 for MXFP4, 6.25 for MXFP6)."""
    return mx_format(fmt).bits + 8.0 / MX_BLOCK


__all__ = ["MXFormat", "MX_FORMATS", "MX_BLOCK", "mx_format", "mx_code_values", "quantize_mx", "dequantize_mx", "pack_codes",
           "unpack_codes", "bits_per_weight"]  # fmt: skip
