"""NF4 (4-bit NormalFloat) weight-only quantisation for very large transformers.

A weight is split into blocks of 64 consecutive values; each block stores its absolute maximum in fp32 and one
4-bit code per value that indexes 16 fixed levels (the quantiles of a standard normal, scaled to [-1, 1]): 4.5
bits per weight. `LinearNF4` keeps packed codes and block maxima; on a B200 its forward expands the codes to
bf16 with one memory-bound kernel (`tfb_nf4_dequant`) into a scratch buffer shared by all layers of the same
shape and runs the tcgen05 GEMM on it; on CPU the expansion is a table lookup in PyTorch. The packed layout (two
codes per byte, first value in the high nibble, row-major blocks) matches the one bitsandbytes writes, so its
checkpoints' `weight` / `absmax` tensors load directly.
Role parity: telefuser/ops/bnb_nf4_linear.py (replace_linear_layers_with_bnb_nf4), which wraps the bitsandbytes package.
"""

from __future__ import annotations

import fnmatch

import torch
from torch import nn

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import native

NF4_LEVELS = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                           -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                           0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023,
                           1.0])  # fmt: skip
NF4_BLOCK = 64


def quantize_nf4(weight: torch.Tensor, block: int = NF4_BLOCK):
    """weight [..] with numel % block == 0 -> (packed uint8 [numel / 2], absmax fp32 [numel / block])."""
    flat = weight.detach().float().reshape(-1)
    if flat.numel() % block or block % 16:
        raise ValueError(f"numel {flat.numel()} must be a multiple of the block size {block} (itself a multiple of 16)")
    blocks = flat.view(-1, block)
    absmax = blocks.abs().amax(dim=1)
    normed = blocks / absmax.clamp_min(1e-30)[:, None]
    levels = NF4_LEVELS.to(flat.device)
    # nearest level by midpoints (levels are sorted)
    codes = torch.bucketize(normed.reshape(-1), (levels[1:] + levels[:-1]) / 2).to(torch.uint8)
    packed = (codes[0::2] << 4) | codes[1::2]
    return packed.contiguous(), absmax.contiguous()


def dequantize_nf4_reference(packed: torch.Tensor, absmax: torch.Tensor, shape, block: int = NF4_BLOCK, dtype=torch.float32):
    codes = torch.stack([packed >> 4, packed & 15], dim=-1).reshape(-1).long()
    vals = NF4_LEVELS.to(packed.device)[codes].view(-1, block) * absmax.float()[:, None]
    return vals.reshape(shape).to(dtype)


def dequantize_nf4(packed: torch.Tensor, absmax: torch.Tensor, shape, block: int = NF4_BLOCK, out: torch.Tensor | None = None):
    """-> bf16 tensor of `shape` on CUDA (native kernel), fp32 reference elsewhere."""
    if not packed.is_cuda:
        return dequantize_nf4_reference(packed, absmax, shape, block)
    numel = packed.numel() * 2
    if out is None:
        out = torch.empty(shape, device=packed.device, dtype=torch.bfloat16)
    code = native.load().tfb_nf4_dequant(packed.data_ptr(), absmax.data_ptr(), out.data_ptr(), numel, block, native.stream_ptr())
    native.check(code, "tfb_nf4_dequant")
    return out


_SCRATCH: dict = {}


def _scratch(shape, device) -> torch.Tensor:
    key = (tuple(shape), str(device), torch.cuda.current_stream(device).cuda_stream)
    buf = _SCRATCH.get(key)
    if buf is None:
        buf = _SCRATCH[key] = torch.empty(shape, device=device, dtype=torch.bfloat16)
    return buf


class LinearNF4(nn.Module):
    """Drop-in for `nn.Linear` with NF4 weights; buffers are named as in bitsandbytes checkpoints."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, block: int = NF4_BLOCK, compute_dtype=torch.bfloat16) -> None:
        super().__init__()
        if (in_features * out_features) % block:
            raise ValueError("in_features * out_features must be a multiple of the NF4 block size")
        self.in_features, self.out_features, self.block, self.compute_dtype = in_features, out_features, block, compute_dtype
        self.register_buffer("weight", torch.zeros(in_features * out_features // 2, dtype=torch.uint8))
        self.register_buffer("absmax", torch.ones(in_features * out_features // block, dtype=torch.float32))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=compute_dtype)) if bias else None

    @classmethod
    def from_linear(cls, linear: nn.Linear, block: int = NF4_BLOCK, compute_dtype=torch.bfloat16) -> "LinearNF4":
        m = cls(linear.in_features, linear.out_features, linear.bias is not None, block, compute_dtype)
        packed, absmax = quantize_nf4(linear.weight, block)
        m.weight, m.absmax = packed.to(linear.weight.device), absmax.to(linear.weight.device)
        if linear.bias is not None:
            m.bias = nn.Parameter(linear.bias.detach().to(compute_dtype), requires_grad=False)
        return m

    def dequantized_weight(self) -> torch.Tensor:
        shape = (self.out_features, self.in_features)
        if self.weight.is_cuda:
            return dequantize_nf4(self.weight, self.absmax, shape, self.block, out=_scratch(shape, self.weight.device))
        return dequantize_nf4_reference(self.weight, self.absmax, shape, self.block)

    def forward(self, x, act=None, residual=None, gate=None):
        w = self.dequantized_weight()
        if not x.is_cuda:
            w = w.to(x.dtype)
        return TF.linear(x, w, self.bias, act=act, residual=residual, gate=gate)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, block={self.block}, bias={self.bias is not None}"


def expand_nf4_weight(weight: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """Packed parameter [N, K / 2] tagged by `quantize_linear_nf4_` -> dense [N, K] (bf16 scratch on CUDA)."""
    absmax, block = weight.tfb_nf4_absmax, getattr(weight, "tfb_nf4_block", NF4_BLOCK)
    if absmax.device != weight.device:  # the module was moved after quantisation
        absmax = weight.tfb_nf4_absmax = absmax.to(weight.device)
    shape = (weight.shape[0], weight.shape[1] * 2)
    if weight.is_cuda:
        return dequantize_nf4(weight.data, absmax, shape, block, out=_scratch(shape, weight.device))
    return dequantize_nf4_reference(weight.data.reshape(-1), absmax, shape, block, dtype)


def quantize_linear_nf4_(lin: nn.Linear, block: int = NF4_BLOCK) -> nn.Linear:
    """In place: the module keeps its class (model code reads `.weight` / `.bias` and calls the functional linear), its
    weight becomes packed codes [N, K / 2] tagged with the block maxima; an `absmax` buffer is registered for checkpoints."""
    if lin.weight.dtype == torch.uint8:
        return lin
    packed, absmax = quantize_nf4(lin.weight.data, block)
    lin.weight = nn.Parameter(packed.view(lin.out_features, lin.in_features // 2), requires_grad=False)
    if "absmax" in lin._buffers:
        lin.absmax = absmax
    else:
        lin.register_buffer("absmax", absmax)
    lin.weight.tfb_nf4_absmax, lin.weight.tfb_nf4_block = lin.absmax, block
    return lin


def quantize_model_nf4_(model: nn.Module, include_names=None, exclude_names=None, block: int = NF4_BLOCK, min_features: int = 64) -> int:
    """In-place NF4 for every `nn.Linear` whose qualified name passes the include / exclude patterns; returns the count."""
    n = 0
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear) or min(m.in_features, m.out_features) < min_features:
            continue
        if m.in_features % block or not _wanted(name, include_names, exclude_names):
            continue
        quantize_linear_nf4_(m, block)
        n += 1
    return n


def _wanted(name: str, include, exclude) -> bool:
    if exclude and any(fnmatch.fnmatch(name, p) or p in name for p in exclude):
        return False
    return not include or any(fnmatch.fnmatch(name, p) or p in name for p in include)


def replace_linear_layers_with_nf4(module: nn.Module, compute_dtype=torch.bfloat16, include_names=None, exclude_names=None,
                                   block: int = NF4_BLOCK, prefix: str = "") -> int:  # fmt: skip
    """Swaps every matching `nn.Linear` under `module` for `LinearNF4` in place; returns how many were replaced.
    Only modules whose call sites use the module's `forward` benefit; functional call sites that read `.weight` of a
    replaced layer must go through `dequantized_weight()`."""
    n = 0
    for name, child in list(module.named_children()):
        full = f"{prefix}.{name}" if prefix else name
        if isinstance(child, nn.Linear) and (child.in_features * child.out_features) % block == 0 and _wanted(full, include_names, exclude_names):
            setattr(module, name, LinearNF4.from_linear(child, block, compute_dtype))
            n += 1
        else:
            n += replace_linear_layers_with_nf4(child, compute_dtype, include_names, exclude_names, block, full)
    return n
