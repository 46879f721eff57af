"""Quantised linear layers: W8A8 FP8 (per-token activation scale x per-output-channel weight scale).

Weights are stored as e4m3 `[out, in]` with `weight_scale [out, 1]` (fp32), the checkpoint layout the
offline converter writes; activations are quantised per token on the fly by a row kernel and the product
runs on the tcgen05 `kind::f8f6f4` GEMM with the scales applied in its epilogue (`ops.functional.linear`
dispatches on the weight dtype, so model code does not change).
`quantize_model_fp8_` converts the selected `nn.Linear` layers of a loaded bf16 model in place.
Role parity: telefuser/ops/linear_fp8.py (`LinearFP8`), ops/fp8_gemm.py, `BaseModel.enable_quant`.
"""

from __future__ import annotations

import fnmatch

import torch
from torch import nn

from . import functional as TF

FP8_MAX = 448.0


def quantize_weight_fp8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[out, in] -> (e4m3 [out, in], fp32 scale [out, 1]); scale = row amax / 448."""
    scale = (w.float().abs().amax(dim=1, keepdim=True) / FP8_MAX).clamp_min(1e-12)
    return (w.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), scale


class _ScaleTagged:
    """Keeps `weight.tfb_scale` (what `ops.functional.linear` reads) pointing at the module's live
    `weight_scale` buffer. `Module.to()` / `.cuda()` / `.cpu()` replace the buffer object but keep the
    Parameter object, deep copies and unpickling rebuild the Parameter without its attributes: after each of
    those the tag is set again, so the GEMM never sees a scale left behind on another device."""

    def _sync(self) -> None:
        if "weight_scale" in self._buffers:
            self.weight.tfb_scale = self.weight_scale
        if "weight_scale_mx" in self._buffers:
            self.weight.tfb_mx_sf = self.weight_scale_mx

    def _load_from_state_dict(self, *a, **kw):
        super()._load_from_state_dict(*a, **kw)
        self._sync()

    def _apply(self, fn, recurse=True):
        r = super()._apply(fn, recurse)
        self._sync()
        return r

    def __setstate__(self, state):
        super().__setstate__(state)
        self._sync()


class LinearFP8(_ScaleTagged, nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.zeros(out_features, in_features, dtype=torch.float8_e4m3fn, device=device),
                                   requires_grad=False)  # fmt: skip
        self.register_buffer("weight_scale", torch.ones(out_features, 1, dtype=torch.float32, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=torch.bfloat16, device=device)) if bias else None
        self._sync()

    @classmethod
    def from_linear(cls, lin: nn.Linear) -> "LinearFP8":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, lin.weight.device)
        q, s = quantize_weight_fp8(lin.weight.data)
        m.weight.data, m.weight_scale = q, s
        if lin.bias is not None:
            m.bias.data = lin.bias.data.to(torch.bfloat16)
        m._sync()
        return m

    def forward(self, x):
        return TF.linear_fp8(x, self.weight, self.weight_scale, self.bias)


class QuantizedLinear(_ScaleTagged, nn.Linear):
    """What an `nn.Linear` becomes when it is quantised in place: still an `nn.Linear` for model code that reads
    `.weight` / `.bias` and calls the functional linear, plus the bookkeeping of `_ScaleTagged`."""

    def forward(self, x):
        return TF.linear_fp8(x, self.weight, self.weight_scale, self.bias)


def quantize_linear_fp8_(lin: nn.Linear) -> nn.Linear:
    """In place: the module stays an `nn.Linear` (its class becomes `QuantizedLinear`), its weight becomes e4m3
    and carries `tfb_scale`; a `weight_scale` buffer is registered for checkpoints."""
    if lin.weight.dtype == torch.float8_e4m3fn:
        return lin
    q, s = quantize_weight_fp8(lin.weight.data)
    lin.weight = nn.Parameter(q, requires_grad=False)
    if "weight_scale" in lin._buffers:
        lin.weight_scale = s
    else:
        lin.register_buffer("weight_scale", s)
    if type(lin) is nn.Linear:
        lin.__class__ = QuantizedLinear
    lin.weight.tfb_scale = lin.weight_scale
    return lin


class QuantizedLinearInt8(_ScaleTagged, nn.Linear):
    """An `nn.Linear` quantised in place to W8A8 on integers: int8 weight with a per-output-channel scale
    (`weight_scale`, tag `weight.tfb_scale`), activations quantised per token, exact int32 accumulation."""

    def forward(self, x):
        return TF.linear_int8(x, self.weight, self.weight_scale, self.bias)


def quantize_linear_int8_(lin: nn.Linear) -> nn.Linear:
    """In place, symmetric int8 (range [-127, 127]); same bookkeeping as `quantize_linear_fp8_`."""
    if lin.weight.dtype in (torch.int8, torch.float8_e4m3fn):
        return lin
    q, s = TF.quantize_weight_int8(lin.weight.data)
    lin.weight = nn.Parameter(q, requires_grad=False)
    if "weight_scale" in lin._buffers:
        lin.weight_scale = s.reshape(-1, 1)
    else:
        lin.register_buffer("weight_scale", s.reshape(-1, 1))
    if type(lin) is nn.Linear:
        lin.__class__ = QuantizedLinearInt8
    lin.weight.tfb_scale = lin.weight_scale
    return lin


class QuantizedLinearMX(_ScaleTagged, nn.Linear):
    """An `nn.Linear` quantised in place to block-scaled MXFP8: e4m3 weight plus one UE8M0 scale per 32 input
    channels, kept in the tile order the tensor core reads (buffer `weight_scale_mx`, tag `weight.tfb_mx_sf`)."""

    def forward(self, x):
        return TF.linear_mxfp8(x, self.weight, self.weight_scale_mx, self.bias)


def quantize_linear_mxfp8_(lin: nn.Linear) -> nn.Linear:
    """In place, block-scaled MXFP8 (needs in_features to be a multiple of 128)."""
    if lin.weight.dtype == torch.float8_e4m3fn:
        return lin
    q, sf = TF.quantize_weight_mxfp8(lin.weight.data)
    lin.weight = nn.Parameter(q, requires_grad=False)
    if "weight_scale_mx" in lin._buffers:
        lin.weight_scale_mx = sf
    else:
        lin.register_buffer("weight_scale_mx", sf)
    if type(lin) is nn.Linear:
        lin.__class__ = QuantizedLinearMX
    lin.weight.tfb_mx_sf = lin.weight_scale_mx
    return lin


def quantize_model_fp8_(model: nn.Module, quantize_modules=("*attn*", "*ffn*"), skip_modules=("head", "time_embedding",
                        "time_projection", "patch_embedding", "text_embedding", "img_emb"), min_features: int = 64,
                        block_scaled: bool = False, int8: bool = False) -> int:  # fmt: skip
    """Quantises every `nn.Linear` whose qualified name matches one of `quantize_modules` (fnmatch) and
    none of `skip_modules` (substring); returns the number of layers converted. `block_scaled=True` selects
    MXFP8 (a scale per 32 input channels) for layers whose input width is a multiple of 128; the others, and
    everything when it is False, get per-channel FP8. `int8=True` selects symmetric int8 weights and activations
    (exact integer accumulation) instead of e4m3."""
    n = 0
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear) or min(m.in_features, m.out_features) < min_features:
            continue
        if m.in_features % 16 or m.out_features % 8:
            continue
        if any(s in name for s in skip_modules) or not any(fnmatch.fnmatchcase(name, p) for p in quantize_modules):
            continue
        if int8:
            quantize_linear_int8_(m)
        elif block_scaled and m.in_features % 128 == 0:
            quantize_linear_mxfp8_(m)
        else:
            quantize_linear_fp8_(m)
        n += 1
    invalidate_fused_caches(model)
    return n


FUSED_CACHE_SLOTS = ("_qkv", "_kv", "_gu", "_fused", "_img", "_txt")


def invalidate_fused_caches(model: nn.Module) -> None:
    """Drops the concatenated-weight views that attention / MLP modules cache (QKV, KV, gate+up, joint streams), so
    the next forward rebuilds them from the converted weights. A slot name that a module uses for a METHOD (the
    builder of such a view) is left alone."""
    for m in model.modules():
        for attr in FUSED_CACHE_SLOTS:
            if attr in m.__dict__ and not callable(m.__dict__[attr]):
                m.__dict__[attr] = None


def resolve_quant_kind(quant) -> str:
    """What a `QuantConfig`, a `QuantType`, a string, a dtype or None asks for: "fp8" (the default), "int8", "mxfp8",
    "nvfp4" or "nf4"."""
    kind = getattr(quant, "quant_type", quant)
    if kind is None:
        return "fp8"
    if isinstance(kind, torch.dtype):
        return {torch.int8: "int8", torch.float8_e4m3fn: "fp8"}.get(kind, "fp8")
    name = (kind.name if hasattr(kind, "name") else str(kind)).lower()
    for key, out in (("nvfp4", "nvfp4"), ("nf4", "nf4"), ("mxfp8", "mxfp8"), ("int8", "int8")):
        if key in name:
            return out
    # MXFP4 / MXFP6 are checkpoint storage formats here (`ops/mxfp.py`); at run time the nearest format with a compute
    # path stands in: the other 4-bit block-scaled format for MXFP4, block-scaled FP8 for MXFP6
    for key, out in (("mxfp4", "nvfp4"), ("mxfp6", "mxfp8")):
        if key in name:
            from telefuser_b200.utils.logging import logger

            logger.warning(f"{key.upper()} has no run-time kernel; layers are quantised as {out.upper()} instead")
            return out
    return "fp8"


def quantize_model_(model: nn.Module, quant, quantize_modules, skip_modules=()) -> int:
    """Quantises the linears of `model` that match `quantize_modules` (fnmatch on qualified names) and none of
    `skip_modules` (substrings) in the format `quant` names; returns the number of layers converted. One entry point
    for every model's `enable_quant`, so each format works for each model family."""
    kind = resolve_quant_kind(quant)
    # a QuantConfig may narrow the selection (its own patterns) and widen the exclusions; what the model itself says
    # must stay unquantised inside a block (routers, modulation tables) is always kept
    quantize_modules = tuple(getattr(quant, "quantize_modules", None) or quantize_modules)
    skip = tuple(dict.fromkeys(tuple(getattr(quant, "skip_modules", None) or ()) + tuple(skip_modules)))
    if kind == "nvfp4":
        from telefuser_b200.ops.nvfp4 import quantize_model_nvfp4_

        return quantize_model_nvfp4_(model, tuple(quantize_modules), skip)
    if kind == "nf4":
        from telefuser_b200.ops.nf4 import quantize_model_nf4_

        n = quantize_model_nf4_(model, tuple(quantize_modules), skip)
        invalidate_fused_caches(model)
        return n
    return quantize_model_fp8_(model, tuple(quantize_modules), skip, block_scaled=kind == "mxfp8", int8=kind == "int8")


# ---------------------------------------------------------------------------------------------------
# quantised side-car checkpoints
# ---------------------------------------------------------------------------------------------------
SIDECAR_FORMAT = "telefuser_b200.quantized_linears.v1"


def stored_format(lin: nn.Module) -> str:
    """How a linear's weight is stored: "dense", "fp8", "int8", "mxfp8", "nvfp4" or "nf4"."""
    w = lin.weight
    if w.dtype == torch.float8_e4m3fn:
        return "mxfp8" if getattr(lin, "weight_scale_mx", None) is not None else "fp8"
    if w.dtype == torch.int8:
        return "int8"
    if w.dtype == torch.uint8:
        return "nvfp4" if getattr(lin, "weight_global_scale", None) is not None else "nf4"
    return "dense"


def dense_weight(lin: nn.Module) -> torch.Tensor:
    """The fp32 matrix [out, in] a (possibly quantised) linear stands for."""
    kind, w = stored_format(lin), lin.weight.data
    if kind == "dense":
        return w.float()
    if kind in ("fp8", "int8"):
        return w.float() * lin.weight_scale.float().reshape(-1, 1)
    if kind == "mxfp8":
        sf = TF.mx_untile_scales(lin.weight_scale_mx, w.shape[0]).float()
        return (w.float().reshape(w.shape[0], -1, 32) * torch.exp2(sf - 127.0).unsqueeze(-1)).reshape(w.shape)
    if kind == "nvfp4":
        from .nvfp4 import dequantize_nvfp4

        return dequantize_nvfp4(w, lin.weight_scale, lin.weight_global_scale, torch.float32)
    from .nf4 import NF4_BLOCK, dequantize_nf4_reference

    shape = (w.shape[0], w.shape[1] * 2)
    return dequantize_nf4_reference(w.reshape(-1), lin.absmax, shape, getattr(w, "tfb_nf4_block", NF4_BLOCK), torch.float32)


def update_weight_(lin: nn.Module, new_dense: torch.Tensor, dtype=torch.bfloat16) -> nn.Module:
    """Replaces what the linear stands for by `new_dense` [out, in], keeping its stored format: the matrix is quantised
    again with fresh scales (used to merge weight deltas such as LoRAs into quantised layers)."""
    kind = stored_format(lin)
    if kind == "dense":
        lin.weight.data.copy_(new_dense.to(lin.weight.dtype))
        return lin
    lin.weight = nn.Parameter(new_dense.to(device=lin.weight.device, dtype=dtype), requires_grad=False)
    if kind == "nvfp4":
        from .nvfp4 import quantize_linear_nvfp4_

        return quantize_linear_nvfp4_(lin)
    if kind == "nf4":
        from .nf4 import quantize_linear_nf4_

        return quantize_linear_nf4_(lin)
    return {"fp8": quantize_linear_fp8_, "int8": quantize_linear_int8_, "mxfp8": quantize_linear_mxfp8_}[kind](lin)


def quantized_state(model: nn.Module) -> dict:
    """Tensors of the quantised linears only, keyed like a state dict: `<name>.weight` (e4m3 bytes as uint8, int8 values
    as they are, or packed NVFP4 codes) with `<name>.weight_scale` (fp32 per output channel; e4m3 per 16 inputs for
    NVFP4), `<name>.weight_scale_mx` (tiled UE8M0 bytes) or `<name>.weight_global_scale` (NVFP4)."""
    out: dict = {}
    for name, m in model.named_modules():
        w = getattr(m, "weight", None)
        if not isinstance(m, (nn.Linear, LinearFP8)) or w is None:
            continue
        nvfp4 = w.dtype == torch.uint8 and hasattr(w, "tfb_nvfp4_sf")
        if w.dtype == torch.float8_e4m3fn:
            out[f"{name}.weight"] = w.data.view(torch.uint8).cpu()
        elif w.dtype == torch.int8 or nvfp4:
            out[f"{name}.weight"] = w.data.cpu()
        else:
            continue
        for buf in ("weight_scale", "weight_scale_mx", "weight_global_scale"):
            if buf in m._buffers:
                t = m._buffers[buf].cpu()
                out[f"{name}.{buf}"] = t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t
    return out


def save_quantized_sidecar(model: nn.Module, path: str) -> int:
    """Writes the quantised linears of `model` next to its bf16 checkpoint (safetensors), so that a later start
    loads the 8-bit weights and their scales as they are instead of quantising again. Returns the layer count."""
    from safetensors.torch import save_file

    state = quantized_state(model)
    layers = sum(1 for k in state if k.endswith(".weight"))
    kinds = set()
    for k, v in state.items():
        if k.endswith(".weight"):
            base = k[: -len(".weight")]
            kinds.add("nvfp4" if f"{base}.weight_global_scale" in state else "int8" if v.dtype == torch.int8
                      else "mxfp8" if f"{base}.weight_scale_mx" in state else "fp8")  # fmt: skip
    save_file({k: v.contiguous() for k, v in state.items()}, path,
              metadata={"format": SIDECAR_FORMAT, "layers": str(layers), "kind": ",".join(sorted(kinds))})  # fmt: skip
    return layers


def load_quantized_sidecar(model: nn.Module, path: str, strict: bool = True) -> int:
    """Turns the linears named in the side-car into their quantised form in place (class swap as
    `quantize_linear_*_`, weights and scales taken from the file). Returns the number of layers converted."""
    from safetensors import safe_open

    with safe_open(path, framework="pt") as f:
        meta = f.metadata() or {}
        if meta.get("format") != SIDECAR_FORMAT:
            raise ValueError(f"{path} is not a quantised side-car (format {meta.get('format')!r})")
        state = {k: f.get_tensor(k) for k in f.keys()}
    return apply_quantized_state_(model, state, strict)


def quantized_state_from_checkpoint(state_dict: dict) -> tuple[dict, dict]:
    """Splits a checkpoint written by the offline converter (`tools/convert.py --quantized`) into (dense state dict,
    quantised layer state in side-car naming). The dense dict holds the de-quantised matrices under the original keys,
    so the model class is recognised and built as usual; the second dict puts the stored payloads and scales back
    afterwards (`apply_quantized_state_`), so the offline-quantised values are used as they are, not quantised again.
    MXFP4 / MXFP6 layers and MXFP8 layers whose width the block-scaled GEMM cannot take stay dense."""
    sides = (".weight_scale", ".weight_sf", ".weight_global_scale", ".weight_mx_format")
    low = (torch.float8_e4m3fn, torch.int8, torch.uint8)
    if not any(k.endswith(sides) and getattr(state_dict.get(k.rsplit(".", 1)[0] + ".weight"), "dtype", None) in low for k in state_dict):
        return state_dict, {}
    from telefuser_b200.tools.convert import dequantize_model

    dense, _ = dequantize_model(state_dict, torch.bfloat16)
    quant: dict = {}
    for k, v in state_dict.items():
        if not k.endswith(".weight"):
            continue
        base = k[: -len(".weight")]
        scale, sf = state_dict.get(f"{base}.weight_scale"), state_dict.get(f"{base}.weight_sf")
        if f"{base}.weight_mx_format" in state_dict or (scale is None and sf is None) or v.dtype not in low:
            continue
        if f"{base}.weight_global_scale" in state_dict:
            quant.update({k: v, f"{base}.weight_scale": scale, f"{base}.weight_global_scale": state_dict[f"{base}.weight_global_scale"]})
        elif sf is not None:
            if v.shape[1] % 128 == 0:
                quant.update({k: v, f"{base}.weight_scale_mx": TF.mx_tile_scales(sf.to(torch.uint8))})
        else:
            quant.update({k: v, f"{base}.weight_scale": scale.float().reshape(-1, 1)})
    return dense, quant


def apply_quantized_state_(model: nn.Module, state: dict, strict: bool = True) -> int:
    """`state`: `<name>.weight` payloads with `<name>.weight_scale` / `.weight_scale_mx` / `.weight_global_scale` (the
    side-car naming). Every named linear of `model` takes the stored form in place; returns the number converted."""
    modules = dict(model.named_modules())
    n = 0
    for key in [k for k in state if k.endswith(".weight")]:
        name = key[: -len(".weight")]
        m = modules.get(name)
        if m is None or not isinstance(m, (nn.Linear, LinearFP8)):
            if strict:
                raise KeyError(f"the side-car names {name!r}, which is not a linear layer of this model")
            continue
        dev = m.weight.device
        w8 = state[key]
        gs = state.get(f"{name}.weight_global_scale")
        if gs is not None:  # NVFP4: packed codes [N, K / 2], e4m3 block scales (stored as bytes), one tensor scale
            from telefuser_b200.ops.nvfp4 import QuantizedLinearNVFP4

            if tuple(w8.shape) != (m.out_features, m.in_features // 2):
                raise ValueError(f"{name}: side-car NVFP4 weight {tuple(w8.shape)} vs layer {(m.out_features, m.in_features)}")
            m.weight = nn.Parameter(w8.to(dev), requires_grad=False)
            for buf, val in (("weight_scale", state[f"{name}.weight_scale"].view(torch.float8_e4m3fn)), ("weight_global_scale", gs)):
                if buf in m._buffers:
                    m._buffers[buf] = val.to(dev)
                else:
                    m.register_buffer(buf, val.to(dev))
            if type(m) is nn.Linear:
                m.__class__ = QuantizedLinearNVFP4
            m.weight.tfb_nvfp4_sf, m.weight.tfb_nvfp4_global = m.weight_scale, m.weight_global_scale
            n += 1
            continue
        if tuple(w8.shape) != tuple(m.weight.shape):
            raise ValueError(f"{name}: side-car weight {tuple(w8.shape)} vs layer {tuple(m.weight.shape)}")
        int8 = w8.dtype == torch.int8
        m.weight = nn.Parameter((w8 if int8 else w8.view(torch.float8_e4m3fn)).to(dev), requires_grad=False)
        mx = state.get(f"{name}.weight_scale_mx")
        per_channel = state.get(f"{name}.weight_scale")
        for buf, val in (("weight_scale_mx", mx), ("weight_scale", per_channel)):
            if val is None:
                m._buffers.pop(buf, None)
            elif buf in m._buffers:
                m._buffers[buf] = val.to(dev)
            else:
                m.register_buffer(buf, val.to(dev))
        if mx is None and per_channel is None:
            raise ValueError(f"{name}: the side-car holds no scale for this layer")
        if type(m) is nn.Linear:
            m.__class__ = QuantizedLinearInt8 if int8 else QuantizedLinearMX if mx is not None else QuantizedLinear
        if hasattr(m.weight, "tfb_scale") and per_channel is None:
            del m.weight.tfb_scale
        m._sync()
        n += 1
    invalidate_fused_caches(model)
    return n
