"""Offline checkpoint converter / quantiser.

    python -m telefuser_b200.tools.convert -s <ckpt file or dir> -o <out dir> [-o_n name]
        [--direction forward|backward --model_type wan_dit] [--rule 'regex=>replacement' ...]
        [--lora_path a.safetensors --lora_strength 1.0]
        [--quantized --linear_dtype fp8|int8|mxfp8|nvfp4|mxfp4|mxfp6 --quantize_modules attn ffn] [--save_by_block]
        [--dequantize [--dtype bfloat16]]

* key mapping: built-in rule sets (diffusers -> native Wan DiT names, and back) plus ad-hoc regex rules
* LoRA merge before any quantisation (same loader as run-time)
* fp8: e4m3 weight + per-output-channel fp32 `weight_scale [out, 1]` (scale = row amax / 448) — the layout
  the W8A8 linear consumes (int8: the same with int8 values in [-127, 127]); mxfp8: e4m3 payload + UE8M0 scale per 32
  input elements in `weight_sf`; nvfp4: packed e2m1 codes + e4m3 `weight_scale` per 16 + fp32 `weight_global_scale`;
  mxfp4 / mxfp6 (`mxfp6_e3m2`, `mxfp6_e2m3`): bit-packed codes + UE8M0 `weight_sf` per 32 + `weight_mx_format`
  (exponent and mantissa widths) — storage formats (`ops/mxfp.py`), expanded again by `--dequantize`
* `--dequantize` turns any checkpoint written by `--quantized` back into dense weights (it runs before `--quantized`,
  so one call can also re-quantise into another format)
* output: one safetensors file, or one file per transformer block plus an index json
Role parity: tools/convert/converter.py:32-937 (key mapping, quantize_model, load_loras, save by block),
tools/convert/quant.py:28-145 (the weight formats).
"""

from __future__ import annotations

import argparse
import json
import os
import re
import shutil
from collections import defaultdict

import torch

from telefuser_b200.utils.logging import logger
from telefuser_b200.utils.model_weight import load_state_dict, save_state_dict

FP8_MAX = 448.0


def get_key_mapping_rules(direction: str, model_type: str) -> list[tuple[str, str]]:
    """Regex rules; `forward` = other layout -> native names, `backward` = native -> other layout."""
    if model_type == "wan_dit":
        fwd = [
            (r"^condition_embedder\.text_embedder\.linear_1\.", "text_embedding.0."),
            (r"^condition_embedder\.text_embedder\.linear_2\.", "text_embedding.2."),
            (r"^condition_embedder\.time_embedder\.linear_1\.", "time_embedding.0."),
            (r"^condition_embedder\.time_embedder\.linear_2\.", "time_embedding.2."),
            (r"^condition_embedder\.time_proj\.", "time_projection.1."),
            (r"^blocks\.(\d+)\.attn1\.to_q\.", r"blocks.\1.self_attn.q."),
            (r"^blocks\.(\d+)\.attn1\.to_k\.", r"blocks.\1.self_attn.k."),
            (r"^blocks\.(\d+)\.attn1\.to_v\.", r"blocks.\1.self_attn.v."),
            (r"^blocks\.(\d+)\.attn1\.to_out\.0\.", r"blocks.\1.self_attn.o."),
            (r"^blocks\.(\d+)\.attn1\.norm_q\.", r"blocks.\1.self_attn.norm_q."),
            (r"^blocks\.(\d+)\.attn1\.norm_k\.", r"blocks.\1.self_attn.norm_k."),
            (r"^blocks\.(\d+)\.attn2\.to_q\.", r"blocks.\1.cross_attn.q."),
            (r"^blocks\.(\d+)\.attn2\.to_k\.", r"blocks.\1.cross_attn.k."),
            (r"^blocks\.(\d+)\.attn2\.to_v\.", r"blocks.\1.cross_attn.v."),
            (r"^blocks\.(\d+)\.attn2\.to_out\.0\.", r"blocks.\1.cross_attn.o."),
            (r"^blocks\.(\d+)\.attn2\.norm_q\.", r"blocks.\1.cross_attn.norm_q."),
            (r"^blocks\.(\d+)\.attn2\.norm_k\.", r"blocks.\1.cross_attn.norm_k."),
            (r"^blocks\.(\d+)\.ffn\.net\.0\.proj\.", r"blocks.\1.ffn.0."),
            (r"^blocks\.(\d+)\.ffn\.net\.2\.", r"blocks.\1.ffn.2."),
            (r"^blocks\.(\d+)\.norm2\.", r"blocks.\1.norm3."),
            (r"^blocks\.(\d+)\.scale_shift_table$", r"blocks.\1.modulation"),
            (r"^proj_out\.", "head.head."),
            (r"^scale_shift_table$", "head.modulation"),
        ]
        bwd = [
            (r"^text_embedding\.0\.", "condition_embedder.text_embedder.linear_1."),
            (r"^text_embedding\.2\.", "condition_embedder.text_embedder.linear_2."),
            (r"^time_embedding\.0\.", "condition_embedder.time_embedder.linear_1."),
            (r"^time_embedding\.2\.", "condition_embedder.time_embedder.linear_2."),
            (r"^time_projection\.1\.", "condition_embedder.time_proj."),
            (r"^blocks\.(\d+)\.self_attn\.([qkv])\.", r"blocks.\1.attn1.to_\2."),
            (r"^blocks\.(\d+)\.self_attn\.o\.", r"blocks.\1.attn1.to_out.0."),
            (r"^blocks\.(\d+)\.self_attn\.norm_([qk])\.", r"blocks.\1.attn1.norm_\2."),
            (r"^blocks\.(\d+)\.cross_attn\.([qkv])\.", r"blocks.\1.attn2.to_\2."),
            (r"^blocks\.(\d+)\.cross_attn\.o\.", r"blocks.\1.attn2.to_out.0."),
            (r"^blocks\.(\d+)\.cross_attn\.norm_([qk])\.", r"blocks.\1.attn2.norm_\2."),
            (r"^blocks\.(\d+)\.ffn\.0\.", r"blocks.\1.ffn.net.0.proj."),
            (r"^blocks\.(\d+)\.ffn\.2\.", r"blocks.\1.ffn.net.2."),
            (r"^blocks\.(\d+)\.norm3\.", r"blocks.\1.norm2."),
            (r"^blocks\.(\d+)\.modulation$", r"blocks.\1.scale_shift_table"),
            (r"^head\.head\.", "proj_out."),
            (r"^head\.modulation$", "scale_shift_table"),
        ]
        return fwd if direction == "forward" else bwd
    if model_type in ("none", "", None):
        return []
    raise ValueError(f"no built-in key mapping for model type {model_type!r}")


def apply_rules(sd: dict, rules: list[tuple[str, str]]) -> dict:
    if not rules:
        return dict(sd)
    comp = [(re.compile(p), r) for p, r in rules]
    out = {}
    for k, v in sd.items():
        nk = k
        for pat, rep in comp:
            nk2 = pat.sub(rep, nk)
            if nk2 != nk:
                nk = nk2
                break
        if nk in out:
            raise ValueError(f"key mapping sends two keys to {nk!r}")
        out[nk] = v
    return out


def quantize_fp8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    scale = (w.float().abs().amax(dim=1, keepdim=True) / FP8_MAX).clamp_min(1e-12)
    return (w.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), scale


def quantize_mxfp8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    from telefuser_b200.ops.functional import quant_mxfp8_reference

    q, sf = quant_mxfp8_reference(w.float())
    return q.view(torch.float8_e4m3fn).reshape(w.shape), sf.reshape(w.shape[0], -1)


def quantize_model(sd: dict, linear_dtype: str = "fp8", quantize_modules=("attn", "ffn"), skip=("norm", "modulation",
                   "embedding", "head", "time_"), min_dim: int = 64) -> tuple[dict, int]:  # fmt: skip
    out, n = {}, 0
    for k, v in sd.items():
        is_target = (k.endswith(".weight") and v.dim() == 2 and min(v.shape) >= min_dim
                     and any(m in k for m in quantize_modules) and not any(s in k for s in skip))  # fmt: skip
        if not is_target or (linear_dtype.startswith("mxfp") and v.shape[1] % 32) or (linear_dtype == "nvfp4" and v.shape[1] % 16):
            out[k] = v
            continue
        base = k[: -len(".weight")]
        if linear_dtype == "fp8":
            q, s = quantize_fp8(v)
            out[k], out[base + ".weight_scale"] = q, s
        elif linear_dtype == "mxfp8":
            q, sf = quantize_mxfp8(v)
            out[k], out[base + ".weight_sf"] = q, sf
        elif linear_dtype == "int8":
            from telefuser_b200.ops.functional import quantize_weight_int8

            q, s = quantize_weight_int8(v)
            out[k], out[base + ".weight_scale"] = q, s.reshape(-1, 1)
        elif linear_dtype == "nvfp4":
            from telefuser_b200.ops.nvfp4 import quantize_nvfp4

            packed, sf, gs = quantize_nvfp4(v)
            out[k], out[base + ".weight_scale"], out[base + ".weight_global_scale"] = packed, sf, gs
        elif linear_dtype in MX_SUBBYTE:
            from telefuser_b200.ops.mxfp import mx_format, quantize_mx

            f = mx_format(linear_dtype)
            packed, sf = quantize_mx(v, f)
            out[k], out[base + ".weight_sf"] = packed, sf
            out[base + ".weight_mx_format"] = torch.tensor([f.exp_bits, f.man_bits], dtype=torch.uint8)
        else:
            raise ValueError(f"unknown linear dtype {linear_dtype!r}")
        n += 1
    return out, n


MX_SUBBYTE = ("mxfp4", "mxfp6", "mxfp6_e2m3", "mxfp6_e3m2")
_SIDE_TENSORS = (".weight_scale", ".weight_sf", ".weight_global_scale", ".weight_mx_format")


def dequantize_model(sd: dict, dtype=torch.bfloat16) -> tuple[dict, int]:
    """Inverse of `quantize_model` for every format it writes: quantised `<name>.weight` entries become dense
    `dtype` matrices and their side tensors are dropped, so a 4- / 6- / 8-bit checkpoint loads anywhere."""
    out, n = {}, 0
    payload_bases = {k[: -len(".weight")] for k, v in sd.items()
                     if k.endswith(".weight") and v.dtype in (torch.float8_e4m3fn, torch.int8, torch.uint8)}  # fmt: skip
    for k, v in sd.items():
        if k.endswith(_SIDE_TENSORS) and k.rsplit(".", 1)[0] in payload_bases:
            continue
        base = k[: -len(".weight")] if k.endswith(".weight") else None
        scale, sf = (sd.get(f"{base}.weight_scale"), sd.get(f"{base}.weight_sf")) if base else (None, None)
        if base is None or (scale is None and sf is None) or v.dtype not in (torch.float8_e4m3fn, torch.int8, torch.uint8):
            out[k] = v  # not a quantised payload (a dense weight next to a tensor that merely shares the suffix)
            continue
        n += 1
        if f"{base}.weight_mx_format" in sd:
            from telefuser_b200.ops.mxfp import MXFormat, dequantize_mx

            e, m = (int(t) for t in sd[f"{base}.weight_mx_format"])
            out[k] = dequantize_mx(v, sf, MXFormat("checkpoint", e, m, 1 if e == 2 else 3), dtype)
        elif f"{base}.weight_global_scale" in sd:
            from telefuser_b200.ops.nvfp4 import dequantize_nvfp4

            out[k] = dequantize_nvfp4(v, scale, sd[f"{base}.weight_global_scale"], dtype)
        elif sf is not None:  # MXFP8: e4m3 payload, UE8M0 byte per 32 input elements
            w = v.float().reshape(v.shape[0], -1, 32) * torch.exp2(sf.float() - 127.0).unsqueeze(-1)
            out[k] = w.reshape(v.shape).to(dtype)
        else:  # e4m3 or int8 with one scale per output channel
            out[k] = (v.float() * scale.float().reshape(-1, 1)).to(dtype)
    return out, n


def save_by_block(sd: dict, out_dir: str, name: str) -> dict:
    groups: dict[str, dict] = defaultdict(dict)
    for k, v in sd.items():
        m = re.match(r"^(?:.*\.)?blocks\.(\d+)\.", k)
        groups[f"block_{int(m.group(1)):03d}" if m else "non_block"][k] = v
    index = {"metadata": {"format": "pt"}, "weight_map": {}}
    for g, part in sorted(groups.items()):
        fn = f"{name}.{g}.safetensors"
        save_state_dict(part, os.path.join(out_dir, fn))
        index["weight_map"].update({k: fn for k in part})
    with open(os.path.join(out_dir, f"{name}.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=2)
    return index


def copy_non_weight_files(source_dir: str, target_dir: str) -> int:
    n = 0
    for root, _dirs, files in os.walk(source_dir):
        for fn in files:
            if fn.endswith((".safetensors", ".pth", ".pt", ".bin", ".ckpt")):
                continue
            rel = os.path.relpath(os.path.join(root, fn), source_dir)
            dst = os.path.join(target_dir, rel)
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            shutil.copy2(os.path.join(root, fn), dst)
            n += 1
    return n


def convert_weights(args) -> dict:
    sd = load_state_dict(args.source)
    rules = get_key_mapping_rules(args.direction, args.model_type)
    for r in args.rule or []:
        pat, rep = r.split("=>", 1)
        rules.append((pat, rep))
    sd = apply_rules(sd, rules)
    merged = 0
    if args.lora_path:
        from torch import nn

        from telefuser_b200.utils.lora import LoRALoader

        params = {k: nn.Parameter(v.float(), requires_grad=False) for k, v in sd.items() if v.is_floating_point()}

        class _Flat(nn.Module):  # exposes the checkpoint's keys as parameter names to the LoRA loader
            def named_parameters(self, *a, **kw):
                return iter(params.items())

            def named_buffers(self, *a, **kw):
                return iter(())

        for lp in args.lora_path:
            merged += LoRALoader().apply_lora(_Flat(), lp, strength=args.lora_strength)["merged"]
        for k, p in params.items():
            sd[k] = p.data.to(sd[k].dtype)
    nq = 0
    if getattr(args, "dequantize", False):
        sd, nq = dequantize_model(sd, getattr(torch, args.dtype or "bfloat16"))
    if args.quantized:
        sd, nq = quantize_model(sd, args.linear_dtype, tuple(args.quantize_modules))
    if args.dtype:
        dt = getattr(torch, args.dtype)
        sd = {k: (v.to(dt) if v.is_floating_point() and v.dtype in (torch.float32, torch.float16, torch.bfloat16)
                  and not k.endswith(_SIDE_TENSORS) else v) for k, v in sd.items()}  # fmt: skip
    os.makedirs(args.output, exist_ok=True)
    if args.save_by_block:
        save_by_block(sd, args.output, args.output_name)
    else:
        save_state_dict(sd, os.path.join(args.output, args.output_name + args.output_ext))
    copied = 0
    if args.copy_no_weight_files and os.path.isdir(args.source):
        copied = copy_non_weight_files(args.source, args.output)
    logger.info(f"converted {len(sd)} tensors ({nq} quantised, {merged} LoRA tensors merged, {copied} files copied)")
    return {"tensors": len(sd), "quantized": nq, "lora_merged": merged, "copied": copied}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="checkpoint converter / quantiser")
    p.add_argument("-s", "--source", required=True)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("-o_n", "--output_name", default="converted")
    p.add_argument("-o_e", "--output_ext", default=".safetensors", choices=[".safetensors", ".pth"])
    p.add_argument("-d", "--direction", default="forward", choices=["forward", "backward"])
    p.add_argument("-t", "--model_type", default="none")
    p.add_argument("--rule", action="append", help="extra regex rule 'pattern=>replacement'")
    p.add_argument("--lora_path", nargs="*")
    p.add_argument("--lora_strength", type=float, default=1.0)
    p.add_argument("--quantized", action="store_true")
    p.add_argument("--linear_dtype", default="fp8", choices=["fp8", "int8", "mxfp8", "nvfp4", *MX_SUBBYTE])
    p.add_argument("--dequantize", action="store_true", help="expand a quantised checkpoint back to dense weights first")
    p.add_argument("--quantize_modules", nargs="*", default=["attn", "ffn"])
    p.add_argument("--dtype", default=None, choices=[None, "bfloat16", "float16", "float32"])
    p.add_argument("-b", "--save_by_block", action="store_true")
    p.add_argument("--copy_no_weight_files", action="store_true")
    return p


def main(argv=None) -> dict:
    return convert_weights(build_parser().parse_args(argv))


if __name__ == "__main__":
    main()
