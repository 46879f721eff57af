"""State-dict converters for the Wan DiT.

`from_official` accepts the checkpoint layout published with the models (which is
this implementation's native layout) and infers the architecture from tensor
shapes; `from_diffusers` renames a diffusers `WanTransformer3DModel` state dict.
Role parity: `WanModelStateDictConverter`, telefuser/models/wan_video_dit.py:1307-1600.
"""

from __future__ import annotations

import re

import torch

_DIFFUSERS_RULES: list[tuple[str, str]] = [
    (r"^condition_embedder\.time_embedder\.linear_1\.", "time_embedding.0."),
    (r"^condition_embedder\.time_embedder\.linear_2\.", "time_embedding.2."),
    (r"^condition_embedder\.time_proj\.", "time_projection.1."),
    (r"^condition_embedder\.text_embedder\.linear_1\.", "text_embedding.0."),
    (r"^condition_embedder\.text_embedder\.linear_2\.", "text_embedding.2."),
    (r"^condition_embedder\.image_embedder\.norm1\.", "img_emb.proj.0."),
    (r"^condition_embedder\.image_embedder\.ff\.net\.0\.proj\.", "img_emb.proj.1."),
    (r"^condition_embedder\.image_embedder\.ff\.net\.2\.", "img_emb.proj.3."),
    (r"^condition_embedder\.image_embedder\.norm2\.", "img_emb.proj.4."),
    (r"^condition_embedder\.image_embedder\.pos_embed$", "img_emb.emb_pos"),
    (r"^proj_out\.", "head.head."),
    (r"^scale_shift_table$", "head.modulation"),
    (r"^blocks\.(\d+)\.scale_shift_table$", r"blocks.\1.modulation"),
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
    (r"^blocks\.(\d+)\.attn2\.add_k_proj\.", r"blocks.\1.cross_attn.k_img."),
    (r"^blocks\.(\d+)\.attn2\.add_v_proj\.", r"blocks.\1.cross_attn.v_img."),
    (r"^blocks\.(\d+)\.attn2\.norm_added_k\.", r"blocks.\1.cross_attn.norm_k_img."),
    (r"^blocks\.(\d+)\.norm2\.", r"blocks.\1.norm3."),
    (r"^blocks\.(\d+)\.ffn\.net\.0\.proj\.", r"blocks.\1.ffn.0."),
    (r"^blocks\.(\d+)\.ffn\.net\.2\.", r"blocks.\1.ffn.2."),
]
_COMPILED = [(re.compile(p), r) for p, r in _DIFFUSERS_RULES]


def rename_diffusers_key(key: str) -> str:
    for pat, rep in _COMPILED:
        new, n = pat.subn(rep, key)
        if n:
            return new
    return key


def infer_wan_config(state_dict: dict[str, torch.Tensor]) -> dict:
    """Architecture hyper-parameters from tensor shapes of an official-layout state dict."""
    pe = state_dict["patch_embedding.weight"]
    dim, in_dim = pe.shape[0], pe.shape[1]
    layers = 1 + max(int(k.split(".")[1]) for k in state_dict if k.startswith("blocks."))
    head_out = state_dict["head.head.weight"].shape[0]
    patch = tuple(pe.shape[2:])
    return {
        "dim": dim,
        "in_dim": in_dim,
        "ffn_dim": state_dict["blocks.0.ffn.0.weight"].shape[0],
        "out_dim": head_out // (patch[0] * patch[1] * patch[2]),
        "text_dim": state_dict["text_embedding.0.weight"].shape[1],
        "freq_dim": state_dict["time_embedding.0.weight"].shape[1],
        "eps": 1e-6,
        "patch_size": patch,
        "num_heads": dim // 128,
        "num_layers": layers,
        "has_image_input": any(k.startswith("img_emb.") for k in state_dict),
        "has_image_pos_emb": "img_emb.emb_pos" in state_dict,
    }


class WanModelStateDictConverter:
    def from_official(self, state_dict: dict) -> tuple[dict, dict]:
        sd = {k: v for k, v in state_dict.items() if not k.startswith("vace")}
        if any(k.startswith("model.diffusion_model.") for k in sd):
            sd = {k.removeprefix("model.diffusion_model."): v for k, v in sd.items()}
        return sd, infer_wan_config(sd)

    def from_diffusers(self, state_dict: dict) -> tuple[dict, dict]:
        sd = {rename_diffusers_key(k): v for k, v in state_dict.items()}
        for k in [k for k in sd if k.endswith("modulation") and sd[k].dim() == 2]:
            sd[k] = sd[k].unsqueeze(0)
        return sd, infer_wan_config(sd)

    def from_civitai(self, state_dict: dict) -> tuple[dict, dict]:
        return self.from_official(state_dict)
