"""LoRA: merge adapters into weights at load time, or keep them as a switchable side network.

`LoRALoader.apply_lora(model, path_or_state_dict, strength)` recognises the usual key spellings
(kohya `lora_up/lora_down(/lora_mid)`, PEFT `lora_A/lora_B` with or without `.default`, diffusers
`_lora.up/_lora.down`, `lora.up/lora.down`, `lora_linear_layer.up/down`, bare `lora_A/lora_B`),
direct-difference keys (`.diff`, `.diff_b`, `.diff_m`) and per-layer `alpha`; delta =
`up @ (mid) @ down * alpha/rank * strength` is added to the matching weight in fp32. Weights stored
as fp8 with a `weight_scale` are de-quantised, merged and re-quantised with a fresh per-row scale.
`LoRANetwork` wraps chosen `nn.Linear` modules to add `multiplier * up(down(x))` at run time.
Role parity: telefuser/utils/lora_loader.py:39-290, utils/lora_network.py:27-230.
"""

from __future__ import annotations

import re

import torch
from torch import nn

from telefuser_b200.utils.logging import logger

# (up suffix, down suffix, mid suffix or None); longest suffixes first so that matching is unambiguous
_PAIR_SUFFIXES = [
    (".lora_linear_layer.up.weight", ".lora_linear_layer.down.weight", None),
    (".lora_B.default.weight", ".lora_A.default.weight", None),
    (".lora_up.weight", ".lora_down.weight", ".lora_mid.weight"),
    ("_lora.up.weight", "_lora.down.weight", None),
    (".lora.up.weight", ".lora.down.weight", None),
    (".lora_B.weight", ".lora_A.weight", None),
    (".lora_B", ".lora_A", None),
]
_DIFF_SUFFIXES = [(".diff_b", ".bias"), (".diff_m", ".modulation"), (".diff", ".weight")]
_PREFIXES = ("diffusion_model.", "model.", "unet.", "transformer.", "base_model.model.")
FP8_MAX = 448.0


def _strip_prefix(key: str) -> str:
    changed = True
    while changed:
        changed = False
        for p in _PREFIXES:
            if key.startswith(p):
                key, changed = key[len(p) :], True
    return key


class LoRALoader:
    def __init__(self, key_mapping_rules: list[tuple[str, str]] | None = None) -> None:
        self.rules = [(re.compile(p), r) for p, r in (key_mapping_rules or [])]

    def map_key(self, key: str) -> str:
        key = _strip_prefix(key)
        for pat, rep in self.rules:
            key = pat.sub(rep, key)
        return key

    # ---- parsing --------------------------------------------------------------
    def extract_lora_pairs(self, sd: dict) -> dict[str, dict]:
        pairs: dict[str, dict] = {}
        for key in sd:
            for up_s, down_s, mid_s in _PAIR_SUFFIXES:
                if not key.endswith(up_s):
                    continue
                base = key[: -len(up_s)]
                down_key = base + down_s
                if down_key not in sd:
                    continue
                entry = {"up": sd[key], "down": sd[down_key], "mid": sd.get(base + mid_s) if mid_s else None,
                         "alpha": None}  # fmt: skip
                for alpha_key in (base + ".alpha", base + ".lora_alpha", base + "_lora.alpha"):
                    if alpha_key in sd:
                        entry["alpha"] = float(sd[alpha_key])
                pairs[self.map_key(base) + ".weight"] = entry
                break
        return pairs

    def extract_lora_diffs(self, sd: dict) -> dict[str, torch.Tensor]:
        diffs = {}
        for key, t in sd.items():
            for suf, target in _DIFF_SUFFIXES:
                if key.endswith(suf):
                    diffs[self.map_key(key[: -len(suf)]) + target] = t
                    break
        return diffs

    # ---- merging ----------------------------------------------------------------
    @staticmethod
    def _delta(entry: dict, alpha: float | None, strength: float, device) -> torch.Tensor:
        up, down = entry["up"].to(device, torch.float32), entry["down"].to(device, torch.float32)
        rank = down.shape[0]
        if up.dim() > 2:  # conv LoRA: flatten the kernel
            d = (up.flatten(1) @ down.flatten(1)).reshape(up.shape[0], down.shape[1], *down.shape[2:])
        elif entry["mid"] is not None:
            d = up @ entry["mid"].to(device, torch.float32).flatten(1) @ down
        else:
            d = up @ down
        a = entry["alpha"] if entry["alpha"] is not None else alpha
        scale = (a / rank) if a is not None else 1.0
        return d * (scale * strength)

    @staticmethod
    def _add_(param: torch.Tensor, delta: torch.Tensor, scale: torch.Tensor | None) -> None:
        if param.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            if scale is None:
                raise ValueError("fp8 weight without weight_scale cannot take a LoRA delta")
            w = param.float() * scale.float().reshape(-1, 1) + delta.reshape(param.shape)
            new_scale = (w.abs().amax(dim=1, keepdim=True) / FP8_MAX).clamp_min(1e-12)
            param.copy_((w / new_scale).clamp(-FP8_MAX, FP8_MAX).to(param.dtype))
            scale.copy_(new_scale.reshape(scale.shape).to(scale.dtype))
        else:
            param.add_(delta.reshape(param.shape).to(param.dtype))

    @torch.no_grad()
    def apply_lora(self, model: nn.Module, lora, alpha: float | None = None, strength: float = 1.0) -> dict:
        """Merges `lora` (path or state dict) into `model`; returns counts of merged / unmatched keys."""
        if isinstance(lora, (str, bytes)) or hasattr(lora, "__fspath__"):
            from telefuser_b200.utils.model_weight import load_state_dict

            lora = load_state_dict(str(lora))
        params = dict(model.named_parameters())
        params.update(dict(model.named_buffers()))
        owners = {f"{name}.weight": m for name, m in model.named_modules() if isinstance(m, nn.Linear)} \
            if callable(getattr(model, "named_modules", None)) else {}  # fmt: skip
        merged, missing, requantised = 0, [], 0
        for key, entry in self.extract_lora_pairs(lora).items():
            p = params.get(key)
            if p is None:
                missing.append(key)
                continue
            owner = owners.get(key)
            if owner is not None and p.dtype in (torch.int8, torch.uint8, torch.float8_e4m3fn):
                # a quantised layer in any stored format: merge on the matrix it stands for, then quantise again
                from telefuser_b200.ops.quant import dense_weight, stored_format, update_weight_

                if stored_format(owner) != "fp8":  # per-channel FP8 keeps the in-place path below (same result, no re-allocation)
                    dense = dense_weight(owner)
                    update_weight_(owner, dense + self._delta(entry, alpha, strength, dense.device).reshape(dense.shape))
                    merged, requantised = merged + 1, requantised + 1
                    continue
            scale = params.get(key[: -len(".weight")] + ".weight_scale")
            self._add_(p.data, self._delta(entry, alpha, strength, p.device), None if scale is None else scale.data)
            merged += 1
            requantised += scale is not None  # in-place FP8: new scales, and fused views hold copies of the old ones
        if requantised and isinstance(model, nn.Module):
            from telefuser_b200.ops.quant import invalidate_fused_caches

            invalidate_fused_caches(model)
        for key, diff in self.extract_lora_diffs(lora).items():
            p = params.get(key)
            if p is None or p.numel() != diff.numel():
                missing.append(key)
                continue
            scale = params.get(key[: -len(".weight")] + ".weight_scale") if key.endswith(".weight") else None
            self._add_(p.data, diff.to(p.device, torch.float32) * strength, None if scale is None else scale.data)
            merged += 1
        if missing:
            logger.warning(f"LoRA: {len(missing)} key(s) matched no parameter, e.g. {missing[:3]}")
        logger.info(f"LoRA: merged {merged} tensors (strength {strength})")
        return {"merged": merged, "missing": missing}


# ---------------------------------------------------------------------------
# run-time (un-merged) LoRA
# ---------------------------------------------------------------------------
def decode_lora_module_name(lora_name: str) -> str:
    """'lora_unet_blocks_0_self_attn_q' -> 'blocks.0.self_attn.q' is ambiguous in general; names made by
    `LoRANetwork` use '-' for '.' so that decoding is exact."""
    return lora_name.split("lora_", 1)[-1].replace("-", ".")


class LoRAModule(nn.Module):
    def __init__(self, name: str, base: nn.Linear, rank: int = 4, alpha: float = 1.0, multiplier: float = 1.0) -> None:
        super().__init__()
        self.lora_name, self.base = name, base
        self.down = nn.Linear(base.in_features, rank, bias=False)
        self.up = nn.Linear(rank, base.out_features, bias=False)
        nn.init.kaiming_uniform_(self.down.weight, a=5**0.5)
        nn.init.zeros_(self.up.weight)
        self.scale, self.multiplier, self.use_lora = alpha / rank, multiplier, True
        self.to(base.weight.device, base.weight.dtype if base.weight.dtype.is_floating_point else torch.bfloat16)

    @property
    def weight(self):  # model code reads `.weight` / `.bias` of its linears directly
        if not self.use_lora:
            return self.base.weight
        return self.base.weight + (self.up.weight @ self.down.weight * (self.scale * self.multiplier)).to(self.base.weight.dtype)

    @property
    def bias(self):
        return self.base.bias

    def set_use_lora(self, flag: bool) -> None:
        self.use_lora = flag

    def forward(self, x):
        y = self.base(x)
        if self.use_lora:
            y = y + self.up(self.down(x.to(self.down.weight.dtype))).to(y.dtype) * (self.scale * self.multiplier)
        return y


class LoRANetwork(nn.Module):
    def __init__(self, model: nn.Module, target_patterns: list[str], rank: int = 4, alpha: float = 1.0,
                 multiplier: float = 1.0) -> None:  # fmt: skip
        super().__init__()
        pats = [re.compile(p) for p in target_patterns]
        self.loras = nn.ModuleDict()
        for name, mod in list(model.named_modules()):
            if isinstance(mod, nn.Linear) and any(p.search(name) for p in pats):
                lora = LoRAModule("lora_" + name.replace(".", "-"), mod, rank, alpha, multiplier)
                parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
                setattr(parent, name.rsplit(".", 1)[-1], lora)
                self.loras[lora.lora_name] = lora
        if not self.loras:
            raise ValueError("no linear layer matched the LoRA target patterns")

    def set_multiplier(self, m: float) -> None:
        for l in self.loras.values():
            l.multiplier = m

    def set_use_lora(self, flag: bool) -> None:
        for l in self.loras.values():
            l.set_use_lora(flag)

    def load_weights(self, sd: dict) -> None:
        """State dict in kohya spelling: `<lora_name>.lora_down.weight` / `.lora_up.weight` / `.alpha`."""
        for name, l in self.loras.items():
            if f"{name}.lora_down.weight" in sd:
                l.down.weight.data.copy_(sd[f"{name}.lora_down.weight"])
                l.up.weight.data.copy_(sd[f"{name}.lora_up.weight"])
                if f"{name}.alpha" in sd:
                    l.scale = float(sd[f"{name}.alpha"]) / l.down.weight.shape[0]


def create_lora_network(model: nn.Module, target_patterns: list[str], rank: int = 4, alpha: float = 1.0,
                        multiplier: float = 1.0) -> LoRANetwork:  # fmt: skip
    return LoRANetwork(model, target_patterns, rank, alpha, multiplier)
