"""Extract a LoRA from the difference of two checkpoints (tuned - base) by truncated SVD.

    python -m telefuser_b200.tools.lora_extract --base base.safetensors --tuned tuned.safetensors \
        -o lora.safetensors --rank 32 [--min_diff 1e-6] [--diff_only_small]

For every 2-D weight whose difference is not negligible: `diff ~= up @ down` with
`up = U[:, :r] * sqrt(S[:r])`, `down = sqrt(S[:r]) * Vt[:r]`, stored as `<key>.lora_up.weight`,
`<key>.lora_down.weight` and `<key>.alpha = r` (scale 1). Differences of 1-D tensors (biases, norms,
modulation tables) are stored as `.diff_b` / `.diff` entries, which the loader adds directly.
Role parity: tools/convert/lora_extractor.py.
"""

from __future__ import annotations

import argparse

import torch

from telefuser_b200.utils.logging import logger
from telefuser_b200.utils.model_weight import load_state_dict, save_state_dict


def extract_lora(base: dict, tuned: dict, rank: int = 32, min_diff: float = 1e-6, device: str = "cpu") -> dict:
    out = {}
    for k, wt in tuned.items():
        wb = base.get(k)
        if wb is None or wb.shape != wt.shape or not wt.is_floating_point():
            continue
        diff = wt.float().to(device) - wb.float().to(device)
        if diff.abs().max().item() <= min_diff:
            continue
        if diff.dim() == 2 and k.endswith(".weight"):
            stem = k[: -len(".weight")]
            r = min(rank, *diff.shape)
            U, S, Vh = torch.linalg.svd(diff, full_matrices=False)
            root = S[:r].sqrt()
            out[f"{stem}.lora_up.weight"] = (U[:, :r] * root).contiguous().cpu()
            out[f"{stem}.lora_down.weight"] = (root[:, None] * Vh[:r]).contiguous().cpu()
            out[f"{stem}.alpha"] = torch.tensor(float(r))
        elif k.endswith(".bias"):
            out[k[: -len(".bias")] + ".diff_b"] = diff.cpu()
        elif k.endswith(".weight"):
            out[k[: -len(".weight")] + ".diff"] = diff.cpu()
        elif k.endswith(".modulation"):
            out[k[: -len(".modulation")] + ".diff_m"] = diff.cpu()
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--base", required=True)
    p.add_argument("--tuned", required=True)
    p.add_argument("-o", "--output", required=True)
    p.add_argument("--rank", type=int, default=32)
    p.add_argument("--min_diff", type=float, default=1e-6)
    p.add_argument("--device", default="cpu")
    a = p.parse_args(argv)
    lora = extract_lora(load_state_dict(a.base), load_state_dict(a.tuned), a.rank, a.min_diff, a.device)
    save_state_dict(lora, a.output)
    logger.info(f"extracted {len(lora)} LoRA tensors at rank {a.rank}")
    return len(lora)


if __name__ == "__main__":
    main()
