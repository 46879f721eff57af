"""Feature-cache benchmark: Wan2.1 text-to-video with and without the adaptive Taylor cache.

    python benchmarks/feature_cache_bench.py --model-root $TF_MODEL_ZOO_PATH/Wan2.1-T2V-1.3B --steps 40 --cfg-scale 6
    python benchmarks/feature_cache_bench.py --random-init --preset wan2.1-t2v-1.3b --steps 40       # no checkpoint needed

Four runs from the same seed: no cache (the reference video), then the cache with Taylor order 0 (reuse the last
residual), 1 and 2. Each row reports the wall time of the pipeline call, the number of denoising steps that ran the
transformer (the others were extrapolated), the speed-up over the uncached run, and PSNR / SSIM of its video against
the uncached one. One JSON line per row and a final summary line.

Role: benchmarks/feature_cache/wan21_1_3b_ada_taylor_cache.py of the reference (same four configurations, same
similarity measures except LPIPS, which needs a downloaded network).
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def build_pipeline(a):
    from telefuser_b200.pipelines.wan.wan21_video import Wan21VideoPipeline

    device = a.device if a.device != "auto" else ("cuda:0" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    if a.random_init or not a.model_root:
        preset = a.preset
        if preset == "tiny":
            from telefuser_b200.models.wan_dit import WanModelConfig

            preset = WanModelConfig(dim=256, ffn_dim=512, num_heads=2, num_layers=2, text_dim=256)
        return Wan21VideoPipeline.from_random_init(preset, device=device, torch_dtype=dtype, seed=a.seed), device
    return Wan21VideoPipeline.from_pretrained(a.model_root, device=device, torch_dtype=dtype), device


def run_once(pipe, a, device: str):
    if device.startswith("cuda"):
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    video = pipe(prompt=a.prompt, negative_prompt=a.negative_prompt, seed=a.seed, height=a.height, width=a.width,
                 num_frames=a.frames, num_inference_steps=a.steps, cfg_scale=a.cfg_scale, sigma_shift=a.sigma_shift,
                 output_type="pt")  # fmt: skip
    if device.startswith("cuda"):
        torch.cuda.synchronize()
    return video[0].float().cpu(), time.perf_counter() - t0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-root", default="")
    ap.add_argument("--random-init", action="store_true")
    ap.add_argument("--preset", default="wan2.1-t2v-1.3b")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--prompt", default="A cat playing the piano in a sunlit room, close-up of paws on the keys.")
    ap.add_argument("--negative-prompt", default="blurry, static, low quality")
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--cfg-scale", type=float, default=6.0)
    ap.add_argument("--sigma-shift", type=float, default=5.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--taylor-threshold", type=int, default=2)
    ap.add_argument("--orders", default="0,1,2")
    ap.add_argument("--model-type", default="", help="name under which calibrated cache parameters are stored")
    a = ap.parse_args(argv)

    from telefuser_b200.core.config import FeatureCacheConfig
    from telefuser_b200.utils.quality import psnr, ssim

    pipe, device = build_pipeline(a)
    stage = pipe.denoise_stage
    if hasattr(stage, "processes"):
        raise SystemExit("run this benchmark on one GPU (the cache setting is applied to the in-process stage)")
    rows = []
    try:
        stage.model_runtime_config.feature_cache_config = FeatureCacheConfig(enabled=False)
        run_once(pipe, a, device)  # warm-up (kernel loading, allocator)
        ref, t_ref = run_once(pipe, a, device)
        rows.append({"config": "no cache", "seconds": round(t_ref, 3), "computed_steps": a.steps, "speedup": 1.0})
        print(json.dumps(rows[-1]), flush=True)
        for order in [int(x) for x in a.orders.split(",") if x != ""]:
            stage.model_runtime_config.feature_cache_config = FeatureCacheConfig(
                enabled=True, model_type=a.model_type or (a.preset if isinstance(a.preset, str) else "wan"),
                n_derivatives=order, taylor_threshold=a.taylor_threshold)  # fmt: skip
            video, t = run_once(pipe, a, device)
            cache = stage.dit.feature_cache
            computed = len(cache.get_compute_steps()) if hasattr(cache, "get_compute_steps") else None
            rows.append({"config": f"adaptive Taylor cache, order {order}", "seconds": round(t, 3), "computed_steps": computed,
                         "speedup": round(t_ref / t, 3), "psnr_db": round(psnr(video, ref), 2), "ssim": round(ssim(video, ref), 4),
                         "finite": bool(torch.isfinite(video).all())})  # fmt: skip
            print(json.dumps(rows[-1]), flush=True)
    finally:
        pipe.close()
    print(json.dumps({"summary": rows, "steps": a.steps, "frames": a.frames, "height": a.height, "width": a.width,
                      "cfg_scale": a.cfg_scale, "device": device}))  # fmt: skip
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
