"""Wan2.2 A14B text-to-video as a service pipeline with the cross-request latent cache.

    telefuser serve examples/wan_video/wan22_14b_text_to_video_service.py -t t2v -g 8 --enable-latent-cache

`run_with_file` forwards `latent_data` (a resume point found by the service's latent cache for a similar earlier
request) to the pipeline and returns the new latent snapshots as `latent_payload`, which the service stores.
`CACHE_CONFIG` overrides the service's cache settings for this pipeline.
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.wan.wan22_video import Wan22VideoPipeline
from telefuser_b200.utils.video import get_target_video_size_from_ratio, save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(
    name="wan22_A14B_t2v_service",
    model_root=os.path.join(TF_MODEL_ZOO_PATH, "Wan2.2-T2V-A14B"),
    negative_prompt="overly saturated colors, overexposed, static, blurry details, subtitles, worst quality, low quality, "
                    "JPEG compression artifacts, ugly, deformed, extra fingers, static frames, cluttered background",
    num_inference_steps=40,
    num_frames=81,
    resolution="720p",
    aspect_ratio="16:9",
    cfg_scale_high=5.0,
    cfg_scale_low=5.0,
    sigma_shift=5.0,
    boundary=0.9,
    sample_solver="euler",
    seed=42,
    target_fps=16,
)
CACHE_CONFIG = dict(
    enable_latent_cache=True,
    latent_cache_dir=os.getenv("TELEFUSER_LATENT_CACHE_DIR", "./latent_cache/wan22_t2v"),
    cache_mode=os.getenv("TELEFUSER_CACHE_MODE", "readwrite"),
)
PIPELINE_MANIFEST = {"tasks": ["t2v"], "media_type": "video", "required_inputs": {"t2v": ["prompt"]}}


def get_pipeline(parallelism: int = 1) -> Wan22VideoPipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    return Wan22VideoPipeline.from_pretrained(PPL_CONFIG["model_root"], parallel_devices=devices,
                                              sample_solver=PPL_CONFIG["sample_solver"])  # fmt: skip


def run_with_file(pipeline, prompt: str, output_path: str, negative_prompt: str = PPL_CONFIG["negative_prompt"],
                  seed: int = PPL_CONFIG["seed"], num_inference_steps: int = PPL_CONFIG["num_inference_steps"],
                  num_frames: int = PPL_CONFIG["num_frames"], resolution: str = PPL_CONFIG["resolution"],
                  aspect_ratio: str = PPL_CONFIG["aspect_ratio"], latent_data: dict | None = None):  # fmt: skip
    height, width = get_target_video_size_from_ratio(resolution, aspect_ratio)
    out = pipeline(prompt=prompt, negative_prompt=negative_prompt, seed=seed, height=height, width=width,
                   num_frames=num_frames, num_inference_steps=num_inference_steps, sigma_shift=PPL_CONFIG["sigma_shift"],
                   cfg_scale_high=PPL_CONFIG["cfg_scale_high"], cfg_scale_low=PPL_CONFIG["cfg_scale_low"],
                   boundary=PPL_CONFIG["boundary"], latent_data=latent_data)  # fmt: skip
    frames, payload = out if isinstance(out, tuple) else (out, None)
    save_video(frames, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path, "latent_payload": payload}
