"""Wan2.1 text-to-video (1.3B or 14B): offline run, and the entry points `telefuser serve` loads.

    python examples/wan_video/wan21_text_to_video.py --model 14b --gpu_num 8 --prompt "a red fox in the snow"
    telefuser serve examples/wan_video/wan21_text_to_video.py -t t2v -g 8 -p 8000

Weights are read from `$TF_MODEL_ZOO_PATH/Wan2.1-T2V-{1.3B,14B}` (official or diffusers layout). With
`TFB_RANDOM_INIT=1` the same architecture is built with random weights, which is what the smoke tests and the
benchmarks use on machines without checkpoints.
"""

from __future__ import annotations

import os

import torch

from telefuser_b200.pipelines.wan.wan21_video import Wan21VideoPipeline
from telefuser_b200.utils.video import get_target_video_size_from_ratio, save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(
    name="wan21_t2v",
    model=os.environ.get("TFB_WAN21_MODEL", "1.3b"),  # "1.3b" | "14b"
    negative_prompt="overexposed, static, blurry details, subtitles, worst quality, low quality, JPEG artifacts, ugly, "
                    "deformed, extra fingers, poorly drawn hands, poorly drawn face, fused fingers, cluttered background",
    num_inference_steps=50,
    num_frames=81,
    resolution="480p",
    aspect_ratio="16:9",
    cfg_scale=5.0,
    sigma_shift=5.0,
    seed=42,
    target_fps=16,
)
PIPELINE_MANIFEST = {"tasks": ["t2v"], "media_type": "video", "required_inputs": {"t2v": ["prompt"]}}
_PRESETS = {"1.3b": ("Wan2.1-T2V-1.3B", "wan2.1-t2v-1.3b"), "14b": ("Wan2.1-T2V-14B", "wan2.1-t2v-14b")}


def layout_for(gpus: int) -> dict:
    """CFG-parallel pair x Ulysses: 2 GPUs split the guidance branches, 4 and 8 add sequence parallelism."""
    if gpus <= 1:
        return {}
    cfg = 2 if gpus % 2 == 0 else 1
    return dict(parallel_devices=list(range(gpus)), cfg_degree=cfg, sp_ulysses_degree=gpus // cfg)


def get_pipeline(parallelism: int = 1, model: str | None = None) -> Wan21VideoPipeline:
    folder, preset = _PRESETS[(model or PPL_CONFIG["model"]).lower()]
    if os.environ.get("TFB_RANDOM_INIT") == "1":
        device = "cuda" if torch.cuda.is_available() else "cpu"
        if os.environ.get("TFB_TINY") == "1":  # a few-thousand-parameter model of the same structure: CPU tests of the serving path
            return Wan21VideoPipeline.from_random_init("tiny", device=device, torch_dtype=torch.bfloat16 if device == "cuda" else torch.float32,
                                                       vae_dim=8, **layout_for(parallelism))  # fmt: skip
        return Wan21VideoPipeline.from_random_init(preset, device=device, torch_dtype=torch.bfloat16, **layout_for(parallelism))
    return Wan21VideoPipeline.from_pretrained(os.path.join(TF_MODEL_ZOO_PATH, folder), **layout_for(parallelism))


def run_with_file(pipeline, prompt: str, output_path: str, negative_prompt: str = PPL_CONFIG["negative_prompt"],
                  seed: int = PPL_CONFIG["seed"], num_inference_steps: int = PPL_CONFIG["num_inference_steps"],
                  num_frames: int = PPL_CONFIG["num_frames"], resolution: str = PPL_CONFIG["resolution"],
                  aspect_ratio: str = PPL_CONFIG["aspect_ratio"], cfg_scale: float = PPL_CONFIG["cfg_scale"],
                  sigma_shift: float = PPL_CONFIG["sigma_shift"], target_fps: int = PPL_CONFIG["target_fps"]):  # fmt: skip
    height, width = get_target_video_size_from_ratio(resolution, aspect_ratio)
    frames = pipeline(prompt=prompt, negative_prompt=negative_prompt, seed=seed, height=height, width=width,
                      num_frames=num_frames, num_inference_steps=num_inference_steps, cfg_scale=cfg_scale,
                      sigma_shift=sigma_shift)  # fmt: skip
    save_video(frames, output_path, fps=target_fps)
    return {"output_path": output_path, "num_frames": len(frames), "height": height, "width": width}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--model", default=PPL_CONFIG["model"], type=click.Choice(["1.3b", "14b"]))
    @click.option("--gpu_num", default=1, type=int)
    @click.option("--prompt", default="A red fox trotting through fresh snow at dawn, breath visible in the cold air.")
    @click.option("--output", default="work_dirs/wan21_t2v.mp4")
    @click.option("--steps", default=PPL_CONFIG["num_inference_steps"], type=int)
    @click.option("--resolution", default=PPL_CONFIG["resolution"])
    def main(model, gpu_num, prompt, output, steps, resolution):
        pipe = get_pipeline(gpu_num, model)
        try:
            print(run_with_file(pipe, prompt, output, num_inference_steps=steps, resolution=resolution))
        finally:
            pipe.close()

    main()
