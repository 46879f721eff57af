"""Wan2.1 image-to-video and first / last-frame-to-video (14B, 480p or 720p): offline run and `telefuser serve` entry
points (tasks i2v, fl2v).

    python examples/wan_video/wan21_image_to_video.py --image first.png --prompt "the camera slowly pushes in" --gpu_num 8
    python examples/wan_video/wan21_image_to_video.py --image first.png --end_image last.png      # interpolate between two frames
    telefuser serve examples/wan_video/wan21_image_to_video.py -t i2v -g 8

Weights: `$TF_MODEL_ZOO_PATH/Wan2.1-I2V-14B-{480P,720P}` (or `Wan2.1-FLF2V-14B-720P` for the two-frame task); the folder
holds the DiT shards, the VAE, the UMT5 text encoder and the CLIP image encoder.
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.wan.wan21_video import Wan21VideoPipeline
from telefuser_b200.utils.video import get_target_video_size_from_ratio, save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(
    name="wan21_i2v",
    model_root=os.path.join(TF_MODEL_ZOO_PATH, os.environ.get("TFB_WAN21_I2V_MODEL", "Wan2.1-I2V-14B-480P")),
    negative_prompt="overexposed, static, blurry details, subtitles, worst quality, low quality, JPEG artifacts, ugly, "
                    "deformed, extra fingers, poorly drawn hands, poorly drawn face, fused fingers, cluttered background",
    num_inference_steps=40, num_frames=81, resolution="480p", aspect_ratio="16:9", cfg_scale=5.0, sigma_shift=3.0, seed=42,
    target_fps=16, tiled=True,
)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["i2v", "fl2v"], "media_type": "video",
                     "required_inputs": {"i2v": ["first_image_path"], "fl2v": ["first_image_path", "last_image_path"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> Wan21VideoPipeline:
    kw = {}
    if parallelism > 1:
        cfg = 2 if parallelism % 2 == 0 else 1
        kw = dict(parallel_devices=list(range(parallelism)), cfg_degree=cfg, sp_ulysses_degree=parallelism // cfg)
    return Wan21VideoPipeline.from_pretrained(model_root, **kw)


def run_with_file(pipeline, first_image_path: str, output_path: str, prompt: str = "", last_image_path: str = "",
                  negative_prompt: str = PPL_CONFIG["negative_prompt"], seed: int = PPL_CONFIG["seed"],
                  num_inference_steps: int = PPL_CONFIG["num_inference_steps"], num_frames: int = PPL_CONFIG["num_frames"],
                  resolution: str = PPL_CONFIG["resolution"], aspect_ratio: str = PPL_CONFIG["aspect_ratio"],
                  cfg_scale: float = PPL_CONFIG["cfg_scale"]):  # fmt: skip
    from PIL import Image

    height, width = get_target_video_size_from_ratio(resolution, aspect_ratio)
    first = Image.open(first_image_path).convert("RGB")
    last = Image.open(last_image_path).convert("RGB") if last_image_path else None
    frames = pipeline(prompt=prompt, negative_prompt=negative_prompt, input_image=first, end_image=last, seed=seed, height=height,
                      width=width, num_frames=num_frames, num_inference_steps=num_inference_steps, cfg_scale=cfg_scale,
                      sigma_shift=PPL_CONFIG["sigma_shift"], tiled=PPL_CONFIG["tiled"])  # fmt: skip
    save_video(frames, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path, "num_frames": len(frames), "height": height, "width": width}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--image", "image_path", required=True)
    @click.option("--end_image", default="")
    @click.option("--prompt", default="The camera slowly pushes in while the scene comes to life, natural motion.")
    @click.option("--output", default="work_dirs/wan21_i2v.mp4")
    @click.option("--gpu_num", default=1, type=int)
    def main(image_path, end_image, prompt, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        pipe = get_pipeline(gpu_num)
        try:
            print(run_with_file(pipe, image_path, output, prompt=prompt, last_image_path=end_image))
        finally:
            pipe.close()

    main()
