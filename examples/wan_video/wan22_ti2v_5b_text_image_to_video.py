"""Wan2.2 TI2V 5B (one DiT, 48-channel VAE with 16x spatial compression): text-to-video, or image-to-video when a
first frame is given; 704 x 1280, 121 frames at 24 fps.

    python examples/wan_video/wan22_ti2v_5b_text_image_to_video.py --prompt "a sea turtle gliding over a reef"
    telefuser serve examples/wan_video/wan22_ti2v_5b_text_image_to_video.py -t t2v -g 4

Weights: `$TF_MODEL_ZOO_PATH/Wan2.2-TI2V-5B` (DiT shards, `Wan2.2_VAE.pth` or `vae/`, UMT5 encoder).
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.wan.wan22_video import Wan22TI2VPipeline
from telefuser_b200.utils.video import save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(
    name="wan22_ti2v_5b", model_root=os.path.join(TF_MODEL_ZOO_PATH, "Wan2.2-TI2V-5B"),
    negative_prompt="overly saturated colors, overexposed, static, blurry details, subtitles, worst quality, low quality, "
                    "JPEG compression artifacts, ugly, deformed, extra fingers, static frames, cluttered background",
    num_inference_steps=50, num_frames=121, height=704, width=1280, cfg_scale=5.0, sigma_shift=5.0, seed=42, target_fps=24,
)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v"], "media_type": "video",
                     "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> Wan22TI2VPipeline:
    kw = {}
    if parallelism > 1:
        cfg = 2 if parallelism % 2 == 0 else 1
        kw = dict(parallel_devices=list(range(parallelism)), cfg_degree=cfg, sp_ulysses_degree=parallelism // cfg)
    return Wan22TI2VPipeline.from_pretrained(model_root, **kw)


def run_with_file(pipeline, prompt: str, output_path: str, first_image_path: str = "",
                  negative_prompt: str = PPL_CONFIG["negative_prompt"], seed: int = PPL_CONFIG["seed"],
                  num_inference_steps: int = PPL_CONFIG["num_inference_steps"], num_frames: int = PPL_CONFIG["num_frames"],
                  height: int = PPL_CONFIG["height"], width: int = PPL_CONFIG["width"], cfg_scale: float = PPL_CONFIG["cfg_scale"]):  # fmt: skip
    from PIL import Image

    image = Image.open(first_image_path).convert("RGB") if first_image_path else None
    frames = pipeline(prompt=prompt, negative_prompt=negative_prompt, input_image=image, seed=seed, height=height, width=width,
                      num_frames=num_frames, num_inference_steps=num_inference_steps, cfg_scale=cfg_scale,
                      sigma_shift=PPL_CONFIG["sigma_shift"])  # fmt: skip
    save_video(frames, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path, "num_frames": len(frames)}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="A sea turtle gliding over a sunlit coral reef, shafts of light, slow tracking shot.")
    @click.option("--image_path", default="")
    @click.option("--output", default="work_dirs/wan22_ti2v.mp4")
    @click.option("--gpu_num", default=1, type=int)
    def main(prompt, image_path, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        pipe = get_pipeline(gpu_num)
        try:
            print(run_with_file(pipe, prompt, output, first_image_path=image_path))
        finally:
            pipe.close()

    main()
