"""LongCat-Video text-to-video / image-to-video / video continuation: offline run and `telefuser serve` entry points.

    python examples/longcat_video/longcat_video_text_to_video.py --prompt "a lighthouse in a storm" --gpu_num 4
    telefuser serve examples/longcat_video/longcat_video_text_to_video.py -t t2v -g 4

Model root (`$TF_MODEL_ZOO_PATH/LongCat-Video`): `dit/diffusion_pytorch_model*.safetensors`, `text_encoder/`
(UMT5-XXL weights), `tokenizer/`, and the Wan2.1 VAE file given by `vae_path`.
"""

from __future__ import annotations

import glob
import os

import torch

from telefuser_b200.core.config import ParallelConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.pipelines.longcat_video.pipeline import LongCatVideoPipeline, LongCatVideoPipelineConfig
from telefuser_b200.utils.video import get_target_video_size_from_ratio, save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(
    name="longcat_video",
    model_root=os.path.join(TF_MODEL_ZOO_PATH, "LongCat-Video"),
    vae_path=os.path.join(TF_MODEL_ZOO_PATH, "Wan2.1-T2V-1.3B", "Wan2.1_VAE.pth"),
    negative_prompt="bright tones, overexposed, static, blurred details, subtitles, worst quality, low quality, ugly, deformed",
    num_inference_steps=50, num_frames=93, resolution="480p", aspect_ratio="16:9", cfg_scale=4.0, sigma_shift=12.0, seed=42,
    target_fps=15, tiled=True,
)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v", "vc"], "media_type": "video",
                     "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"], "vc": ["ref_video_path"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> LongCatVideoPipeline:
    from transformers import AutoTokenizer

    mm = ModuleManager(torch_dtype=torch.bfloat16, device="cpu")
    mm.load_model(sorted(glob.glob(os.path.join(model_root, "dit", "*.safetensors"))))
    mm.load_model(sorted(glob.glob(os.path.join(model_root, "text_encoder", "*.safetensors"))))
    mm.load_model(PPL_CONFIG["vae_path"])
    mm.add_module(AutoTokenizer.from_pretrained(os.path.join(model_root, "tokenizer")), "tokenizer")
    cfg = LongCatVideoPipelineConfig()
    if parallelism > 1:
        cfg.dit_config.parallel_config = ParallelConfig(device_ids=list(range(parallelism)), sp_ulysses_degree=parallelism)
        cfg.enable_denoising_parallel = True
    pipe = LongCatVideoPipeline(device="cuda", torch_dtype=torch.bfloat16)
    pipe.init(mm, cfg)
    return pipe


def run_with_file(pipeline, prompt: str = "", output_path: str = "output.mp4", first_image_path: str = "",
                  ref_video_path: str = "", negative_prompt: str = PPL_CONFIG["negative_prompt"], seed: int = PPL_CONFIG["seed"],
                  num_inference_steps: int = PPL_CONFIG["num_inference_steps"], num_frames: int = PPL_CONFIG["num_frames"],
                  resolution: str = PPL_CONFIG["resolution"], aspect_ratio: str = PPL_CONFIG["aspect_ratio"],
                  cfg_scale: float = PPL_CONFIG["cfg_scale"]):  # fmt: skip
    from PIL import Image

    from telefuser_b200.utils.video import VideoData

    height, width = get_target_video_size_from_ratio(resolution, aspect_ratio)
    image = Image.open(first_image_path).convert("RGB") if first_image_path else None
    video = VideoData(ref_video_path, height=height, width=width).raw_data() if ref_video_path else None
    frames = pipeline(prompt=prompt, negative_prompt=negative_prompt, input_image=image, input_video=video, seed=seed,
                      height=height, width=width, num_frames=num_frames, cfg_scale=cfg_scale,
                      num_inference_steps=num_inference_steps, tiled=PPL_CONFIG["tiled"], sigma_shift=PPL_CONFIG["sigma_shift"])  # fmt: skip
    save_video(frames, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path, "num_frames": len(frames)}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="A lighthouse on a cliff in a winter storm, waves breaking far below, slow aerial orbit.")
    @click.option("--image_path", default="")
    @click.option("--output", default="work_dirs/longcat_video.mp4")
    @click.option("--gpu_num", default=1, type=int)
    def main(prompt, image_path, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        pipe = get_pipeline(gpu_num)
        try:
            print(run_with_file(pipe, prompt, output, first_image_path=image_path))
        finally:
            pipe.close()

    main()
