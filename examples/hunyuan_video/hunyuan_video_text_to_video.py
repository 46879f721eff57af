"""HunyuanVideo-1.5 text-to-video / image-to-video, optionally with the 720p super-resolution pass: offline run and
`telefuser serve` entry points.

    python examples/hunyuan_video/hunyuan_video_text_to_video.py --prompt "a kite over dunes" --gpu_num 8
    telefuser serve examples/hunyuan_video/hunyuan_video_text_to_video.py -t t2v -g 8

Model root (`$TF_MODEL_ZOO_PATH/HunyuanVideo-1.5`, official layout): `transformer/<version>/`, `vae/`,
`text_encoder/llm/`, `text_encoder/Glyph-SDXL-v2/` + `text_encoder/byt5-small/`, `vision_encoder/siglip/` (image to
video), `upsampler/720p_sr_distilled/` and `transformer/720p_sr_distilled/` (super-resolution).
"""

from __future__ import annotations

import glob
import os

import torch

from telefuser_b200.core.config import ParallelConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.pipelines.hunyuan_video_1_5.pipeline import (HunyuanTextEncodingStage, HunyuanVideo15Pipeline,
                                                                 HunyuanVideo15PipelineConfig)
from telefuser_b200.utils.video import save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="hunyuan_video_15", model_root=os.path.join(TF_MODEL_ZOO_PATH, "HunyuanVideo-1.5"),
                  transformer_version="480p_t2v", i2v_transformer_version="480p_i2v", sr_version="720p_sr_distilled",
                  enable_sr=False, height=480, width=848, num_frames=121, num_inference_steps=50, cfg_scale=6.0, sigma_shift=5.0,
                  seed=42, target_fps=24, negative_prompt="")  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v"], "media_type": "video",
                     "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"]}}  # fmt: skip


def _weights(folder: str) -> list:
    return sorted(glob.glob(os.path.join(folder, "*.safetensors")))


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"], image_to_video: bool = False):
    from telefuser_b200.models.hunyuan_video_dit import HunyuanVideoDiT
    from telefuser_b200.models.hunyuan_video_encoders import (HunyuanVideoByT5Encoder, HunyuanVideoImageEncoder,
                                                              HunyuanVideoTextEncoder)
    from telefuser_b200.models.hunyuan_video_vae import HunyuanVideoVAE, SRTo720pUpsampler

    version = PPL_CONFIG["i2v_transformer_version" if image_to_video else "transformer_version"]
    mm = ModuleManager(torch_dtype=torch.bfloat16, device="cpu")
    mm.load_model(_weights(os.path.join(model_root, "transformer", version)), name="hunyuan_video_dit", model_class=HunyuanVideoDiT)
    upsampler = None
    if PPL_CONFIG["enable_sr"]:
        mm.load_model(_weights(os.path.join(model_root, "transformer", PPL_CONFIG["sr_version"])), name="hunyuan_video_sr_dit",
                      model_class=HunyuanVideoDiT)  # fmt: skip
        upsampler = SRTo720pUpsampler.from_pretrained(os.path.join(model_root, "upsampler", PPL_CONFIG["sr_version"])).to("cuda")
    vae = HunyuanVideoVAE.from_pretrained(os.path.join(model_root, "vae"), torch_dtype=torch.bfloat16).to("cuda")
    llm = HunyuanVideoTextEncoder.from_pretrained(os.path.join(model_root, "text_encoder", "llm"), torch_dtype=torch.bfloat16)
    byt5 = None
    if os.path.isdir(os.path.join(model_root, "text_encoder", "Glyph-SDXL-v2")):
        byt5 = HunyuanVideoByT5Encoder.from_pretrained(os.path.join(model_root, "text_encoder"), device="cuda")
    vision = None
    if image_to_video:
        enc = HunyuanVideoImageEncoder.from_pretrained(os.path.join(model_root, "vision_encoder", "siglip"), device="cuda")
        vision = lambda img: enc.encode_images(img).last_hidden_state  # noqa: E731
    cfg = HunyuanVideo15PipelineConfig()
    cfg.sigma_shift = PPL_CONFIG["sigma_shift"]
    if parallelism > 1:
        cfg.dit_config.parallel_config = ParallelConfig(device_ids=list(range(parallelism)), sp_ulysses_degree=parallelism)
        cfg.enable_denoising_parallel = True
    pipe = HunyuanVideo15Pipeline(device="cuda", torch_dtype=torch.bfloat16)
    pipe.init(mm, cfg, text_stage=HunyuanTextEncodingStage(llm.to("cuda"), byt5), vision_stage=vision, vae=vae, upsampler=upsampler)
    return pipe


def run_with_file(pipeline, prompt: str, output_path: str, first_image_path: str = "",
                  negative_prompt: str = PPL_CONFIG["negative_prompt"], seed: int = PPL_CONFIG["seed"],
                  height: int = PPL_CONFIG["height"], width: int = PPL_CONFIG["width"], num_frames: int = PPL_CONFIG["num_frames"],
                  num_inference_steps: int = PPL_CONFIG["num_inference_steps"], cfg_scale: float = PPL_CONFIG["cfg_scale"]):  # fmt: skip
    from PIL import Image

    image = Image.open(first_image_path).convert("RGB") if first_image_path else None
    frames = pipeline(prompt, negative_prompt=negative_prompt, input_image=image, seed=seed, height=height, width=width,
                      num_frames=num_frames, cfg_scale=cfg_scale, num_inference_steps=num_inference_steps,
                      enable_sr=PPL_CONFIG["enable_sr"])  # fmt: skip
    save_video(frames, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path, "num_frames": len(frames)}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="A red kite pulling hard over wind-carved dunes, low sun, sand streaming off the crests.")
    @click.option("--image_path", default="")
    @click.option("--output", default="work_dirs/hunyuan_video.mp4")
    @click.option("--gpu_num", default=1, type=int)
    def main(prompt, image_path, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        pipe = get_pipeline(gpu_num, image_to_video=bool(image_path))
        try:
            print(run_with_file(pipe, prompt, output, first_image_path=image_path))
        finally:
            pipe.close()

    main()
