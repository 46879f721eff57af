"""Z-Image-Turbo text-to-image (9 steps, no guidance): offline run and `telefuser serve` entry points (task t2i).

    python examples/z_image/z_image_turbo_text_to_image.py --prompt "a paper boat on a puddle, macro"
    telefuser serve examples/z_image/z_image_turbo_text_to_image.py -t t2i

Model root (`$TF_MODEL_ZOO_PATH/Z-Image-Turbo`, diffusers layout): `transformer/`, `vae/`, `text_encoder/`, `tokenizer/`.
"""

from __future__ import annotations

import glob
import os

import torch

from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.pipelines.z_image.pipeline import ZImagePipeline, ZImagePipelineConfig

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="z_image_turbo_t2i", model_root=os.path.join(TF_MODEL_ZOO_PATH, "Z-Image-Turbo"), seed=42, cfg_scale=0.0,
                  num_inference_steps=9, height=1024, width=1024)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2i"], "media_type": "image", "required_inputs": {"t2i": ["prompt"]}}


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> ZImagePipeline:
    from transformers import AutoModelForCausalLM, AutoTokenizer

    from telefuser_b200.models.autoencoder_kl import AutoencoderKL
    from telefuser_b200.models.hf_text_encoders import ZImageTextEncoder

    mm = ModuleManager(torch_dtype=torch.bfloat16, device="cpu")
    mm.load_model(sorted(glob.glob(os.path.join(model_root, "transformer", "*.safetensors"))))
    mm.load_model(os.path.join(model_root, "vae"), name="z_image_vae", model_class=AutoencoderKL)
    lm = AutoModelForCausalLM.from_pretrained(os.path.join(model_root, "text_encoder"), torch_dtype=torch.bfloat16)
    mm.add_module(ZImageTextEncoder(lm), "text_encoder")
    mm.add_module(AutoTokenizer.from_pretrained(os.path.join(model_root, "tokenizer")), "tokenizer")
    pipe = ZImagePipeline(device="cuda", torch_dtype=torch.bfloat16)
    pipe.init(mm, ZImagePipelineConfig())
    return pipe


def run_with_file(pipeline, prompt: str, output_path: str, negative_prompt: str = "", seed: int = PPL_CONFIG["seed"],
                  num_inference_steps: int = PPL_CONFIG["num_inference_steps"], cfg_scale: float = PPL_CONFIG["cfg_scale"],
                  height: int = PPL_CONFIG["height"], width: int = PPL_CONFIG["width"]):  # fmt: skip
    images = pipeline(prompt, negative_prompt=negative_prompt, seed=seed, height=height, width=width, cfg_scale=cfg_scale,
                      num_inference_steps=num_inference_steps)  # fmt: skip
    images[0].save(output_path)
    return {"output_path": output_path}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="A folded paper boat on a rain puddle, macro, city lights reflected in the water.")
    @click.option("--output", default="work_dirs/z_image_turbo.png")
    def main(prompt, output):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        print(run_with_file(get_pipeline(), prompt, output))

    main()
