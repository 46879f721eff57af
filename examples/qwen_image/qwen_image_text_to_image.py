"""Qwen-Image text-to-image: offline run and `telefuser serve` entry points (task t2i).

    python examples/qwen_image/qwen_image_text_to_image.py --prompt "a tram in Lisbon, watercolor"
    telefuser serve examples/qwen_image/qwen_image_text_to_image.py -t t2i -g 2
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.qwen_image.pipeline import QwenImagePipeline

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="qwen_image_t2i", model_root=os.path.join(TF_MODEL_ZOO_PATH, "Qwen-Image"), num_inference_steps=40,
                  cfg_scale=4.0, height=1328, width=1328, seed=42, negative_prompt=" ")  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2i"], "media_type": "image", "required_inputs": {"t2i": ["prompt"]}}


def get_pipeline(parallelism: int = 1) -> QwenImagePipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    return QwenImagePipeline.from_pretrained(PPL_CONFIG["model_root"], parallel_devices=devices)


def run_with_file(pipeline, prompt: str, output_path: str, negative_prompt: str = PPL_CONFIG["negative_prompt"],
                  seed: int = PPL_CONFIG["seed"], num_inference_steps: int = PPL_CONFIG["num_inference_steps"],
                  cfg_scale: float = PPL_CONFIG["cfg_scale"], height: int = PPL_CONFIG["height"],
                  width: int = PPL_CONFIG["width"]):  # fmt: skip
    from PIL import Image

    image = pipeline(prompt=prompt, negative_prompt=negative_prompt, cfg_scale=cfg_scale, seed=seed, height=height, width=width,
                     num_inference_steps=num_inference_steps)  # fmt: skip
    arr = ((image[0].float().cpu().clamp(-1, 1) + 1) * 127.5).round().byte()
    arr = arr[:, 0] if arr.ndim == 4 else arr  # the video VAE returns [C, 1, H, W]
    Image.fromarray(arr.permute(1, 2, 0).numpy()).save(output_path)
    return {"output_path": output_path}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="A yellow tram climbing a steep Lisbon street, loose watercolor, morning light.")
    @click.option("--output", default="work_dirs/qwen_image.png")
    @click.option("--gpu_num", default=1, type=int)
    def main(prompt, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        print(run_with_file(get_pipeline(gpu_num), prompt, output))

    main()
