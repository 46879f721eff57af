"""FLUX.2 [klein] text-to-image (4 steps, no guidance) with optional reference images.

    python examples/flux2_klein/flux2_klein_text_to_image.py --prompt "a brass telescope on a windowsill"
    telefuser serve examples/flux2_klein/flux2_klein_text_to_image.py -t t2i
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.flux2_klein.pipeline import Flux2KleinPipeline

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="flux2_klein_t2i", model_root=os.path.join(TF_MODEL_ZOO_PATH, "FLUX.2-klein-4B"),
                  num_inference_steps=4, cfg_scale=1.0, height=1024, width=1024, seed=42)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2i", "i2i"], "media_type": "image",
                     "required_inputs": {"t2i": ["prompt"], "i2i": ["prompt", "first_image_path"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1) -> Flux2KleinPipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    return Flux2KleinPipeline.from_pretrained(PPL_CONFIG["model_root"], parallel_devices=devices)


def run_with_file(pipeline, prompt: str, output_path: str, first_image_path: str | None = None,
                  seed: int = PPL_CONFIG["seed"], num_inference_steps: int = PPL_CONFIG["num_inference_steps"],
                  cfg_scale: float = PPL_CONFIG["cfg_scale"], height: int = PPL_CONFIG["height"],
                  width: int = PPL_CONFIG["width"]):  # fmt: skip
    refs = None
    if first_image_path:
        from PIL import Image

        refs = [Image.open(first_image_path).convert("RGB")]
    images = pipeline(prompt=prompt, seed=seed, height=height, width=width, cfg_scale=cfg_scale,
                      num_inference_steps=num_inference_steps, reference_images=refs)  # fmt: skip
    images[0].save(output_path)
    return {"output_path": output_path}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="A brass telescope on a sunlit windowsill, shallow depth of field.")
    @click.option("--output", default="work_dirs/flux2_klein.png")
    def main(prompt, output):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        print(run_with_file(get_pipeline(), prompt, output))

    main()
