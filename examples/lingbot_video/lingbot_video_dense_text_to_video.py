"""LingBot-Video dense 1.3B: text to image, text to video and image to video on one GPU (or `-g N` for Ulysses).

    python examples/lingbot_video/lingbot_video_dense_text_to_video.py --prompt "..." [--image first.png] [--num_frames 1]
    telefuser serve examples/lingbot_video/lingbot_video_dense_text_to_video.py -t t2v
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.lingbot_video import LingBotVideoPipeline

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="lingbot_video_dense_t2v", model_root=os.path.join(TF_MODEL_ZOO_PATH, "lingbot", "lingbot-video-dense-1.3b"),
                  num_frames=81, height=480, width=832, num_inference_steps=50, guidance_scale=3.0, shift=3.0, seed=42,
                  target_fps=24, supports_refiner=False)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v", "t2i"], "media_type": "video",
                     "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"], "t2i": ["prompt"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1) -> LingBotVideoPipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    return LingBotVideoPipeline.from_pretrained(PPL_CONFIG["model_root"], parallel_devices=devices,
                                                guidance_scale=PPL_CONFIG["guidance_scale"],
                                                num_inference_steps=PPL_CONFIG["num_inference_steps"], shift=PPL_CONFIG["shift"])  # fmt: skip


def run_with_file(pipeline, prompt: str, output_path: str, seed: int = PPL_CONFIG["seed"],
                  num_frames: int = PPL_CONFIG["num_frames"], height: int = PPL_CONFIG["height"],
                  width: int = PPL_CONFIG["width"], first_image_path: str | None = None, negative_prompt: str | None = None):  # fmt: skip
    """Same request handling as the MoE example (prompt files, one-frame requests saved as PNG); no refiner."""
    import importlib.util

    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("_lingbot_video_moe_example", os.path.join(here, "lingbot_video_moe_text_to_video.py"))
    moe = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(moe)
    moe.PPL_CONFIG = {**moe.PPL_CONFIG, "target_fps": PPL_CONFIG["target_fps"]}
    return moe.run_with_file(pipeline, prompt, output_path, seed=seed, num_frames=num_frames, height=height, width=width,
                             first_image_path=first_image_path, negative_prompt=negative_prompt, refine=False)  # fmt: skip


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--gpu_num", default=1, type=int)
    @click.option("--prompt", default="A red kite rising over a wheat field at dusk.")
    @click.option("--image", "image_path", default=None)
    @click.option("--num_frames", default=PPL_CONFIG["num_frames"], type=int)
    @click.option("--output", default="work_dirs/lingbot_video_dense.mp4")
    def main(gpu_num, prompt, image_path, num_frames, output):
        print(run_with_file(get_pipeline(gpu_num), prompt, output, num_frames=num_frames, first_image_path=image_path))

    main()
