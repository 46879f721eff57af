"""LingBot-Video (128-expert MoE DiT) text-to-video; `-g 8` runs CFG x Ulysses with the experts spread over the
same ranks (expert parallelism by peer-memory dispatch / combine).

    python examples/lingbot_video/lingbot_video_moe_text_to_video.py --gpu_num 8 --prompt "..."
    telefuser serve examples/lingbot_video/lingbot_video_moe_text_to_video.py -t t2v -g 8
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.lingbot_video.pipeline import LingBotVideoPipeline, LingBotVideoRequest
from telefuser_b200.utils.video import save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="lingbot_video_moe_t2v", model_root=os.path.join(TF_MODEL_ZOO_PATH, "lingbot", "lingbot-video-moe"),
                  num_frames=81, height=480, width=832, num_inference_steps=50, guidance_scale=3.0, shift=3.0, seed=42,
                  target_fps=16)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v"], "media_type": "video", "required_inputs": {"t2v": ["prompt"]}}


def get_pipeline(parallelism: int = 1) -> LingBotVideoPipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    return LingBotVideoPipeline.from_pretrained(PPL_CONFIG["model_root"], parallel_devices=devices,
                                                expert_parallel=parallelism > 1,
                                                guidance_scale=PPL_CONFIG["guidance_scale"],
                                                num_inference_steps=PPL_CONFIG["num_inference_steps"], shift=PPL_CONFIG["shift"])  # fmt: skip


def run_with_file(pipeline, prompt: str, output_path: str, seed: int = PPL_CONFIG["seed"],
                  num_frames: int = PPL_CONFIG["num_frames"], height: int = PPL_CONFIG["height"],
                  width: int = PPL_CONFIG["width"]):  # fmt: skip
    result = pipeline.generate(LingBotVideoRequest(caption=prompt, num_frames=num_frames, height=height, width=width, seed=seed))
    save_video(result.output, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--gpu_num", default=1, type=int)
    @click.option("--prompt", default="A paper boat drifting along a rain-filled gutter, low camera following it.")
    @click.option("--output", default="work_dirs/lingbot_video.mp4")
    def main(gpu_num, prompt, output):
        pipe = get_pipeline(gpu_num)
        print(run_with_file(pipe, prompt, output))

    main()
