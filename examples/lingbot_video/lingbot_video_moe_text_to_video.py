"""LingBot-Video (128-expert MoE DiT, 30B-A3B) text / image to video, with the optional high-resolution refiner pass.
`-g 8` runs CFG x Ulysses with the experts spread over the same ranks (expert parallelism by peer-memory dispatch /
combine).

    python examples/lingbot_video/lingbot_video_moe_text_to_video.py --gpu_num 8 --prompt "..." [--refine]
    python examples/lingbot_video/lingbot_video_moe_text_to_video.py --prompt rewritten_prompt.json
    telefuser serve examples/lingbot_video/lingbot_video_moe_text_to_video.py -t t2v -g 8

`--prompt` is a caption or the JSON file a prompt rewriter wrote (structured caption + duration). A request of one
frame (task t2i) is saved as a PNG. With `--refine` the base video is resampled to `refiner_height x refiner_width`,
noised to `refiner_t_thresh` and denoised by the refiner transformer under `<model_root>/refiner`.
"""

from __future__ import annotations

import os

import torch

from telefuser_b200.pipelines.lingbot_video import (LingBotVideoPipeline, LingBotVideoRequest, load_lingbot_video_prompt,
                                                    num_frames_from_duration, preprocess_ti2v_image)  # fmt: skip
from telefuser_b200.pipelines.lingbot_video.refiner import LingBotVideoRefinerStage, first_frame_for_refiner, prepare_refiner_video
from telefuser_b200.utils.video import save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="lingbot_video_moe_t2v", model_root=os.path.join(TF_MODEL_ZOO_PATH, "lingbot", "lingbot-video-moe"),
                  num_frames=81, height=480, width=832, num_inference_steps=50, guidance_scale=3.0, shift=3.0, seed=42,
                  target_fps=24, supports_refiner=True, enable_refiner=False, refiner_height=1088, refiner_width=1920,
                  refiner_steps=8, refiner_guidance_scale=3.0, refiner_shift=3.0, refiner_t_thresh=0.85, refiner_tail_steps=2,
                  refiner_co_resident=False)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v", "t2i"], "media_type": "video",
                     "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"], "t2i": ["prompt"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1) -> LingBotVideoPipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    pipe = LingBotVideoPipeline.from_pretrained(PPL_CONFIG["model_root"], parallel_devices=devices,
                                                expert_parallel=parallelism > 1,
                                                guidance_scale=PPL_CONFIG["guidance_scale"],
                                                num_inference_steps=PPL_CONFIG["num_inference_steps"], shift=PPL_CONFIG["shift"])  # fmt: skip
    pipe.refiner_parallelism = parallelism
    return pipe


def build_refiner(pipeline: LingBotVideoPipeline) -> LingBotVideoRefinerStage:
    """The refiner is a second MoE transformer with its own weights; it shares the VAE and the prompt embeddings."""
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.pipelines.lingbot_video import LingBotVideoDenoisingStage

    root = os.path.join(PPL_CONFIG["model_root"], "refiner")
    if not os.path.isdir(root):
        raise FileNotFoundError(f"{root}: the refiner checkpoint is a separate download")
    mm = ModuleManager(torch_dtype=pipeline.torch_dtype, device=str(pipeline.device))
    if not mm.load_model(root):
        raise ValueError(f"{root}: not a LingBot-Video transformer checkpoint")
    stage = LingBotVideoDenoisingStage("refiner", mm, pipeline.config.dit_config)
    stage.onload_models_flag = True
    return LingBotVideoRefinerStage(stage, pipeline.vae_stage, device=pipeline.device, torch_dtype=pipeline.torch_dtype)


def run_with_file(pipeline, prompt: str, output_path: str, seed: int = PPL_CONFIG["seed"],
                  num_frames: int = PPL_CONFIG["num_frames"], height: int = PPL_CONFIG["height"],
                  width: int = PPL_CONFIG["width"], first_image_path: str | None = None, negative_prompt: str | None = None,
                  refine: bool = PPL_CONFIG["enable_refiner"]):  # fmt: skip
    if prompt.endswith(".json") and os.path.isfile(prompt):
        prompt, duration = load_lingbot_video_prompt(prompt)
        if duration is not None:
            num_frames = num_frames_from_duration(duration, PPL_CONFIG["target_fps"])
    image = None
    image_path = first_image_path
    if image_path:
        import numpy as np
        from PIL import Image

        rgb = torch.from_numpy(np.array(Image.open(image_path).convert("RGB"))).permute(2, 0, 1)[None].float()
        image = preprocess_ti2v_image(rgb, height, width)[:, :, 0] * 2 - 1
    if num_frames == 1:
        refine = False
        output_path = os.path.splitext(output_path)[0] + ".png"
    result = pipeline.generate(LingBotVideoRequest(caption=prompt, num_frames=num_frames, height=height, width=width, seed=seed,
                                                   image=image), negative_caption=negative_prompt)  # fmt: skip
    video = result.output
    if refine:
        if not PPL_CONFIG["refiner_co_resident"]:
            release = getattr(pipeline.denoising_stage, "offload_models", None)  # make room for the refiner's weights
            if callable(release):
                release()
        refiner = build_refiner(pipeline)
        rh, rw = PPL_CONFIG["refiner_height"], PPL_CONFIG["refiner_width"]
        up, facts = prepare_refiner_video(video.float(), PPL_CONFIG["target_fps"], rh, rw, sample_fps=PPL_CONFIG["target_fps"])
        first = first_frame_for_refiner(image_path, rh, rw, height, width) if image_path else None
        cond = result.prompt_conditions
        video = refiner.refine(up, cond["positive_prompt_embeds"], cond["negative_prompt_embeds"],
                               num_inference_steps=PPL_CONFIG["refiner_steps"], guidance_scale=PPL_CONFIG["refiner_guidance_scale"],
                               shift=PPL_CONFIG["refiner_shift"], t_thresh=PPL_CONFIG["refiner_t_thresh"],
                               tail_steps=PPL_CONFIG["refiner_tail_steps"], clean_first_frame=first, seed=seed,
                               before_decode=refiner.close)  # fmt: skip
    if num_frames == 1:
        from telefuser_b200.utils.video import frames_to_uint8_array
        from PIL import Image

        os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
        Image.fromarray(frames_to_uint8_array(video)[0]).save(output_path)
    else:
        save_video(video, output_path, fps=PPL_CONFIG["target_fps"])
    return {"output_path": output_path, "refined": bool(refine), "num_frames": num_frames}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--gpu_num", default=1, type=int)
    @click.option("--prompt", default="A paper boat drifting along a rain-filled gutter, low camera following it.")
    @click.option("--image", "image_path", default=None, help="first frame for image-to-video")
    @click.option("--num_frames", default=PPL_CONFIG["num_frames"], type=int, help="1 for a still image, else 4n+1")
    @click.option("--refine/--no-refine", default=PPL_CONFIG["enable_refiner"])
    @click.option("--output", default="work_dirs/lingbot_video.mp4")
    def main(gpu_num, prompt, image_path, num_frames, refine, output):
        pipe = get_pipeline(gpu_num)
        print(run_with_file(pipe, prompt, output, num_frames=num_frames, first_image_path=image_path, refine=refine))

    main()
