"""LiveAct speech-driven portrait video (task s2v): a first frame, an audio track and a prompt give a lip-synced clip,
generated chunk by chunk over a compressed memory of the earlier chunks.

    python examples/liveact/liveact_speech_to_video.py --image face.png --audio speech.wav --gpu_num 4
    telefuser serve examples/liveact/liveact_speech_to_video.py -t s2v -g 4

Model root (`$TF_MODEL_ZOO_PATH/LiveAct`): the DiT shards, the Wan2.1 VAE, the CLIP image encoder and the UMT5 text
encoder files; `wav2vec_dir` holds the Wav2Vec2 audio encoder in transformers layout.
"""

from __future__ import annotations

import os

import torch

from telefuser_b200.core.config import ParallelConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.pipelines.liveact.pipeline import LiveActPipeline, LiveActPipelineConfig
from telefuser_b200.utils.video import save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="liveact_s2v", model_root=os.path.join(TF_MODEL_ZOO_PATH, "LiveAct"),
                  wav2vec_dir=os.path.join(TF_MODEL_ZOO_PATH, "chinese-wav2vec2-base"), height=480, width=832, fps=24,
                  num_inference_steps=3, seed=42, fp8_kv_cache=False)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["s2v"], "media_type": "video", "required_inputs": {"s2v": ["first_image_path", "audio_path"]}}


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> LiveActPipeline:
    from telefuser_b200.models.wav2vec2 import Wav2Vec2Model

    mm = ModuleManager(torch_dtype=torch.bfloat16, device="cpu")
    mm.load_models([os.path.join(model_root, "diffusion_pytorch_model-*.safetensors"),
                    os.path.join(model_root, "Wan2.1_VAE.pth"),
                    os.path.join(model_root, "models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth"),
                    os.path.join(model_root, "models_t5_umt5-xxl-enc-bf16.pth")])  # fmt: skip
    mm.add_module(Wav2Vec2Model.from_pretrained(PPL_CONFIG["wav2vec_dir"], torch_dtype=torch.bfloat16).eval(), "wav2vec2")
    cfg = LiveActPipelineConfig()
    cfg.fp8_kv_cache = PPL_CONFIG["fp8_kv_cache"]
    if parallelism > 1:
        cfg.dit_config.parallel_config = ParallelConfig(device_ids=list(range(parallelism)), sp_ulysses_degree=parallelism)
        cfg.enable_denoising_parallel = True
    pipe = LiveActPipeline(device="cuda", torch_dtype=torch.bfloat16)
    pipe.init(mm, cfg)
    return pipe


def run_with_file(pipeline, first_image_path: str, audio_path: str, output_path: str, prompt: str = "",
                  seed: int = PPL_CONFIG["seed"], height: int = PPL_CONFIG["height"], width: int = PPL_CONFIG["width"],
                  fps: int = PPL_CONFIG["fps"], num_inference_steps: int = PPL_CONFIG["num_inference_steps"]):  # fmt: skip
    from PIL import Image

    frames = pipeline(prompt, Image.open(first_image_path).convert("RGB"), audio_path=audio_path, seed=seed, height=height,
                      width=width, fps=fps, num_inference_steps=num_inference_steps)  # fmt: skip
    save_video(frames, output_path, fps=fps)  # the audio track is muxed by the caller (no muxer in this package)
    return {"output_path": output_path, "num_frames": len(frames)}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--image", "image_path", required=True)
    @click.option("--audio", "audio_path", required=True)
    @click.option("--prompt", default="a person speaking to the camera, natural head motion")
    @click.option("--output", default="work_dirs/liveact.mp4")
    @click.option("--gpu_num", default=1, type=int)
    def main(image_path, audio_path, prompt, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        pipe = get_pipeline(gpu_num)
        try:
            print(run_with_file(pipe, image_path, audio_path, output, prompt=prompt))
        finally:
            pipe.close()

    main()
