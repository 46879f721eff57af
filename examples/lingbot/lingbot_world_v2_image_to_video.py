"""LingBot-World v2 (camera-controlled causal world model): offline chunked generation and the interactive
streaming service.

    python examples/lingbot/lingbot_world_v2_image_to_video.py --gpu_num 4 --image first.jpg
    telefuser stream-serve examples/lingbot/lingbot_world_v2_image_to_video.py --gpu-num 4 -p 8088

Stage placement on one node follows `resolve_stage_devices`: with 2 or 4 GPUs all of them run the DiT (Ulysses)
and the VAE encode / decode actors share GPUs 0 and 1 with it; with 5 or 6 GPUs the last GPU belongs to the VAE
alone. With `TFB_RANDOM_INIT=1` the 14B architecture is built with random weights (benchmarks, smoke tests).
"""

from __future__ import annotations

import os
from pathlib import Path

import torch

from telefuser_b200.core.config import CompileConfig, ModelRuntimeConfig, ParallelConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.pipelines.lingbot_world.service import LingBotWorldFastService, LingBotWorldFastSessionConfig
from telefuser_b200.pipelines.lingbot_world_v2 import LingBotWorldV2Pipeline, LingBotWorldV2PipelineConfig, resolve_stage_devices

TF_MODEL_ZOO_PATH = Path(os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")).expanduser()
PPL_CONFIG = dict(
    vae_path=str(TF_MODEL_ZOO_PATH / "Wan2.2-I2V-A14B" / "Wan2.1_VAE.pth"),
    text_encoder_path=str(TF_MODEL_ZOO_PATH / "Wan2.2-I2V-A14B" / "models_t5_umt5-xxl-enc-bf16.pth"),
    dit_dir=str(TF_MODEL_ZOO_PATH / "lingbot" / "lingbot-world-v2-14b-causal-fast" / "transformers"),
    parallelism=1, vae_encode_device_id=0, vae_decode_device_id=0, resolution=(480, 832), frame_num=77, chunk_size=4,
    sample_shift=10.0, seed=42, target_fps=16, max_duration_seconds=120.0, local_attn_size=18, sink_size=6,
    timestep_indices=(0, 250, 500, 750), control_move_step=0.10, control_yaw_step_degrees=0.5,
    compile_config=CompileConfig(enabled=True), torch_dtype=torch.bfloat16,
)  # fmt: skip


def _modules(device: str, dtype) -> ModuleManager:
    from telefuser_b200.models.lingbot_world_dit import LingBotWorldFastDiT
    from telefuser_b200.models.umt5 import WanTextEncoder
    from telefuser_b200.models.wan_vae import WanVideoVAE

    mm = ModuleManager(torch_dtype=dtype, device=device)
    if os.environ.get("TFB_RANDOM_INIT") == "1":
        from telefuser_b200.testing.synthetic import random_init_

        tiny = os.environ.get("TFB_TINY") == "1"
        kw = dict(in_dim=36, local_attn_size=PPL_CONFIG["local_attn_size"], sink_size=PPL_CONFIG["sink_size"])
        if tiny:  # a few thousand parameters: service smoke tests on CPU
            kw.update(dim=64, ffn_dim=128, num_heads=2, num_layers=2, text_dim=64)
        with torch.device(device):
            dit, vae = LingBotWorldFastDiT(**kw).to(dtype), WanVideoVAE(**({"dim": 8} if tiny else {})).to(dtype)
        dit.dtype = dtype
        mm.add_module(random_init_(dit).eval(), "lingbot_world_fast_dit")
        mm.add_module(random_init_(vae, std=0.02).eval(), "wan_video_vae")
        text_dim = kw.get("text_dim", 4096)  # a short random UMT5 stack of the right width stands in for the prompt encoder
        with torch.device(device):
            te = WanTextEncoder(vocab=4096, dim=text_dim, dim_attn=text_dim, dim_ffn=2 * text_dim,
                                num_heads=max(1, text_dim // 64), num_layers=2).to(dtype)  # fmt: skip
        mm.add_module(random_init_(te, seed=1).eval(), "random_text_encoder")
        return mm
    shards = sorted(str(p) for p in Path(PPL_CONFIG["dit_dir"]).glob("model-*-of-*.safetensors"))
    mm.load_model(shards, model_class=LingBotWorldFastDiT, name="lingbot_world_fast_dit")
    mm.load_model(PPL_CONFIG["vae_path"], model_class=WanVideoVAE, name="wan_video_vae")
    mm.load_model(PPL_CONFIG["text_encoder_path"], model_class=WanTextEncoder, name="wan_video_text_encoder")
    return mm


def get_pipeline(parallelism: int = PPL_CONFIG["parallelism"]) -> LingBotWorldV2Pipeline:
    dit_devices, enc_dev, dec_dev = resolve_stage_devices(parallelism, PPL_CONFIG["vae_encode_device_id"],
                                                          PPL_CONFIG["vae_decode_device_id"])  # fmt: skip
    dtype = PPL_CONFIG["torch_dtype"]
    on_gpu = torch.cuda.is_available()
    device = f"cuda:{dit_devices[0]}" if on_gpu else "cpu"

    def rc(device_id: int, parallel: ParallelConfig | None = None) -> ModelRuntimeConfig:
        return ModelRuntimeConfig(device_type="cuda" if on_gpu else "cpu", device_id=device_id, torch_dtype=dtype,
                                  parallel_config=parallel or ParallelConfig(), compile_config=PPL_CONFIG["compile_config"])  # fmt: skip

    par = ParallelConfig(device_ids=dit_devices, sp_ulysses_degree=len(dit_devices)) if len(dit_devices) > 1 else None
    config = LingBotWorldV2PipelineConfig(
        dit_config=rc(dit_devices[0], par), vae_encode_config=rc(enc_dev), vae_decode_config=rc(dec_dev),
        text_encoding_config=rc(dit_devices[0]), chunk_size=PPL_CONFIG["chunk_size"], sample_shift=PPL_CONFIG["sample_shift"],
        local_attn_size=PPL_CONFIG["local_attn_size"], sink_size=PPL_CONFIG["sink_size"],
        timestep_indices=PPL_CONFIG["timestep_indices"], fps=PPL_CONFIG["target_fps"], enable_denoising_parallel=par is not None)  # fmt: skip
    pipe = LingBotWorldV2Pipeline(device=device, torch_dtype=dtype)
    mm = _modules(device, dtype)
    text_stage = None
    if mm.fetch_module("random_text_encoder") is not None:
        from telefuser_b200.pipelines.wan.stages import TextEncodingStage
        from telefuser_b200.testing.synthetic import HashTokenizer

        text_stage = TextEncodingStage("text_encoding", mm, config.text_encoding_config, config.max_sequence_length,
                                       text_encoder=mm.fetch_module("random_text_encoder"), tokenizer=HashTokenizer(4096, 512))  # fmt: skip
        text_stage.onload_models_flag = True
    pipe.init(mm, config, text_stage=text_stage)
    return pipe


def get_service(gpu_num: int = 1) -> LingBotWorldFastService:
    """Entry point of `telefuser stream-serve`: one pipeline, sessions created per client."""
    h, w = PPL_CONFIG["resolution"]
    defaults = LingBotWorldFastSessionConfig(height=h, width=w, seed=PPL_CONFIG["seed"], fps=PPL_CONFIG["target_fps"],
                                             max_duration_seconds=PPL_CONFIG["max_duration_seconds"],
                                             move_step=PPL_CONFIG["control_move_step"],
                                             turn_step_deg=PPL_CONFIG["control_yaw_step_degrees"], hud=True)  # fmt: skip
    return LingBotWorldFastService(get_pipeline(gpu_num), defaults, warmup=torch.cuda.is_available())


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--gpu_num", default=1, type=int)
    @click.option("--image", default=None, help="first frame; a grey image when omitted")
    @click.option("--prompt", default="A calm lakeside with a lone tree, distant snow-capped mountains, drifting clouds.")
    @click.option("--output", default="work_dirs/lingbot_world_v2.mp4")
    def main(gpu_num, image, prompt, output):
        from PIL import Image

        from telefuser_b200.utils.video import save_video

        h, w = PPL_CONFIG["resolution"]
        img = Image.open(image).convert("RGB") if image else Image.new("RGB", (w, h), (128, 128, 128))
        pipe = get_pipeline(gpu_num)
        try:
            video, metrics = pipe.generate_video(prompt, img, PPL_CONFIG["frame_num"], h, w, seed=PPL_CONFIG["seed"])
            save_video(video, output, fps=PPL_CONFIG["target_fps"])
            print({"output_path": output, "chunk_period_p50_s": metrics.get("chunk_period_p50_s")})
        finally:
            pipe.close()

    main()
