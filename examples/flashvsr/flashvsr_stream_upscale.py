"""FlashVSR streaming video super-resolution (task vsr): a clip is upscaled chunk by chunk, every chunk continuing
from the frames and the sparse-attention cache of the one before.

    python examples/flashvsr/flashvsr_stream_upscale.py --input clip_480p.mp4 --scale 2.25
    telefuser serve examples/flashvsr/flashvsr_stream_upscale.py -t vsr

Model root (`$TF_MODEL_ZOO_PATH/FlashVSR-v1.1-BF16`): the streaming DiT file and the tiny conditional decoder file.
"""

from __future__ import annotations

import os

import torch

from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.pipelines.flashvsr.pipeline import FlashVSRPipelineConfig, FlashVSRStreamPipeline
from telefuser_b200.utils.video import VideoData, save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="flashvsr_stream", model_root=os.path.join(TF_MODEL_ZOO_PATH, "FlashVSR-v1.1-BF16"),
                  dit_filename="flashvsr11_dit_streaming_dmd_5dc619.safetensors", vae_filename="TCDecoder.ckpt", scale=2.25,
                  seed=0, sparse_ratio=2.0, kv_ratio=3, local_range=11, fps=16, first_chunk_size=25, chunk_size=16)  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["vsr"], "media_type": "video", "required_inputs": {"vsr": ["ref_video_path"]}}


def chunk_bounds(frame_count: int, first: int = PPL_CONFIG["first_chunk_size"], step: int = PPL_CONFIG["chunk_size"]) -> list:
    """[(start, end), ...]: a longer first chunk fills the temporal context, equal chunks follow."""
    out, pos = [(0, min(first, frame_count))], first
    while pos < frame_count:
        out.append((pos, min(pos + step, frame_count)))
        pos += step
    return out


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> FlashVSRStreamPipeline:
    mm = ModuleManager(torch_dtype=torch.bfloat16, device="cpu")
    mm.load_models([os.path.join(model_root, PPL_CONFIG["dit_filename"]), os.path.join(model_root, PPL_CONFIG["vae_filename"])])
    pipe = FlashVSRStreamPipeline(device="cuda", torch_dtype=torch.bfloat16)
    pipe.init(mm, FlashVSRPipelineConfig())
    return pipe


def run_with_file(pipeline, ref_video_path: str, output_path: str, scale: float = PPL_CONFIG["scale"],
                  seed: int = PPL_CONFIG["seed"], sparse_ratio: float = PPL_CONFIG["sparse_ratio"],
                  kv_ratio: int = PPL_CONFIG["kv_ratio"], local_range: int = PPL_CONFIG["local_range"]):  # fmt: skip
    frames_in = VideoData(ref_video_path).raw_data()
    pipeline.clean_cache()
    frames_out: list = []
    for start, end in chunk_bounds(len(frames_in)):
        frames_out.extend(pipeline(seed=seed, LQ_video=frames_in[start:end], sparse_ratio=sparse_ratio, kv_ratio=kv_ratio,
                                   local_range=local_range, scale=scale))  # fmt: skip
    save_video(frames_out, output_path, fps=PPL_CONFIG["fps"])
    return {"output_path": output_path, "num_frames": len(frames_out)}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--input", "input_video", required=True)
    @click.option("--output", default="work_dirs/flashvsr.mp4")
    @click.option("--scale", default=PPL_CONFIG["scale"], type=float)
    def main(input_video, output, scale):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        print(run_with_file(get_pipeline(), input_video, output, scale=scale))

    main()
