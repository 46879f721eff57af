"""LTX-2.3 text / image to video with stereo audio (two stages, latent upsampling between them): offline run and
`telefuser serve` entry points.

    python examples/ltx_video/ltx23_text_to_video.py --prompt "waves on a pebble beach, gulls calling"
    telefuser serve examples/ltx_video/ltx23_text_to_video.py -t t2v

Model root (`$TF_MODEL_ZOO_PATH/LTX-2.3`): the shared checkpoint, the spatial upsampler file and the Gemma-3 text
encoder folder, as `LTX23VideoPipeline.from_pretrained` documents.
"""

from __future__ import annotations

import os

from telefuser_b200.pipelines.ltx_video import LTX23VideoPipeline
from telefuser_b200.utils.video import save_video

TF_MODEL_ZOO_PATH = os.environ.get("TF_MODEL_ZOO_PATH", "model_zoo")
PPL_CONFIG = dict(name="ltx23_t2v", model_root=os.path.join(TF_MODEL_ZOO_PATH, "LTX-2.3"), height=1024, width=1536, num_frames=121,
                  frame_rate=24.0, seed=0, negative_prompt="worst quality, inconsistent motion, blurry, jittery, distorted",
                  quant=os.environ.get("TFB_LTX_QUANT", ""))  # fmt: skip
PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v"], "media_type": "video",
                     "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"]}}  # fmt: skip


def get_pipeline(parallelism: int = 1, model_root: str = PPL_CONFIG["model_root"]) -> LTX23VideoPipeline:
    devices = list(range(parallelism)) if parallelism > 1 else None
    pipe = LTX23VideoPipeline.from_pretrained(model_root, enable_parallel=parallelism > 1, parallel_devices=devices)
    if PPL_CONFIG["quant"]:  # "nf4": the 22B transformer in 4.5 bits per weight
        pipe.stage1_denoise_stage.dit.enable_quant(PPL_CONFIG["quant"])
    return pipe


def run_with_file(pipeline, prompt: str, output_path: str, first_image_path: str = "",
                  negative_prompt: str = PPL_CONFIG["negative_prompt"], seed: int = PPL_CONFIG["seed"],
                  height: int = PPL_CONFIG["height"], width: int = PPL_CONFIG["width"], num_frames: int = PPL_CONFIG["num_frames"]):  # fmt: skip
    from PIL import Image

    image = Image.open(first_image_path).convert("RGB") if first_image_path else None
    frames, waveform, sample_rate = pipeline(prompt, negative_prompt=negative_prompt, input_image=image, seed=seed, height=height,
                                             width=width, num_frames=num_frames, frame_rate=PPL_CONFIG["frame_rate"])  # fmt: skip
    save_video(frames, output_path, fps=int(PPL_CONFIG["frame_rate"]))
    out = {"output_path": output_path, "num_frames": len(frames)}
    if waveform is not None:
        from telefuser_b200.utils.video import save_wav

        out["audio_path"] = save_wav(waveform, os.path.splitext(output_path)[0] + ".wav", sample_rate)
    return out


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="Waves folding over a pebble beach at dusk, gulls calling, the hiss of retreating water.")
    @click.option("--image_path", default="")
    @click.option("--output", default="work_dirs/ltx23.mp4")
    @click.option("--gpu_num", default=1, type=int)
    def main(prompt, image_path, output, gpu_num):
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        print(run_with_file(get_pipeline(gpu_num), prompt, output, first_image_path=image_path))

    main()
