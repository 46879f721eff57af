"""LTX-2.3 two-stage text / image -> video + audio pipeline.

Stage 1 denoises video and audio jointly at half resolution with multi-modal guidance; the video latents are
upsampled x2 in latent space and stage 2 refines both streams at full resolution with a short fixed sigma
schedule and no guidance. The video VAE then decodes tile by tile and the audio decoder + vocoder turn the audio
latents into a stereo waveform. `__call__` returns (frames, waveform [2, samples], sample rate).
Role parity: telefuser/pipelines/ltx_video/ltx23_video.py:34-518.
"""

from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass, field
from typing import Any, Sequence

import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.models.ltx_video_vae import VIDEO_SCALE_FACTORS
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

from .dit_denoising import AudioLatentShape, DitDenoisingStage, MultiModalGuiderParams
from .stages import DEFAULT_TILE_SIZE, DEFAULT_TILE_STRIDE, GemmaTextEncodingStage, UpsamplerStage, VAEStage

DEFAULT_VIDEO_STG_BLOCKS, DEFAULT_AUDIO_STG_BLOCKS = [28], [28]
DEFAULT_NUM_INFERENCE_STEPS = 30
LATENT_TOKEN_CHANNELS = 128


def assert_resolution(height: int, width: int, is_two_stage: bool) -> None:
    divisor = 64 if is_two_stage else 32
    if height % divisor or width % divisor:
        raise ValueError(f"resolution {height}x{width} must be a multiple of {divisor} for the "
                         f"{'two' if is_two_stage else 'one'}-stage pipeline")  # fmt: skip


@dataclass
class LTXVideoPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    upsampler_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_stage1_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_stage2_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sample_solver: str = "euler"
    enable_denoising_parallel: bool = False
    enable_vae_parallel: bool = False
    enable_vae_ray: bool = False
    stage2_lora_strength: float = 1.0
    batched_guidance: bool = True  # the up-to-four guidance passes of a stage-1 step run as one batch


class LTX23VideoPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = self.width_division_factor = 64
        self.base_fps = 24
        self._audio_decoder = self._vocoder = self._audio_sample_rate = None
        self._ltx_checkpoint_paths = None

    def _get_stages(self) -> list:
        return [self.text_encoding_stage, self.vae_stage, self.stage1_denoise_stage, self.upsampler_stage, self.stage2_denoise_stage]

    def _scheduler(self, solver: str):
        if solver == "euler":
            return FlowMatchScheduler(template="LTX.2")
        if solver == "unipc":
            from telefuser_b200.schedulers.unipc import FlowUniPCMultistepScheduler

            return FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        raise NotImplementedError(f"solver {solver} is not supported")

    def init(self, module_manager: Any, config: LTXVideoPipelineConfig, *, text_stage=None, audio_decoder=None, vocoder=None) -> None:
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.module_manager, self.config = module_manager, config
        self.vae_stage = VAEStage("vae", module_manager, config.vae_config)
        self.stage1_denoise_stage = DitDenoisingStage("stage1_denoise", module_manager, config.dit_stage1_config, "ltx_dit",
                                                      self._scheduler(config.sample_solver), batched_guidance=config.batched_guidance)  # fmt: skip
        self.stage2_denoise_stage = DitDenoisingStage("stage2_denoise", module_manager, config.dit_stage2_config, "ltx_dit",
                                                      self._scheduler(config.sample_solver))  # fmt: skip
        self.upsampler_stage = UpsamplerStage("upsampler", module_manager, config.upsampler_config)
        self.text_encoding_stage = text_stage or GemmaTextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        for stage in self._get_stages():
            stage.onload_models_flag = True
        if config.enable_vae_parallel:
            self.vae_stage = ParallelWorker(self.vae_stage)
        if config.enable_denoising_parallel:
            self.stage1_denoise_stage = ParallelWorker(self.stage1_denoise_stage)
            self.stage2_denoise_stage = ParallelWorker(self.stage2_denoise_stage)
        fetched = module_manager.fetch_module("ltx_dit", require_model_path=True)
        self._ltx_checkpoint_paths = fetched[1] if fetched else None
        if audio_decoder is not None:
            self._audio_decoder, self._vocoder = audio_decoder, vocoder
            self._audio_sample_rate = int(vocoder.output_sampling_rate)

    # ---- audio decoding --------------------------------------------------------------------------
    def _ensure_audio_decoder_loaded(self) -> None:
        """Builds the audio decoder and vocoder from the `config` metadata of the shared checkpoint and loads their weights."""
        if self._audio_decoder is not None and self._vocoder is not None:
            return
        from safetensors import safe_open

        from telefuser_b200.models.ltx_audio_vae import AudioDecoderConfigurator, VocoderConfigurator

        paths = self._ltx_checkpoint_paths
        if paths is None:
            raise ValueError("no LTX checkpoint path is known; pass audio_decoder / vocoder to init() instead")
        paths = [paths] if isinstance(paths, str) else list(paths)
        with safe_open(paths[0], framework="pt") as f:
            meta = f.metadata() or {}
        if "config" not in meta:
            raise ValueError("the LTX checkpoint has no `config` metadata to configure the audio decoder / vocoder")
        config = json.loads(meta["config"])
        dec_sd, voc_sd = {}, {}
        for p in paths:
            with safe_open(p, framework="pt", device="cpu") as f:
                for k in f.keys():
                    if k.startswith("audio_vae.decoder."):
                        dec_sd[k[len("audio_vae.decoder."):]] = f.get_tensor(k)
                    elif k.startswith("audio_vae.per_channel_statistics."):
                        dec_sd["per_channel_statistics." + k[len("audio_vae.per_channel_statistics."):]] = f.get_tensor(k)
                    elif k.startswith("vocoder."):
                        voc_sd[k[len("vocoder."):]] = f.get_tensor(k)
        decoder, vocoder = AudioDecoderConfigurator.from_config(config), VocoderConfigurator.from_config(config)
        decoder.load_state_dict(dec_sd, strict=False)
        vocoder.load_state_dict(voc_sd, strict=False)
        self._audio_decoder = decoder.to(self.device, self.torch_dtype).eval()
        self._vocoder = vocoder.to(self.device, self.torch_dtype).eval()
        self._audio_sample_rate = int(vocoder.output_sampling_rate)

    @torch.no_grad()
    def _decode_audio(self, audio_latents: torch.Tensor):
        self._ensure_audio_decoder_loaded()
        mel = self._audio_decoder(audio_latents.to(self.device, next(self._audio_decoder.parameters()).dtype))
        return self._vocoder(mel).squeeze(0).float().detach(), self._audio_sample_rate

    # ---- noise -------------------------------------------------------------------------------------
    def _init_video_noise(self, height: int, width: int, num_frames: int, seed):
        f = (num_frames - 1) // VIDEO_SCALE_FACTORS.time + 1
        tokens = f * (height // VIDEO_SCALE_FACTORS.height) * (width // VIDEO_SCALE_FACTORS.width)
        return self.generate_noise((1, tokens, LATENT_TOKEN_CHANNELS), seed=seed, device=self.device, dtype=torch.float32)

    def _init_audio_noise(self, num_frames: int, frame_rate: float, seed):
        s = AudioLatentShape.from_duration(1, float(num_frames) / float(frame_rate))
        return self.generate_noise((1, s.frames, s.channels * s.mel_bins), seed=seed, device=self.device, dtype=torch.float32)

    @staticmethod
    def _wait(x):
        return x() if callable(x) else x

    @torch.no_grad()
    def __call__(self, prompt: str, negative_prompt: str = "", input_image=None, seed: int | None = None, height: int = 1024,
                 width: int = 1536, num_frames: int = 121, num_inference_steps: int = DEFAULT_NUM_INFERENCE_STEPS,
                 frame_rate: float | None = None, tiled: bool = True, tile_size=DEFAULT_TILE_SIZE, tile_stride=DEFAULT_TILE_STRIDE,
                 input_image_frame_idx: int = 0, input_image_strength: float = 1.0, video_cfg_scale: float = 3.0,
                 video_stg_scale: float = 1.0, video_rescale_scale: float = 0.7, video_modality_scale: float = 3.0, video_skip_step: int = 0,
                 video_stg_blocks: Sequence[int] | None = None, audio_cfg_scale: float = 7.0, audio_stg_scale: float = 1.0,
                 audio_rescale_scale: float = 0.7, audio_modality_scale: float = 3.0, audio_skip_step: int = 0,
                 audio_stg_blocks: Sequence[int] | None = None, return_latents: bool = False):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        assert_resolution(height, width, is_two_stage=True)
        frame_rate = frame_rate or float(self.base_fps)
        vparams = MultiModalGuiderParams(video_cfg_scale, video_stg_scale, list(video_stg_blocks if video_stg_blocks is not None else DEFAULT_VIDEO_STG_BLOCKS),
                                         video_rescale_scale, video_modality_scale, video_skip_step)  # fmt: skip
        aparams = MultiModalGuiderParams(audio_cfg_scale, audio_stg_scale, list(audio_stg_blocks if audio_stg_blocks is not None else DEFAULT_AUDIO_STG_BLOCKS),
                                         audio_rescale_scale, audio_modality_scale, audio_skip_step)  # fmt: skip
        noise1_v, noise1_a = self._init_video_noise(height // 2, width // 2, num_frames, seed), self._init_audio_noise(num_frames, frame_rate, seed)
        noise2_v, noise2_a = self._init_video_noise(height, width, num_frames, seed), self._init_audio_noise(num_frames, frame_rate, seed)
        use_negative = video_cfg_scale != 1.0 and audio_cfg_scale != 1.0
        embs = self._wait(self.text_encoding_stage.process([prompt] + ([negative_prompt] if use_negative else [])))
        positive, negative = embs[0], (embs[1] if use_negative else None)
        cond1 = None
        if input_image is not None:
            cond1 = self._wait(self.vae_stage.process("encode_image", input_image, height // 2, width // 2, input_image_frame_idx,
                                                      input_image_strength))  # fmt: skip
        common = dict(num_frames=num_frames, frame_rate=frame_rate, positive_context=positive, negative_context=negative,
                      num_inference_steps=num_inference_steps, video_guider_params=vparams, audio_guider_params=aparams)  # fmt: skip
        v1, a1 = self._wait(self.stage1_denoise_stage.process(height=height // 2, width=width // 2, conditionings=cond1, video_noise=noise1_v,
                                                              audio_noise=noise1_a, **common))  # fmt: skip
        upscaled = self._wait(self.upsampler_stage.process(v1.latent[:1]))
        cond2 = self._wait(self.vae_stage.process("encode_image", input_image, height, width, input_image_frame_idx, input_image_strength))
        sigmas2 = DitDenoisingStage.stage2_sigmas(self.device)
        v2, a2 = self._wait(self.stage2_denoise_stage.process(height=height, width=width, conditionings=cond2, video_noise=noise2_v,
                                                              audio_noise=noise2_a, initial_video_latent=upscaled,
                                                              initial_audio_latent=a1.latent, sigmas=sigmas2,
                                                              noise_scale=float(sigmas2[0]), simple_denoise=True, **common))  # fmt: skip
        if return_latents:
            return v2.latent, a2.latent
        gen = None if seed is None else torch.Generator(device=self.device).manual_seed(seed)
        frames = self._wait(self.vae_stage.process("decode_video", v2.latent, gen, tiled=tiled, tile_size=tile_size, tile_stride=tile_stride))
        waveform, rate = self._decode_audio(a2.latent)
        return self.tensor2video(frames[0]), waveform, rate

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device: str = "cuda", torch_dtype: torch.dtype = torch.bfloat16, cache_dir=None,
                        attention_config=None, enable_parallel: bool = False, parallel_devices=None, sample_solver: str = "euler",
                        **kwargs) -> "LTX23VideoPipeline":  # fmt: skip
        """Model root layout: one shared `*.safetensors` checkpoint (transformer, VAEs, vocoder, connectors), a
        `*upscaler*` / `*upsampler*` safetensors file and a Gemma-3 folder (one that holds `tokenizer.model`)."""
        from telefuser_b200.core.module_manager import ModuleManager
        from telefuser_b200.models.ltx_dit import LTXVideoTransformer
        from telefuser_b200.models.ltx_gemma_text_encoder import GemmaTextEncoder, LTXEmbeddingsProcessor
        from telefuser_b200.models.ltx_upsampler import LTXSpatialUpsampler
        from telefuser_b200.models.ltx_video_vae import LTXVideoVAE
        from telefuser_b200.utils.hf import resolve_hf_path

        root = resolve_hf_path(model_id_or_path, cache_dir)
        files = sorted(glob.glob(os.path.join(root, "*.safetensors")))
        is_up = lambda p: any(t in os.path.basename(p).lower() for t in ("upscaler", "upsampler"))  # noqa: E731
        ups = [p for p in files if is_up(p)]
        ckpts = [p for p in files if not is_up(p) and "lora" not in os.path.basename(p).lower()]
        gemma = next((os.path.dirname(p) for p in glob.glob(os.path.join(root, "**", "tokenizer.model"), recursive=True)), None)
        if not ckpts or not ups or gemma is None:
            raise ValueError(f"{root}: need a transformer checkpoint, a spatial upsampler and a Gemma folder "
                             f"(found {len(ckpts)}, {len(ups)}, {gemma})")  # fmt: skip
        mm = ModuleManager(torch_dtype=torch_dtype, device="cpu")
        for name, klass in (("ltx_dit", LTXVideoTransformer), ("ltx_video_vae", LTXVideoVAE), ("ltx_embeddings_processor", LTXEmbeddingsProcessor)):
            mm.load_model(ckpts[0], device="cpu", torch_dtype=torch_dtype, name=name, model_class=klass)
        mm.load_model(ups[0], device="cpu", torch_dtype=torch_dtype, name="ltx_spatial_upsampler", model_class=LTXSpatialUpsampler)
        mm.load_from_huggingface(gemma, "gemma_text_encoder", GemmaTextEncoder, torch_dtype=torch_dtype, device="cpu")
        config = LTXVideoPipelineConfig(sample_solver=sample_solver)
        if attention_config is not None:
            config.dit_stage1_config.attention_config = config.dit_stage2_config.attention_config = attention_config
        if enable_parallel and parallel_devices:
            for c in (config.dit_stage1_config, config.dit_stage2_config):
                c.parallel_config.device_ids, c.parallel_config.sp_ulysses_degree = parallel_devices, len(parallel_devices)
            config.enable_denoising_parallel = True
        for k, v in kwargs.items():
            if hasattr(config, k):
                setattr(config, k, v)
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config)
        return pipe
