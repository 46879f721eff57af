"""LiveAct real-time speech-driven video pipeline.

The video grows block by block (6 latent frames first, 8 afterwards). Per block: the matching stretch of audio
is resampled to 16 kHz and encoded by Wav2Vec2 (all hidden layers, one vector per video frame, a window of 5
frames around each frame), the DiT runs three fixed Euler steps (timesteps 1000, 937.5, 833.3 -> 0) with one KV
memory per (step, layer), optionally with audio classifier-free guidance on the last two steps against a second
memory fed with silent audio, and the Wan VAE decodes the new latents together with the last 3 latents of the
previous block (whose 9 frames are dropped again) so that the causal decoder sees continuous context.
Role parity: telefuser/pipelines/liveact/{pipeline,denoising,audio_encoding}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from telefuser_b200.cache.kv_cache import KVCacheManager
from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.utils.func import auto_async_call

TIMESTEPS = [1000.0, 937.5, 833.33333333, 0.0]
VAE_STRIDE = (4, 8, 8)
PATCH_SIZE = (1, 2, 2)
LATENT_CHANNELS = 16


def resample_to_16k(audio: torch.Tensor, sr: int, gain: float = 3.0) -> torch.Tensor:
    """[channels, samples] at `sr` Hz -> 16 kHz (polyphase filter), scaled by the gain the model was trained with."""
    if sr != 16000:
        from math import gcd

        from scipy.signal import resample_poly

        g = gcd(int(sr), 16000)
        audio = torch.from_numpy(resample_poly(audio.cpu().numpy(), 16000 // g, int(sr) // g, axis=-1).astype(np.float32))
    return audio.cpu().float() * gain


def load_audio(path: str) -> tuple[torch.Tensor, int]:
    """-> ([channels, samples] float in [-1, 1], sample rate); WAV through scipy, other containers through torchaudio."""
    if path.lower().endswith(".wav"):
        from scipy.io import wavfile

        sr, data = wavfile.read(path)
        x = torch.from_numpy(np.asarray(data))
        x = x.float() / (32768.0 if data.dtype == np.int16 else (2147483648.0 if data.dtype == np.int32 else 1.0))
        return (x[None] if x.dim() == 1 else x.t().contiguous()), int(sr)
    import torchaudio

    return torchaudio.load(path)


@dataclass
class LiveActPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    clip_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    audio_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    audio_window: int = 5
    stream_audio: bool = True  # re-encode the audio of every block (exact) instead of encoding the whole track once
    block_sizes: tuple = (6, 8)
    fp8_kv_cache: bool = False
    offload_cache: bool = False
    mean_memory: bool = False
    enable_denoising_parallel: bool = False
    enable_vae_parallel: bool = False


class AudioEncodingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, audio_window: int = 5, encoder=None) -> None:
        super().__init__(name, config)
        self.audio_encoder = encoder if encoder is not None else module_manager.fetch_module("wav2vec2")
        self.audio_processor = getattr(self.audio_encoder, "audio_processor", None)
        self.audio_window = audio_window
        self.model_names = ["audio_encoder"]
        half = audio_window // 2
        self._window = torch.arange(-half, half + 1)
        self._audio, self._sr, self._fps, self._pre = None, None, 24, None

    def duration(self) -> float:
        return 0.0 if self._audio is None else self._audio.shape[1] / self._sr

    def extract_features(self, audio_16k: torch.Tensor, seq_len: int) -> torch.Tensor:
        """mono waveform [samples] -> [seq_len, layers, C] (all transformer layers, one vector per video frame)."""
        if self.audio_processor is not None:
            values = self.audio_processor(audio_16k.cpu().numpy(), sampling_rate=16000, return_tensors="pt").input_values
        else:  # zero mean, unit variance, as the stock feature extractor does
            values = ((audio_16k - audio_16k.mean()) / torch.sqrt(audio_16k.var() + 1e-7))[None]
        p = next(self.audio_encoder.parameters())
        out = self.audio_encoder(values.to(self.device, p.dtype), seq_len=seq_len, output_hidden_states=True)
        return torch.stack(out.hidden_states[1:], dim=1).squeeze(0).transpose(0, 1)

    def windows(self, emb: torch.Tensor, start: int, end: int) -> torch.Tensor:
        """[frames, layers, C] -> [1, end - start, window, layers, C]; indices past the ends repeat the edge frame."""
        idx = torch.arange(start, end, device=emb.device)[:, None] + self._window.to(emb.device)[None, :]
        return emb[idx.clamp(0, emb.shape[0] - 1)][None]

    @torch.no_grad()
    def process_stream_audio_segment(self, audio_start_idx: int, audio_end_idx: int, fps: int, frame_num: int):
        a = int(self._sr * (audio_start_idx / fps))
        b = min(int(self._sr * ((audio_end_idx + 2) / fps)), self._audio.shape[1])
        wave = resample_to_16k(self._audio[:1, a:b], self._sr)[0]
        return self.windows(self.extract_features(wave, frame_num), 0, frame_num).to(self.torch_dtype)

    def process_pre_encoded_segment(self, audio_start_idx: int, audio_end_idx: int):
        if self._pre is None:
            raise ValueError("no pre-encoded audio: call process(stream_audio=False) first")
        return self.windows(self._pre.to(self.device), audio_start_idx, audio_end_idx).to(self.torch_dtype)

    @with_model_offload(["audio_encoder"])
    @torch.no_grad()
    def process(self, audio_path=None, audio=None, sr: int = 16000, fps: int = 24, video_length=None, stream_audio: bool = True):
        if audio_path is not None:
            audio, sr = load_audio(audio_path)
        if audio is None:
            raise ValueError("either audio_path or audio must be given")
        self._audio, self._sr, self._fps = audio, sr, fps
        self._pre = None
        if not stream_audio:
            n = video_length or int(self.duration() * fps)
            self._pre = self.extract_features(resample_to_16k(audio, sr)[0], n)
        return (None if stream_audio else self._pre), self.duration()


class LiveActDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, fp8_kv_cache: bool = False,
                 offload_cache: bool = False, mean_memory: bool = False, dit=None) -> None:  # fmt: skip
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module("liveact_dit")
        self.dit.set_mean_memory(mean_memory)
        self.model_names = ["dit"]
        self.fp8_kv_cache, self.offload_cache = fp8_kv_cache, offload_cache
        self.kv_cache_manager = self._null_audio_manager = None
        self._tokens_per_frame = None
        if config.quant_config.enabled and config.parallel_config.world_size == 1 and hasattr(self.dit, "enable_quant"):
            from telefuser_b200.ops.quant import quantize_model_fp8_

            quantize_model_fp8_(self.dit, ("blocks.*",), ("modulation", "memory_proj"))

    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.dit.device_mesh = pmesh.create_device_mesh_from_config(cfg)
        if cfg.sp_degree > 1:
            self.dit.enable_usp()
        if cfg.enable_fsdp:
            from telefuser_b200.parallel.fsdp import shard_model

            shard_model(self.dit, self.device, wrap_module_names=self.dit.get_fsdp_module_names())

    def init_kv_cache(self, tokens_per_frame: int, num_timesteps: int = 3) -> KVCacheManager:
        from telefuser_b200.parallel import shard as pshard

        sp = pshard._sp(None)[1] if self.dit.usp_flag else 1
        m = KVCacheManager(num_timesteps, self.dit.num_layers, self.fp8_kv_cache, self.offload_cache)
        m.allocate((1, 6 * tokens_per_frame, self.dit.num_heads // sp, self.dit.head_dim), self.torch_dtype, self.device)
        return m

    def clear_kv_cache(self) -> None:
        for m in (self.kv_cache_manager, self._null_audio_manager):
            if m is not None:
                m.clear()
        self.kv_cache_manager = self._null_audio_manager = self._tokens_per_frame = None

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latent, context, clip_fea, audio_embedding, y, tokens_per_frame: int, audio_cfg: float = 1.0,
                num_inference_steps: int = 3, seed: int | None = None, block_sizes=(6, 8)):  # fmt: skip
        """latent [C, f, h, w] noise of one block (f = 6: first block, 8: later) -> denoised latent."""
        first = latent.shape[1] == block_sizes[0]
        start_idx = 0 if first else block_sizes[0] * tokens_per_frame
        end_idx = (block_sizes[0] if first else sum(block_sizes)) * tokens_per_frame
        if self.kv_cache_manager is None or self._tokens_per_frame != tokens_per_frame:
            self.kv_cache_manager = self.init_kv_cache(tokens_per_frame, num_inference_steps)
            self._tokens_per_frame, self._null_audio_manager = tokens_per_frame, None
        if audio_cfg > 1.0 and self._null_audio_manager is None:
            self._null_audio_manager = self.init_kv_cache(tokens_per_frame, num_inference_steps)
        y_slice = y[:, :, start_idx // tokens_per_frame : end_idx // tokens_per_frame].squeeze(0)
        latent = latent.to(self.device, torch.float32)
        ctx = context if isinstance(context, (list, tuple)) else [context[0] if context.dim() == 3 else context]
        for i in range(len(TIMESTEPS) - 1):
            t = torch.tensor([TIMESTEPS[i]], device=self.device)
            kw = dict(context=ctx, clip_fea=clip_fea, y=[y_slice], start_idx=start_idx, end_idx=end_idx)
            x_in = [latent.to(self.torch_dtype)]
            pred = self.dit(x_in, t, audio=audio_embedding, kv_cache=self.kv_cache_manager.get_timestep_caches(i), **kw)[0]
            if audio_cfg > 1.0 and i in (1, 2):
                silent = self.dit(x_in, t, audio=torch.zeros_like(audio_embedding),
                                  kv_cache=self._null_audio_manager.get_timestep_caches(i), **kw)[0]  # fmt: skip
                pred = silent + audio_cfg * (pred - silent)
            latent = latent - pred.float() * ((TIMESTEPS[i] - TIMESTEPS[i + 1]) / 1000)
        return latent.to(self.torch_dtype)


class LiveActPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = self.width_division_factor = 16

    def _get_stages(self) -> list:
        return [self.audio_encoding_stage, self.denoise_stage, self.text_encoding_stage, self.clip_encoding_stage, self.vae_stage]

    def init(self, module_manager, config: LiveActPipelineConfig, text_stage=None, clip_stage=None, audio_stage=None):
        from telefuser_b200.pipelines.wan.stages import ClipEncodingStage, TextEncodingStage, VAEStage
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.vae_stage = VAEStage("vae", module_manager, config.vae_config)
        self.clip_encoding_stage = clip_stage or ClipEncodingStage("clip_encoding", module_manager, config.clip_config)
        self.text_encoding_stage = text_stage or TextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        self.audio_encoding_stage = audio_stage or AudioEncodingStage("audio_encoding", module_manager, config.audio_config,
                                                                      config.audio_window)  # fmt: skip
        self.denoise_stage = LiveActDenoisingStage("denoise", module_manager, config.dit_config, config.fp8_kv_cache,
                                                   config.offload_cache, config.mean_memory)  # fmt: skip
        for s in (self.vae_stage, self.denoise_stage):
            s.onload_models_flag = True
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)
        if config.enable_vae_parallel:
            self.vae_stage = ParallelWorker(self.vae_stage)

    def preprocess_image(self, image, height: int, width: int) -> torch.Tensor:
        """Centre crop to the target aspect ratio, resize, scale to [-1, 1] -> [1, 3, H, W]."""
        from PIL import Image

        w0, h0 = image.size
        scale = max(height / h0, width / w0)
        image = image.convert("RGB").resize((max(width, round(w0 * scale)), max(height, round(h0 * scale))), Image.LANCZOS)
        left, top = (image.size[0] - width) // 2, (image.size[1] - height) // 2
        arr = np.asarray(image.crop((left, top, left + width, top + height)), dtype=np.float32)
        return torch.from_numpy(arr).permute(2, 0, 1).unsqueeze(0) / 127.5 - 1.0

    @torch.no_grad()
    def __call__(self, prompt: str, input_image, audio_path=None, audio=None, audio_sr: int = 16000, seed=None,
                 height: int = 480, width: int = 832, fps: int = 24, num_inference_steps: int = 3, audio_cfg: float = 1.0,
                 output_type: str = "pil"):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        image = input_image if isinstance(input_image, torch.Tensor) else self.preprocess_image(input_image, height, width)
        prompt_emb = self.text_encoding_stage.process([prompt])[0]
        clip_fea = self.clip_encoding_stage.process(image)
        stream = self.config.stream_audio
        _, duration = self.audio_encoding_stage.process(audio_path=audio_path, audio=audio, sr=audio_sr, fps=fps, stream_audio=stream)
        blocks = self.config.block_sizes
        frames_per_iter = (sum(blocks) - 1) * VAE_STRIDE[0] + 1
        iterations = int(duration / (VAE_STRIDE[0] * blocks[-1] / fps)) + 1
        y = auto_async_call(self.vae_stage.process, "encode_image", image, None, frames_per_iter, tiled=False, concat_mask=True)()
        tpf = (height // (PATCH_SIZE[1] * VAE_STRIDE[1])) * (width // (PATCH_SIZE[2] * VAE_STRIDE[2]))
        gen = None if seed is None else torch.Generator().manual_seed(seed)
        getattr(self.denoise_stage, "clear_kv_cache", lambda: None)()  # a new video starts with empty memories
        videos, prev = [], None
        for it in range(iterations):
            shift = max(it - 1, 0) * blocks[-1] * VAE_STRIDE[0]
            a0, a1 = shift, frames_per_iter + shift
            if stream:
                audio_emb = self.audio_encoding_stage.process_stream_audio_segment(a0, a1, fps, frames_per_iter)
            else:
                audio_emb = self.audio_encoding_stage.process_pre_encoded_segment(a0, a1)
            f = min(it, 1)
            noise = torch.randn((LATENT_CHANNELS, blocks[f], height // VAE_STRIDE[1], width // VAE_STRIDE[2]), generator=gen)
            latent = auto_async_call(self.denoise_stage.process, latent=noise.to(self.device, self.torch_dtype), context=prompt_emb,
                                     clip_fea=clip_fea, audio_embedding=audio_emb, y=y, tokens_per_frame=tpf, audio_cfg=audio_cfg,
                                     num_inference_steps=num_inference_steps, seed=seed, block_sizes=blocks)()  # fmt: skip
            if f == 0:
                frames = auto_async_call(self.vae_stage.process, "decode_video", latent.unsqueeze(0))()[0]
            else:  # decode with 3 latents of context; their 9 frames were already emitted
                ctx = torch.cat([prev[:, -3:], latent], dim=1).unsqueeze(0)
                frames = auto_async_call(self.vae_stage.process, "decode_video", ctx)()[0, :, 9:]
            prev = latent
            videos.append(frames.float().cpu())
        video = torch.cat(videos, dim=1)
        return video if output_type == "pt" else self.tensor2video(video)
