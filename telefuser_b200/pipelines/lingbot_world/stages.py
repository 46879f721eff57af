"""Stages of the LingBot-World streaming pipeline: condition encode, chunk denoise, chunk decode.

Every stage keeps per-session state under a `cache_handle` (KV caches, scheduler, RNG, VAE
causal state), so the stages can live in separate worker processes / GPUs and serve many
sessions. Unlike the reference (telefuser/pipelines/lingbot_world_fast/denoising.py:49-299,
vae_stage.py), chunk tensors are returned on the stage's device; they only move to the host
when a worker boundary or the client requires it.

A chunk = `chunk_size` latent frames. Denoising runs the few-step schedule (model forward,
x0 = x_t - sigma * v, re-noise to the next timestep with fresh noise) and then one extra
forward at t = 0 on the clean latent, which writes the chunk's final K/V into the rolling
cache (5 forwards per chunk for a 4-step schedule).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.schedulers.unipc import FlowUniPCMultistepScheduler


def select_timesteps(scheduler: FlowUniPCMultistepScheduler, indices: tuple, shift: float,
                     num_train_timesteps: int = 1000) -> torch.Tensor:  # fmt: skip
    if not indices:
        raise ValueError("timestep indices must not be empty")
    if any(not isinstance(i, int) or isinstance(i, bool) for i in indices):
        raise ValueError(f"timestep indices must be integers, got {indices!r}")
    if any(i < 0 or i >= num_train_timesteps for i in indices):
        raise ValueError(f"timestep indices must be in [0, {num_train_timesteps}), got {indices!r}")
    if tuple(sorted(indices)) != tuple(indices) or len(set(indices)) != len(indices):
        raise ValueError(f"timestep indices must be strictly increasing, got {indices!r}")
    scheduler.set_timesteps(num_train_timesteps, shift=shift)
    return scheduler.timesteps[list(indices)].clone()


@dataclass
class DenoisingCacheState:
    scheduler: FlowUniPCMultistepScheduler
    timesteps: torch.Tensor
    model_cache: Any
    generator: torch.Generator
    noise_generator: torch.Generator
    noise_shape: tuple
    chunks_done: int = 0


class LingBotWorldFastDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, dit=None) -> None:
        super().__init__(name, model_runtime_config)
        self.dit = dit if dit is not None else module_manager.fetch_module("lingbot_world_fast_dit")
        if self.dit is None:
            raise ValueError("LingBot denoising stage requires a loaded lingbot_world_fast_dit module")
        self.dit.set_attention_config(model_runtime_config.attention_config)
        self.model_names = ["dit"]
        self._caches: dict[int, DenoisingCacheState] = {}
        self.mesh = pmesh.get_mesh()

    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.mesh = pmesh.create_device_mesh_from_config(cfg)
        self.dit.device_mesh = self.mesh
        if cfg.sp_ulysses_degree > 1:
            if self.dit.num_heads % cfg.sp_ulysses_degree:
                raise ValueError(f"{self.dit.num_heads} heads are not divisible by Ulysses degree {cfg.sp_ulysses_degree}")
            self.dit.enable_usp()
        if cfg.enable_fsdp:
            from telefuser_b200.parallel.fsdp import shard_model

            self.dit = shard_model(self.dit, self.device, wrap_module_names=self.dit.get_fsdp_module_names())

    # ---- session state ------------------------------------------------------------
    @with_model_offload(["dit"])
    def initialize_cache(self, cache_handle: int, batch_size: int, kv_size: int, max_sequence_length: int,
                         sample_shift: float, generator_state, noise_generator_state, noise_shape,
                         timestep_indices: tuple = (0, 179, 358, 679), frame_tokens: int | None = None) -> bool:  # fmt: skip
        if cache_handle in self._caches:
            raise ValueError(f"Cache handle {cache_handle} is already registered")
        sched = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        ts = select_timesteps(sched, tuple(timestep_indices), sample_shift)
        gen = torch.Generator(device=self.device)
        ngen = torch.Generator(device=self.device)
        for g, st in ((gen, generator_state), (ngen, noise_generator_state)):
            if isinstance(st, int):
                g.manual_seed(st)
            else:
                g.set_state(torch.as_tensor(st, dtype=torch.uint8))
        if frame_tokens is None:
            frame_tokens = (noise_shape[3] // self.dit.patch_size[1]) * (noise_shape[4] // self.dit.patch_size[2])
        cache = self.dit.new_cache_state(batch_size, kv_size, frame_tokens, device=self.device, dtype=self.torch_dtype,
                                         ulysses_degree=self.mesh.size("ulysses"))  # fmt: skip
        self._caches[cache_handle] = DenoisingCacheState(sched, ts, cache, gen, ngen, tuple(noise_shape))
        return True

    def release_cache(self, cache_handle: int) -> bool:
        return self._caches.pop(cache_handle, None) is not None

    def cache_bytes(self, cache_handle: int) -> int:
        return self._caches[cache_handle].model_cache.nbytes()

    # ---- snapshot / resume ------------------------------------------------------------------
    def snapshot_cache(self, cache_handle: int) -> dict:
        """Session state of this stage as CPU tensors and plain values (picklable): the K/V history of every block,
        both random generators and the chunk counter. With `restore_cache` on a fresh stage (after a worker
        restart, or on another replica) the session continues with the same chunks it would have produced."""
        st = self._state(cache_handle)
        return {"chunks_done": st.chunks_done, "noise_shape": list(st.noise_shape), "timesteps": st.timesteps.cpu(),
                "generator": st.generator.get_state(), "noise_generator": st.noise_generator.get_state(),
                "model_cache": st.model_cache.snapshot()}  # fmt: skip

    def restore_cache(self, cache_handle: int, snap: dict) -> bool:
        """The handle must have been registered by `initialize_cache` with the session's shapes."""
        st = self._state(cache_handle)
        if tuple(snap["noise_shape"]) != tuple(st.noise_shape):
            raise ValueError("the snapshot belongs to a session of another resolution or chunk size")
        st.model_cache.restore(snap["model_cache"])
        st.generator.set_state(torch.as_tensor(snap["generator"], dtype=torch.uint8))
        st.noise_generator.set_state(torch.as_tensor(snap["noise_generator"], dtype=torch.uint8))
        st.timesteps = snap["timesteps"].to(st.timesteps.device)
        st.chunks_done = int(snap["chunks_done"])
        return True

    def _state(self, cache_handle: int) -> DenoisingCacheState:
        try:
            return self._caches[cache_handle]
        except KeyError as e:
            raise KeyError(f"Unknown cache handle {cache_handle}") from e

    def _next_noise(self, st: DenoisingCacheState) -> torch.Tensor:
        return torch.randn(st.noise_shape, generator=st.noise_generator, device=self.device, dtype=torch.float32)

    def advance_noise(self, cache_handle: int) -> bool:
        """Keeps the noise RNG in step when a chunk is served from a cache instead of being denoised."""
        self._next_noise(self._state(cache_handle))
        return True

    # ---- the chunk ---------------------------------------------------------------------
    @staticmethod
    def flow_to_x0(flow_pred, xt, timestep, scheduler):
        idx = int(torch.argmin((scheduler.timesteps.double() - float(timestep)).abs()))
        sigma = scheduler.sigmas[idx].double()
        return (xt.double() - sigma * flow_pred.double()).to(flow_pred.dtype)

    def denoise_chunk(self, latent, condition, prompt_emb, st: DenoisingCacheState, control, current_start,
                      max_attention_size):  # fmt: skip
        cur = latent
        n = len(st.timesteps)
        for i in range(n):
            t = st.timesteps[i].view(1).to(self.device)
            pred = self.dit(cur.to(self.torch_dtype), t.float(), prompt_emb, y=condition, control_tensor=control,
                            cache=st.model_cache, current_start=current_start, max_attention_size=max_attention_size)  # fmt: skip
            x0 = self.flow_to_x0(pred, cur.float(), t[0], st.scheduler)
            if i < n - 1:
                noise = torch.randn(x0.shape, generator=st.generator, device=x0.device, dtype=x0.dtype)
                cur = st.scheduler.add_noise(x0, noise, st.timesteps[i + 1].view(1))
            else:
                cur = x0
        return cur

    @with_model_offload(["dit"])
    @torch.no_grad()
    def denoise_and_update_cache(self, cache_handle: int, condition_chunk, prompt_emb, control_chunk, current_start: int,
                                 max_attention_size: int, cached_latent=None):  # fmt: skip
        """One chunk: denoise from fresh noise, then the commit pass. With `cached_latent` (the clean latent this very
        chunk had in an earlier session of the same world) the denoising steps are skipped: both random generators
        are advanced by what those steps would have drawn and only the commit pass runs, so the rolling cache and the
        generators end up exactly where a full run leaves them."""
        st = self._state(cache_handle)
        cond = condition_chunk.to(self.device, self.torch_dtype)
        ctrl = None if control_chunk is None else control_chunk.to(self.device, self.torch_dtype)
        emb = prompt_emb.to(self.device, self.torch_dtype)
        if cached_latent is None:
            clean = self.denoise_chunk(self._next_noise(st), cond, emb, st, ctrl, current_start, max_attention_size)
        else:
            self._next_noise(st)
            for _ in range(len(st.timesteps) - 1):  # the re-noising draws between denoising steps
                torch.randn(st.noise_shape, generator=st.generator, device=self.device, dtype=self.torch_dtype)
            clean = cached_latent.to(self.device, self.torch_dtype)
        # commit pass: K/V of the clean latent become the history that later chunks attend to
        self.dit(clean.to(self.torch_dtype), torch.zeros(1, device=self.device), emb, y=cond, control_tensor=ctrl,
                 cache=st.model_cache, current_start=current_start, max_attention_size=max_attention_size)  # fmt: skip
        st.chunks_done += 1
        return clean


@dataclass
class _EncodeState:
    condition_image: torch.Tensor | None
    stream: Any = None


class LingBotWorldFastVAEEncodeStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, model_runtime_config)
        self.vae = vae if vae is not None else module_manager.fetch_module("wan_video_vae")
        if self.vae is None:
            raise ValueError("LingBot VAE encode stage requires a loaded wan_video_vae module")
        self.model_names = ["vae"]
        self._caches: dict[int, _EncodeState] = {}

    def initialize_cache(self, cache_handle: int, condition_image: torch.Tensor) -> bool:
        if cache_handle in self._caches:
            raise ValueError(f"VAE encode cache handle {cache_handle} is already registered")
        self._caches[cache_handle] = _EncodeState(condition_image, self.vae.new_stream("encode"))
        return True

    @with_model_offload(["vae"])
    @torch.no_grad()
    def encode_condition_chunk(self, cache_handle: int, chunk_index: int, chunk_count: int, chunk_size: int,
                               height: int, width: int) -> torch.Tensor:  # fmt: skip
        """[1, 4 + z, chunk_size, h, w]: frame mask (first frame of the first chunk = 1) + encoded condition video."""
        st = self._caches[cache_handle]
        first = chunk_index == 0
        p = next(self.vae.parameters())
        frames = 1 + 4 * (chunk_size - 1) if first else 4 * chunk_size
        video = torch.zeros(1, 3, frames, height, width, device=self.device, dtype=p.dtype)
        if first:
            if st.condition_image is None:
                raise RuntimeError("The first condition chunk requires the session image tensor")
            video[0, :, 0] = st.condition_image.to(self.device, p.dtype)
        latent = self.vae.cached_encode(video, st.stream)[0]
        if latent.shape[1] != chunk_size:
            raise RuntimeError(f"VAE condition chunk has {latent.shape[1]} latent frames, expected {chunk_size}")
        mask = torch.zeros(4, chunk_size, latent.shape[2], latent.shape[3], device=latent.device, dtype=latent.dtype)
        if first:
            mask[:, 0] = 1
            st.condition_image = None
        return torch.cat([mask, latent], dim=0).unsqueeze(0)

    def release_cache(self, cache_handle: int) -> bool:
        return self._caches.pop(cache_handle, None) is not None


class LingBotWorldFastVAEDecodeStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, model_runtime_config)
        self.vae = vae if vae is not None else module_manager.fetch_module("wan_video_vae")
        if self.vae is None:
            raise ValueError("LingBot VAE decode stage requires a loaded wan_video_vae module")
        self.model_names = ["vae"]
        self._caches: dict[int, Any] = {}

    def initialize_cache(self, cache_handle: int) -> bool:
        if cache_handle in self._caches:
            raise ValueError(f"VAE decode cache handle {cache_handle} is already registered")
        self._caches[cache_handle] = self.vae.new_stream("decode")
        return True

    @with_model_offload(["vae"])
    @torch.no_grad()
    def decode_chunk(self, cache_handle: int, latents: torch.Tensor, to_uint8: bool = False) -> torch.Tensor:
        """[1, 3, T, H, W] in [-1, 1] (or uint8 [T, H, W, 3] frames ready for the encoder / client)."""
        frames = self.vae.cached_decode(latents.to(self.device), self._caches[cache_handle])
        if to_uint8:
            from telefuser_b200.ops import functional as TF

            return TF.frames_to_uint8(frames[0])  # one pass on the device; the host copy moves 1 byte per channel
        return frames

    def release_cache(self, cache_handle: int) -> bool:
        return self._caches.pop(cache_handle, None) is not None
