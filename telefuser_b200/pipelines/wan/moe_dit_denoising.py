"""Denoising with two expert DiTs (Wan2.2 A14B): a high-noise model down to `boundary`, a low-noise model after.

The loop is the single-model loop (`WanDenoisingStage`): guidance combine and Euler update in one fused pass,
CFG-parallel pair over peer memory. Added here: the switch of the active model when the timestep drops below
boundary * 1000 (with its own guidance scale, feature cache and CPU offload hand-over), resuming from a
cached latent at `skip_step`, and snapshots of the latent before the steps named in `saved_steps`.
Role parity: telefuser/pipelines/wan_video/moe_dit_denoising.py:26-409.
"""

from __future__ import annotations

from typing import Any

import torch

from telefuser_b200.core.config import ModelRuntimeConfig, WeightOffloadType
from telefuser_b200.parallel import mesh as pmesh

from .denoising import WanDenoisingStage
from .latent_data_utils import parse_latent_data


class MoeDitDenoisingStage(WanDenoisingStage):
    def __init__(self, name: str, module_manager: Any, dit_high_runtime_config: ModelRuntimeConfig,
                 dit_low_runtime_config: ModelRuntimeConfig, scheduler: Any, dits=None) -> None:  # fmt: skip
        high, low = dits if dits is not None else module_manager.fetch_module("wan_video_dit", index=2)
        super().__init__(name, module_manager, dit_high_runtime_config, scheduler, dit=high)
        self.num_train_timesteps = 1000
        self.dit_high, self.dit_low = high, low
        self.dit_high_runtime_config, self.dit_low_runtime_config = dit_high_runtime_config, dit_low_runtime_config
        self.dit_low.set_attention_config(dit_low_runtime_config.attention_config)
        self.model_names = ["dit_high", "dit_low"]
        self._resident = {"high": False, "low": False}
        off = dit_low_runtime_config.offload_config.offload_type
        if not dit_low_runtime_config.parallel_config.enable_fsdp:
            if off == WeightOffloadType.SEQUENTIAL_CPU_OFFLOAD:
                self.dit_low.enable_sequential_cpu_offload(self.device)
            if off == WeightOffloadType.ASYNC_CPU_OFFLOAD:
                self.dit_low.enable_async_offload(self.device, dit_low_runtime_config.offload_config)
        if self.dit_low_runtime_config.lora_configs:
            from telefuser_b200.utils.lora import LoRALoader

            for cfg in self.dit_low_runtime_config.lora_configs:
                LoRALoader().apply_lora(self.dit_low, cfg.path, strength=cfg.strength)

    def _offloads(self, which: str) -> bool:
        cfg = self.dit_high_runtime_config if which == "high" else self.dit_low_runtime_config
        return cfg.offload_config.offload_type != WeightOffloadType.NO_CPU_OFFLOAD

    def _activate(self, which: str):
        """Makes one expert resident (moving the other to the host when its config offloads) and current."""
        other = "low" if which == "high" else "high"
        models = {"high": self.dit_high, "low": self.dit_low}
        if self._offloads(other) and self._resident[other]:
            models[other].offload_device()
            self._resident[other] = False
        if self._offloads(which) or not self._resident[which]:
            models[which].onload_device(self.device)
            self._resident[which] = True
        self.dit = models[which]
        return self.dit

    def parallel_models(self) -> None:
        for dit, cfg in ((self.dit_high, self.dit_high_runtime_config), (self.dit_low, self.dit_low_runtime_config)):
            self.dit, self.model_runtime_config = dit, cfg
            super().parallel_models()
            if dit is self.dit_high:
                self.dit_high = self.dit
            else:
                self.dit_low = self.dit
        self.dit, self.model_runtime_config = self.dit_high, self.dit_high_runtime_config

    @torch.no_grad()
    def process(self, latents, num_inference_steps, ref_latent=None, prompt_emb_posi=None, prompt_emb_nega=None,
                cfg_scale_high: float = 5.0, cfg_scale_low: float = 5.0, sigma_shift: float = 5.0, boundary: float = 0.875,
                latent_data: dict | None = None):  # fmt: skip
        if isinstance(num_inference_steps, int):
            self.scheduler.set_timesteps(num_inference_steps, shift=sigma_shift)
        else:  # (high steps, low steps) for the mixed schedule
            self.scheduler.set_timesteps(num_inference_steps, shift=sigma_shift, boundary=boundary)
            num_inference_steps = num_inference_steps[0]
        timesteps = self.scheduler.timesteps
        total = len(timesteps)
        boundary_t = boundary * self.num_train_timesteps
        cached, start, saved = parse_latent_data(latent_data, tuple(latents.shape), total)
        latents = (cached if cached is not None else latents).to(device=self.device, dtype=torch.float32)
        saved, snapshots = frozenset(saved), {}
        which = "low" if (start > 0 and float(timesteps[start]) < boundary_t) else "high"
        cfgs = {"high": (self.dit_high_runtime_config, cfg_scale_high), "low": (self.dit_low_runtime_config, cfg_scale_low)}
        dit = self._activate(which)
        self.setup_feature_cache(dit, cfgs[which][0].feature_cache_config, num_inference_steps, init_step=start)
        dit.feature_cache.reset()
        self.mesh = getattr(dit, "device_mesh", None) or pmesh.get_mesh()
        for i in range(start, total):
            t = timesteps[i]
            if which == "high" and float(t) < boundary_t:
                which = "low"
                dit = self._activate("low")
                self.setup_feature_cache(dit, cfgs["low"][0].feature_cache_config, num_inference_steps, init_step=i)
                dit.feature_cache.reset()
            ts = t.reshape(1).to(device=self.device, dtype=torch.float32).expand(latents.shape[0])
            x_in = latents if ref_latent is None else torch.cat([latents, ref_latent.to(latents)], dim=1)
            scale = cfgs[which][1]
            cond, uncond = self.predict_noise_with_cfg(x_in.to(self.torch_dtype), ts, prompt_emb_posi, prompt_emb_nega, None,
                                                       scale, total - i - 1)  # fmt: skip
            if i in saved:
                snapshots[i] = latents.detach().cpu()
            sigma, nxt = self.scheduler.sigma_pair(t)
            latents = self.guided_step(latents, cond, uncond, scale, nxt - sigma)
        if self._offloads("low") and self._resident["low"]:
            self.dit_low.offload_device()
            self._resident["low"] = False
        if latent_data is not None:
            return latents, {"latent_states_dict": snapshots, "saved_steps": sorted(saved), "final_step": total - 1}
        return latents
