"""Denoising stage of the Wan pipelines: the timestep loop around the DiT.

Per step: one DiT forward per guidance branch (both on this rank, or one each
under CFG parallelism), then guidance ``u + s (c - u)`` and the flow-matching
Euler update fused into a single pass over the fp32 latents. Latents stay in
fp32 for the whole loop; only the DiT input is cast to the compute dtype.

Reference behaviour: ``telefuser/pipelines/wan_video/single_dit_denoising.py:24-262``
(predict_noise_with_cfg :79-158, process :164-237, parallel_models :239-262).
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig, WeightOffloadType
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard


class _PeerPrediction:
    """This rank's branch of a CFG-parallel pair; the partner's branch is read from its memory."""

    def __init__(self, tensor: torch.Tensor) -> None:
        self.tensor = tensor


class WanDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, scheduler: Any,
                 dit: Any | None = None) -> None:  # fmt: skip
        super().__init__(name, model_runtime_config)
        self.dit = dit if dit is not None else module_manager.fetch_module("wan_video_dit")
        self.dit.set_attention_config(model_runtime_config.attention_config)
        self.model_names = ["dit"]
        self.scheduler = scheduler
        self.mesh = pmesh.get_mesh()
        self.step_callback = None  # optional fn(step_index, latents) for latent-cache snapshots
        self._load_loras(module_manager)
        off = model_runtime_config.offload_config.offload_type
        fsdp = model_runtime_config.parallel_config.enable_fsdp
        if off == WeightOffloadType.SEQUENTIAL_CPU_OFFLOAD and not fsdp:
            self.dit.enable_sequential_cpu_offload(self.device)
        if off == WeightOffloadType.ASYNC_CPU_OFFLOAD and not fsdp:
            self.dit.enable_async_offload(self.device, model_runtime_config.offload_config)
        if model_runtime_config.parallel_config.world_size == 1 and model_runtime_config.compile_config.enabled:
            self.dit.compile(model_runtime_config.compile_config)

    def _load_loras(self, module_manager) -> None:
        if not self.model_runtime_config.lora_configs:
            return
        from telefuser_b200.utils.lora import LoRALoader

        loader = LoRALoader()
        for cfg in self.model_runtime_config.lora_configs:
            loader.apply_lora(self.dit, cfg.path, strength=cfg.strength)

    # ---- per-rank set-up -----------------------------------------------------
    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.mesh = pmesh.create_device_mesh_from_config(cfg)
        self.configure_device_waits()
        self.dit.device_mesh = self.mesh
        self.dit.set_attention_config(self.model_runtime_config.attention_config)
        if cfg.sp_degree > 1:
            self.dit.enable_usp()
        if cfg.pp_degree > 1:
            from telefuser_b200.parallel.pp import stage_block_range

            start, end = stage_block_range(self.dit.num_layers, cfg.pp_degree, self.mesh.coord("pp"))
            self.dit.enable_pp(start, end, self.mesh.group("pp"))
        if cfg.tp_degree > 1:
            from telefuser_b200.parallel.tp import parallelize_module

            parallelize_module(self.dit, self.mesh, self.dit.get_tp_plan())
        if cfg.enable_fsdp:
            from telefuser_b200.parallel.fsdp import shard_model

            self.dit = shard_model(self.dit, self.device, wrap_module_names=self.dit.get_fsdp_module_names())
        if self.model_runtime_config.compile_config.enabled:
            self.dit.compile(self.model_runtime_config.compile_config)

    # ---- one guidance evaluation ---------------------------------------------------
    def predict_noise_with_cfg(self, latents, timestep, prompt_emb_posi, prompt_emb_nega, clip_feature, cfg_scale,
                               numeral_timestep: int = 0):  # fmt: skip
        """Returns (cond, uncond) predictions; `uncond` is None when guidance is off.
        `numeral_timestep` = denoising steps still to run after this one (selects dense / sparse attention)."""
        use_cfg = cfg_scale != 1.0 and prompt_emb_nega is not None
        kw = dict(clip_feature=clip_feature, numeral_timestep=numeral_timestep)
        if use_cfg and self.mesh.size("cfg") == 2:
            is_cond = self.mesh.coord("cfg") == 0
            ctx = prompt_emb_posi if is_cond else prompt_emb_nega
            mine = self.dit(latents, timestep, ctx, cond_flag=is_cond, **kw)
            if mine is None:  # not the last pipeline stage: nothing to combine here
                return None, None
            if self.mesh.fused and mine.is_cuda:
                return _PeerPrediction(mine), None  # combined by peer loads inside the step kernel
            return pshard.cfg_parallel_unshard(mine, self.mesh)
        cond = self.dit(latents, timestep, prompt_emb_posi, cond_flag=True, **kw)
        if not use_cfg:
            return cond, None
        uncond = self.dit(latents, timestep, prompt_emb_nega, cond_flag=False, **kw)
        return cond, uncond

    def guided_step(self, latents, cond, uncond, cfg_scale, dsigma):
        """Guidance combine + flow-matching Euler update (one kernel; the CFG-parallel form reads the
        partner rank's prediction over NVLink instead of all-gathering it first)."""
        if isinstance(cond, _PeerPrediction):
            from telefuser_b200.parallel.symm import cfg_combine_step_fused, get_workspace

            pred = cond.tensor
            ws = get_workspace(self.mesh.group("cfg"), pred.numel() * pred.element_size() + 4096)
            return cfg_combine_step_fused(latents, pred, ws, cfg_scale, float(dsigma))
        return TF.cfg_euler_step(latents, cond, uncond, cfg_scale, dsigma)

    # ---- the loop ---------------------------------------------------------------------
    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, num_inference_steps, ref_latent=None, prompt_emb_posi=None, prompt_emb_nega=None,
                clip_feature=None, cfg_scale=5.0, sigma_shift=5.0, skip_step: int = 0):  # fmt: skip
        """latents: [B, C, F, H, W]; returns the denoised latents (fp32)."""
        self.scheduler.set_timesteps(num_inference_steps, shift=sigma_shift)
        self.setup_feature_cache(self.dit, self.model_runtime_config.feature_cache_config, num_inference_steps,
                                 init_step=skip_step)  # fmt: skip
        self.dit.feature_cache.reset()
        latents = latents.to(device=self.device, dtype=torch.float32)
        pp = self.mesh.size("pp") > 1
        timesteps = self.scheduler.timesteps
        for i in range(skip_step, len(timesteps)):
            t = timesteps[i]
            ts = t.reshape(1).to(device=self.device, dtype=torch.float32).expand(latents.shape[0])
            x_in = latents if ref_latent is None else torch.cat([latents, ref_latent.to(latents)], dim=1)
            x_in = x_in.to(self.torch_dtype)
            cond, uncond = self.predict_noise_with_cfg(x_in, ts, prompt_emb_posi, prompt_emb_nega, clip_feature,
                                                       cfg_scale, len(timesteps) - i - 1)  # fmt: skip
            sigma, nxt = self.scheduler.sigma_pair(t)
            if pp:
                src = self.mesh.ranks("pp")[-1]
                if self.mesh.coord("pp") == self.mesh.size("pp") - 1:
                    latents = self.guided_step(latents, cond, uncond, cfg_scale, nxt - sigma)
                dist.broadcast(latents, src=src, group=self.mesh.group("pp"))
            else:
                latents = self.guided_step(latents, cond, uncond, cfg_scale, nxt - sigma)
            if self.step_callback is not None:
                self.step_callback(i, latents)
            self.check_device_waits()  # non-blocking: sees the word posted one step ago
        self.check_device_waits(final=True)
        return latents


# Name used by pipeline files written for the reference.
SingleDitDenoisingStage = WanDenoisingStage
