"""Denoising for Wan2.2 TI2V (5B): image conditioning by latent replacement and per-token timesteps.

With a reference image the first latent frame (and the last, with an end image) is the encoded image itself:
it is written back into the latents after every step, and the model is told that those tokens are clean by a
per-token timestep (0 on conditioned frames, t elsewhere), one value per 2x2 latent patch.
Role parity: telefuser/pipelines/wan_video/ti2v_denoising.py:27-396.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from telefuser_b200.core.base_stage import with_model_offload

from .denoising import WanDenoisingStage


def per_token_timestep(timestep: torch.Tensor, mask: torch.Tensor, patch=(1, 2, 2)) -> torch.Tensor:
    """timestep [1]; mask [C, T, H, W] (0 = conditioned) -> [1, T * H/ph * W/pw]."""
    m = mask[0, :, :: patch[1], :: patch[2]]
    return (m.flatten() * timestep.reshape(1)).unsqueeze(0)


class TI2VDenoisingStage(WanDenoisingStage):
    def _replace(self, latents, mask, start_latent, end_latent):
        latents = ((1.0 - mask) * start_latent + mask * latents[0]).unsqueeze(0)
        if end_latent is not None:
            latents[0, :, -1:] = end_latent
        return latents

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, num_inference_steps, ref_latent=None, ref_mask=None, prompt_emb_posi=None,
                prompt_emb_nega=None, cfg_scale: float = 5.0, sigma_shift: float = 5.0):  # fmt: skip
        self.scheduler.set_timesteps(num_inference_steps, shift=sigma_shift)
        self.setup_feature_cache(self.dit, self.model_runtime_config.feature_cache_config, num_inference_steps)
        self.dit.feature_cache.reset()
        latents = latents.to(device=self.device, dtype=torch.float32)
        mask = start_latent = end_latent = None
        if ref_latent is not None and ref_mask is not None:
            mask = torch.ones(latents.shape[1:], device=self.device, dtype=torch.float32)
            mask[:, 0] = 0
            if isinstance(ref_latent, (tuple, list)):
                start_latent, end_latent = (r.to(self.device, torch.float32) for r in ref_latent)
                mask[:, -1] = 0
            else:
                start_latent = ref_latent.to(self.device, torch.float32)
            latents = self._replace(latents, mask, start_latent, end_latent)
        pp = self.mesh.size("pp") > 1
        last_stage = (not pp) or self.mesh.coord("pp") == self.mesh.size("pp") - 1
        timesteps = self.scheduler.timesteps
        patch = tuple(getattr(self.dit, "patch_size", (1, 2, 2)))
        for i, t in enumerate(timesteps):
            ts = t.reshape(1).to(device=self.device, dtype=torch.float32)
            ts = per_token_timestep(ts, mask, patch) if mask is not None else ts.expand(latents.shape[0])
            cond, uncond = self.predict_noise_with_cfg(latents.to(self.torch_dtype), ts, prompt_emb_posi, prompt_emb_nega,
                                                       None, cfg_scale, len(timesteps) - i - 1)  # fmt: skip
            sigma, nxt = self.scheduler.sigma_pair(t)
            if last_stage:
                latents = self.guided_step(latents, cond, uncond, cfg_scale, nxt - sigma)
                if mask is not None:
                    latents = self._replace(latents, mask, start_latent, end_latent)
            if pp:
                dist.broadcast(latents, src=self.mesh.ranks("pp")[-1], group=self.mesh.group("pp"))
        return latents
