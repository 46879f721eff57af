"""Public LingBot-World v2 pipeline: the causal-fast engine of `pipelines.lingbot_world` fixed to what the
published v2 checkpoint supports (camera control; 18 latent frames of local attention with 6 sink frames; the four
distilled timesteps 0 / 250 / 500 / 750), plus the placement of its three stage groups on the GPUs of one node.

Role parity: telefuser/pipelines/lingbot_world_v2/pipeline.py:14-30 and the placement rules of
examples/lingbot/lingbot_world_v2_image_to_video_h100.py:92-106.
"""

from __future__ import annotations

from dataclasses import dataclass

from telefuser_b200.pipelines.lingbot_world.pipeline import LingBotWorldFastPipeline, LingBotWorldFastPipelineConfig


@dataclass
class LingBotWorldV2PipelineConfig(LingBotWorldFastPipelineConfig):
    control_type: str = "cam"
    local_attn_size: int = 18
    sink_size: int = 6
    timestep_indices: tuple = (0, 250, 500, 750)


def resolve_stage_devices(gpu_count: int, default_vae_encode: int = 0, default_vae_decode: int = 0):
    """(DiT device ids, VAE-encode device, VAE-decode device) for `gpu_count` GPUs.

    The sequence-parallel DiT group wants a size that divides the head count (40): 1, 2, 4, 5 or 8. With 2 or 4
    GPUs all of them run the DiT and the two VAE actors share GPUs 0 and 1 with it (encode and decode then overlap
    each other). With 5 or 6 GPUs the last one is left to the VAE alone, so encode / decode never contend with a
    DiT rank. Any other count runs the DiT on all GPUs and both VAE actors on the configured defaults."""
    if gpu_count < 1:
        raise ValueError(f"at least one GPU is needed, got {gpu_count}")
    if gpu_count in (2, 4):
        return list(range(gpu_count)), 0, 1
    if gpu_count in (5, 6):
        return list(range(gpu_count - 1)), gpu_count - 1, gpu_count - 1
    return list(range(gpu_count)), default_vae_encode, default_vae_decode


class LingBotWorldV2Pipeline(LingBotWorldFastPipeline):
    def init(self, module_manager, config: LingBotWorldV2PipelineConfig, text_stage=None):
        if config.control_type != "cam":
            raise ValueError(f"the v2 causal-fast checkpoint is camera-controlled only (got control_type={config.control_type!r})")
        super().init(module_manager, config, text_stage=text_stage)
