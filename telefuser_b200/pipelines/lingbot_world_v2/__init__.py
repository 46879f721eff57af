"""LingBot-World v2 (causal-fast checkpoint, camera control) on the shared chunk-autoregressive engine."""

from .pipeline import LingBotWorldV2Pipeline, LingBotWorldV2PipelineConfig, resolve_stage_devices

__all__ = ["LingBotWorldV2Pipeline", "LingBotWorldV2PipelineConfig", "resolve_stage_devices"]
