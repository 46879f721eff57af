from .dit_denoising import (
    AudioLatentShape,
    ConditioningItemAttentionStrengthWrapper,
    DitDenoisingStage,
    LatentState,
    MultiModalGuider,
    MultiModalGuiderParams,
    VideoConditionByKeyframeIndex,
    VideoConditionByLatentIndex,
)
from .pipeline import LTX23VideoPipeline, LTXVideoPipelineConfig
from .stages import GemmaTextEncodingStage, UpsamplerStage, VAEStage

__all__ = ["AudioLatentShape", "ConditioningItemAttentionStrengthWrapper", "DitDenoisingStage", "GemmaTextEncodingStage",
           "LTX23VideoPipeline", "LTXVideoPipelineConfig", "LatentState", "MultiModalGuider", "MultiModalGuiderParams",
           "UpsamplerStage", "VAEStage", "VideoConditionByKeyframeIndex", "VideoConditionByLatentIndex"]  # fmt: skip
