from .pipeline import (LongCatDitDenoisingStage, LongCatRefineDenoisingStage, LongCatTextEncodingStage, LongCatVideoPipeline,
                       LongCatVideoPipelineConfig, bsa_align_resolution, cfg_zero_star)  # fmt: skip

__all__ = ["LongCatDitDenoisingStage", "LongCatRefineDenoisingStage", "LongCatTextEncodingStage", "LongCatVideoPipeline",
           "LongCatVideoPipelineConfig", "bsa_align_resolution", "cfg_zero_star"]  # fmt: skip
