from .pipeline import (ZImageDenoisingStage, ZImagePipeline, ZImagePipelineConfig, ZImageTextEncodingStage, ZImageVAEStage,
                       guided_prediction, tiled_decode)  # fmt: skip

__all__ = ["ZImageDenoisingStage", "ZImagePipeline", "ZImagePipelineConfig", "ZImageTextEncodingStage", "ZImageVAEStage",
           "guided_prediction", "tiled_decode"]  # fmt: skip
