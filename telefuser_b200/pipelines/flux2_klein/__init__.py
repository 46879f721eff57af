from .pipeline import (Flux2DenoisingStage, Flux2KleinPipeline, Flux2KleinPipelineConfig, Flux2TextEncodingStage,
                       Flux2VAEStage)  # fmt: skip

__all__ = ["Flux2DenoisingStage", "Flux2KleinPipeline", "Flux2KleinPipelineConfig", "Flux2TextEncodingStage",
           "Flux2VAEStage"]  # fmt: skip
