from .pipeline import (LingBotVideoDenoisingStage, LingBotVideoGeneration, LingBotVideoPipeline,
                       LingBotVideoPipelineConfig, LingBotVideoRequest, compute_refiner_sigmas, latent_shape,
                       prepare_refiner_latent, reinject_ti2v_condition)  # fmt: skip

__all__ = ["LingBotVideoDenoisingStage", "LingBotVideoGeneration", "LingBotVideoPipeline", "LingBotVideoPipelineConfig",
           "LingBotVideoRequest", "compute_refiner_sigmas", "latent_shape", "prepare_refiner_latent",
           "reinject_ti2v_condition"]  # fmt: skip
