from .pipeline import (LingBotVideoDenoisingStage, LingBotVideoGeneration, LingBotVideoPipeline,
                       LingBotVideoPipelineConfig, LingBotVideoRequest, compute_refiner_sigmas, latent_shape,
                       prepare_refiner_latent, reinject_ti2v_condition)  # fmt: skip

from .data import (DEFAULT_NEGATIVE_PROMPT, DEFAULT_NEGATIVE_PROMPT_IMAGE, LingBotVideoModelConfig, default_negative_caption,
                   load_lingbot_video_model_config, load_lingbot_video_prompt, num_frames_from_duration,
                   parse_lingbot_video_prompt, preprocess_ti2v_image, smart_resize)  # fmt: skip

__all__ = ["DEFAULT_NEGATIVE_PROMPT", "DEFAULT_NEGATIVE_PROMPT_IMAGE", "LingBotVideoModelConfig", "default_negative_caption",
           "load_lingbot_video_model_config", "load_lingbot_video_prompt", "num_frames_from_duration", "parse_lingbot_video_prompt",
           "preprocess_ti2v_image", "smart_resize","LingBotVideoDenoisingStage", "LingBotVideoGeneration", "LingBotVideoPipeline", "LingBotVideoPipelineConfig",
           "LingBotVideoRequest", "compute_refiner_sigmas", "latent_shape", "prepare_refiner_latent",
           "reinject_ti2v_condition"]  # fmt: skip
