from .pipeline import FlashVSRDenoisingStage, FlashVSRPipelineConfig, FlashVSRStreamPipeline, FlashVSRVAEStage, prepare_input_tensor

__all__ = ["FlashVSRDenoisingStage", "FlashVSRPipelineConfig", "FlashVSRStreamPipeline", "FlashVSRVAEStage",
           "prepare_input_tensor"]  # fmt: skip
