from .realesrgan_upscale import RealESRGANStage
from .vfi import RiftVFIStage

__all__ = ["RealESRGANStage", "RiftVFIStage"]
