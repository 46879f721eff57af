"""Wan2.1 / Wan2.2 pipelines; classes are imported on first access."""

_EXPORTS = {
    "Wan21VideoPipeline": "wan21_video", "Wan21VideoPipelineConfig": "wan21_video",
    "Wan22VideoPipeline": "wan22_video", "Wan22VideoPipelineConfig": "wan22_video",
    "Wan22TI2VPipeline": "wan22_video", "Wan22TI2VPipelineConfig": "wan22_video",
    "AsyncWan22VideoPipeline": "async_wan22_video", "AsyncWan22VideoPipelineConfig": "async_wan22_video",
}  # fmt: skip
__all__ = sorted(_EXPORTS)


def __getattr__(name: str):
    if name in _EXPORTS:
        from importlib import import_module

        return getattr(import_module(f"{__name__}.{_EXPORTS[name]}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
