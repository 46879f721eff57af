"""Feature-cache interface: lets a DiT skip its block stack on some denoising steps.

Interface parity with the reference's ``telefuser/feature_cache/base.py:28-150``.
"""

from __future__ import annotations

from abc import ABC, abstractmethod

import torch


class BaseFeatureCache(ABC):
    @abstractmethod
    def should_compute(self, is_cond: bool) -> bool:
        """True when the block stack must run this step. Advances the branch's step counter."""

    @abstractmethod
    def update(self, output: torch.Tensor, ori_input: torch.Tensor, is_cond: bool) -> None:
        """Records a freshly computed block-stack output."""

    @abstractmethod
    def approximate(self, input: torch.Tensor, is_cond: bool) -> torch.Tensor:  # noqa: A002
        """Returns an approximation of the block-stack output for `input`."""

    def reset(self) -> None:
        return None


class NoOpCache(BaseFeatureCache):
    def should_compute(self, is_cond: bool) -> bool:
        return True

    def update(self, output, ori_input, is_cond) -> None:
        return None

    def approximate(self, input, is_cond):  # noqa: A002
        return input


def create_feature_cache(cache_type: str = "none", **kwargs) -> BaseFeatureCache:
    if cache_type == "none":
        return NoOpCache()
    if cache_type == "ada_taylor":
        from .ada_taylor import AdaTaylorCache

        return AdaTaylorCache(**kwargs)
    if cache_type == "calibrator":
        from .ada_taylor import AdaTaylorCacheCalibrator

        return AdaTaylorCacheCalibrator(**kwargs)
    raise ValueError(f"Unknown cache_type: {cache_type}. Expected: none, ada_taylor, calibrator")
