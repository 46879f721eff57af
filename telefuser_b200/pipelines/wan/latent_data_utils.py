"""Validation of the cross-request latent cache hand-off (`latent_data` of a generation request).

`latent_data = {"cached_latent": tensor, "skip_step": k, "saved_steps": [...]}` lets a request resume from the
latent another request saved before step k and asks for snapshots before further steps. A cache whose shape does
not match, whose skip step is out of range, or that is not a tensor is ignored (the request then runs in full).
Role parity: telefuser/pipelines/wan_video/latent_data_utils.py:11-53.
"""

from __future__ import annotations

import torch

from telefuser_b200.utils.logging import logger


def parse_latent_data(latent_data: dict | None, expected_shape: tuple, total_steps: int):
    """-> (cached latent or None, first step to run, sorted steps to snapshot in [first, total))."""
    if not latent_data:
        return None, 0, []
    cached = latent_data.get("cached_latent")
    skip = int(latent_data.get("skip_step") or 0)
    saved = [int(s) for s in (latent_data.get("saved_steps") or [])]
    if cached is not None and not isinstance(cached, torch.Tensor):
        logger.warning(f"[latent_cache] cached_latent is a {type(cached).__name__}, not a tensor: ignored")
        cached = None
    if cached is not None and tuple(cached.shape) != tuple(expected_shape):
        logger.warning(f"[latent_cache] cached shape {tuple(cached.shape)} != {tuple(expected_shape)}: ignored")
        cached = None
    if skip >= total_steps:
        logger.warning(f"[latent_cache] skip_step {skip} >= {total_steps} steps: ignored")
        cached = None
    if cached is None or skip <= 0:
        cached, skip = None, 0
    return cached, skip, sorted({s for s in saved if skip <= s < total_steps})
