"""Per-session request record of the LingBot-World pipeline and the frame-count rule.

A session asks for `frame_num = 4n + 1` video frames; the model produces latent frames in chunks of `chunk_size`, so
only lengths with a whole number of chunks can be generated. `frame_policy` says what happens otherwise: "truncate"
(the default) rounds the request down to the last whole chunk, "strict" refuses it.
Role parity: telefuser/pipelines/lingbot_world_fast/session.py:20-67.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

FRAME_POLICIES = ("strict", "truncate")


def _is_count(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def resolve_lingbot_frame_count(frame_num: int, chunk_size: int, frame_policy: str = "truncate") -> tuple[int, int]:
    """(video frames actually generated, latent frames) for a request of `frame_num` frames."""
    if not _is_count(chunk_size) or chunk_size < 1:
        raise ValueError(f"chunk_size counts latent frames per chunk and must be a positive integer, got {chunk_size!r}")
    if not _is_count(frame_num):
        raise ValueError(f"frame_num must be an integer, got {frame_num!r}")
    if frame_policy not in FRAME_POLICIES:
        raise ValueError(f"frame_policy is one of {FRAME_POLICIES}, got {frame_policy!r}")
    if frame_num < 1 or (frame_num - 1) % 4:
        raise ValueError(f"frame_num must have the form 4n+1 (the VAE packs 4 frames per latent frame), got {frame_num}")
    latent = (frame_num - 1) // 4 + 1
    whole = latent - latent % chunk_size
    if whole < chunk_size or (frame_policy == "strict" and whole != latent):
        raise ValueError(f"{frame_num} frames are {latent} latent frames, not a whole number of chunks of {chunk_size}"
                         + ("" if whole >= chunk_size else " (shorter than the first chunk)"))  # fmt: skip
    return 4 * (whole - 1) + 1, whole


@dataclass
class LingBotWorldFastSessionConfig:
    """What one generation / interactive session asks for."""

    prompt: str
    image: object  # PIL image or a [3, H, W] tensor in [-1, 1]
    control_mode: str = "cam"  # "cam": camera rays; "act": rays + action vector
    fps: int = 16
    chunk_size: int = 3
    frame_num: int = 81
    frame_policy: str = "truncate"
    sample_shift: float = 10.0
    seed: int = 42
    max_attention_size: int | None = None
    max_sequence_length: int = 512
    # camera calibration: (fx, fy, cx, cy) or one row per frame (the first row is used), measured on an image of
    # intrinsics_width x intrinsics_height pixels; None: a pinhole with focal length = image width
    intrinsics: object | None = None
    intrinsics_width: int | None = None
    intrinsics_height: int | None = None
    # key-driven control of the interactive service
    control_move_step: float = 0.05
    control_lateral_step: float = 0.05
    control_yaw_step_degrees: float = 2.0
    control_pitch_step_degrees: float = 2.0
    control_pitch_limit_degrees: float = 85.0
    control_translation_scale: float = 3.0  # multiplier of the normalised frame-to-frame translation given to the DiT
    show_control_hud: bool = True
    benchmark_metrics: bool = False

    def validate(self, pipeline_control_type: str | None = None) -> "LingBotWorldFastSessionConfig":
        """Checks the record and rewrites `frame_num` to the number of frames that will be generated."""
        if pipeline_control_type is not None and self.control_mode != pipeline_control_type:
            raise ValueError(f"the session asks for control mode {self.control_mode!r} but the loaded model takes "
                             f"{pipeline_control_type!r}")  # fmt: skip
        pair = (self.intrinsics_width, self.intrinsics_height)
        if (pair[0] is None) != (pair[1] is None):
            raise ValueError("intrinsics_width and intrinsics_height name one calibration image: give both or neither")
        if pair[0] is not None:
            if self.intrinsics is None:
                raise ValueError("a calibration size without intrinsics has nothing to apply to")
            for name, v in zip(("intrinsics_width", "intrinsics_height"), pair):
                if not _is_count(v) or v < 1:
                    raise ValueError(f"{name} must be a positive integer, got {v!r}")
        self.frame_num, _ = resolve_lingbot_frame_count(self.frame_num, self.chunk_size, self.frame_policy)
        return self


class LingBotWorldFastSessionStatus(str, Enum):
    """Life cycle of a session's caches: usable, unusable after a failed chunk, or returned."""

    READY = "ready"
    POISONED = "poisoned"
    RELEASED = "released"


__all__ = ["resolve_lingbot_frame_count", "LingBotWorldFastSessionConfig", "LingBotWorldFastSessionStatus", "FRAME_POLICIES"]
