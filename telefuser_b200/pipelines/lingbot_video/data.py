"""Request-side contracts of LingBot-Video: captions, default negative captions, frame counts, checkpoint
architecture records and the TI2V condition frame.

LingBot-Video is conditioned on STRUCTURED captions: the positive prompt is the JSON a prompt rewriter produces, and the
classifier-free-guidance branch uses a JSON "universal negative" that differs between still images and videos. The text
encoder sees these as strings, so the serialisation (key order, separators) is part of the contract.
Role parity: telefuser/pipelines/lingbot_video/data.py:16-206.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

import torch

# ---- default negative captions ------------------------------------------------------------------------------------
_QUALITY = ["low quality", "worst quality", "blurry", "pixelated", "jpeg artifacts", "low resolution"]
_EXPOSURE = ["underexposed", "overexposed", "invisible subject", "subject hidden in darkness"]
_STYLE = ["painting", "illustration", "drawing", "cartoon", "3d render", "cgi", "sketch", "digital art"]
_FRAMING = ["pillarboxed", "side bars", "portrait image in landscape frame"]
_MOTION = ["flickering", "jittery", "motion blur", "temporal inconsistency", "warping", "morphing", "incoherent motion",
           "unnatural movement", "static object with sudden jump", "frame-to-frame inconsistency"]  # fmt: skip


def _negative(video: bool) -> str:
    """The universal negative caption as the text encoder must see it (`json.dumps` default separators)."""
    groups = {
        "visual_quality": _QUALITY + (["unstable color", "color flicker"] if video else []) + _EXPOSURE,
        "artistic_style": _STYLE,
        "composition_and_content": ["text", "watermark", "signature", "logo"] + (["subtitles"] if video else []) + _FRAMING,
    }
    if video:
        groups["temporal_and_motion_stability"] = _MOTION
    groups["material_and_structure"] = (["plastic-like glass", "unrealistic texture", "deformed bottle"]
                                        + (["liquid freezing improperly"] if video else []) + ["distorted reflections"])  # fmt: skip
    return json.dumps({"universal_negative": groups})


DEFAULT_NEGATIVE_PROMPT = _negative(video=True)
DEFAULT_NEGATIVE_PROMPT_IMAGE = _negative(video=False)


def default_negative_caption(num_frames: int) -> str:
    """Guidance-branch caption for a request of `num_frames` frames: the still-image form for 1, the video form otherwise."""
    return DEFAULT_NEGATIVE_PROMPT_IMAGE if num_frames == 1 else DEFAULT_NEGATIVE_PROMPT


# ---- captions and durations -----------------------------------------------------------------------------------------
RUNTIME_PROMPT_FIELDS = frozenset({"duration", "fps", "height", "width", "num_frames", "resolution", "ratio"})


def validate_frame_count(num_frames: int) -> int:
    """1 (a still image) or 4n + 1 (the VAE packs four frames per latent frame after the first)."""
    if num_frames < 1 or (num_frames - 1) % 4:
        raise ValueError(f"num_frames must be 1 or 4n+1, got {num_frames}")
    return num_frames


def num_frames_from_duration(duration: float, fps: int = 24) -> int:
    """Smallest 4n + 1 frame count that covers `duration` seconds at `fps` (0 s -> 1 frame)."""
    if duration < 0 or fps <= 0:
        raise ValueError(f"a duration is non-negative and a frame rate positive, got {duration} s at {fps} fps")
    frames = int(float(duration) * fps)
    return ((frames - 1) // 4 + 1) * 4 + 1


def parse_lingbot_video_prompt(payload) -> tuple[str, float | None]:
    """(caption text, duration or None) from a prompt-rewriter sample: a dict, or a list whose first entry is one.
    The caption is `payload["caption"]` when present, else the sample without its run-time fields (duration, fps,
    size ...); structured captions are serialised compactly, exactly as the rewriter's own tooling does."""
    if isinstance(payload, list):
        if not payload:
            raise ValueError("an empty list holds no prompt sample")
        payload = payload[0]
    if not isinstance(payload, dict):
        raise ValueError(f"a prompt sample is a dict (or a list of them), got {type(payload).__name__}")
    caption = payload["caption"] if "caption" in payload else {k: v for k, v in payload.items() if k not in RUNTIME_PROMPT_FIELDS}
    text = json.dumps(caption, ensure_ascii=False, separators=(",", ":")) if isinstance(caption, (dict, list)) else str(caption)
    if not text:
        raise ValueError("the prompt sample has an empty caption")
    duration = payload.get("duration")
    return text, (None if duration is None else float(duration))


def load_lingbot_video_prompt(path) -> tuple[str, float | None]:
    return parse_lingbot_video_prompt(json.loads(Path(path).read_text(encoding="utf-8")))


# ---- checkpoint architecture ----------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LingBotVideoModelConfig:
    """The architecture values a dense / MoE / refiner checkpoint's `config.json` fixes."""

    variant: str = "dense"
    num_layers: int = 24
    hidden_size: int = 2048
    num_heads: int = 16
    in_channels: int = 16
    patch_size: tuple = (1, 2, 2)
    text_dim: int = 2560
    intermediate_size: int = 6144
    num_experts: int = 0
    top_k: int = 0

    def __post_init__(self) -> None:
        if self.variant not in ("dense", "moe", "refiner"):
            raise ValueError(f"LingBot-Video has dense, moe and refiner checkpoints, not {self.variant!r}")
        if min(self.num_layers, self.hidden_size, self.num_heads) <= 0:
            raise ValueError("layer count, width and head count must be positive")
        if self.variant != "dense" and (self.num_experts <= 0 or self.top_k <= 0):
            raise ValueError(f"a {self.variant} checkpoint needs num_experts and top_k")


def load_lingbot_video_model_config(path, variant: str = "dense") -> LingBotVideoModelConfig:
    """Reads a transformer `config.json` (or the folder that holds it)."""
    p = Path(path)
    raw = json.loads((p / "config.json" if p.is_dir() else p).read_text(encoding="utf-8"))
    names = {"depth": "num_layers", "hidden_size": "hidden_size", "num_attention_heads": "num_heads", "in_channels": "in_channels",
             "text_dim": "text_dim", "intermediate_size": "intermediate_size"}  # fmt: skip
    missing = [k for k in (*names, "patch_size") if k not in raw]
    if missing:
        raise ValueError(f"the transformer config lacks {missing}")
    experts = int(raw.get("num_experts", 0))
    return LingBotVideoModelConfig(variant=variant, patch_size=tuple(int(v) for v in raw["patch_size"]), num_experts=experts,
                                   top_k=int(raw.get("num_experts_per_tok", 0)) if experts else 0,
                                   **{ours: int(raw[theirs]) for theirs, ours in names.items()})  # fmt: skip


# ---- image geometry -------------------------------------------------------------------------------------------------
def smart_resize(height: int, width: int, factor: int, min_pixels: int = 4 * 28**2, max_pixels: int = 16384 * 28**2) -> tuple[int, int]:
    """Size the vision tower resamples an image to: both sides multiples of `factor`, area within [min, max] pixels,
    aspect ratio kept as well as the grid allows."""
    if min_pixels > max_pixels:
        raise ValueError("min_pixels exceeds max_pixels")
    if min(height, width) <= 0 or max(height, width) / min(height, width) > 200:
        raise ValueError(f"an image of {height} x {width} is empty or thinner than 1:200")
    h, w = max(factor, round(height / factor) * factor), max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        shrink = math.sqrt(height * width / max_pixels)
        h, w = math.floor(height / shrink / factor) * factor, math.floor(width / shrink / factor) * factor
    elif h * w < min_pixels:
        grow = math.sqrt(min_pixels / (height * width))
        h, w = math.ceil(height * grow / factor) * factor, math.ceil(width * grow / factor) * factor
    return h, w


def preprocess_ti2v_image(image: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """RGB image [B, 3, H, W] with values 0..255 -> condition frame [B, 3, 1, height, width] in [0, 1]: scaled so that it
    covers the target, centre-cropped. The interpolation runs on uint8 values (results are truncated back to uint8), which
    is what the checkpoints were trained against."""
    if image.ndim != 4 or image.shape[1] != 3:
        raise ValueError(f"the condition image is [B, 3, H, W], got {tuple(image.shape)}")
    h0, w0 = image.shape[-2:]
    scale = max(height / h0, width / w0)
    rh, rw = max(math.ceil(h0 * scale), height), max(math.ceil(w0 * scale), width)
    resized = torch.nn.functional.interpolate(image.to(torch.uint8), size=(rh, rw), mode="bilinear", align_corners=False)
    top, left = int(round((rh - height) / 2.0)), int(round((rw - width) / 2.0))
    return resized[:, :, top : top + height, left : left + width].float().div(255.0).unsqueeze(2)


__all__ = ["DEFAULT_NEGATIVE_PROMPT", "DEFAULT_NEGATIVE_PROMPT_IMAGE", "default_negative_caption", "RUNTIME_PROMPT_FIELDS",
           "validate_frame_count", "num_frames_from_duration", "parse_lingbot_video_prompt", "load_lingbot_video_prompt",
           "LingBotVideoModelConfig", "load_lingbot_video_model_config", "smart_resize", "preprocess_ti2v_image"]  # fmt: skip
