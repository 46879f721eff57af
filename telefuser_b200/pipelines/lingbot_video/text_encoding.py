"""Prompt encoding of the LingBot-Video pipelines with a Qwen3-VL language model.

The caption is placed in a fixed "enhance this prompt" chat template; an optional conditioning frame (TI2V) is put
in front of it as one vision segment. The stage returns the encoder's hidden states of the user part only: the
tokens of the template's system preamble are counted once (by tokenising the preamble alone) and cut off, and for
a single prompt the right padding is cut as well. `hidden_state_skip_layer = n` takes the n-th hidden state from
the end (0 = last layer's output before the final norm of `output_hidden_states`), `None` takes `last_hidden_state`.

The stage is a callable: `stage(caption)` -> (embeddings [B, L, C], mask [B, L]), which is what
`LingBotVideoPipeline.init(text_stage=...)` expects.
Role parity: telefuser/pipelines/lingbot_video/text_encoding.py:38-140.
"""

from __future__ import annotations

import math
from typing import Any

import torch

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig

SYSTEM_PREAMBLE = (
    "<|im_start|>system\nGiven a user input that may include a text prompt alone, a text prompt with an image reference, or a text "
    'prompt with a video reference or a video reference alone, generate an "Enhanced prompt" that provides detailed visual '
    "descriptions suitable for video generation. Evaluate the level of detail in the user's input: if it is simple, enrich it by "
    "adding specifics about colors, shapes, sizes, textures, lighting, motion dynamics, camera movement, temporal progression, and "
    "spatial relationships to create vivid, concrete, and temporally coherent scenes to create vivid and concrete scenes. Please "
    "generate only the enhanced description for the prompt below and avoid including any additional commentary or evaluations:"
    "<|im_end|>\n<|im_start|>user\n"
)
TEMPLATE_TAIL = "<|im_end|>\n<|im_start|>assistant\n"
VISION_SEGMENT = "<|vision_start|><|image_pad|><|vision_end|>"
MERGE = 2  # spatial merge of the vision tower: one language token per 2 x 2 patches
MIN_VISION_TOKENS, MAX_VISION_TOKENS = 4, 16384


def fit_to_patch_grid(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Nearest size whose sides are multiples of `factor` and whose area lies in [min_pixels, max_pixels],
    keeping the aspect ratio (the resize rule of the Qwen-VL image processors)."""
    if min(height, width) <= 0:
        raise ValueError("image sides must be positive")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        shrink = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / shrink / factor) * factor)
        w = max(factor, math.floor(width / shrink / factor) * factor)
    elif h * w < min_pixels:
        grow = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * grow / factor) * factor
        w = math.ceil(width * grow / factor) * factor
    return h, w


class LingBotVideoTextEncodingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, *, text_encoder=None,
                 processor=None, token_length: int = 37698, hidden_state_skip_layer: int | None = 0) -> None:  # fmt: skip
        super().__init__(name, model_runtime_config)
        self.text_encoder = text_encoder if text_encoder is not None else module_manager.fetch_module("text_encoder")
        self.processor = processor if processor is not None else module_manager.fetch_module("processor")
        if self.text_encoder is None or self.processor is None:
            raise ValueError("the LingBot-Video text stage needs a `text_encoder` and a `processor`")
        self.token_length = token_length
        self.hidden_state_skip_layer = hidden_state_skip_layer
        self.model_names = ["text_encoder"]
        self._preamble_tokens: int | None = None

    # ---- template bookkeeping -------------------------------------------------------
    def preamble_length(self) -> int:
        """Number of tokens the system preamble takes; they carry no information about the caption."""
        if self._preamble_tokens is None:
            ids = self.processor(text=SYSTEM_PREAMBLE, images=None, videos=None, return_tensors="pt")["input_ids"]
            self._preamble_tokens = int(ids.shape[1])
        return self._preamble_tokens

    def vision_patch_size(self) -> int:
        holders = (getattr(getattr(self.text_encoder, "config", None), "vision_config", None),
                   getattr(getattr(self.processor, "image_processor", None), "config", None),
                   getattr(self.processor, "image_processor", None))  # fmt: skip
        for h in holders:
            if getattr(h, "patch_size", None) is not None:
                return int(h.patch_size)
        return 16

    def prepare_ti2v_vlm_image(self, pixel_values: torch.Tensor):
        """First frame of a [1, 3, F, H, W] clip in [0, 1] -> PIL image sized to the vision tower's patch grid."""
        from PIL import Image

        if pixel_values.ndim != 5 or pixel_values.shape[:2] != (1, 3) or pixel_values.shape[2] < 1:
            raise ValueError(f"expected conditioning pixels of shape [1, 3, F, H, W], got {tuple(pixel_values.shape)}")
        frame = (pixel_values[0, :, 0].detach().float().cpu().clamp(0, 1) * 255).byte().permute(1, 2, 0).numpy()
        image = Image.fromarray(frame, mode="RGB")
        cell = self.vision_patch_size() * MERGE
        h, w = fit_to_patch_grid(image.height, image.width, cell, MIN_VISION_TOKENS * cell * cell,
                                 MAX_VISION_TOKENS * cell * cell)  # fmt: skip
        return image.resize((w, h))

    # ---- encoding -----------------------------------------------------------------------
    @with_model_offload(["text_encoder"])
    @torch.no_grad()
    def encode(self, prompt, *, images=None, video_metadata=None):
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        lead = VISION_SEGMENT if images is not None else ""
        texts = [SYSTEM_PREAMBLE + lead + p + TEMPLATE_TAIL for p in prompts]
        inputs = self.processor(text=texts, images=images, videos=None, video_metadata=video_metadata, do_resize=False,
                                truncation=True, max_length=self.token_length, padding="longest", return_tensors="pt")  # fmt: skip
        inputs = inputs.to(self.device)
        skip = self.hidden_state_skip_layer
        out = self.text_encoder(**inputs, output_hidden_states=skip is not None)
        hidden = out.last_hidden_state if skip is None else out.hidden_states[-(skip + 1)]
        mask = inputs["attention_mask"]
        cut = self.preamble_length()
        hidden, mask = hidden[:, cut:], mask[:, cut:]
        if hidden.shape[0] == 1:  # one prompt: nothing to pad against
            n = int(mask[0].sum())
            hidden, mask = hidden[:, :n], mask[:, :n]
        return hidden, mask

    def process(self, prompt, **kwargs):
        return self.encode(prompt, **kwargs)

    __call__ = process
