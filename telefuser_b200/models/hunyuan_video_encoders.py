"""HunyuanVideo-1.5 conditioning encoders: chat-templated LLM prompt encoder, glyph (ByT5) encoder for quoted text,
SigLIP image encoder.

All three wrap transformers models (as the reference does); this module holds the logic around them: the system
prompt templates and the removal of their tokens from the hidden states (`crop_start` is found by locating the
user-turn marker), taking a hidden state a few layers before the last, extraction and style-tagging of quoted
strings for the glyph branch, and zero states when a prompt has no quoted text. Models and tokenizers can be
injected, so the logic is testable without checkpoints.
Role parity: telefuser/models/hunyuan_video_text_encoder.py:20-461, hunyuan_video_byt5.py:21-433,
hunyuan_video_image_encoder.py:20-222.
"""

from __future__ import annotations

import copy
import json
import os
import re
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch
from torch import nn

_IMAGE_SYSTEM = ("You are a helpful assistant. Describe the image by detailing the following aspects: "
                 "1. The main content and theme of the image. "
                 "2. The color, shape, size, texture, quantity, text, and spatial relationships of the objects. "
                 "3. The background environment, light, style and atmosphere.")  # fmt: skip
_VIDEO_SYSTEM = ("You are a helpful assistant. Describe the video by detailing the following aspects: "
                 "1. The main content and theme of the video. "
                 "2. The color, shape, size, texture, quantity, text, and spatial relationships of the objects. "
                 "3. Actions, events, behaviors temporal relationships, physical movement changes of the objects. "
                 "4. background environment, light, style and atmosphere. "
                 "5. camera angles, movements, and transitions used in the video.")  # fmt: skip
PROMPT_TEMPLATE = {
    "li-dit-encode-image-json": {"template": [{"role": "system", "content": _IMAGE_SYSTEM}, {"role": "user", "content": "{}"}], "crop_start": -1},
    "li-dit-encode-video-json": {"template": [{"role": "system", "content": _VIDEO_SYSTEM}, {"role": "user", "content": "{}"}], "crop_start": -1},
}
PRECISION_TO_TYPE = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
USER_TURN_MARKER = "<|im_start|>user\n"


@dataclass
class TextEncoderModelOutput:
    hidden_state: torch.Tensor | None = None
    attention_mask: torch.Tensor | None = None
    hidden_states_list: tuple | None = None


class HunyuanVideoTextEncoder(nn.Module):
    def __init__(self, text_encoder_type: str = "llm", max_length: int = 1000, text_encoder_precision: str | None = None,
                 text_encoder_path: str | None = None, tokenizer_type: str | None = None, tokenizer_path: str | None = None,
                 output_key: str | None = None, use_attention_mask: bool = True, prompt_template: dict | None = None,
                 prompt_template_video: dict | None = None, hidden_state_skip_layer: int | None = None, apply_final_norm: bool = False,
                 reproduce: bool = False, device=None, model: nn.Module | None = None, tokenizer: Any = None) -> None:  # fmt: skip
        super().__init__()
        if text_encoder_type != "llm":
            raise ValueError(f"unsupported text encoder type {text_encoder_type}")
        self.text_encoder_type, self.max_length, self.precision, self.model_path = text_encoder_type, max_length, text_encoder_precision, text_encoder_path
        self.tokenizer_type, self.tokenizer_path = tokenizer_type or text_encoder_type, tokenizer_path or text_encoder_path
        self.use_attention_mask, self.hidden_state_skip_layer, self.apply_final_norm, self.reproduce = use_attention_mask, hidden_state_skip_layer, apply_final_norm, reproduce
        self.prompt_template, self.prompt_template_video = copy.deepcopy(prompt_template), copy.deepcopy(prompt_template_video)
        for t in (self.prompt_template, self.prompt_template_video):
            if t is not None and (not isinstance(t, dict) or "{}" not in str(t.get("template"))):
                raise ValueError("a prompt template is a dict whose 'template' has a {} placeholder")
        self.use_template, self.use_video_template = self.prompt_template is not None, self.prompt_template_video is not None
        self.output_key = output_key or "last_hidden_state"
        if model is None:
            from transformers import AutoModel, AutoTokenizer

            model = AutoModel.from_pretrained(self.model_path)
            model = getattr(model, "language_model", model)
            tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_path, padding_side="right")
        if not hasattr(model, "final_layer_norm") and hasattr(model, "norm"):
            model.final_layer_norm = model.norm
        if self.precision is not None:
            model = model.to(PRECISION_TO_TYPE[self.precision])
        self.model, self.tokenizer = model.requires_grad_(False).eval(), tokenizer
        if device is not None:
            self.model = self.model.to(device)
        for kind, t in (("image", self.prompt_template), ("video", self.prompt_template_video)):
            if t is not None:
                self.text2tokens("a photo of a cat", data_type=kind)  # fixes crop_start once

    @property
    def dtype(self) -> torch.dtype:
        return next(self.model.parameters()).dtype

    @property
    def device(self) -> torch.device:
        return next(self.model.parameters()).device

    @staticmethod
    def apply_text_to_template(text, template, prevent_empty_text: bool = True):
        if isinstance(template, str):
            return template.format(text)
        if isinstance(template, list):
            out = copy.deepcopy(template)
            for item in out:
                if isinstance(item, dict) and "content" in item:
                    item["content"] = item["content"].format(text if text else (" " if prevent_empty_text else ""))
            return out
        raise TypeError(f"unsupported template type {type(template)}")

    def calculate_crop_start(self, tokenized) -> int:
        """Index of the first token after the user-turn marker (0 when the marker is absent)."""
        ids = tokenized["input_ids"][0].tolist()
        marker = self.tokenizer(USER_TURN_MARKER, add_special_tokens=False)["input_ids"]
        for i in range(len(ids) - len(marker) + 1):
            if ids[i : i + len(marker)] == marker:
                return i + len(marker)
        return 0

    def _tokenize(self, text, as_chat: bool, max_length: int):
        kw = dict(truncation=True, max_length=max_length, padding="max_length", return_tensors="pt")
        if as_chat:
            return self.tokenizer.apply_chat_template(text, add_generation_prompt=True, tokenize=True, return_dict=True, **kw)
        return self.tokenizer(text, return_length=False, return_overflowing_tokens=False, return_attention_mask=True, **kw)

    def text2tokens(self, text, data_type: str = "image", max_length: int | None = None):
        max_length = max_length or self.max_length
        crop_start, as_chat = 0, False
        if self.use_template or self.use_video_template:
            if data_type not in ("image", "video"):
                raise ValueError(f"unsupported data type {data_type}")
            holder = self.prompt_template if data_type == "image" else self.prompt_template_video
            template, crop_start = holder["template"], holder.get("crop_start", -1)
            if isinstance(text, (list, tuple)):
                text = [self.apply_text_to_template(t, template) for t in text]
                as_chat = isinstance(text[0], list)
            elif isinstance(text, str):
                text = self.apply_text_to_template(text, template)
                as_chat = isinstance(text, list)
            else:
                raise TypeError(f"unsupported text type {type(text)}")
            if crop_start == -1:
                crop_start = holder["crop_start"] = self.calculate_crop_start(self._tokenize(text, as_chat, 256))
        return self._tokenize(text, as_chat, max_length + max(crop_start, 0))

    @torch.no_grad()
    def encode(self, batch_encoding, use_attention_mask=None, output_hidden_states: bool = False, do_sample=None,
               hidden_state_skip_layer=None, return_texts: bool = False, data_type: str = "image", device=None, is_uncond: bool = False):  # fmt: skip
        device = device if device is not None else self.device
        use_mask = self.use_attention_mask if use_attention_mask is None else use_attention_mask
        skip = self.hidden_state_skip_layer if hidden_state_skip_layer is None else hidden_state_skip_layer
        mask = batch_encoding["attention_mask"].to(device) if use_mask else None
        out = self.model(input_ids=batch_encoding["input_ids"].to(device), attention_mask=mask,
                         output_hidden_states=output_hidden_states or skip is not None)  # fmt: skip
        if skip is not None:
            last = out.hidden_states[-(skip + 1)]
            if skip > 0 and self.apply_final_norm:
                last = self.model.final_layer_norm(last)
        else:
            last = out[self.output_key]
        if self.use_template:
            holder = self.prompt_template if data_type == "image" else self.prompt_template_video
            crop = holder.get("crop_start", 0)
            if crop > 0:
                last, mask = last[:, crop:], (mask[:, crop:] if use_mask else None)
        return TextEncoderModelOutput(last, mask, out.hidden_states if output_hidden_states else None)

    def forward(self, text, use_attention_mask=None, output_hidden_states: bool = False, do_sample: bool = False, hidden_state_skip_layer=None,
                return_texts: bool = False, data_type: str = "image"):  # fmt: skip
        return self.encode(self.text2tokens(text, data_type=data_type, max_length=self.max_length), use_attention_mask, output_hidden_states,
                           do_sample, hidden_state_skip_layer, return_texts, data_type=data_type)  # fmt: skip

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16, **kwargs) -> "HunyuanVideoTextEncoder":
        return cls("llm", 1000, "bf16" if torch_dtype == torch.bfloat16 else "fp16", path, "llm",
                   prompt_template=PROMPT_TEMPLATE["li-dit-encode-image-json"], prompt_template_video=PROMPT_TEMPLATE["li-dit-encode-video-json"],
                   hidden_state_skip_layer=2, apply_final_norm=False, reproduce=False)  # fmt: skip


# ---- glyph encoder ---------------------------------------------------------------------------------
def extract_glyph_texts(prompt: str) -> list:
    """Strings inside straight or curly double quotes, in order; duplicates are dropped when there are several."""
    found = [a or b for a, b in re.findall(r"\"(.*?)\"|“(.*?)”", prompt)]
    return list(dict.fromkeys(found)) if len(found) > 1 else found


@dataclass
class ByT5Config:
    byt5_name: str = "google/byt5-small"
    max_length: int = 256
    hidden_dim: int = 1472
    color_ann_path: str | None = None
    font_ann_path: str | None = None
    checkpoint_path: str | None = None


def _load_json(path: str | None) -> dict:
    if path and os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


class MultilingualPromptFormat:
    """Prefixes each glyph string with its `<color-i>` and `<ll-font-j>` tokens when the index files know them."""

    def __init__(self, font_path: str | None = None, color_path: str | None = None) -> None:
        self.idx_font_dict, self.idx_color_dict = _load_json(font_path), _load_json(color_path)

    def format_prompt(self, glyph_texts: list, text_styles: list) -> str:
        parts = []
        for text, style in zip(glyph_texts, text_styles):
            color = f"<color-{style['color']}>" if style.get("color") is not None and self.idx_color_dict else ""
            family, font = style.get("font-family"), ""
            if family is not None and family in self.idx_font_dict:
                font = f"<{family[:2] if len(family) >= 2 else 'en'}-font-{self.idx_font_dict[family]}>"
            parts.append(f"{color}{font}{text}")
        return " ".join(parts)


class HunyuanVideoByT5Encoder(nn.Module):
    def __init__(self, config: ByT5Config, torch_dtype: torch.dtype = torch.bfloat16, device=None, model: nn.Module | None = None,
                 tokenizer: Any = None) -> None:  # fmt: skip
        super().__init__()
        self.config, self.max_length, self.torch_dtype = config, config.max_length, torch_dtype
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        if model is None:
            from transformers import AutoTokenizer, T5ForConditionalGeneration

            tokenizer = AutoTokenizer.from_pretrained(config.byt5_name)
            model = T5ForConditionalGeneration.from_pretrained(config.byt5_name, torch_dtype=torch_dtype).get_encoder()
        self.model, self.tokenizer = model, tokenizer
        self._add_special_tokens(config)
        if config.checkpoint_path and os.path.exists(config.checkpoint_path):
            self._load_checkpoint(config.checkpoint_path)
        self.model = self.model.requires_grad_(False).eval().to(self.device)
        self.prompt_format = MultilingualPromptFormat(config.font_ann_path, config.color_ann_path)

    def _add_special_tokens(self, config: ByT5Config) -> None:
        colors, fonts = _load_json(config.color_ann_path), _load_json(config.font_ann_path)
        tokens = [f"<color-{i}>" for i in range(len(colors))] + [f"<{code[:2]}-font-{fonts[code]}>" for code in fonts]
        if tokens:
            self.tokenizer.add_tokens(tokens, special_tokens=True)
            self.model.resize_token_embeddings(len(self.tokenizer), mean_resizing=False)

    def _load_checkpoint(self, path: str) -> None:
        sd = torch.load(path, map_location="cpu", weights_only=True)
        if "state_dict" in sd:
            prefix = "module.text_tower.encoder."
            sd = {k[len(prefix):]: v for k, v in sd["state_dict"].items() if k.startswith(prefix)}
        self.model.load_state_dict(sd)

    @property
    def dtype(self) -> torch.dtype:
        return next(self.model.parameters()).dtype

    def tokenize(self, text: str, max_length: int | None = None):
        enc = self.tokenizer(text, padding="max_length", max_length=max_length or self.max_length, truncation=True, add_special_tokens=True,
                             return_tensors="pt")  # fmt: skip
        return enc["input_ids"], enc["attention_mask"]

    @torch.no_grad()
    def encode(self, input_ids, attention_mask):
        return self.model(input_ids.to(self.device), attention_mask=attention_mask.float().to(self.device)).last_hidden_state

    def process_prompt(self, prompt: str, device=None):
        """-> (states [1, max_length, hidden], mask [1, max_length]); zeros when the prompt quotes nothing."""
        device = device or self.device
        glyphs = extract_glyph_texts(prompt)
        if not glyphs:
            return (torch.zeros((1, self.max_length, self.config.hidden_dim), device=device),
                    torch.zeros((1, self.max_length), device=device, dtype=torch.int64))  # fmt: skip
        text = self.prompt_format.format_prompt(glyphs, [{"color": None, "font-family": None} for _ in glyphs])
        ids, mask = (t.to(device) for t in self.tokenize(text))
        return self.encode(ids, mask), mask

    def forward(self, prompt, device=None) -> dict:
        pairs = [self.process_prompt(p, device) for p in ([prompt] if isinstance(prompt, str) else prompt)]
        return {"byt5_text_states": torch.cat([p[0].to(self.dtype) for p in pairs]), "byt5_text_mask": torch.cat([p[1] for p in pairs])}

    @classmethod
    def from_pretrained(cls, root: str, torch_dtype: torch.dtype = torch.bfloat16, max_length: int = 256, device=None, **kwargs):
        enc = os.path.join(root, "text_encoder")
        glyph = os.path.join(enc, "Glyph-SDXL-v2")
        cfg = ByT5Config(os.path.join(enc, "byt5-small"), max_length, 1472, os.path.join(glyph, "assets", "color_idx.json"),
                         os.path.join(glyph, "assets", "multilingual_10-lang_idx.json"), os.path.join(glyph, "checkpoints", "byt5_model.pt"))  # fmt: skip
        if not os.path.exists(cfg.byt5_name):
            cfg.byt5_name = "google/byt5-small"
        return cls(cfg, torch_dtype=torch_dtype, device=device)


def load_glyph_byT5_v2(args: dict, device) -> dict:  # noqa: N802
    n = args.get("byt5_max_length", 256)
    enc = HunyuanVideoByT5Encoder(ByT5Config(args.get("byT5_google_path", "google/byt5-small"), n, 1472, args.get("multilingual_prompt_format_color_path"),
                                             args.get("multilingual_prompt_format_font_path"), args.get("byT5_ckpt_path")), torch.bfloat16, device)  # fmt: skip
    return {"byt5_tokenizer": enc.tokenizer, "byt5_model": enc.model, "byt5_max_length": n}


# ---- image encoder ---------------------------------------------------------------------------------
@dataclass
class VisionEncoderOutput:
    last_hidden_state: torch.Tensor | None = None
    pooler_output: torch.Tensor | None = None
    hidden_states: tuple | None = None


class HunyuanVideoImageEncoder(nn.Module):
    """SigLIP vision tower + its image processor; uint8 arrays are preprocessed, dicts of tensors pass through."""

    def __init__(self, model: nn.Module, processor: Any, dtype: torch.dtype = torch.float16, device=None) -> None:
        super().__init__()
        self.model = model.to(dtype=dtype).requires_grad_(False)
        self.processor, self.dtype = processor, dtype
        if device is not None:
            self.model = self.model.to(device)

    @classmethod
    def from_pretrained(cls, root: str, torch_dtype: torch.dtype = torch.float16, device=None) -> "HunyuanVideoImageEncoder":
        from transformers import SiglipImageProcessor, SiglipVisionModel

        return cls(SiglipVisionModel.from_pretrained(root, subfolder="image_encoder"),
                   SiglipImageProcessor.from_pretrained(root, subfolder="feature_extractor"), torch_dtype,
                   torch.device(device) if isinstance(device, str) else device)  # fmt: skip

    @property
    def device(self) -> torch.device:
        return next(self.model.parameters()).device

    @property
    def hidden_size(self) -> int:
        return self.model.config.hidden_size

    def preprocess_images(self, images: np.ndarray) -> dict:
        return self.processor.preprocess(images=images, return_tensors="pt")

    @torch.no_grad()
    def encode_images(self, images) -> VisionEncoderOutput:
        if isinstance(images, np.ndarray):
            images = {k: v.to(device=self.device, dtype=self.dtype) for k, v in self.preprocess_images(images).items()}
        out = self.model(**images)
        return VisionEncoderOutput(out.last_hidden_state, getattr(out, "pooler_output", None), getattr(out, "hidden_states", None))

    forward = encode_images


def resize_and_center_crop(image: np.ndarray, target_width: int, target_height: int) -> np.ndarray:
    """Lanczos resize so that the target is covered, then crop the centre."""
    from PIL import Image

    if (target_height, target_width) == image.shape[:2]:
        return image
    pil = Image.fromarray(image)
    w, h = pil.size
    s = max(target_width / w, target_height / h)
    rw, rh = int(round(w * s)), int(round(h * s))
    pil = pil.resize((rw, rh), Image.LANCZOS)
    return np.array(pil.crop(((rw - target_width) / 2, (rh - target_height) / 2, (rw + target_width) / 2, (rh + target_height) / 2)))
