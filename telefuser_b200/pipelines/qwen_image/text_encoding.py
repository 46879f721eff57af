"""Qwen-Image prompt encoding: chat template, Qwen2.5-VL hidden states, template tokens dropped, ragged batch padded.

The prompt is wrapped in a fixed system / user template; the encoder's last hidden state is taken, each sample is
cut to its valid tokens, the first `drop` tokens (the template's system part: 34 for generation, 64 for editing)
are removed, and the samples are right-padded to a common length with a 0 / 1 mask. Edit prompts carry the input
images through the vision tower ("Picture i: <vision tokens>" per image in the multi-image form).
The stage is callable as `stage(prompt)` / `stage(prompt, images)` -> (embeddings [B, L, C], mask [B, L]).
Role parity: telefuser/pipelines/qwen_image/text_encoding.py:22-223.
"""

from __future__ import annotations

import torch

GENERATE_TEMPLATE = ("<|im_start|>system\nDescribe the image by detailing the color, shape, size, texture, quantity, text, spatial "
                     "relationships of the objects and background:<|im_end|>\n<|im_start|>user\n{}<|im_end|>\n<|im_start|>assistant\n")  # fmt: skip
EDIT_SYSTEM_PROMPT = ("Describe the key features of the input image (color, shape, size, texture, objects, background), then explain how the "
                      "user's text instruction should alter or modify the image. Generate a new image that meets the user's requirements "
                      "while maintaining consistency with the original.")  # fmt: skip
EDIT_TEMPLATE = ("<|im_start|>system\n" + EDIT_SYSTEM_PROMPT + "<|im_end|>\n<|im_start|>user\n<|vision_start|><|image_pad|><|vision_end|>{}"
                 "<|im_end|>\n<|im_start|>assistant\n")  # fmt: skip
EDIT_PLUS_TEMPLATE = "<|im_start|>system\n" + EDIT_SYSTEM_PROMPT + "<|im_end|>\n<|im_start|>user\n{}<|im_end|>\n<|im_start|>assistant\n"
PICTURE_TEMPLATE = "Picture {}: <|vision_start|><|image_pad|><|vision_end|>"
GENERATE_DROP, EDIT_DROP = 34, 64


def pack_valid_tokens(hidden: torch.Tensor, mask: torch.Tensor, drop: int, max_len: int | None = None):
    """[B, T, C] with a 0 / 1 mask -> the valid tokens of each sample minus its first `drop`, right-padded: ([B, L, C], [B, L])."""
    rows = [h[m.bool()][drop:] for h, m in zip(hidden, mask)]
    L = max(r.shape[0] for r in rows)
    emb = torch.stack([torch.cat([r, r.new_zeros(L - r.shape[0], r.shape[1])]) for r in rows])
    msk = torch.stack([torch.cat([torch.ones(r.shape[0], dtype=torch.long, device=r.device),
                                  torch.zeros(L - r.shape[0], dtype=torch.long, device=r.device)]) for r in rows])  # fmt: skip
    return (emb, msk) if max_len is None else (emb[:, :max_len], msk[:, :max_len])


class QwenImageTextEncodingStage:
    def __init__(self, text_encoder, tokenizer, processor=None, device="cuda", torch_dtype=torch.bfloat16, max_length: int = 1024) -> None:
        self.text_encoder, self.tokenizer, self.processor = text_encoder, tokenizer, processor
        self.device, self.torch_dtype, self.tokenizer_max_length = torch.device(device), torch_dtype, max_length

    @staticmethod
    def _repeat(emb, mask, n: int):
        return (emb, mask) if n == 1 else (emb.repeat_interleave(n, dim=0), mask.repeat_interleave(n, dim=0))

    @torch.no_grad()
    def encode_prompt(self, prompt, num_images_per_prompt: int = 1, max_sequence_length: int = 1024):
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        tok = self.tokenizer([GENERATE_TEMPLATE.format(p) for p in prompts], max_length=self.tokenizer_max_length + GENERATE_DROP,
                             padding=True, truncation=True, return_tensors="pt")  # fmt: skip
        ids, mask = tok["input_ids"].to(self.device), tok["attention_mask"].to(self.device)
        hidden = self.text_encoder(input_ids=ids, attention_mask=mask, output_hidden_states=True)[-1]
        emb, m = pack_valid_tokens(hidden, mask, GENERATE_DROP, max_sequence_length)
        return self._repeat(emb.to(self.device, self.torch_dtype), m, num_images_per_prompt)

    @torch.no_grad()
    def encode_prompt_with_image(self, prompt, image: list, num_images_per_prompt: int = 1, is_edit_plus: bool = True):
        if self.processor is None:
            raise RuntimeError("editing prompts need the Qwen2-VL processor")
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        if is_edit_plus:
            pictures = "".join(PICTURE_TEMPLATE.format(i + 1) for i in range(len(image)))
            texts = [EDIT_PLUS_TEMPLATE.format(pictures + p) for p in prompts]
        else:
            texts = [EDIT_TEMPLATE.format(p) for p in prompts]
        inputs = self.processor(text=texts, images=image, padding=True, return_tensors="pt").to(self.device)
        hidden = self.text_encoder(input_ids=inputs.input_ids, attention_mask=inputs.attention_mask, pixel_values=inputs.pixel_values,
                                   image_grid_thw=inputs.image_grid_thw, output_hidden_states=True)[-1]  # fmt: skip
        emb, m = pack_valid_tokens(hidden, inputs.attention_mask, EDIT_DROP)
        return self._repeat(emb.to(self.device, self.torch_dtype), m, num_images_per_prompt)

    def process(self, prompt, negative_prompt=None, num_images_per_prompt: int = 1, edit_image=None, is_edit_plus: bool = False):
        """-> (embeddings, mask, negative embeddings or None, negative mask or None)."""
        if edit_image is None:
            enc = lambda p: self.encode_prompt(p, num_images_per_prompt)  # noqa: E731
        else:
            enc = lambda p: self.encode_prompt_with_image(p, edit_image, num_images_per_prompt, is_edit_plus)  # noqa: E731
        pos = enc(prompt)
        neg = enc(negative_prompt) if negative_prompt is not None else (None, None)
        return (*pos, *neg)

    def __call__(self, prompt, images=None):
        return self.encode_prompt(prompt) if images is None else self.encode_prompt_with_image(prompt, list(images))
