"""LTX-2 prompt path: Gemma-3 hidden states -> per-modality prompt embeddings.

Every hidden state of the language model (embedding output + each layer) is normalised and concatenated on the
feature axis, projected to the transformer widths by the feature extractor (V1: one shared projection after a
per-sample min / max normalisation; V2: per-token RMS normalisation and one projection per modality), then refined
by a small 1-D transformer (`Embeddings1DConnector`) in which padding positions are replaced by learned register
tokens so the diffusion model always sees a dense, fixed-length context.
The language model itself is the transformers implementation of Gemma-3 (a library model, as in the reference);
the connector runs on this package's attention / GEMM kernels.
Role parity: telefuser/models/ltx_gemma_text_encoder.py:108-1000.
"""

from __future__ import annotations

import math
from typing import NamedTuple

import torch
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.ltx_dit import (
    LTX23_DEV_TRANSFORMER_CONFIG,
    Attention,
    FeedForward,
    LTXRopeType,
    precompute_freqs_cis,
)
from telefuser_b200.ops import functional as TF

GEMMA3_TEXT_HIDDEN_SIZE, GEMMA3_TEXT_LAYERS = 3840, 48

GEMMA3_CONFIG_FOR_LTX = {
    "architectures": ["Gemma3ForConditionalGeneration"], "boi_token_index": 255999, "eoi_token_index": 256000, "eos_token_id": [1, 106],
    "image_token_index": 262144, "initializer_range": 0.02, "mm_tokens_per_image": 256, "model_type": "gemma3", "torch_dtype": "bfloat16",
    "text_config": {
        "attention_bias": False, "attention_dropout": 0.0, "attn_logit_softcapping": None, "final_logit_softcapping": None, "head_dim": 256,
        "hidden_activation": "gelu_pytorch_tanh", "hidden_size": GEMMA3_TEXT_HIDDEN_SIZE, "initializer_range": 0.02,
        "intermediate_size": 15360, "max_position_embeddings": 131072, "model_type": "gemma3_text", "num_attention_heads": 16,
        "num_hidden_layers": GEMMA3_TEXT_LAYERS, "num_key_value_heads": 8, "query_pre_attn_scalar": 256, "rms_norm_eps": 1e-06,
        "rope_local_base_freq": 10000, "rope_scaling": {"factor": 8.0, "rope_type": "linear"}, "rope_theta": 1000000,
        "sliding_window": 1024, "sliding_window_pattern": 6, "use_cache": True, "vocab_size": 262208},
    "vision_config": {
        "attention_dropout": 0.0, "hidden_act": "gelu_pytorch_tanh", "hidden_size": 1152, "image_size": 896, "intermediate_size": 4304,
        "layer_norm_eps": 1e-06, "model_type": "siglip_vision_model", "num_attention_heads": 16, "num_channels": 3,
        "num_hidden_layers": 27, "patch_size": 14, "vision_use_head": False},
}  # fmt: skip


class LTXVGemmaTokenizer:
    """Left-padded fixed-length tokenisation; `tokenize_with_weights` returns (token id, attention flag) pairs."""

    def __init__(self, tokenizer_path: str, max_length: int = 256) -> None:
        from transformers import AutoTokenizer

        self.tokenizer = AutoTokenizer.from_pretrained(tokenizer_path, local_files_only=True, model_max_length=max_length)
        self.tokenizer.padding_side = "left"
        if self.tokenizer.pad_token is None:
            self.tokenizer.pad_token = self.tokenizer.eos_token
        self.max_length = max_length

    def tokenize_with_weights(self, text: str, return_word_ids: bool = False) -> dict:
        enc = self.tokenizer(text.strip(), padding="max_length", max_length=self.max_length, truncation=True, return_tensors="pt")
        triples = [(t, a, i) for i, (t, a) in enumerate(zip(enc.input_ids[0], enc.attention_mask[0]))]
        return {"gemma": triples if return_word_ids else [(t, a) for t, a, _ in triples]}


def _norm_and_concat_padded_batch(encoded: torch.Tensor, sequence_lengths: torch.Tensor, padding_side: str = "right") -> torch.Tensor:
    """[B, T, D, L] -> [B, T, D * L]: per sample and layer, centre on the mean of the valid tokens and scale to a range of 8."""
    b, t, d, l = encoded.shape  # noqa: E741
    idx = torch.arange(t, device=encoded.device)[None]
    if padding_side == "right":
        valid = idx < sequence_lengths[:, None]
    elif padding_side == "left":
        valid = idx >= t - sequence_lengths[:, None]
    else:
        raise ValueError(f"padding_side must be 'left' or 'right', got {padding_side}")
    valid = valid[:, :, None, None]
    eps = 1e-6
    mean = encoded.masked_fill(~valid, 0.0).sum(dim=(1, 2), keepdim=True) / ((sequence_lengths * d).view(b, 1, 1, 1) + eps)
    lo = encoded.masked_fill(~valid, float("inf")).amin(dim=(1, 2), keepdim=True)
    hi = encoded.masked_fill(~valid, float("-inf")).amax(dim=(1, 2), keepdim=True)
    out = (8 * (encoded - mean) / (hi - lo + eps)).masked_fill(~valid, 0.0)
    return out.reshape(b, t, d * l)


def norm_and_concat_per_token_rms(encoded: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
    """[B, T, D, L] -> [B, T, D * L]: RMS-normalise every token in every layer; padding tokens become zero."""
    b, t, d, l = encoded.shape  # noqa: E741
    normed = encoded * torch.rsqrt(encoded.pow(2).mean(dim=2, keepdim=True) + 1e-6)
    return normed.reshape(b, t, d * l) * attention_mask.bool().unsqueeze(-1).to(normed.dtype)


def _stack_layers(hidden_states) -> torch.Tensor:
    return torch.stack(list(hidden_states), dim=-1) if isinstance(hidden_states, (list, tuple)) else hidden_states


class FeatureExtractorV1(nn.Module):
    def __init__(self, aggregate_embed: nn.Module, is_av: bool = False) -> None:
        super().__init__()
        self.aggregate_embed, self.is_av = aggregate_embed, is_av

    def forward(self, hidden_states, attention_mask, padding_side: str = "left"):
        enc = _stack_layers(hidden_states)
        normed = _norm_and_concat_padded_batch(enc, attention_mask.sum(dim=-1), padding_side).to(enc.dtype)
        feats = TF.linear(normed, self.aggregate_embed.weight, self.aggregate_embed.bias)
        return feats, (feats if self.is_av else None)


class FeatureExtractorV2(nn.Module):
    def __init__(self, video_aggregate_embed: nn.Linear, embedding_dim: int, audio_aggregate_embed: nn.Linear | None = None) -> None:
        super().__init__()
        self.video_aggregate_embed, self.audio_aggregate_embed, self.embedding_dim = video_aggregate_embed, audio_aggregate_embed, embedding_dim

    def forward(self, hidden_states, attention_mask, padding_side: str = "left"):
        enc = _stack_layers(hidden_states)
        normed = norm_and_concat_per_token_rms(enc, attention_mask).to(enc.dtype)
        out = []
        for proj in (self.video_aggregate_embed, self.audio_aggregate_embed):
            if proj is None:
                out.append(None)
                continue
            scaled = normed * math.sqrt(proj.out_features / self.embedding_dim)
            out.append(TF.linear(scaled, proj.weight, proj.bias))
        return out[0], out[1]


class _BasicTransformerBlock1D(nn.Module):
    def __init__(self, dim: int, heads: int, dim_head: int, rope_type: LTXRopeType = LTXRopeType.INTERLEAVED,
                 apply_gated_attention: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.attn1 = Attention(dim, heads=heads, dim_head=dim_head, rope_type=rope_type, apply_gated_attention=apply_gated_attention)
        self.ff = FeedForward(dim, dim)

    def forward(self, x, attention_mask=None, pe=None):
        x = x + self.attn1(TF.rmsnorm_modulate(x, None, None, None, 1e-6), mask=attention_mask, pe=pe)
        return self.ff(TF.rmsnorm_modulate(x, None, None, None, 1e-6), residual=x)


class Embeddings1DConnector(nn.Module):
    def __init__(self, attention_head_dim: int = 128, num_attention_heads: int = 30, num_layers: int = 2,
                 positional_embedding_theta: float = 10000.0, positional_embedding_max_pos=None, causal_temporal_positioning: bool = False,
                 num_learnable_registers: int | None = 128, rope_type: LTXRopeType = LTXRopeType.INTERLEAVED,
                 double_precision_rope: bool = False, apply_gated_attention: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.num_attention_heads, self.inner_dim = num_attention_heads, num_attention_heads * attention_head_dim
        self.causal_temporal_positioning, self.positional_embedding_theta = causal_temporal_positioning, positional_embedding_theta
        self.positional_embedding_max_pos = positional_embedding_max_pos or [1]
        self.rope_type, self.double_precision_rope = rope_type, double_precision_rope
        self.transformer_1d_blocks = nn.ModuleList(
            [_BasicTransformerBlock1D(self.inner_dim, num_attention_heads, attention_head_dim, rope_type, apply_gated_attention) for _ in range(num_layers)])  # fmt: skip
        self.num_learnable_registers = num_learnable_registers
        if num_learnable_registers:
            self.learnable_registers = nn.Parameter(torch.rand(num_learnable_registers, self.inner_dim, dtype=torch.bfloat16) * 2.0 - 1.0)

    def _replace_padded_with_learnable_registers(self, x, attention_mask):
        """Valid tokens move to the front (order kept); every other position takes the register of its index."""
        T = x.shape[1]
        if T % self.num_learnable_registers:
            raise ValueError(f"sequence length {T} must be a multiple of the {self.num_learnable_registers} registers")
        registers = self.learnable_registers.repeat(T // self.num_learnable_registers, 1).to(x.dtype)
        valid = attention_mask.reshape(x.shape[0], T) >= -9000.0
        order = torch.argsort((~valid).to(torch.int8), dim=1, stable=True)
        moved = x.gather(1, order[..., None].expand_as(x))
        keep = torch.arange(T, device=x.device)[None] < valid.sum(dim=1, keepdim=True)
        return torch.where(keep[..., None], moved, registers[None]), torch.zeros_like(attention_mask)

    def forward(self, hidden_states, attention_mask=None):
        dense = False
        if self.num_learnable_registers:
            hidden_states, attention_mask = self._replace_padded_with_learnable_registers(hidden_states, attention_mask)
            dense = True  # the additive mask is now all zeros
        grid = torch.arange(hidden_states.shape[1], dtype=torch.float32, device=hidden_states.device)[None, None]
        pe = precompute_freqs_cis(grid, self.inner_dim, torch.float32, self.positional_embedding_theta, self.positional_embedding_max_pos,
                                  False, self.num_attention_heads, self.rope_type, self.double_precision_rope)  # fmt: skip
        for blk in self.transformer_1d_blocks:
            hidden_states = blk(hidden_states, attention_mask=None if dense else attention_mask, pe=pe)
        return TF.rmsnorm_modulate(hidden_states, None, None, None, 1e-6), attention_mask


def _connector_from(tc: dict, prefix: str) -> Embeddings1DConnector:
    get = lambda key, default: tc.get(prefix + key, tc.get("connector_" + key, default))  # noqa: E731
    return Embeddings1DConnector(attention_head_dim=get("attention_head_dim", 128), num_attention_heads=get("num_attention_heads", 30),
                                 num_layers=get("num_layers", 2), positional_embedding_max_pos=tc.get("connector_positional_embedding_max_pos", [1]),
                                 rope_type=LTXRopeType(tc.get("rope_type", "interleaved")),
                                 double_precision_rope=tc.get("frequencies_precision", False) == "float64",
                                 apply_gated_attention=tc.get("connector_apply_gated_attention", False))  # fmt: skip


class Embeddings1DConnectorConfigurator:
    @classmethod
    def from_config(cls, config: dict) -> Embeddings1DConnector:
        return _connector_from(config.get("transformer", {}), "connector_")


class AudioEmbeddings1DConnectorConfigurator:
    @classmethod
    def from_config(cls, config: dict) -> Embeddings1DConnector:
        return _connector_from(config.get("transformer", {}), "audio_connector_")


class EmbeddingsProcessorOutput(NamedTuple):
    video_encoding: torch.Tensor
    audio_encoding: torch.Tensor | None
    attention_mask: torch.Tensor


def convert_to_additive_mask(attention_mask: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """{0, 1} [B, T] -> [B, 1, 1, T] with 0 for valid and -max for padding."""
    m = (attention_mask.to(torch.int64) - 1).to(dtype)
    return m.reshape(attention_mask.shape[0], 1, -1, attention_mask.shape[-1]) * torch.finfo(dtype).max


class EmbeddingsProcessor(nn.Module):
    def __init__(self, *, feature_extractor: nn.Module | None = None, video_connector: Embeddings1DConnector,
                 audio_connector: Embeddings1DConnector | None = None) -> None:  # fmt: skip
        super().__init__()
        self.feature_extractor, self.video_connector, self.audio_connector = feature_extractor, video_connector, audio_connector

    def create_embeddings(self, video_features, audio_features, additive_attention_mask):
        if (self.audio_connector is None) != (audio_features is None):
            raise ValueError("audio features and the audio connector must be given together")
        video, vmask = self.video_connector(video_features, additive_attention_mask)
        binary = (vmask < 1e-6).to(torch.int64).reshape(video.shape[0], video.shape[1], 1)
        video = video * binary.to(video.dtype)
        audio = self.audio_connector(audio_features, additive_attention_mask)[0] if self.audio_connector is not None else None
        return video, audio, binary.squeeze(-1)

    def process_hidden_states(self, hidden_states, attention_mask, padding_side: str = "left") -> EmbeddingsProcessorOutput:
        if self.feature_extractor is None:
            raise ValueError("a feature extractor is needed to process hidden states")
        v, a = self.feature_extractor(hidden_states, attention_mask, padding_side)
        return EmbeddingsProcessorOutput(*self.create_embeddings(v, a, convert_to_additive_mask(attention_mask, v.dtype)))


_V2_EXPECTED_CONFIG = {"caption_proj_before_connector": True, "caption_projection_first_linear": False, "caption_proj_input_norm": False,
                       "caption_projection_second_linear": False}  # fmt: skip


def _create_feature_extractor(tc: dict, embedding_dim: int = GEMMA3_TEXT_HIDDEN_SIZE, num_layers: int = GEMMA3_TEXT_LAYERS + 1) -> nn.Module:
    """V1 when the config names none of the V2 keys; V2 needs all four at their expected values."""
    flat = embedding_dim * num_layers
    present = tc.keys() & _V2_EXPECTED_CONFIG.keys()
    if not present:
        return FeatureExtractorV1(nn.Linear(flat, embedding_dim, bias=False), is_av=True)
    wrong = sorted(k for k in _V2_EXPECTED_CONFIG if tc.get(k, None) != _V2_EXPECTED_CONFIG[k])
    if wrong:
        raise NotImplementedError("unsupported caption projection config: " + ", ".join(f"{k}={tc.get(k)!r}" for k in wrong))
    return FeatureExtractorV2(nn.Linear(flat, tc["num_attention_heads"] * tc["attention_head_dim"], bias=True), embedding_dim,
                              nn.Linear(flat, tc["audio_num_attention_heads"] * tc["audio_attention_head_dim"], bias=True))  # fmt: skip


class EmbeddingsProcessorConfigurator:
    @classmethod
    def from_config(cls, config: dict, embedding_dim: int = GEMMA3_TEXT_HIDDEN_SIZE, num_layers: int = GEMMA3_TEXT_LAYERS + 1) -> EmbeddingsProcessor:
        return EmbeddingsProcessor(feature_extractor=_create_feature_extractor(config.get("transformer", {}), embedding_dim, num_layers),
                                   video_connector=Embeddings1DConnectorConfigurator.from_config(config),
                                   audio_connector=AudioEmbeddings1DConnectorConfigurator.from_config(config))  # fmt: skip


class LTXEmbeddingsProcessor(EmbeddingsProcessor):
    def __init__(self, config: dict | None = None, embedding_dim: int = GEMMA3_TEXT_HIDDEN_SIZE, num_layers: int = GEMMA3_TEXT_LAYERS + 1) -> None:
        config = config or LTX23_DEV_TRANSFORMER_CONFIG
        super().__init__(feature_extractor=_create_feature_extractor(config["transformer"], embedding_dim, num_layers),
                         video_connector=Embeddings1DConnectorConfigurator.from_config(config),
                         audio_connector=AudioEmbeddings1DConnectorConfigurator.from_config(config))  # fmt: skip

    @staticmethod
    def state_dict_converter():
        return LTXEmbeddingsProcessorStateDictConverter()


class LTXEmbeddingsProcessorStateDictConverter:
    _PREFIXES = {
        "text_embedding_projection.aggregate_embed.": "feature_extractor.aggregate_embed.",
        "text_embedding_projection.video_aggregate_embed.": "feature_extractor.video_aggregate_embed.",
        "text_embedding_projection.audio_aggregate_embed.": "feature_extractor.audio_aggregate_embed.",
        "model.diffusion_model.video_embeddings_connector.": "video_connector.",
        "model.diffusion_model.audio_embeddings_connector.": "audio_connector.",
        "model.diffusion_model.video_embedding_connector.": "video_connector.",
        "model.diffusion_model.audio_embedding_connector.": "audio_connector.",
    }

    def from_official(self, sd: dict):
        out = {}
        for k, v in sd.items():
            for src, dst in self._PREFIXES.items():
                if k.startswith(src):
                    out[dst + k[len(src):]] = v
                    break
        return (out or dict(sd)), {}

    from_diffusers = from_official


class GemmaTextEncoder(BaseModel):
    """Wraps a transformers `Gemma3ForConditionalGeneration`; forward returns every hidden state of the language model."""

    def __init__(self, model=None, dtype: torch.dtype = torch.bfloat16, config: dict | None = None) -> None:
        super().__init__()
        if model is None:
            from transformers import Gemma3Config, Gemma3ForConditionalGeneration

            model = Gemma3ForConditionalGeneration(Gemma3Config.from_dict(dict(config or GEMMA3_CONFIG_FOR_LTX)))
        self.model, self._dtype = model, dtype

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype | None = None, device_map: str | None = None,
                        local_files_only: bool = True, **kwargs) -> "GemmaTextEncoder":  # fmt: skip
        from transformers import Gemma3ForConditionalGeneration

        model = Gemma3ForConditionalGeneration.from_pretrained(path, torch_dtype=torch_dtype, local_files_only=local_files_only, **kwargs)
        module = cls(model=model, dtype=torch_dtype or next(model.parameters()).dtype).eval().requires_grad_(False)
        return module.to(device_map) if device_map not in (None, "auto") else module

    def forward(self, input_ids, attention_mask=None, output_hidden_states: bool = True, **kwargs):
        out = self.model.model(input_ids=input_ids, attention_mask=attention_mask, output_hidden_states=output_hidden_states, **kwargs)
        return out.hidden_states

    @staticmethod
    def state_dict_converter():
        return GemmaTextEncoderStateDictConverter()


class GemmaTextEncoderStateDictConverter:
    """Accepts language-model-only, `model.`-rooted and fully wrapped key layouts; ties the output head to the embedding."""

    @staticmethod
    def _convert(sd: dict):
        out = {}
        for k, v in sd.items():
            k = k.replace("lanuage_model", "language_model").replace("language_model.model.", "language_model.")
            if k.startswith(("model.model.", "model.lm_head.")):
                out[k] = v
            elif k.startswith(("model.", "lm_head.")):
                out["model." + k] = v
            else:
                out["model.model." + k] = v
        if out and "model.lm_head.weight" not in out:
            for cand in ("model.model.language_model.embed_tokens.weight", "model.model.embed_tokens.weight"):
                if cand in out:
                    out["model.lm_head.weight"] = out[cand]
                    break
        return out, {}

    def from_official(self, sd: dict):
        return self._convert(sd)

    from_diffusers = from_official


class GemmaTextEncoderConfigurator:
    @classmethod
    def from_config(cls, config: dict | None = None) -> GemmaTextEncoder:
        from transformers import Gemma3Config, Gemma3ForConditionalGeneration

        with torch.device("meta"):
            model = Gemma3ForConditionalGeneration(Gemma3Config.from_dict(dict(GEMMA3_CONFIG_FOR_LTX)))
        return GemmaTextEncoder(model=model)


LTXTextEncoder = GemmaTextEncoder
