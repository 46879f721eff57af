"""Language-model prompt encoders that are transformers models behind this package's model interface.

`QwenImageTextEncoder` (Qwen2.5-VL 7B, returns every hidden state; takes pixel inputs for the edit pipelines) and
`ZImageTextEncoder` (Qwen3 4B). The reference wraps the same library classes; the diffusion transformers they
feed run on this package's kernels. Constructors accept size overrides so tests can build small instances.
Role parity: telefuser/models/qwen_image_text_encoder.py:11-196, telefuser/models/z_image_text_encoder.py:9-81.
"""

from __future__ import annotations

from torch import nn

from telefuser_b200.core.base_model import BaseModel

_QWEN25_VL_TEXT = dict(
    attention_dropout=0.0, bos_token_id=151643, eos_token_id=151645, hidden_act="silu", hidden_size=3584, initializer_range=0.02,
    intermediate_size=18944, max_position_embeddings=128000, max_window_layers=28, num_attention_heads=28, num_hidden_layers=28,
    num_key_value_heads=4, rms_norm_eps=1e-06, rope_scaling={"mrope_section": [16, 24, 24], "rope_type": "default", "type": "default"},
    rope_theta=1000000.0, use_cache=True, use_sliding_window=False, vocab_size=152064)  # fmt: skip
_QWEN25_VL_VISION = dict(
    depth=32, fullatt_block_indexes=[7, 15, 23, 31], hidden_act="silu", hidden_size=1280, in_channels=3, in_chans=3, initializer_range=0.02,
    intermediate_size=3420, model_type="qwen2_5_vl", num_heads=16, out_hidden_size=3584, patch_size=14, spatial_merge_size=2,
    spatial_patch_size=14, temporal_patch_size=2, tokens_per_second=2, window_size=112)  # fmt: skip
_QWEN3_4B = dict(
    attention_bias=False, attention_dropout=0.0, bos_token_id=151643, eos_token_id=151645, head_dim=128, hidden_act="silu", hidden_size=2560,
    initializer_range=0.02, intermediate_size=9728, max_position_embeddings=40960, max_window_layers=36, model_type="qwen3",
    num_attention_heads=32, num_hidden_layers=36, num_key_value_heads=8, rms_norm_eps=1e-06, rope_scaling=None, rope_theta=1000000,
    sliding_window=None, tie_word_embeddings=True, use_cache=True, use_sliding_window=False, vocab_size=151936)  # fmt: skip


class QwenImageTextEncoder(BaseModel):
    def __init__(self, text_overrides: dict | None = None, vision_overrides: dict | None = None) -> None:
        super().__init__()
        from transformers import Qwen2_5_VLConfig, Qwen2_5_VLModel

        text = {**_QWEN25_VL_TEXT, **(text_overrides or {})}
        vision = {**_QWEN25_VL_VISION, **(vision_overrides or {})}
        text_cfg = {**text, "model_type": "qwen2_5_vl_text", "layer_types": ["full_attention"] * text["num_hidden_layers"], "sliding_window": None,
                    "image_token_id": None, "video_token_id": None, "vision_end_token_id": 151653, "vision_start_token_id": 151652,
                    "vision_token_id": 151654}  # fmt: skip
        config = Qwen2_5_VLConfig(**{**text, "architectures": ["Qwen2_5_VLForConditionalGeneration"], "model_type": "qwen2_5_vl",
                                     "image_token_id": 151655, "video_token_id": 151656, "vision_end_token_id": 151653,
                                     "vision_start_token_id": 151652, "vision_token_id": 151654, "sliding_window": 32768,
                                     "tie_word_embeddings": False, "text_config": text_cfg, "vision_config": vision})  # fmt: skip
        self.model = Qwen2_5_VLModel(config)
        self.lm_head = nn.Linear(config.text_config.hidden_size, config.text_config.vocab_size, bias=False)
        self.config = config

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, inputs_embeds=None, pixel_values=None, pixel_values_videos=None,
                image_grid_thw=None, video_grid_thw=None, **kwargs):  # fmt: skip
        """-> tuple of hidden states (embedding output and every layer)."""
        kwargs.pop("output_hidden_states", None)
        kwargs.pop("output_attentions", None)
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids, inputs_embeds=inputs_embeds,
                         pixel_values=pixel_values, pixel_values_videos=pixel_values_videos, image_grid_thw=image_grid_thw,
                         video_grid_thw=video_grid_thw, output_attentions=False, output_hidden_states=True, return_dict=True, **kwargs)  # fmt: skip
        return out.hidden_states

    def get_tp_plan(self) -> dict:
        """Column / row roles of the language-model linears, keyed by module path."""
        plan = {}
        for i in range(len(self.model.language_model.layers)):
            base = f"model.language_model.layers.{i}."
            plan.update({base + "self_attn.q_proj": "colwise", base + "self_attn.k_proj": "colwise", base + "self_attn.v_proj": "colwise",
                         base + "self_attn.o_proj": "rowwise", base + "mlp.gate_proj": "colwise", base + "mlp.up_proj": "colwise",
                         base + "mlp.down_proj": "rowwise"})  # fmt: skip
        return plan

    @staticmethod
    def state_dict_converter():
        return QwenImageTextEncoderStateDictConverter()


class QwenImageTextEncoderStateDictConverter:
    """Official layout: `visual.*` and `model.*` (language model) at the root, plus `lm_head`."""

    def from_official(self, sd: dict):
        out = {}
        for k, v in sd.items():
            if k.startswith("visual."):
                k = "model." + k
            elif k.startswith("model.") and not k.startswith(("model.language_model.", "model.visual.")):
                k = "model.language_model." + k[len("model."):]
            out[k] = v
        return out, {}

    from_diffusers = from_official


class ZImageTextEncoder(BaseModel):
    def __init__(self, overrides: dict | None = None) -> None:
        super().__init__()
        from transformers import Qwen3Config, Qwen3Model

        self.config = Qwen3Config(**{**_QWEN3_4B, **(overrides or {})})
        self.model = Qwen3Model(self.config)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, output_hidden_states: bool = True, **kwargs):
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                         output_hidden_states=output_hidden_states, **kwargs)  # fmt: skip
        return out.hidden_states

    @staticmethod
    def state_dict_converter():
        return ZImageTextEncoderStateDictConverter()


class ZImageTextEncoderStateDictConverter:
    def from_diffusers(self, sd: dict):
        return dict(sd), {}

    from_official = from_diffusers
