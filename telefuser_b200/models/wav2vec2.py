"""Wav2Vec2 speech encoder whose convolutional features are resampled to one vector per video frame.

A thin subclass of the `transformers` Wav2Vec2 model (library code: the convolutional feature extractor and
the transformer encoder are used as they are): between the two, the feature sequence is linearly interpolated
to `seq_len` (the number of video frames of the audio segment), so that every hidden state lines up with a
frame. `feature_extract` / `encode` expose the two halves for callers that cache the features.
Role parity: telefuser/models/wav2vec2.py:14-154.
"""

from __future__ import annotations

import torch.nn.functional as F
from transformers import Wav2Vec2FeatureExtractor
from transformers import Wav2Vec2Model as _HFWav2Vec2Model
from transformers.modeling_outputs import BaseModelOutput

__all__ = ["Wav2Vec2Model", "linear_interpolation"]


def linear_interpolation(features, seq_len: int):
    """[B, T, C] -> [B, seq_len, C] (align_corners)."""
    return F.interpolate(features.transpose(1, 2), size=seq_len, align_corners=True, mode="linear").transpose(1, 2)


class Wav2Vec2Model(_HFWav2Vec2Model):
    audio_processor: Wav2Vec2FeatureExtractor | None = None

    @classmethod
    def from_pretrained(cls, path, *args, **kwargs):
        model = super().from_pretrained(path, *args, **kwargs)
        model.audio_processor = Wav2Vec2FeatureExtractor.from_pretrained(path, *args, **kwargs)
        return model

    def feature_extract(self, input_values, seq_len: int):
        return linear_interpolation(self.feature_extractor(input_values).transpose(1, 2), seq_len)

    def encode(self, extract_features, attention_mask=None, mask_time_indices=None, output_attentions=None,
               output_hidden_states=None, return_dict=None):  # fmt: skip
        output_hidden_states = self.config.output_hidden_states if output_hidden_states is None else output_hidden_states
        return_dict = getattr(self.config, "return_dict", True) if return_dict is None else return_dict
        if attention_mask is not None:
            attention_mask = self._get_feature_vector_attention_mask(extract_features.shape[1], attention_mask, add_adapter=False)
        hidden, _ = self.feature_projection(extract_features)
        hidden = self._mask_hidden_states(hidden, mask_time_indices=mask_time_indices, attention_mask=attention_mask)
        enc = self.encoder(hidden, attention_mask=attention_mask, output_attentions=output_attentions,
                           output_hidden_states=output_hidden_states, return_dict=return_dict)  # fmt: skip
        hidden = enc[0]
        if self.adapter is not None:
            hidden = self.adapter(hidden)
        if not return_dict:
            return (hidden,) + enc[1:]
        return BaseModelOutput(last_hidden_state=hidden, hidden_states=enc.hidden_states, attentions=enc.attentions)

    def forward(self, input_values, seq_len: int, attention_mask=None, mask_time_indices=None, output_attentions=None,
                output_hidden_states=None, return_dict=None):  # fmt: skip
        return self.encode(self.feature_extract(input_values, seq_len), attention_mask, mask_time_indices, output_attentions,
                           output_hidden_states, return_dict)  # fmt: skip
