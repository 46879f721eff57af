"""Qwen-Image VAE (single-frame form of a causal video VAE) and the transformers-backed prompt encoders."""

import pytest
import torch
import torch.nn.functional as F

from telefuser_b200.models import qwen_image_vae as Q
from telefuser_b200.models.hf_text_encoders import QwenImageTextEncoder, ZImageTextEncoder


def _vae():
    torch.manual_seed(0)
    vae = Q.QwenImageVAE(base_dim=16, z_dim=16, dim_mult=(1, 2, 2, 2), num_res_blocks=1, attn_scales=[0.25])
    for p in vae.parameters():
        torch.nn.init.normal_(p, std=0.1)
    return vae.float().eval()


def test_qwen_image_vae_shapes_and_single_frame_equivalence():
    vae = _vae()
    x = torch.randn(2, 3, 32, 48)
    z = vae.encode(x)
    assert z.shape == (2, 16, 4, 6) and vae.decode(z).shape == x.shape
    # the 2-D form equals the 5-D causal conv on one frame padded with two zero frames in front
    conv = vae.encoder.conv_in
    ref = F.conv3d(F.pad(x.unsqueeze(2), (1, 1, 1, 1, 2, 0)), conv.weight, conv.bias).squeeze(2)
    assert torch.allclose(conv(x), ref, atol=1e-5)
    # weights keep the video checkpoint's layout, temporal resamplers included
    keys = set(vae.state_dict())
    assert vae.encoder.conv_in.weight.shape == (16, 3, 3, 3, 3) and any("time_conv" in k for k in keys)
    assert vae.decoder.up_blocks[0].resnets[0].norm1.gamma.shape == (32, 1, 1, 1) and vae.decoder.mid_block.attentions[0].norm.gamma.shape == (32, 1, 1)
    # latent statistics: decode(encode-normalised) inverts the normalisation
    mean, inv_std = vae._stats(z)
    assert torch.allclose((z / inv_std + mean - mean) * inv_std, z, atol=1e-5)
    norm = Q.QwenImageRMS_norm(8, images=False)
    y = norm(torch.randn(1, 8, 4, 4))
    assert torch.allclose(y.pow(2).sum(dim=1), torch.full((1, 4, 4), 8.0), atol=1e-4)


@pytest.mark.gpu
def test_qwen_image_vae_gpu_bf16():
    vae = _vae()
    x = torch.randn(1, 3, 64, 64)
    ref = vae.decode(vae.encode(x))
    g = _vae().to("cuda", torch.bfloat16)
    out = g.decode(g.encode(x.to("cuda", torch.bfloat16))).float().cpu()
    assert (out - ref).abs().max() < 0.05 * max(1.0, float(ref.abs().max()))


def test_prompt_encoders_tiny():
    z = ZImageTextEncoder(dict(hidden_size=32, intermediate_size=64, num_attention_heads=2, num_key_value_heads=1, head_dim=16,
                               num_hidden_layers=2, vocab_size=100, max_window_layers=2)).eval()  # fmt: skip
    hs = z(torch.randint(0, 100, (1, 6)), torch.ones(1, 6, dtype=torch.long))
    assert len(hs) == 3 and hs[-1].shape == (1, 6, 32)
    q = QwenImageTextEncoder(dict(hidden_size=32, intermediate_size=64, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=2,
                                  vocab_size=2000, max_window_layers=2, rope_scaling={"mrope_section": [2, 3, 3], "rope_type": "default", "type": "default"}),
                             dict(depth=1, hidden_size=16, intermediate_size=32, num_heads=2, out_hidden_size=32, fullatt_block_indexes=[0])).eval()  # fmt: skip
    hs = q(torch.randint(0, 1000, (1, 6)), torch.ones(1, 6, dtype=torch.long))
    assert len(hs) == 3 and hs[-1].shape == (1, 6, 32) and len(q.get_tp_plan()) == 14
    sd, _ = q.state_dict_converter().from_official({"visual.a": 1, "model.layers.0.w": 2, "lm_head.weight": 3})
    assert sorted(sd) == ["lm_head.weight", "model.language_model.layers.0.w", "model.visual.a"]
    assert set(sd) <= {k.split(".weight")[0] + ".weight" if k.endswith(".weight") else k for k in sd}
