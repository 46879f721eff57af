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
    with torch.no_grad():
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


def test_qwen_image_text_stage_packing():
    from types import SimpleNamespace

    from telefuser_b200.pipelines.qwen_image.text_encoding import (GENERATE_DROP, GENERATE_TEMPLATE, QwenImageTextEncodingStage,
                                                                    pack_valid_tokens)

    hidden = torch.arange(2 * 6 * 2, dtype=torch.float32).view(2, 6, 2)
    mask = torch.tensor([[1, 1, 1, 1, 1, 0], [1, 1, 1, 0, 0, 0]])
    emb, m = pack_valid_tokens(hidden, mask, drop=2)
    assert emb.shape == (2, 3, 2) and m.tolist() == [[1, 1, 1], [1, 0, 0]] and torch.equal(emb[0], hidden[0, 2:5]) and bool((emb[1, 1:] == 0).all())
    assert pack_valid_tokens(hidden, mask, 2, max_len=2)[0].shape == (2, 2, 2)

    class Tok:
        def __call__(self, texts, max_length=None, padding=True, truncation=True, return_tensors="pt"):
            rows = [[ord(c) % 50 + 1 for c in t] for t in texts]
            n = max(len(r) for r in rows)
            ids = torch.tensor([r + [0] * (n - len(r)) for r in rows])
            return {"input_ids": ids, "attention_mask": (ids > 0).long()}

    encoder = lambda input_ids, attention_mask, output_hidden_states=True, **kw: (None, input_ids[..., None].float().repeat(1, 1, 4))  # noqa: E731
    stage = QwenImageTextEncodingStage(encoder, Tok(), device="cpu", torch_dtype=torch.float32)
    emb, m = stage(["a cat", "a much longer prompt"])
    base = len(GENERATE_TEMPLATE.format("")) - GENERATE_DROP
    assert emb.shape == (2, base + 20, 4) and m.sum(dim=1).tolist() == [base + 5, base + 20]
    pos, pm, neg, nm = stage.process("x", "y", num_images_per_prompt=2)
    assert pos.shape[0] == 2 and neg.shape == pos.shape and torch.equal(pm, nm)
    proc = lambda text, images, padding=True, return_tensors="pt": SimpleNamespace(  # noqa: E731
        to=lambda dev: SimpleNamespace(input_ids=torch.ones(1, 70, dtype=torch.long), attention_mask=torch.ones(1, 70, dtype=torch.long),
                                       pixel_values=torch.zeros(4, 8), image_grid_thw=torch.tensor([[1, 2, 2]])), text=text)  # fmt: skip
    stage.processor = proc
    e2, m2 = stage("make it blue", images=[torch.zeros(3, 8, 8)])
    assert e2.shape == (1, 6, 4) and int(m2.sum()) == 6  # 70 valid tokens minus the 64 template tokens
