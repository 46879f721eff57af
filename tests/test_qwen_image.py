"""Qwen-Image MM-DiT and pipeline: rope layout, checkpoint key names, batch / edit / mask handling,
norm-preserving guidance, end-to-end latents on CPU; bf16 forward on GPUs against fp32."""

import pytest
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.qwen_image_dit import QwenEmbedRope, QwenImageDiT, timestep_embedding
from telefuser_b200.pipelines.qwen_image import QwenImagePipeline, QwenImagePipelineConfig, norm_preserving_cfg


def small(dtype=torch.float32, device="cpu", head_dim=32, axes=(8, 12, 12), heads=2, layers=2):
    torch.manual_seed(0)
    m = QwenImageDiT(num_layers=layers, dim=heads * head_dim, num_heads=heads, head_dim=head_dim, text_dim=48, axes_dim=axes)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    m = m.to(dtype).to(device).eval()
    m.dtype = dtype
    return m


def test_rope_positions_are_centred_and_text_follows_the_image():
    rope = QwenEmbedRope(10000.0, (8, 12, 12))
    (ic, isn), (tc, ts) = rope([(1, 4, 6)], 5, "cpu")
    assert ic.shape == (24, 16) and tc.shape == (5, 16)
    assert torch.allclose(ic**2 + isn**2, torch.ones_like(ic), atol=1e-6)
    # token (h=2, w=3) sits at the centre: height index 0, width index 0 -> zero angle on those axes
    centre = 2 * 6 + 3
    assert torch.allclose(isn[centre, 4:], torch.zeros(12), atol=1e-7)
    # text positions start at max(h//2, w//2) = 3 on every axis
    assert torch.allclose(ts[0, 0], torch.sin(torch.tensor(3.0)), atol=1e-6)
    emb = timestep_embedding(torch.tensor([0.5]))
    assert emb.shape == (1, 256) and torch.allclose(emb[0, 0], torch.cos(torch.tensor(500.0)), atol=1e-4)


def test_key_names_follow_the_public_checkpoint_and_forward_variants_agree():
    m = small()
    keys = set(m.state_dict())
    for k in ("time_text_embed.timestep_embedder.linear_1.weight", "txt_norm.weight", "img_in.weight",
              "transformer_blocks.0.img_mod.1.weight", "transformer_blocks.0.attn.add_q_proj.bias",
              "transformer_blocks.0.attn.norm_added_k.weight", "transformer_blocks.0.attn.to_out.0.weight",
              "transformer_blocks.1.txt_mlp.net.0.proj.weight", "transformer_blocks.1.img_mlp.net.2.bias",
              "norm_out.linear.weight", "proj_out.bias"):  # fmt: skip
        assert k in keys, k
    with torch.device("meta"):
        full = QwenImageDiT(num_layers=1)
    assert full.state_dict()["transformer_blocks.0.img_mod.1.weight"].shape == (18432, 3072)
    lat, t = torch.randn(2, 16, 8, 12), torch.tensor([300.0, 300.0])
    emb = torch.randn(2, 7, 48)
    mask = torch.ones(2, 7, dtype=torch.long)
    mask[:, 5:] = 0
    both = m(lat, t, emb, mask)
    one = m(lat[1:], t[1:], emb[1:, :5])
    assert both.shape == lat.shape and (both[1:] - one).abs().max() <= 1e-5  # batch == per sample, mask == cut text
    edit = m(lat[:1], t[:1], emb[:1], mask[:1], edit_latents=[torch.randn(1, 16, 4, 4)])
    assert edit.shape == (1, 16, 8, 12) and not torch.allclose(edit, both[:1])


def test_guidance_keeps_the_conditional_norm_and_pipeline_runs():
    c, u = torch.randn(1, 4, 8, 8), torch.randn(1, 4, 8, 8)
    g = norm_preserving_cfg(c, u, 4.0)
    assert torch.allclose(g.norm(dim=-1), c.norm(dim=-1), atol=1e-5)
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(small(), "qwen_image_dit")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = QwenImagePipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, QwenImagePipelineConfig(dit_config=rc(), text_encoding_config=rc(), vae_config=rc()))
    pos, neg = torch.randn(1, 6, 48), torch.randn(1, 3, 48)
    a = pipe(prompt_emb=pos, negative_prompt_emb=neg, cfg_scale=3.0, num_inference_steps=3, seed=1, height=64, width=96)
    b = pipe(prompt_emb=pos, negative_prompt_emb=neg, cfg_scale=3.0, num_inference_steps=3, seed=1, height=64, width=96)
    assert a.shape == (1, 16, 8, 12) and torch.isfinite(a).all() and torch.equal(a, b)
    e = pipe(prompt_emb=pos, cfg_scale=1.0, num_inference_steps=2, seed=1, height=64, width=96,
             edit_image_latents=torch.randn(1, 16, 8, 8))  # fmt: skip
    assert e.shape == a.shape


@pytest.mark.gpu
def test_gpu_bf16_forward_tracks_cpu_fp32():
    ref_m = small(head_dim=128, axes=(16, 56, 56))
    lat, t, emb = torch.randn(1, 16, 32, 48), torch.tensor([700.0]), torch.randn(1, 11, 48)
    ref = ref_m(lat, t, emb)
    gpu_m = small(torch.bfloat16, "cuda", head_dim=128, axes=(16, 56, 56))
    got = gpu_m(lat.cuda().bfloat16(), t.cuda(), emb.cuda().bfloat16()).float().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err
