"""HunyuanVideo-1.5 DiT and pipeline: rope tables, key names, token stream assembly, the base and the
super-resolution denoising stages on CPU; bf16 forward on GPUs."""

import pytest
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.hunyuan_video_dit import ByT5Mapper, HunyuanVideoDiT, rope_tables
from telefuser_b200.pipelines.hunyuan_video_1_5 import HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig
from telefuser_b200.pipelines.hunyuan_video_1_5.pipeline import empty_condition, image_condition


def small(dtype=torch.float32, device="cpu", head_dim=32, axes=(8, 12, 12), in_channels=4, extra_cond=0, **kw):
    torch.manual_seed(0)
    m = HunyuanVideoDiT(patch_size=(1, 1, 1), in_channels=in_channels, hidden_size=2 * head_dim, heads_num=2,
                        mm_double_blocks_depth=2, mm_single_blocks_depth=1, rope_dim_list=axes, text_states_dim=24,
                        vision_states_dim=20, **kw)  # fmt: skip
    m.byt5_in = ByT5Mapper(16, 2 * head_dim, 2 * head_dim, 2 * head_dim, False)
    if extra_cond:  # the super-resolution model takes more condition channels
        m.img_in.proj = torch.nn.Conv3d(in_channels * 2 + 1 + extra_cond, 2 * head_dim, 1)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    m = m.to(dtype).to(device).eval()
    m.dtype = dtype
    return m


def test_rope_and_key_names():
    cos, sin = rope_tables((8, 12, 12), (2, 3, 4), 256.0, "cpu")
    assert cos.shape == (24, 16) and torch.allclose(cos**2 + sin**2, torch.ones_like(cos), atol=1e-6)
    assert torch.allclose(sin[12, 0], torch.sin(torch.tensor(1.0))) and torch.allclose(sin[1, 10], torch.sin(torch.tensor(1.0)))
    keys = set(small(guidance_embed=True, use_meanflow=True).state_dict())
    for k in ("img_in.proj.weight", "txt_in.input_embedder.weight", "txt_in.individual_token_refiner.blocks.1.self_attn_qkv.bias",
              "txt_in.c_embedder.linear_2.weight", "time_in.mlp.2.bias", "guidance_in.mlp.0.weight", "time_r_in.mlp.0.weight",
              "double_blocks.0.img_mod.linear.weight", "double_blocks.1.txt_attn_k_norm.weight", "double_blocks.0.img_mlp.fc2.bias",
              "single_blocks.0.linear2.fc.weight", "single_blocks.0.modulation.linear.bias", "final_layer.adaLN_modulation.1.weight",
              "cond_type_embedding.weight", "vision_in.proj.3.weight", "byt5_in.fc3.bias"):  # fmt: skip
        assert k in keys, k
    with torch.device("meta"):
        full = HunyuanVideoDiT(mm_double_blocks_depth=1)
    assert full.state_dict()["img_in.proj.weight"].shape == (2048, 65, 1, 1, 1)


def test_token_streams_and_batches():
    m = small()
    x, t = torch.randn(1, 9, 2, 4, 4), torch.tensor([600.0])
    txt, mask = torch.randn(1, 7, 24), torch.tensor([[1, 1, 1, 1, 0, 0, 0]])
    a = m(x, t, txt, None, mask)
    assert a.shape == (1, 4, 2, 4, 4)
    assert torch.allclose(a, m(x, t, txt[:, :4], None, None), atol=1e-5)  # masked == cut
    zero_vis = m(x, t, txt, None, mask, vision_states=torch.zeros(1, 5, 20))
    assert torch.allclose(zero_vis, a, atol=1e-6)  # text-to-video: zero vision states add no tokens
    vis = m(x, t, txt, None, mask, vision_states=torch.randn(1, 5, 20), mask_type="i2v")
    glyph = m(x, t, txt, None, mask, byt5_text_states=torch.randn(1, 6, 16), byt5_text_mask=torch.tensor([[1, 1, 0, 0, 0, 0]]))
    assert not torch.allclose(vis, a, atol=1e-4) and not torch.allclose(glyph, a, atol=1e-4)
    two = m(torch.cat([x, 2 * x]), torch.tensor([600.0, 600.0]), torch.cat([txt, txt]), None, torch.cat([mask, mask]))
    assert torch.allclose(two[:1], a, atol=1e-5)


def test_conditions_and_pipeline_with_sr():
    lat = torch.randn(1, 4, 3, 4, 4)
    cond = image_condition(torch.ones(1, 4, 1, 4, 4), lat)
    assert cond.shape == (1, 5, 3, 4, 4) and cond[:, :4, 0].min() == 1 and cond[:, :, 1:].abs().max() == 0 and cond[0, 4, 0, 0, 0] == 1
    assert empty_condition(lat).abs().max() == 0
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(small(), "hunyuan_video_dit")
    mm.add_module(small(extra_cond=5), "hunyuan_video_sr_dit")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = HunyuanVideo15Pipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, HunyuanVideo15PipelineConfig(dit_config=rc(), sr_dit_config=rc(), vae_config=rc(), text_encoding_config=rc()))
    text = dict(text_states=torch.randn(1, 6, 24), mask=torch.ones(1, 6, dtype=torch.long))
    neg = dict(text_states=torch.randn(1, 6, 24), mask=torch.ones(1, 6, dtype=torch.long))
    kw = dict(text=text, negative_text=neg, seed=0, height=64, width=64, num_frames=9, num_inference_steps=3, cfg_scale=3.0,
              latent_channels=4)  # fmt: skip
    a = pipe(**kw)
    assert a.shape == (1, 4, 3, 4, 4) and torch.isfinite(a).all() and torch.equal(a, pipe(**kw))
    i2v = pipe(image_latents=torch.randn(1, 4, 1, 4, 4), vision_states=torch.randn(1, 5, 20), **kw)
    assert not torch.allclose(i2v, a, atol=1e-3)
    sr = pipe(enable_sr=True, sr_height=128, sr_width=128, sr_num_inference_steps=4, **kw)
    assert sr.shape == (1, 4, 3, 8, 8) and torch.isfinite(sr).all()


@pytest.mark.gpu
def test_gpu_bf16_forward_tracks_cpu_fp32():
    ref_m = small(head_dim=128, axes=(16, 56, 56))
    x, t, txt = torch.randn(1, 9, 2, 16, 16), torch.tensor([700.0]), torch.randn(1, 24, 24)
    vis = torch.randn(1, 8, 20)
    ref = ref_m(x, t, txt, vision_states=vis, mask_type="i2v")
    gpu_m = small(torch.bfloat16, "cuda", head_dim=128, axes=(16, 56, 56))
    got = gpu_m(x.cuda().bfloat16(), t.cuda(), txt.cuda().bfloat16(), vision_states=vis.cuda().bfloat16(), mask_type="i2v").float().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err


def test_pipeline_with_vae_upsampler_and_text_stage():
    from types import SimpleNamespace

    from telefuser_b200.models.hunyuan_video_vae import HunyuanVideoVAE, SRTo720pUpsampler
    from telefuser_b200.pipelines.hunyuan_video_1_5 import HunyuanTextEncodingStage

    torch.manual_seed(0)
    vae = HunyuanVideoVAE(latent_channels=4, block_out_channels=(16, 32, 64, 64), layers_per_block=1, ffactor_spatial=8, ffactor_temporal=4,
                          sample_size=64).float().eval()  # fmt: skip
    up = SRTo720pUpsampler(in_channels=4, out_channels=4, hidden_channels=8, num_blocks=1, global_residual=True).float().eval()
    llm = lambda p, data_type="video": SimpleNamespace(hidden_state=torch.randn(1, 6, 24), attention_mask=torch.ones(1, 6, dtype=torch.long))  # noqa: E731
    glyph = lambda p: {"byt5_text_states": torch.zeros(1, 5, 16), "byt5_text_mask": torch.zeros(1, 5, dtype=torch.long)}  # noqa: E731
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(small(), "hunyuan_video_dit")
    mm.add_module(small(extra_cond=5), "hunyuan_video_sr_dit")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = HunyuanVideo15Pipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, HunyuanVideo15PipelineConfig(dit_config=rc(), sr_dit_config=rc(), vae_config=rc(), text_encoding_config=rc()),
              text_stage=HunyuanTextEncodingStage(llm, glyph), vae=vae, upsampler=up)  # fmt: skip
    frames = pipe("a fox", input_image=torch.rand(1, 3, 32, 32) * 2 - 1, seed=0, height=32, width=32, num_frames=5, num_inference_steps=2,
                  cfg_scale=2.0, latent_channels=4, spatial_factor=8, enable_sr=True, sr_height=64, sr_width=64, sr_num_inference_steps=2)  # fmt: skip
    assert len(frames) == 5 and frames[0].size == (64, 64)
