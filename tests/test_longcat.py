"""LongCat-Video: rope tables, per-frame modulation with clean conditioning frames, KV-cache continuation,
3-D block-sparse attention, LoRA switches, guidance rescaling and the pipeline modes on CPU; bf16 on GPUs."""

import pytest
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.longcat_video_dit import LongCatVideoTransformer3DModel, rope_tables_3d
from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import sparse_attention as SA
from telefuser_b200.pipelines.longcat_video import (LongCatVideoPipeline, LongCatVideoPipelineConfig, bsa_align_resolution,
                                                    cfg_zero_star)  # fmt: skip


def small(dtype=torch.float32, device="cpu", head_dim=48, depth=2, **kw):
    torch.manual_seed(0)
    m = LongCatVideoTransformer3DModel(in_channels=16, out_channels=16, hidden_size=2 * head_dim, depth=depth, num_heads=2,
                                       caption_channels=24, mlp_ratio=4, adaln_tembed_dim=32, **kw)  # fmt: skip
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    m = m.to(dtype).to(device).eval()
    m.dtype = dtype
    return m


def test_rope_and_keys():
    cos, sin = rope_tables_3d(48, (2, 3, 4))
    assert cos.shape == (24, 24) and torch.allclose(cos**2 + sin**2, torch.ones_like(cos), atol=1e-6)
    assert torch.allclose(sin[0], torch.zeros(24)) and torch.allclose(sin[12, 0], torch.sin(torch.tensor(1.0)))  # frame axis first
    keys = set(small().state_dict())
    for k in ("x_embedder.proj.weight", "t_embedder.mlp.2.bias", "y_embedder.y_proj.0.weight", "blocks.0.adaLN_modulation.1.weight",
              "blocks.0.attn.qkv.bias", "blocks.1.attn.k_norm.weight", "blocks.0.cross_attn.kv_linear.weight",
              "blocks.0.pre_crs_attn_norm.bias", "blocks.1.ffn.w3.weight", "final_layer.adaLN_modulation.1.bias",
              "final_layer.linear.weight"):  # fmt: skip
        assert k in keys, k
    with torch.device("meta"):
        full = LongCatVideoTransformer3DModel(depth=1)
    assert full.state_dict()["blocks.0.ffn.w1.weight"].shape == (11008, 4096)


def test_conditioning_frames_and_kv_cache_agree():
    m = small()
    x, y = torch.randn(1, 16, 3, 8, 8), torch.randn(1, 1, 6, 24)
    mask = torch.tensor([[1, 1, 1, 1, 0, 0]])
    t = torch.tensor([[0.0, 600.0, 600.0]])
    joint = m(x, t, y, mask, num_cond_latents=1)
    assert joint.shape == x.shape and joint.dtype == torch.float32
    m.cache_clean_latents(x[:, :, :1])
    assert len(m.kv_cache_dict) == 2 and m.kv_cache_dict[0][0].shape == (1, 16, 2, 48)
    cont = m(x[:, :, 1:], torch.tensor([600.0]), y, mask, num_cond_latents=1)
    m.clear_cache()
    # the new frames see the same keys / values either way (conditioning frames never look at the noisy ones)
    assert torch.allclose(cont, joint[:, :, 1:], atol=1e-4)
    two = m(torch.cat([x, x * 0.5]), torch.tensor([600.0, 300.0]), torch.cat([y, y * 2]), torch.cat([mask, mask]))
    one = m(x * 0.5, torch.tensor([300.0]), y * 2, mask)
    assert torch.allclose(two[1:], one, atol=1e-5)  # samples only see their own text


def test_bsa_3d_dense_limit_and_model_switch():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 4 * 8 * 8, 2, 16) for _ in range(3))
    blocks = SA.to_3d_blocks(q, (4, 8, 8), (4, 4, 4))
    assert torch.equal(SA.from_3d_blocks(blocks, (4, 8, 8), (4, 4, 4)), q)
    dense = SA.bsa_3d_attention(q, k, v, (4, 8, 8), sparsity=0.0)
    assert torch.allclose(dense, TF.attention_reference(q, k, v), atol=1e-5)
    sparse = SA.bsa_3d_attention(q, k, v, (4, 8, 8), sparsity=0.75)
    assert torch.isfinite(sparse).all() and not torch.allclose(sparse, dense, atol=1e-3)
    m = small()
    x, y = torch.randn(1, 16, 4, 16, 16), torch.randn(1, 1, 4, 24)
    base = m(x, torch.tensor([500.0]), y)
    m.enable_bsa()
    assert not torch.allclose(m(x, torch.tensor([500.0]), y), base, atol=1e-4)
    m.disable_bsa()
    assert torch.equal(m(x, torch.tensor([500.0]), y), base)
    assert bsa_align_resolution(720, 1280) == (704, 1216) and bsa_align_resolution(960, 960) == (960, 960)


def test_lora_switches_restore_the_weights():
    m = small()
    w0 = m.blocks[0].attn.proj.weight.detach().clone()
    lora = {"blocks.0.attn.proj.lora_A.weight": torch.randn(4, 96) * 0.1, "blocks.0.attn.proj.lora_B.weight": torch.randn(96, 4) * 0.1}
    m.load_lora(lora, "refinement_lora")
    m.enable_loras(["refinement_lora"])
    assert not torch.allclose(m.blocks[0].attn.proj.weight, w0) and m.active_loras == ["refinement_lora"]
    m.disable_all_loras()
    assert torch.allclose(m.blocks[0].attn.proj.weight, w0, atol=1e-6) and m.active_loras == []


def test_guidance_and_pipeline_modes():
    p, n = torch.randn(1, 4, 2, 3, 3), torch.randn(1, 4, 2, 3, 3)
    a = (p * n).sum() / (n * n).sum()
    assert torch.allclose(cfg_zero_star(p, n, 3.0), n * a + 3 * (p - n * a), atol=1e-5)
    assert torch.allclose(cfg_zero_star(p, p, 3.0), p, atol=1e-5)
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(small(), "longcat_video_dit")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = LongCatVideoPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, LongCatVideoPipelineConfig(dit_config=rc(), vae_config=rc(), text_encoding_config=rc(), enable_refine=True,
                                             refine_num_steps=4, enable_refine_bsa=False))  # fmt: skip
    stage = pipe.denoise_stage
    assert torch.allclose(stage.get_timesteps_sigmas(4, use_distill=True), torch.tensor([1.0, 0.76, 0.5, 0.26]))
    pos = (torch.randn(1, 1, 5, 24), torch.ones(1, 5, dtype=torch.long))
    neg = (torch.randn(1, 1, 5, 24), torch.ones(1, 5, dtype=torch.long))
    kw = dict(prompt_embeds=pos, negative_prompt_embeds=neg, height=64, width=64, num_frames=9, num_inference_steps=3, seed=0)
    a = pipe(**kw)
    assert a.shape == (1, 16, 3, 8, 8) and torch.isfinite(a).all() and torch.equal(a, pipe(**kw))
    prev = torch.randn(1, 16, 4, 8, 8)  # continuation from the latents of an earlier clip (13 frames -> 3 latent frames)
    kw17 = {**kw, "num_frames": 17}  # 5 latent frames: 3 conditioning + 2 new
    joint = pipe(input_video=prev, need_encode=False, **kw17)
    assert joint.shape == (1, 16, 5, 8, 8) and torch.equal(joint[:, :, :3], prev[:, :, -3:].to(joint))
    cached = pipe(input_video=prev, need_encode=False, use_kv_cache=True, **kw17)
    assert cached.shape == joint.shape and torch.allclose(cached, joint, atol=1e-2)
    hf = pipe(enhance_hf=True, **{**kw, "num_inference_steps": 6})
    tail = stage.scheduler.timesteps[-10:]
    assert torch.allclose(tail, torch.linspace(500, 50, 10)) and (stage.scheduler.timesteps[:-10] > 500).all() and hf.shape == a.shape
    refined = pipe(enable_refine=True, refine_height=128, refine_width=128, refine_t_thresh=0.5, **kw)
    assert refined.shape == (1, 16, 3, 16, 16) and torch.isfinite(refined).all()


@pytest.mark.gpu
def test_gpu_bf16_forward_tracks_cpu_fp32():
    ref_m = small(head_dim=128)
    x, y, t = torch.randn(1, 16, 2, 32, 32), torch.randn(1, 1, 9, 24), torch.tensor([[0.0, 700.0]])
    ref = ref_m(x, t, y, num_cond_latents=1)
    gpu_m = small(torch.bfloat16, "cuda", head_dim=128)
    got = gpu_m(x.cuda().bfloat16(), t.cuda(), y.cuda().bfloat16(), num_cond_latents=1).float().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err
