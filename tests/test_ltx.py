"""LTX-2 audio-video transformer: structure, rotary tables, perturbations, x0 wrapper; bf16 kernels vs fp32 on the GPU."""

import pytest
import torch

from telefuser_b200.models import ltx_dit as M

KW = dict(num_attention_heads=2, attention_head_dim=64, in_channels=8, out_channels=8, num_layers=2, cross_attention_dim=128,
          audio_num_attention_heads=2, audio_attention_head_dim=32, audio_in_channels=6, audio_out_channels=6,
          audio_cross_attention_dim=64, av_ca_timestep_scale_multiplier=1000)  # fmt: skip


def _model(rope="split", gated=True, caln=True, model_type=M.LTXModelType.AudioVideo, seed=0):
    torch.manual_seed(seed)
    m = M.LTXModel(model_type=model_type, rope_type=M.LTXRopeType(rope), double_precision_rope=rope == "split",
                   apply_gated_attention=gated, cross_attention_adaln=caln, **KW)  # fmt: skip
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    return m.float().eval()


def _inputs(B=2, grid=(3, 2, 2), Ta=7, device="cpu", dtype=torch.float32):
    torch.manual_seed(1)
    f, h, w = torch.meshgrid(*[torch.arange(n) for n in grid], indexing="ij")
    start = torch.stack([f.flatten() * 8.0 / 25, h.flatten() * 32.0, w.flatten() * 32.0])
    vpos = torch.stack([start, start + torch.tensor([8 / 25, 32.0, 32.0])[:, None]], dim=-1)[None].repeat(B, 1, 1, 1)
    astart = torch.arange(Ta)[None].float() * 0.04
    apos = torch.stack([astart, astart + 0.04], dim=-1)[None].repeat(B, 1, 1, 1)
    Tv = vpos.shape[2]
    sig = torch.linspace(0.7, 0.3, B)
    v = M.Modality(latent=torch.randn(B, Tv, 8).to(device, dtype), sigma=sig.to(device), positions=vpos.to(device),
                   timesteps=sig[:, None, None].expand(B, Tv, 1).clone().to(device), context=torch.randn(B, 5, 128).to(device, dtype),
                   context_mask=torch.tensor([[1, 1, 1, 1, 1], [1, 1, 1, 0, 0]][:B]).to(device))  # fmt: skip
    a = M.Modality(latent=torch.randn(B, Ta, 6).to(device, dtype), sigma=(sig * 0.9).to(device), positions=apos.to(device),
                   timesteps=(sig * 0.9)[:, None, None].expand(B, Ta, 1).clone().to(device),
                   context=torch.randn(B, 5, 64).to(device, dtype), context_mask=None)  # fmt: skip
    return v, a


def test_rotary_tables_and_application():
    pos = torch.rand(1, 3, 5, 2) * 10
    cos, sin = M.precompute_freqs_cis(pos, 48, torch.float32, use_middle_indices_grid=True, num_attention_heads=2)
    assert cos.shape == (1, 5, 48) and torch.allclose(cos**2 + sin**2, torch.ones_like(cos), atol=1e-5)
    x = torch.randn(1, 5, 48)
    y = M.apply_rotary_emb(x, (cos, sin))
    assert torch.allclose(y.unflatten(-1, (-1, 2)).norm(dim=-1), x.unflatten(-1, (-1, 2)).norm(dim=-1), atol=1e-5)
    c2, s2 = M.precompute_freqs_cis(pos, 52, torch.float32, use_middle_indices_grid=True, num_attention_heads=2,
                                    rope_type=M.LTXRopeType.SPLIT, double_precision=True)  # fmt: skip
    assert c2.shape == (1, 2, 5, 13) and torch.all(c2[:, 0, :, :2] == 1) and torch.all(s2[:, 0, :, :2] == 0)  # 26 - 8*3 = 2 pad slots in front
    x = torch.randn(1, 5, 52)
    y = M.apply_rotary_emb(x, (c2, s2), M.LTXRopeType.SPLIT)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # a position at the middle of the range has angle 0
    c3, s3 = M.precompute_freqs_cis(torch.full((1, 1, 4, 2), 10.0), 16, torch.float32, max_pos=[20], use_middle_indices_grid=True)
    assert torch.allclose(c3, torch.ones_like(c3)) and torch.allclose(s3, torch.zeros_like(s3), atol=1e-6)


@pytest.mark.parametrize("rope,gated,caln", [("interleaved", False, False), ("split", True, True)])
def test_forward_shapes_and_batch_independence(rope, gated, caln):
    m = _model(rope, gated, caln)
    v, a = _inputs()
    vx, ax = m(v, a)
    assert vx.shape == (2, 12, 8) and ax.shape == (2, 7, 6)
    first = lambda m_: M.Modality(**{k: (t[:1] if isinstance(t, torch.Tensor) else t) for k, t in m_.__dict__.items()})  # noqa: E731
    v1, a1 = first(v), first(a)
    vx1, ax1 = m(v1, a1)
    assert torch.allclose(vx1[0], vx[0], atol=1e-5) and torch.allclose(ax1[0], ax[0], atol=1e-5)
    # a disabled video stream passes through untouched and still conditions the audio stream
    v_off = M.Modality(**{**v.__dict__, "enabled": False})
    vx_off, ax_off = m(v_off, a)
    assert not torch.allclose(vx_off, vx) and ax_off.shape == ax.shape


def test_perturbations():
    m = _model()
    v, a = _inputs()
    P, T = M.Perturbation, M.PerturbationType
    base_v, base_a = m(v, a)
    skip0 = M.BatchedPerturbationConfig([M.PerturbationConfig([P(T.SKIP_VIDEO_SELF_ATTN, None), P(T.SKIP_A2V_CROSS_ATTN, [1])]),
                                         M.PerturbationConfig.empty()])  # fmt: skip
    pv, pa = m(v, a, skip0)
    assert torch.allclose(pv[1], base_v[1], atol=1e-5) and not torch.allclose(pv[0], base_v[0], atol=1e-4)
    both = M.BatchedPerturbationConfig([M.PerturbationConfig([P(T.SKIP_VIDEO_SELF_ATTN, None), P(T.SKIP_A2V_CROSS_ATTN, [1])])] * 2)
    bv, _ = m(v, a, both)
    assert torch.allclose(bv[0], pv[0], atol=1e-5)  # the whole-batch shortcut equals the masked form
    cfg = M.PerturbationConfig([P(T.SKIP_V2A_CROSS_ATTN, [0])])
    assert cfg.is_perturbed(T.SKIP_V2A_CROSS_ATTN, 0) and not cfg.is_perturbed(T.SKIP_V2A_CROSS_ATTN, 1)
    assert not M.PerturbationConfig(None).is_perturbed(T.SKIP_V2A_CROSS_ATTN, 0)


def test_single_modality_models_and_x0():
    m = _model(model_type=M.LTXModelType.VideoOnly)
    assert not hasattr(m, "audio_patchify_proj") and not hasattr(m.transformer_blocks[0], "audio_attn1")
    v, a = _inputs()
    vx, ax = m(v, None)
    assert ax is None and vx.shape == (2, 12, 8)
    with pytest.raises(ValueError):
        m(v, a)
    den, _ = M.X0Model(m)(v, None)
    assert torch.allclose(den, v.latent - vx * v.timesteps, atol=1e-6)
    assert torch.allclose(M.to_velocity(v.latent[:1], 0.7, den[:1]), vx[:1], atol=1e-5)
    ma = _model(model_type=M.LTXModelType.AudioOnly)
    _, ax = ma(None, a)
    assert ax.shape == (2, 7, 6)


def test_wrapper_config_and_converter():
    cfg = {"transformer": {**M.LTX23_DEV_TRANSFORMER_CONFIG["transformer"], "num_layers": 1, "num_attention_heads": 2,
                           "audio_num_attention_heads": 2, "cross_attention_dim": 256, "audio_cross_attention_dim": 128}}  # fmt: skip
    net = M.LTXVideoTransformer(cfg)
    vm = net.velocity_model
    assert vm.rope_type == M.LTXRopeType.SPLIT and vm.double_precision_rope and vm.cross_attention_adaln
    assert not hasattr(vm, "caption_projection") and vm.transformer_blocks[0].scale_shift_table.shape == (9, 256)
    assert vm.transformer_blocks[0].attn1.to_gate_logits is not None and net.get_fsdp_module_names() == net.layer_name_list
    sd = {"model.diffusion_model." + k: v for k, v in vm.state_dict().items()}
    sd["vae.decoder.conv_in.weight"] = torch.zeros(1)
    conv, _ = net.state_dict_converter().from_official(sd)
    assert set(conv) == set(net.state_dict())
    with_cap = M.build_ltx_model_from_config({"transformer": {"num_layers": 1, "num_attention_heads": 2, "audio_num_attention_heads": 2,
                                                              "caption_channels": 40}})  # fmt: skip
    assert with_cap.caption_projection.linear_1.in_features == 40 and with_cap.audio_caption_projection.linear_2.out_features == 128


@pytest.mark.gpu
def test_gpu_bf16_matches_fp32():
    m = _model()
    v, a = _inputs(B=1, grid=(4, 6, 8), Ta=40)
    v = M.Modality(**{**v.__dict__, "context_mask": None})
    ref_v, ref_a = m(v, a)
    mg = _model().to("cuda", torch.bfloat16)
    vg, ag = _inputs(B=1, grid=(4, 6, 8), Ta=40, device="cuda", dtype=torch.bfloat16)
    vg = M.Modality(**{**vg.__dict__, "context_mask": None})
    out_v, out_a = mg(vg, ag)
    for o, r in ((out_v, ref_v), (out_a, ref_a)):
        err = (o.float().cpu() - r).abs().max().item()
        assert err < 0.04 * max(1.0, r.abs().max().item()), err


@pytest.mark.gpu
def test_gpu_batched_passes_with_perturbations():
    """Batch of two with different prompts and perturbations (the batched-guidance form) on the native kernels."""
    P, T = M.Perturbation, M.PerturbationType
    ptb = lambda: M.BatchedPerturbationConfig([M.PerturbationConfig.empty(),  # noqa: E731
                                               M.PerturbationConfig([P(T.SKIP_VIDEO_SELF_ATTN, [1]), P(T.SKIP_A2V_CROSS_ATTN, None), P(T.SKIP_AUDIO_SELF_ATTN, [0])])])
    m = _model()
    v, a = _inputs(B=2, grid=(4, 6, 8), Ta=40)
    v = M.Modality(**{**v.__dict__, "context_mask": None})
    ref_v, ref_a = m(v, a, ptb())
    mg = _model().to("cuda", torch.bfloat16)
    vg, ag = _inputs(B=2, grid=(4, 6, 8), Ta=40, device="cuda", dtype=torch.bfloat16)
    vg = M.Modality(**{**vg.__dict__, "context_mask": None})
    out_v, out_a = mg(vg, ag, ptb())
    for o, r in ((out_v, ref_v), (out_a, ref_a)):
        err = (o.float().cpu() - r).abs().max().item()
        assert err < 0.04 * max(1.0, r.abs().max().item()), err
    x0_v, _ = M.X0Model(mg)(vg, ag, ptb())
    assert x0_v.shape == vg.latent.shape and bool(torch.isfinite(x0_v.float()).all())
