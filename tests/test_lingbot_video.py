"""LingBot-Video transformers (dense and mixture of experts): checkpoint fingerprints, batching rule,
routed experts against a dense evaluation, Ulysses and expert parallelism on gloo ranks; on GPUs the
RMSNorm glue kernels and the bf16 forward against the fp32 CPU path."""

import pytest
import torch

from telefuser_b200.models.lingbot_video import (LingBotVideoConfig, LingBotVideoTransformer3DModel,
                                                 infer_lingbot_video_config, joint_position_ids, rope_tables)  # fmt: skip
from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import moe as MOE
from telefuser_b200.testing.lingbot_video_checks import make_inputs, make_model, spawn
from telefuser_b200.utils.model_weight import hash_state_dict_keys


def test_presets_reproduce_the_public_checkpoint_fingerprints():
    for preset, want, params in (("dense-1.3b", "2bcf511fe5e0000519394d242b4d8abd", 1.357e9),
                                 ("moe-30b-a3b", "65b83aa625cd362ff5ff3409fb367a6f", 30.08e9)):  # fmt: skip
        with torch.device("meta"):
            m = LingBotVideoTransformer3DModel(LingBotVideoConfig.preset(preset))
        assert hash_state_dict_keys(m.state_dict(), with_shape=True) == want
        assert abs(sum(p.numel() for p in m.parameters()) - params) / params < 0.01
        cfg = infer_lingbot_video_config({k: v for k, v in m.state_dict().items()})
        assert cfg["depth"] == m.config.depth and cfg.get("num_experts", 0) == m.config.num_experts


def test_batch_with_text_mask_equals_per_sample_runs():
    m = make_model("tiny")
    x = torch.randn(2, 16, 2, 8, 8)
    t = torch.tensor([200.0, 800.0])
    txt = torch.randn(2, 6, 32)
    mask = torch.tensor([[1, 1, 1, 1, 1, 1], [1, 1, 1, 0, 0, 0]])
    both = m(x, t, txt, mask)
    one = m(x[1:], t[1:], txt[1:, :3])
    assert both.shape == x.shape and torch.isfinite(both).all()
    assert (both[1:] - one).abs().max() <= 1e-5


def test_positions_and_rope_tables():
    pos = joint_position_ids(3, 2, 2, 2, "cpu")
    assert pos.shape == (11, 3) and pos[0].tolist() == [4, 0, 0] and pos[7].tolist() == [5, 1, 1]
    assert pos[8:].tolist() == [[1, 0, 0], [2, 0, 0], [3, 0, 0]]
    cos, sin = rope_tables(pos, (16, 24, 24), 256.0)
    assert cos.shape == (11, 32) and torch.allclose(cos**2 + sin**2, torch.ones_like(cos), atol=1e-6)


def test_routed_experts_equal_dense_evaluation():
    torch.manual_seed(0)
    T, C, I, E, K = 33, 64, 32, 8, 3
    x = torch.randn(T, C)
    w13, w2 = torch.randn(E, 2 * I, C) * 0.1, torch.randn(E, C, I) * 0.1
    ids, w = MOE.route_topk(torch.randn(T, E), 2, 1, K, torch.randn(E) * 0.1, 2.0)
    assert ((ids // 4) == (ids[:, :1] // 4)).all()  # one group of the two survives
    got = MOE.experts_forward(x, ids, w, w13, w2)
    dense = torch.zeros(T, C)
    for t in range(T):
        for k in range(K):
            e = int(ids[t, k])
            h = w13[e] @ x[t]
            dense[t] += w[t, k] * (w2[e] @ (torch.nn.functional.silu(h[:I]) * h[I:]))
    assert (got - dense).abs().max() <= 1e-4


def test_fp8_experts_follow_the_bf16_experts_and_the_model_switch():
    torch.manual_seed(0)
    T, C, I, E, K = 40, 64, 64, 8, 2
    x = torch.randn(T, C)
    w13, w2 = torch.randn(E, 2 * I, C) * 0.1, torch.randn(E, C, I) * 0.1
    ids, w = MOE.route_topk(torch.randn(T, E), 1, 1, K)
    q13, s13 = MOE.quantize_expert_weight_fp8(w13)
    q2, s2 = MOE.quantize_expert_weight_fp8(w2)
    assert q13.dtype == torch.float8_e4m3fn and s13.shape == (E, 2 * I) and s2.shape == (E, C)
    assert torch.allclose(q13.float() * s13.unsqueeze(2), w13, atol=(w13.abs().amax(2, keepdim=True) / 16).max().item())
    assert torch.equal((q13.float().abs().amax(2) - 448).abs() < 1e-3, torch.ones(E, 2 * I, dtype=torch.bool))  # full range used
    ref = MOE.experts_forward(x, ids, w, w13, w2)
    got = MOE.experts_forward_fp8(x, ids, w, q13, s13, q2, s2)
    assert torch.equal(got, MOE.experts_forward_fp8_reference(x, ids.long(), w, q13, s13, q2, s2))
    assert (got - ref).norm() / ref.norm() < 0.09  # two GEMMs with e4m3 operands on both sides
    res = torch.randn(T, C)
    assert torch.allclose(MOE.experts_forward_fp8(x, ids, w, q13, s13, q2, s2, residual=res), got + res, atol=1e-5)
    with pytest.raises(ValueError, match="quantised"):
        MOE.experts_forward_fp8(x, ids, w, w13, s13, q2, s2)
    with pytest.raises(ValueError, match="stacked"):
        MOE.quantize_expert_weight_fp8(w13[0])

    m = make_model("tiny-moe", hidden_size=128, num_attention_heads=2, moe_intermediate_size=64, intermediate_size=256)
    lat, ts, txt = make_inputs(text_dim=m.config.text_dim, size=8)
    with torch.no_grad():
        base = m(lat, ts, txt)
        banks = sum(1 for b in m.blocks if hasattr(b.ffn, "experts"))
        linears_only = make_model("tiny-moe", hidden_size=128, num_attention_heads=2, moe_intermediate_size=64, intermediate_size=256).enable_quant("int8")
        n = m.enable_quant("fp8")
        assert banks > 0 and n == linears_only + banks  # the stacked experts are counted on top of the block linears
        ex = next(b.ffn.experts for b in m.blocks if hasattr(b.ffn, "experts"))
        assert ex.w1.dtype == ex.w2.dtype == ex.w3.dtype == torch.float8_e4m3fn and ex.w1_scale.shape == ex.w1.shape[:2]
        assert ex.fused_w13_scale().shape == (ex.w1.shape[0], 2 * ex.w1.shape[1])
        assert {"w1_scale", "w2_scale", "w3_scale"} <= {k.rsplit(".", 1)[1] for k in m.state_dict() if ".experts." in k}
        out = m(lat, ts, txt)
        assert torch.isfinite(out).all() and (out - base).norm() / base.norm() < 0.15
        assert m.quantize_experts_fp8_() == banks and torch.equal(m(lat, ts, txt), out)  # a second call changes nothing
    from telefuser_b200.parallel.expert import ExpertParallelState

    with pytest.raises(ValueError, match="unsharded"):
        ExpertParallelState.shard_(ex, None)


def test_ulysses2_and_expert_parallel2_match_single_process():
    for preset in ("tiny", "tiny-moe"):
        m = make_model(preset)
        x, t, txt = make_inputs()
        ref = m(x, t, txt)
        got = spawn(2, preset, "ulysses")  # 128 video + 7 text tokens: odd length, padded to 136
        assert (ref - got).abs().max() <= 1e-5, preset
    m = make_model("tiny-moe")
    ref = m(*make_inputs())
    assert (ref - spawn(2, "tiny-moe", "ep")).abs().max() <= 1e-5
    assert (ref - spawn(2, "tiny-moe", "both")).abs().max() <= 1e-5


def test_pipeline_generate_cfg_modes_ti2v_and_refiner():
    import numpy as np

    from telefuser_b200.core.config import ModelRuntimeConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.lingbot_video import (LingBotVideoPipeline, LingBotVideoPipelineConfig,
                                                        LingBotVideoRequest, compute_refiner_sigmas, latent_shape,
                                                        reinject_ti2v_condition)  # fmt: skip
    from telefuser_b200.testing.synthetic import random_init_

    assert latent_shape(17, 32, 48) == (5, 4, 6)
    sig = compute_refiner_sigmas(1.0, 0.0, 10, 3.0, 0.5, tail_steps=2)
    assert abs(sig[0] - 0.5) < 1e-6 and np.all(np.diff(sig) < 0) and sig[-1] > 0
    lat, cond = torch.zeros(1, 2, 4, 2, 2), torch.ones(1, 2, 1, 2, 2)
    mask = torch.tensor([True, False, False, False])
    assert reinject_ti2v_condition(lat, cond, mask)[:, :, 0].eq(1).all() and reinject_ti2v_condition(lat, cond, mask)[:, :, 1:].eq(0).all()

    def build(batch_cfg):
        mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
        mm.add_module(make_model("tiny-moe"), "lingbot_video_moe_transformer")
        mm.add_module(random_init_(WanVideoVAE(dim=8).float(), std=0.05).eval(), "wan_video_vae")
        rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
        cfg = LingBotVideoPipelineConfig(text_encoding_config=rc(), dit_config=rc(), vae_config=rc(), num_inference_steps=3,
                                         guidance_scale=3.0, batch_cfg=batch_cfg)  # fmt: skip
        pipe = LingBotVideoPipeline(device="cpu", torch_dtype=torch.float32)
        pipe.init(mm, cfg)
        return pipe

    pos, neg = torch.randn(1, 6, 32), torch.randn(1, 4, 32)
    req = LingBotVideoRequest(num_frames=5, height=32, width=32, seed=3)
    a = build(False).generate(req, prompt_embeds=pos, negative_prompt_embeds=neg, decode=False).output
    b = build(True).generate(req, prompt_embeds=pos, negative_prompt_embeds=neg, decode=False).output
    assert a.shape == (1, 16, 2, 4, 4) and torch.isfinite(a).all()
    assert (a - b).abs().max() <= 1e-4  # one batched forward == two sequential forwards
    pipe = build(False)
    img = torch.rand(1, 3, 32, 32) * 2 - 1
    out = pipe.generate(LingBotVideoRequest(num_frames=5, height=32, width=32, image=img), prompt_embeds=pos,
                        negative_prompt_embeds=neg, decode=True)  # fmt: skip
    assert out.output.shape[-3:] == (5, 32, 32) and out.prompt_conditions["has_visual_condition"]
    r = pipe.refine(a, pos, neg, t_thresh=0.4, num_inference_steps=6)
    assert r.shape == a.shape and torch.isfinite(r).all()


def _rel(a, b):
    """Largest error relative to 1 + |reference| (outputs are bf16: half an ulp is 2^-9 of the value)."""
    return ((a - b).abs() / (1 + b.abs())).max().item()


@pytest.mark.gpu
def test_rms_glue_kernels_match_reference():
    torch.manual_seed(0)
    B, S, C = 1, 777, 2048
    x = torch.randn(B, S, C, device="cuda").bfloat16()
    y = torch.randn(B, S, C, device="cuda").bfloat16()
    w = torch.rand(C, device="cuda") + 0.5
    shift, scale, gate = (torch.randn(1, 1, C, device="cuda") for _ in range(3))
    got = TF.rmsnorm_modulate(x, w, shift, scale)
    want = TF.rmsnorm_modulate(x.float().cpu(), w.cpu(), shift.cpu(), scale.cpu())
    assert _rel(got.float().cpu(), want) <= 1.5e-2
    got = TF.rmsnorm_gate_residual(x, y, w, gate)
    want = TF.rmsnorm_gate_residual(x.float().cpu(), y.float().cpu(), w.cpu(), gate.cpu())
    assert _rel(got.float().cpu(), want) <= 1.5e-2
    per_tok = torch.randn(1, S, C, device="cuda")
    got = TF.rmsnorm_modulate(x, None, per_tok, None)
    want = TF.rmsnorm_modulate(x.float().cpu(), None, per_tok.cpu(), None)
    assert _rel(got.float().cpu(), want) <= 1.5e-2
    for H, D in ((16, 128), (4, 64), (2, 192)):
        qkv = torch.randn(1, 301, 3 * H * D, device="cuda").bfloat16()
        ref = qkv.float().cpu()
        wq, wk = torch.rand(D) + 0.5, torch.rand(D) + 0.5
        ang = torch.randn(301, D // 2)
        q, k = (qkv[..., i * H * D : (i + 1) * H * D].unflatten(-1, (H, D)) for i in range(2))
        TF.headnorm_rope_(q, wq.cuda(), ang.cos().cuda(), ang.sin().cuda(), 1e-6, k=k, weight_k=wk.cuda())
        rq, rk = (ref[..., i * H * D : (i + 1) * H * D].unflatten(-1, (H, D)).clone() for i in range(2))
        TF.headnorm_rope_(rq, wq, ang.cos(), ang.sin(), 1e-6, k=rk, weight_k=wk)
        assert _rel(q.float().cpu(), rq) <= 1.5e-2 and _rel(k.float().cpu(), rk) <= 1.5e-2
        assert torch.equal(qkv[..., 2 * H * D :].float().cpu(), ref[..., 2 * H * D :])  # v untouched


@pytest.mark.gpu
@pytest.mark.parametrize("preset", ["tiny", "tiny-moe"])
def test_gpu_bf16_forward_tracks_cpu_fp32(preset):
    over = dict(hidden_size=256, num_attention_heads=2, axes_dims=(32, 48, 48), moe_intermediate_size=128)  # head_dim 128
    ref_m = make_model(preset, **over)
    x, t, txt = make_inputs(frames=2, size=16, text_len=9)
    ref = ref_m(x, t, txt)
    gpu_m = make_model(preset, torch.bfloat16, "cuda", **over)
    got = gpu_m(x.cuda().bfloat16(), t.cuda(), txt.cuda().bfloat16()).float().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err


@pytest.mark.gpu
@pytest.mark.multi_gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_over_peer_memory_matches_single_gpu():
    over = dict(hidden_size=256, num_attention_heads=2, axes_dims=(32, 48, 48), moe_intermediate_size=128)
    kw = dict(frames=2, size=16, text_len=8)  # 520 tokens: divisible by 2
    single = make_model("tiny-moe", torch.bfloat16, "cuda", **over)
    x, t, txt = make_inputs(**kw)
    ref = single(x.cuda().bfloat16(), t.cuda(), txt.cuda().bfloat16()).float().cpu()
    for mode in ("ep", "both"):
        got = spawn(2, "tiny-moe", mode, backend="nccl", dtype=torch.bfloat16, overrides=over, **kw)
        err = ((got - ref).norm() / ref.norm()).item()
        assert err < 2e-2, (mode, err)
