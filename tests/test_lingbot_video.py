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


def test_request_side_contracts(tmp_path):
    import hashlib
    import json

    from telefuser_b200.pipelines.lingbot_video import data as D

    # the guidance-branch captions are strings the text encoder was trained with: pinned by content hash
    assert hashlib.sha256(D.DEFAULT_NEGATIVE_PROMPT.encode()).hexdigest()[:16] == "43704d85b3951aed"
    assert hashlib.sha256(D.DEFAULT_NEGATIVE_PROMPT_IMAGE.encode()).hexdigest()[:16] == "7e277788a8bb3d2f"
    video, image = (json.loads(D.default_negative_caption(n))["universal_negative"] for n in (81, 1))
    assert "temporal_and_motion_stability" in video and "temporal_and_motion_stability" not in image
    assert "subtitles" in video["composition_and_content"] and "subtitles" not in image["composition_and_content"]
    assert list(video) == ["visual_quality", "artistic_style", "composition_and_content", "temporal_and_motion_stability", "material_and_structure"]

    assert [D.num_frames_from_duration(d) for d in (0, 0.1, 1, 3.3, 5)] == [1, 5, 25, 81, 121] and D.num_frames_from_duration(2, 16) == 33
    for bad in ((-1, 24), (1, 0)):
        with pytest.raises(ValueError):
            D.num_frames_from_duration(*bad)
    assert D.validate_frame_count(1) == 1 and D.validate_frame_count(81) == 81
    with pytest.raises(ValueError, match="4n\\+1"):
        D.validate_frame_count(80)

    sample = {"subject": "a fox", "scene": {"time": "dawn"}, "duration": 5, "fps": 24, "resolution": "480p"}
    assert D.parse_lingbot_video_prompt(sample) == ('{"subject":"a fox","scene":{"time":"dawn"}}', 5.0)  # run-time fields stay out
    assert D.parse_lingbot_video_prompt([{"caption": "plain text"}]) == ("plain text", None)
    assert D.parse_lingbot_video_prompt({"caption": {"主体": "狐狸"}, "duration": "2.5"}) == ('{"主体":"狐狸"}', 2.5)
    for bad, msg in (([], "empty list"), ("text", "is a dict"), ({"caption": ""}, "empty caption")):
        with pytest.raises(ValueError, match=msg):
            D.parse_lingbot_video_prompt(bad)
    (tmp_path / "p.json").write_text(json.dumps([sample]), encoding="utf-8")
    assert D.load_lingbot_video_prompt(tmp_path / "p.json")[1] == 5.0

    cfg = {"depth": 48, "hidden_size": 2048, "num_attention_heads": 16, "in_channels": 16, "patch_size": [1, 2, 2], "text_dim": 2560,
           "intermediate_size": 768, "num_experts": 128, "num_experts_per_tok": 8}  # fmt: skip
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    moe = D.load_lingbot_video_model_config(tmp_path, variant="moe")
    assert (moe.num_layers, moe.num_heads, moe.patch_size, moe.num_experts, moe.top_k) == (48, 16, (1, 2, 2), 128, 8)
    dense = {k: v for k, v in cfg.items() if not k.startswith("num_experts")}
    (tmp_path / "dense.json").write_text(json.dumps(dense))
    assert D.load_lingbot_video_model_config(tmp_path / "dense.json").top_k == 0
    with pytest.raises(ValueError, match="needs num_experts"):
        D.load_lingbot_video_model_config(tmp_path / "dense.json", variant="refiner")
    (tmp_path / "short.json").write_text(json.dumps({"depth": 2}))
    with pytest.raises(ValueError, match="lacks"):
        D.load_lingbot_video_model_config(tmp_path / "short.json")
    with pytest.raises(ValueError, match="not 'turbo'"):
        D.LingBotVideoModelConfig(variant="turbo")

    assert D.smart_resize(1080, 1920, factor=32) == (1088, 1920) and D.smart_resize(20, 20, factor=32) == (64, 64)
    big = D.smart_resize(6000, 9000, factor=32)
    assert big[0] % 32 == 0 and big[1] % 32 == 0 and big[0] * big[1] <= 16384 * 28**2 and abs(big[0] / big[1] - 2 / 3) < 0.01
    with pytest.raises(ValueError, match="thinner"):
        D.smart_resize(10, 4000, factor=32)

    img = torch.arange(3 * 40 * 60, dtype=torch.float32).reshape(1, 3, 40, 60) % 256
    frame = D.preprocess_ti2v_image(img, 32, 32)
    assert frame.shape == (1, 3, 1, 32, 32) and 0 <= frame.min() and frame.max() <= 1
    assert torch.equal(frame * 255, (frame * 255).round())  # uint8 interpolation: only whole grey levels come out
    same = D.preprocess_ti2v_image(img, 40, 60)
    assert torch.equal(same[:, :, 0] * 255, img)  # no resize needed: the frame is the image
    with pytest.raises(ValueError, match="condition image"):
        D.preprocess_ti2v_image(img[0], 32, 32)


def test_default_negative_follows_the_request_mode():
    from telefuser_b200.core.config import ModelRuntimeConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.pipelines.lingbot_video import LingBotVideoPipeline, LingBotVideoPipelineConfig, LingBotVideoRequest
    from telefuser_b200.pipelines.lingbot_video import data as D

    m = make_model("tiny")
    seen = []

    def text_stage(caption):
        seen.append(caption)
        g = torch.Generator().manual_seed(len(caption))
        return torch.randn(1, 5, m.config.text_dim, generator=g)

    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(m, "lingbot_video_transformer")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = LingBotVideoPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, LingBotVideoPipelineConfig(text_encoding_config=rc(), dit_config=rc(), vae_config=rc(), num_inference_steps=1), text_stage=text_stage)
    pipe.generate(LingBotVideoRequest("a fox", num_frames=5, height=32, width=32), decode=False)
    pipe.generate(LingBotVideoRequest("a fox", num_frames=1, height=32, width=32), decode=False)
    pipe.generate(LingBotVideoRequest("a fox", num_frames=1, height=32, width=32), negative_caption="mine", decode=False)
    assert seen == ["a fox", D.DEFAULT_NEGATIVE_PROMPT, "a fox", D.DEFAULT_NEGATIVE_PROMPT_IMAGE, "a fox", "mine"]
    with pytest.raises(ValueError, match="one-frame request"):
        pipe.generate(LingBotVideoRequest("a fox", num_frames=1, height=32, width=32, image=torch.zeros(1, 3, 32, 32)), decode=False)


def test_refiner_hand_off_from_video_to_video(tmp_path):
    import numpy as np
    from PIL import Image

    from telefuser_b200.core.config import ModelRuntimeConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.lingbot_video import LingBotVideoPipeline, LingBotVideoPipelineConfig
    from telefuser_b200.pipelines.lingbot_video import refiner as R
    from telefuser_b200.testing.synthetic import random_init_

    # frame budget: clips faster than the training rate are thinned, counts are cut to 4n+1, short clips repeat their end
    assert R.compute_training_frame_budget(81, 16) == (81, 16.0, 21)
    frames, fps, latents = R.compute_training_frame_budget(121, 30)
    assert (frames, latents) == (93, 24) and abs(fps - 93 / 121 * 30) < 1e-9
    assert R.compute_training_frame_budget(0, 24) == (1, 0.0, 1)
    with pytest.raises(ValueError, match="positive"):
        R.compute_training_frame_budget(10, 0)
    assert R.compute_training_aligned_indices(9, 5).tolist() == [0, 2, 4, 6, 8] and R.compute_training_aligned_indices(3, 5).tolist() == [0, 1, 2, 2, 2]
    assert R.compute_training_aligned_indices(0, 2).tolist() == [0, 0] and R.compute_training_aligned_indices(4, 0).numel() == 0
    clip = torch.linspace(-1, 1, 30).view(1, 1, 30, 1, 1).expand(1, 3, 30, 8, 12).contiguous()
    up, facts = R.prepare_refiner_video(clip, 30.0, 16, 24, max_frames=13)
    assert up.shape == (1, 3, 13, 16, 24) and facts["truncated_by_max_frames"] and facts["sample_frame_uncapped"] == 21 and facts["t_vae"] == 4
    assert torch.allclose(up[0, 0, :, 0, 0], clip[0, 0, np.linspace(0, 29, 13, dtype=int), 0, 0], atol=1e-6)  # constant frames survive the resize
    same, f2 = R.prepare_refiner_video(clip[:, :, :9], 16.0, 8, 12)
    assert torch.equal(same, clip[:, :, :9]) and not f2["truncated_by_max_frames"]
    with pytest.raises(ValueError, match=r"\[B, 3, F, H, W\]"):
        R.prepare_refiner_video(clip[0], 16.0, 8, 12)
    assert R.refiner_size(480, 832) == (1088, 1872)

    # a wide image is cropped to the LOW-resolution run's aspect ratio before it is resized
    arr = np.zeros((40, 120, 3), dtype=np.uint8)
    arr[:, 40:80] = 255  # white centre third
    Image.fromarray(arr).save(tmp_path / "first.png")
    first = R.first_frame_for_refiner(tmp_path / "first.png", 32, 32, geometry_height=16, geometry_width=16)
    assert first.shape == (1, 3, 1, 32, 32) and first.min() >= -1 and first.max() <= 1 and first.mean() > 0.95  # only the centre is left

    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(make_model("tiny-moe"), "lingbot_video_moe_transformer")
    mm.add_module(random_init_(WanVideoVAE(dim=8).float(), std=0.05).eval(), "wan_video_vae")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = LingBotVideoPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, LingBotVideoPipelineConfig(text_encoding_config=rc(), dit_config=rc(), vae_config=rc(), num_inference_steps=2))
    stage = R.LingBotVideoRefinerStage(pipe.denoising_stage, pipe.vae_stage, device="cpu", torch_dtype=torch.float32)
    pos, neg = torch.randn(1, 6, 32), torch.randn(1, 4, 32)
    low = torch.rand(1, 3, 9, 16, 16) * 2 - 1
    video, _ = R.prepare_refiner_video(low, 16.0, 32, 32)
    called = []
    out = stage.refine(video, pos, neg, num_inference_steps=4, t_thresh=0.5, tail_steps=1, seed=3, before_decode=lambda: called.append(1))
    assert out.shape == (1, 3, 9, 32, 32) and torch.isfinite(out).all() and called == [1]
    assert torch.equal(out, stage.refine(video, pos, neg, num_inference_steps=4, t_thresh=0.5, tail_steps=1, seed=3))
    lat = stage.refine(video, pos, neg, num_inference_steps=4, t_thresh=0.5, tail_steps=1, seed=3, decode=False)
    # the stage is the pipeline's latent-level `refine` with the VAE around it
    enc = pipe.vae_stage.process("encode_video", video).float()
    assert torch.allclose(lat, pipe.refine(enc, pos, neg, t_thresh=0.5, num_inference_steps=4, tail_steps=1, seed=3), atol=1e-5)
    # image-conditioned: frame 0 of the result is the clean first frame's latent
    clean = torch.rand(1, 3, 32, 32) * 2 - 1
    lat_c = stage.refine(video, pos, neg, num_inference_steps=4, t_thresh=0.5, seed=3, clean_first_frame=clean, decode=False)
    want0 = pipe.vae_stage.process("encode_video", clean.unsqueeze(2)).float()[:, :, :1]
    assert torch.allclose(lat_c[:, :, :1], want0, atol=1e-6) and not torch.allclose(lat_c[:, :, 1:], lat[:, :, 1:])
    with pytest.raises(ValueError, match="injected noise"):
        stage.refine(video, pos, neg, noise=torch.zeros(1, 16, 1, 4, 4))
