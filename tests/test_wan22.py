"""Wan2.2: 48-channel VAE building blocks and streaming, the latent-cache hand-off, the two-expert denoising
stage (switch at the boundary, resume from a cached latent) and TI2V conditioning with per-token timesteps."""

import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.models.wan22_vae import AvgDown3D, DupUp3D, VideoVAE22, Wan22VideoVAE, patchify, unpatchify
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.pipelines.wan.latent_data_utils import parse_latent_data
from telefuser_b200.pipelines.wan.moe_dit_denoising import MoeDitDenoisingStage
from telefuser_b200.pipelines.wan.ti2v_denoising import TI2VDenoisingStage, per_token_timestep
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler
from telefuser_b200.testing.distributed_checks import make_tiny_inputs, make_tiny_model, tiny_wan_denoise


def test_vae22_blocks_and_streaming():
    x = torch.randn(1, 3, 5, 8, 12)
    p = patchify(x)
    assert p.shape == (1, 12, 5, 4, 6) and torch.equal(unpatchify(p), x)
    assert p[0, 1 * 4 + 1 * 2 + 0, 2, 1, 3] == x[0, 1, 2, 2, 7]  # channel (c=1, col offset 1, row offset 0)
    down = AvgDown3D(4, 8, factor_t=2, factor_s=2)
    y = down(torch.ones(1, 4, 3, 4, 4))  # odd length: one zero frame is padded in front
    assert y.shape == (1, 8, 2, 2, 2) and torch.allclose(y[:, :, 1], torch.ones(1, 8, 2, 2))
    assert y[:, 0::2, 0].abs().max() == 0 and (y[:, 1::2, 0] == 1).all()  # a group = one time offset of one channel
    up = DupUp3D(8, 4, factor_t=2, factor_s=2)
    z = torch.randn(1, 8, 2, 3, 3)
    assert up(z).shape == (1, 4, 4, 6, 6) and up(z, first_chunk=True).shape == (1, 4, 3, 6, 6)
    torch.manual_seed(0)
    vae = VideoVAE22(dim=16, dec_dim=16, z_dim=8).eval()
    scale = [torch.zeros(8), torch.ones(8)]
    video = torch.randn(1, 3, 9, 32, 32)
    with torch.no_grad():
        lat = vae.encode(video, scale)
        assert lat.shape == (1, 8, 3, 2, 2)
        es = vae.new_encoder_state()
        parts = [vae.encode_chunk(video[:, :, :1], es, scale), vae.encode_chunk(video[:, :, 1:5], es, scale),
                 vae.encode_chunk(video[:, :, 5:], es, scale)]  # fmt: skip
        assert torch.allclose(torch.cat(parts, 2), lat, atol=1e-6)
        full = vae.decode(lat, scale)
        assert full.shape == video.shape
        ds = vae.new_decoder_state()
        chunks = torch.cat([vae.decode_chunk(lat[:, :, :1], ds, scale), vae.decode_chunk(lat[:, :, 1:], ds, scale)], 2)
        assert torch.allclose(chunks, full, atol=1e-6)
    wrapper = Wan22VideoVAE(z_dim=8, dim=16, dec_dim=16)
    assert wrapper.upsampling_factor == 16 and len(wrapper.mean) == 8
    assert "model.decoder.upsamples.0.upsamples.3.resample.1.weight" in wrapper.state_dict()
    with torch.no_grad():
        out = wrapper.decode(torch.randn(1, 8, 2, 4, 6), tiled=True, tile_size=(3, 4), tile_stride=(2, 2))
    assert out.shape == (1, 3, 5, 64, 96)


def test_latent_data_validation():
    lat = torch.zeros(1, 16, 3, 8, 8)
    assert parse_latent_data(None, lat.shape, 10) == (None, 0, [])
    c, s, saved = parse_latent_data({"cached_latent": lat, "skip_step": 4, "saved_steps": [2, 6, 6, 12]}, lat.shape, 10)
    assert c is lat and s == 4 and saved == [6]
    assert parse_latent_data({"cached_latent": lat, "skip_step": 10}, lat.shape, 10)[:2] == (None, 0)
    assert parse_latent_data({"cached_latent": lat[:, :8], "skip_step": 3}, lat.shape, 10)[:2] == (None, 0)
    assert parse_latent_data({"cached_latent": "x", "skip_step": 3, "saved_steps": [1]}, lat.shape, 10) == (None, 0, [1])


class _Counting(torch.nn.Module):
    def __init__(self, model):
        super().__init__()
        self.model, self.calls = model, 0

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.model, name)

    def forward(self, *a, **k):
        self.calls += 1
        return self.model(*a, **k)


def _moe_stage(high, low):
    cfg = lambda: ModelRuntimeConfig(torch_dtype=torch.float32, device_type="cpu")  # noqa: E731
    pmesh.set_mesh(None)
    stage = MoeDitDenoisingStage("denoise", None, cfg(), cfg(), FlowMatchScheduler("Wan"), dits=(high, low))
    stage.mesh = pmesh.get_mesh()
    return stage


def test_two_expert_denoising_switches_and_resumes():
    ref = tiny_wan_denoise(steps=6)  # one model for all steps
    latents, ctx, neg = make_tiny_inputs()
    high, low = _Counting(make_tiny_model()), _Counting(make_tiny_model())
    stage = _moe_stage(high, low)
    out = stage.process(latents, 6, None, ctx, neg, 5.0, 5.0, 5.0, 0.875)
    assert torch.allclose(out, ref, atol=1e-5)  # identical experts == single model
    steps_high = int((stage.scheduler.timesteps >= 875).sum())
    assert 0 < steps_high < 6 and high.calls == 2 * steps_high and low.calls == 2 * (6 - steps_high)
    other = _moe_stage(make_tiny_model(), make_tiny_model(seed=5))
    diff = other.process(latents, 6, None, ctx, neg, 5.0, 3.0, 5.0, 0.875)
    assert not torch.allclose(diff, ref, atol=1e-3)
    full, payload = other.process(latents, 6, None, ctx, neg, 5.0, 3.0, 5.0, 0.875, latent_data={"saved_steps": [3]})
    assert torch.equal(full, diff) and payload["final_step"] == 5 and list(payload["latent_states_dict"]) == [3]
    resumed, _ = other.process(torch.zeros_like(latents), 6, None, ctx, neg, 5.0, 3.0, 5.0, 0.875,
                               latent_data={"cached_latent": payload["latent_states_dict"][3], "skip_step": 3})  # fmt: skip
    assert torch.allclose(resumed, full, atol=1e-6)


def test_ti2v_keeps_the_reference_frame_and_marks_it_clean():
    mask = torch.ones(16, 3, 8, 8)
    mask[:, 0] = 0
    ts = per_token_timestep(torch.tensor([700.0]), mask)
    assert ts.shape == (1, 3 * 4 * 4) and ts[0, :16].abs().max() == 0 and (ts[0, 16:] == 700).all()
    latents, ctx, neg = make_tiny_inputs()
    cfg = ModelRuntimeConfig(torch_dtype=torch.float32, device_type="cpu")
    pmesh.set_mesh(None)
    stage = TI2VDenoisingStage("denoise", None, cfg, FlowMatchScheduler("Wan"), dit=make_tiny_model())
    stage.mesh = pmesh.get_mesh()
    stage.onload_models_flag = True
    ref = torch.randn(16, 1, 8, 8)
    out = stage.process(latents, 4, ref, 9, ctx, neg, 5.0, 5.0)
    assert out.shape == latents.shape and torch.equal(out[0, :, :1], ref) and torch.isfinite(out).all()
    end = torch.randn(16, 1, 8, 8)
    both = stage.process(latents, 4, (ref, end), 9, ctx, neg, 5.0, 5.0)
    assert torch.equal(both[0, :, :1], ref) and torch.equal(both[0, :, -1:], end)
    plain = stage.process(latents, 4, None, None, ctx, neg, 5.0, 5.0)
    assert torch.allclose(plain, tiny_wan_denoise(steps=4), atol=1e-5)


def test_async_pipeline_emits_stage_events(tmp_path):
    import asyncio

    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.wan.async_wan22_video import AsyncWan22VideoPipeline, AsyncWan22VideoPipelineConfig

    torch.manual_seed(0)
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(make_tiny_model(), "wan_video_dit")
    mm.add_module(make_tiny_model(seed=3), "wan_video_dit")
    mm.add_module(WanVideoVAE(z_dim=16, dim=8).eval(), "wan_video_vae")
    rc = lambda: ModelRuntimeConfig(torch_dtype=torch.float32, device_type="cpu")  # noqa: E731

    class Text:
        def process(self, prompts):
            return [torch.randn(1, 8, 256) for _ in prompts]

    pipe = AsyncWan22VideoPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, AsyncWan22VideoPipelineConfig(vae_config=rc(), dit_high_config=rc(), dit_low_config=rc(), text_encoding_config=rc(),
                                                name="unit", output_root=str(tmp_path)), text_stage=Text())  # fmt: skip

    async def run(**kw):
        events = []
        async for e in pipe.agenerate(request_id="r1", prompt="x", height=64, width=64, num_frames=5, num_inference_steps=2,
                                      file_ext=".frames", **kw):  # fmt: skip
            events.append(e)
        await pipe.astop()
        return events

    events = asyncio.run(run())
    assert [e["type"] for e in events] == ["stage_end"] * 5 + ["final"]
    assert [e["stage"]["name"] for e in events[:5]] == ["text_encoding", "vae_encode", "denoise", "vae_decode", "artifact_save"]
    assert all(e["v"] == "teleai.v2.event.v1" and e["seq"] == i + 1 for i, e in enumerate(events))
    art = events[-1]["payload"]["artifacts"][0]
    assert art["num_frames"] == 5 and art["height"] == 64 and events[-1]["payload"]["params_snapshot"]["num_frames"] == 5
    bad = asyncio.run(run(cfg_scale_high="not a number"))
    assert bad[-1]["type"] == "error" and bad[-1]["error"]["stage"]["name"] in ("text_encoding", "denoise")
