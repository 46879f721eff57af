"""LTX-2 components around the transformer and the two-stage pipeline on tiny random models."""

import pytest
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models import ltx_audio_vae as A
from telefuser_b200.models import ltx_dit as D
from telefuser_b200.models import ltx_gemma_text_encoder as G
from telefuser_b200.models import ltx_upsampler as U
from telefuser_b200.models import ltx_video_vae as V
from telefuser_b200.pipelines.ltx_video import dit_denoising as DD
from telefuser_b200.pipelines.ltx_video.pipeline import LTX23VideoPipeline, LTXVideoPipelineConfig, assert_resolution
from telefuser_b200.pipelines.ltx_video.stages import GemmaTextEncodingStage, VAEStage

ENC = (("res_x", 1), ("compress_space_res", {"multiplier": 1}), ("compress_time_res", {"multiplier": 1}), ("compress_all_res", {"multiplier": 1}),
       ("compress_all_res", {"multiplier": 1}))  # fmt: skip
DEC = (("res_x", 1), ("compress_space", {"multiplier": 2}), ("compress_time", {"multiplier": 2}), ("compress_all", {"multiplier": 2}),
       ("compress_all", {"multiplier": 1}))  # fmt: skip


def _vae(latent=128, base=16, **kw):
    torch.manual_seed(0)
    vae = V.LTXVideoVAE(latent_channels=latent, encoder_blocks=ENC, decoder_blocks=DEC, decoder_base_channels=base, **kw)
    for p in vae.parameters():
        torch.nn.init.normal_(p, std=0.05)
    return vae.float().eval()


def _dit(layers=2):
    torch.manual_seed(0)
    net = D.LTXVideoTransformer({"transformer": dict(num_attention_heads=2, attention_head_dim=16, num_layers=layers, cross_attention_dim=32,
                                                      audio_num_attention_heads=2, audio_attention_head_dim=8, audio_cross_attention_dim=16,
                                                      av_ca_timestep_scale_multiplier=1000, rope_type="split", frequencies_precision="float64",
                                                      apply_gated_attention=True, cross_attention_adaln=True,
                                                      caption_proj_before_connector=True)})  # fmt: skip
    for p in net.parameters():
        torch.nn.init.normal_(p, std=0.05)
    net.dtype = torch.float32
    return net.float().eval()


def test_video_vae_shapes_tiling_and_converter():
    vae = _vae(latent=8, base=4)
    x = torch.randn(1, 3, 17, 64, 96)
    z = vae.encode(x)
    assert z.shape == (1, 8, 3, 2, 3)
    assert vae.encode(torch.randn(1, 3, 20, 64, 64)).shape[2] == 3  # 20 frames are cropped to 17
    rec = next(vae.decode(z))
    assert rec.shape == x.shape
    # causal encoder: the first latent frame depends on the first pixel frame only
    x2 = x.clone()
    x2[:, :, 1:] += 1.0
    assert torch.allclose(vae.encode(x2)[:, :, 0], z[:, :, 0], atol=1e-5)
    # a window that covers everything gives one tile equal to the plain decode; smaller windows stream the same frame count
    whole = torch.cat(list(vae.decode(z, tiled=True, tile_size=(64, 512), tile_stride=(40, 448))), dim=2)
    assert torch.allclose(whole, rec, atol=1e-5)
    zl = torch.randn(1, 8, 7, 4, 6)
    chunks = list(vae.decode(zl, tiled=True, tile_size=(32, 64), tile_stride=(16, 32)))
    assert len(chunks) > 1 and sum(c.shape[2] for c in chunks) == 49 and chunks[0].shape[-2:] == (128, 192)
    assert V.get_video_chunks_number(49, True, (32, 64), (16, 32)) == 3 and V.get_video_chunks_number(49) == 1
    with pytest.raises(ValueError):
        list(vae.decode(zl, tiled=True, tile_size=(32, 48), tile_stride=(16, 32)))
    sd = {"vae.encoder." + k: v for k, v in vae.encoder.state_dict().items() if "per_channel" not in k}
    sd.update({"vae.decoder." + k: v for k, v in vae.decoder.state_dict().items() if "per_channel" not in k})
    sd.update({"vae.per_channel_statistics.std-of-means": torch.ones(8), "vae.per_channel_statistics.mean-of-means": torch.zeros(8),
               "model.diffusion_model.x": torch.zeros(1)})  # fmt: skip
    conv, _ = vae.state_dict_converter().from_official(sd)
    assert set(conv) == set(vae.state_dict())


def test_tile_planning():
    iv = V.split_with_symmetric_overlaps(4, 1)(10)
    assert iv.starts == [0, 3, 6] and iv.ends == [4, 7, 10] and iv.left_ramps == [0, 1, 1] and iv.right_ramps == [1, 1, 0]
    tl = V.split_temporal_latents(4, 1)(10)
    assert tl.starts == [0, 2, 5] and tl.left_ramps == [0, 2, 2]
    tf = V.split_temporal_frames(32, 16)(49)
    assert tf.ends == [33, 49, 49] and tf.right_ramps == [0, 0, 0]
    sl, mask = V.map_temporal_interval_to_frame(2, 6, 2, 1, 8)
    assert (sl.start, sl.stop) == (16, 41) and mask.shape == (25,) and mask[0] == 0 and mask[9] == 1 and 0 < mask[-1] < 1
    m = V.compute_trapezoidal_mask_1d(8, 2, 2)
    assert torch.allclose(m, torch.tensor([1 / 3, 2 / 3, 1, 1, 1, 1, 2 / 3, 1 / 3]))
    tiles = V.create_tiles((1, 8, 7, 4, 6), [None, None, V.split_temporal_latents(4, 2), None, V.split_with_symmetric_overlaps(4, 1)],
                           [None, None, (V.map_temporal_interval_to_frame, 8), None, (V.map_spatial_interval_to_pixel, 32)])  # fmt: skip
    assert len(tiles) == 6 and tiles[0].blend_mask.shape == (1, 1, 25, 1, 128)


def test_upsampler_and_audio():
    up = U.LTXSpatialUpsampler(in_channels=8, mid_channels=32, num_blocks_per_stage=1).float().eval()
    z = torch.randn(1, 8, 3, 4, 6)
    assert up(z).shape == (1, 8, 3, 8, 12)
    vae = _vae(latent=8, base=4)
    vae.encoder.per_channel_statistics.get_buffer("std-of-means").fill_(2.0)
    out = U.upsample_video(z, vae.encoder, up)
    assert torch.allclose(out, up(z * 2.0) / 2.0, atol=1e-5)
    assert U.LatentUpsamplerConfigurator.from_config({"in_channels": 8, "mid_channels": 32, "rational_resampler": True, "spatial_scale": 1.5})(z).shape[-2:] == (6, 9)
    dec = A.AudioDecoder(ch=16, out_ch=2, ch_mult=(1, 2, 4), num_res_blocks=1, attn_resolutions={8}, resolution=16, z_channels=8, mel_bins=64)
    dec.per_channel_statistics = A.PerChannelStatistics(128)
    dec = dec.float().eval()
    za = torch.randn(1, 8, 5, 16)
    mel = dec(za)
    assert mel.shape == (1, 2, 17, 64)
    # without the attention blocks the decoder is causal along time: earlier mel frames do not change
    cdec = A.AudioDecoder(ch=16, out_ch=2, ch_mult=(1, 2, 4), num_res_blocks=1, attn_resolutions=set(), mid_block_add_attention=False,
                          resolution=16, z_channels=8, mel_bins=64)  # fmt: skip
    cdec.per_channel_statistics = A.PerChannelStatistics(128)
    cdec = cdec.float().eval()
    za2 = za.clone()
    za2[:, :, 3:] += 1.0
    assert torch.allclose(cdec(za2)[:, :, :9], cdec(za)[:, :, :9], atol=1e-5) and not torch.allclose(cdec(za2)[:, :, 9:], cdec(za)[:, :, 9:], atol=1e-3)
    cfg = {"vocoder": {"vocoder": {"upsample_rates": [4, 2], "upsample_kernel_sizes": [8, 4], "upsample_initial_channel": 32,
                                   "resblock_kernel_sizes": [3], "resblock_dilation_sizes": [[1, 3, 5]]},
                       "bwe": {"upsample_rates": [8, 4], "upsample_kernel_sizes": [16, 8], "upsample_initial_channel": 32, "resblock_kernel_sizes": [3],
                               "resblock_dilation_sizes": [[1, 3, 5]], "n_fft": 64, "hop_length": 16, "num_mels": 64}}}  # fmt: skip
    voc = A.VocoderConfigurator.from_config(cfg).float().eval()
    assert isinstance(voc, A.VocoderWithBWE) and voc.vocoder.is_amp and voc(mel).shape == (1, 2, 17 * 8 * 2)
    plain = A.VocoderConfigurator.from_config({"vocoder": cfg["vocoder"]["vocoder"]}).float().eval()
    wav = plain(mel)
    assert wav.shape == (1, 2, 136) and wav.abs().max() <= 1.0
    f = A.kaiser_sinc_filter1d(0.25, 0.3, 12)
    assert abs(float(f.sum()) - 1.0) < 1e-6 and torch.allclose(f, f.flip(-1), atol=1e-7)
    d, v = A.split_audio_state_dicts({"audio_vae.decoder.conv_in.conv.weight": 1, "audio_vae.per_channel_statistics.std-of-means": 2, "vocoder.conv_pre.weight": 3, "x": 4})
    assert set(d) == {"conv_in.conv.weight", "per_channel_statistics.std-of-means"} and set(v) == {"conv_pre.weight"}


def test_text_embeddings_processor():
    torch.manual_seed(0)
    tc = {"transformer": dict(num_attention_heads=2, attention_head_dim=16, audio_num_attention_heads=2, audio_attention_head_dim=8,
                              connector_num_attention_heads=2, connector_attention_head_dim=16, audio_connector_num_attention_heads=2,
                              audio_connector_attention_head_dim=8, connector_num_layers=1, rope_type="split", frequencies_precision="float64",
                              connector_apply_gated_attention=True, caption_proj_before_connector=True, caption_projection_first_linear=False,
                              caption_proj_input_norm=False, caption_projection_second_linear=False)}  # fmt: skip
    proc = G.LTXEmbeddingsProcessor(tc, embedding_dim=12, num_layers=4).float().eval()
    assert isinstance(proc.feature_extractor, G.FeatureExtractorV2) and proc.audio_connector.inner_dim == 16
    hs = tuple(torch.randn(2, 128, 12) for _ in range(4))
    mask = torch.zeros(2, 128, dtype=torch.long)
    mask[0, 100:] = 1
    mask[1, 64:] = 1
    out = proc.process_hidden_states(hs, mask, "left")
    assert out.video_encoding.shape == (2, 128, 32) and out.audio_encoding.shape == (2, 128, 16) and bool(out.attention_mask.all())
    regs = proc.video_connector._replace_padded_with_learnable_registers(torch.zeros(2, 128, 32), G.convert_to_additive_mask(mask, torch.float32))[0]
    assert torch.allclose(regs[0, 28:], proc.video_connector.learnable_registers[28:].float()) and bool((regs[0, :28] == 0).all())
    assert isinstance(G._create_feature_extractor({}, 12, 4), G.FeatureExtractorV1)
    with pytest.raises(NotImplementedError):
        G._create_feature_extractor({"caption_proj_before_connector": True}, 12, 4)
    sd, _ = proc.state_dict_converter().from_official({"model.diffusion_model.video_embeddings_connector.learnable_registers": 1,
                                                       "text_embedding_projection.video_aggregate_embed.weight": 2, "vae.x": 3})  # fmt: skip
    assert set(sd) == {"video_connector.learnable_registers", "feature_extractor.video_aggregate_embed.weight"}
    conv, _ = G.GemmaTextEncoderStateDictConverter().from_official({"language_model.model.embed_tokens.weight": 1, "model.vision_tower.w": 2})
    assert set(conv) == {"model.model.language_model.embed_tokens.weight", "model.model.vision_tower.w", "model.lm_head.weight"}
    padded = GemmaTextEncodingStage.pad_inputs_for_attention_alignment({"input_ids": torch.ones(1, 13, dtype=torch.long), "attention_mask": torch.ones(1, 13, dtype=torch.long)})
    assert padded["input_ids"].shape == (1, 16) and int(padded["attention_mask"].sum()) == 13


def test_latent_tools_conditioning_and_guider():
    shape = DD.VideoLatentShape.from_pixels(1, 17, 64, 96)
    assert tuple(shape) == (1, 128, 3, 2, 3) and DD.AudioLatentShape.from_duration(1, 121 / 24).frames == 126
    tools = DD.VideoLatentTools(DD.VideoLatentPatchifier(1), shape, fps=24.0)
    s = tools.create_initial_state("cpu", torch.float32, torch.randn(*shape))
    assert s.latent.shape == (1, 18, 128) and s.positions.shape == (1, 3, 18, 2) and s.denoise_mask.shape == (1, 18, 1)
    assert torch.equal(tools.unpatchify(s).latent, tools.patchifier.unpatchify(s.latent, shape))
    # first latent frame spans pixel frame 0 only, the next one frames 1..8, in seconds
    assert torch.allclose(s.positions[0, 0, 0], torch.tensor([0.0, 1 / 24])) and torch.allclose(s.positions[0, 0, 6], torch.tensor([1 / 24, 9 / 24]))
    assert torch.allclose(s.positions[0, 1, 3], torch.tensor([32.0, 64.0]))
    ap = DD.AudioPatchifier(1).get_patch_grid_bounds(DD.AudioLatentShape(1, 8, 3, 16))
    assert torch.allclose(ap[0, 0], torch.tensor([[0.0, 0.01], [0.01, 0.05], [0.05, 0.09]]))
    cond = DD.VideoConditionByLatentIndex(torch.ones(1, 128, 1, 2, 3), strength=0.75, latent_idx=1).apply_to(s, tools)
    assert bool((cond.latent[:, 6:12] == 1).all()) and torch.allclose(cond.denoise_mask[:, 6:12], torch.tensor(0.25)) and bool((cond.denoise_mask[:, :6] == 1).all())
    with pytest.raises(DD.ConditioningError):
        DD.VideoConditionByLatentIndex(torch.ones(1, 128, 1, 3, 3), 1.0, 0).apply_to(s, tools)
    key = DD.ConditioningItemAttentionStrengthWrapper(DD.VideoConditionByKeyframeIndex(torch.ones(1, 128, 1, 2, 3), frame_idx=8, strength=1.0), 0.5)
    k = key.apply_to(s, tools)
    assert k.latent.shape[1] == 24 and k.attention_mask.shape == (1, 24, 24) and float(k.attention_mask[0, 0, 20]) == 0.5 and float(k.attention_mask[0, 20, 21]) == 1.0
    assert torch.allclose(k.positions[0, 0, 18], torch.tensor([8 / 24, 16 / 24]))
    k2 = DD.VideoConditionByKeyframeIndex(torch.ones(1, 128, 1, 2, 3), frame_idx=16, strength=1.0).apply_to(k, tools)
    assert k2.attention_mask.shape == (1, 30, 30) and float(k2.attention_mask[0, 18, 24]) == 0.0 and float(k2.attention_mask[0, 0, 24]) == 1.0
    cleared = tools.clear_conditioning(k2)
    assert cleared.latent.shape[1] == 18 and cleared.attention_mask is None
    noised = DD.GaussianNoiser(torch.full((1, 18, 128), 5.0))(cond, 0.5)
    assert torch.allclose(noised.latent[:, 6:12], torch.tensor(0.125 * 5 + 0.875)) and torch.allclose(noised.latent[:, :6], 0.5 * 5 + 0.5 * cond.latent[:, :6])
    g = DD.MultiModalGuider(DD.MultiModalGuiderParams(cfg_scale=3.0, stg_scale=1.0, modality_scale=2.0, skip_step=1))
    c, u, p, m = (torch.full((4,), v) for v in (1.0, 0.5, 0.25, 0.0))
    assert torch.allclose(g.calculate(c, u, p, m), torch.full((4,), 1 + 2 * 0.5 + 0.75 + 1.0))
    assert g.do_unconditional_generation() and g.do_perturbed_generation() and g.do_isolated_modality_generation()
    assert [g.should_skip_step(i) for i in range(4)] == [False, True, False, True]
    r = DD.MultiModalGuider(DD.MultiModalGuiderParams(cfg_scale=2.0, rescale_scale=1.0))
    cc, uu = torch.randn(100), torch.randn(100)
    assert abs(float(r.calculate(cc, uu, 0.0, 0.0).std()) - float(cc.std())) < 1e-4
    assert DD.resolve_context({"video_encoding": c, "audio_encoding": u})[1] is u and DD.resolve_context([c, u, m])[0] is c
    with pytest.raises(TypeError):
        DD.resolve_context(c)


def test_denoising_stage_guidance_and_conditioning():
    dit = _dit()
    stage = DD.DitDenoisingStage("denoise", None, ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32), dit=dit)
    stage.onload_models_flag = True
    ctx = (torch.randn(1, 8, 32), torch.randn(1, 8, 16))
    neg = (torch.randn(1, 8, 32), torch.randn(1, 8, 16))
    nv, na = torch.randn(1, 2 * 2 * 2, 128), torch.randn(1, 9, 128)
    full = DD.MultiModalGuiderParams(cfg_scale=3.0, stg_scale=1.0, stg_blocks=[1], rescale_scale=0.7, modality_scale=3.0)
    kw = dict(height=64, width=64, num_frames=9, frame_rate=24.0, positive_context=ctx, num_inference_steps=2, video_noise=nv, audio_noise=na)
    v, a = stage.process(conditionings=None, negative_context=neg, video_guider_params=full, audio_guider_params=full, **kw)
    assert v.latent.shape == (1, 128, 2, 2, 2) and a.latent.shape == (1, 8, 9, 16) and stage.forward_calls == 8
    assert bool(torch.isfinite(v.latent).all()) and bool(torch.isfinite(a.latent).all())
    off = DD.MultiModalGuiderParams()
    stage.forward_calls = 0
    v0, a0 = stage.process(conditionings=None, negative_context=None, video_guider_params=off, audio_guider_params=off, **kw)
    assert stage.forward_calls == 2
    v1, _ = stage.process(conditionings=None, negative_context=None, video_guider_params=off, audio_guider_params=off, simple_denoise=True, **kw)
    assert torch.allclose(v0.latent, v1.latent, atol=1e-5)
    # a fully clamped first frame comes back unchanged; the other frame is generated
    cond = torch.cat([torch.zeros(1, 1, 1, 2, 2), torch.full((1, 128, 1, 2, 2), 0.3)], dim=1)
    vc, _ = stage.process(conditionings=cond, negative_context=None, video_guider_params=off, audio_guider_params=off, **kw)
    assert torch.allclose(vc.latent[:, :, 0], torch.tensor(0.3), atol=1e-5) and not torch.allclose(vc.latent[:, :, 1], torch.tensor(0.3), atol=1e-2)
    # stage-2 form: fixed sigmas, start from given latents re-noised to the first sigma
    sig = DD.DitDenoisingStage.stage2_sigmas("cpu")
    stage.forward_calls = 0
    v2, a2 = stage.process(conditionings=None, negative_context=None, video_guider_params=off, audio_guider_params=off, sigmas=sig,
                           noise_scale=float(sig[0]), initial_video_latent=v0.latent, initial_audio_latent=a0.latent, simple_denoise=True, **kw)  # fmt: skip
    assert stage.forward_calls == 3 and v2.latent.shape == v0.latent.shape
    with pytest.raises(ValueError):
        stage.process(conditionings=torch.zeros(1, 5, 1, 2, 2), negative_context=None, video_guider_params=off, audio_guider_params=off, **kw)


class _TextStage:
    onload_models_flag = True

    def process(self, prompts):
        g = torch.Generator().manual_seed(len(prompts[0]))
        return [G.EmbeddingsProcessorOutput(torch.randn(1, 8, 32, generator=g), torch.randn(1, 8, 16, generator=g), torch.ones(1, 8)) for _ in prompts]


def test_two_stage_pipeline_end_to_end():
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    vae = _vae()
    mm.add_module(_dit(1), "ltx_dit")
    mm.add_module(vae, "ltx_video_vae")
    mm.add_module(U.LTXSpatialUpsampler(mid_channels=32, num_blocks_per_stage=1).float().eval(), "ltx_spatial_upsampler")
    dec = A.AudioDecoder(ch=16, out_ch=2, ch_mult=(1, 2), num_res_blocks=1, attn_resolutions=set(), resolution=16, z_channels=8, mel_bins=64)
    dec.per_channel_statistics = A.PerChannelStatistics(128)
    voc = A.Vocoder(upsample_rates=[4, 2], upsample_kernel_sizes=[8, 4], upsample_initial_channel=16, resblock_kernel_sizes=[3],
                    resblock_dilation_sizes=[[1, 3, 5]], output_sampling_rate=24000)  # fmt: skip
    pipe = LTX23VideoPipeline(device="cpu", torch_dtype=torch.float32)
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    cfg = LTXVideoPipelineConfig(vae_config=rc(), upsampler_config=rc(), dit_stage1_config=rc(), dit_stage2_config=rc(), text_encoding_config=rc())
    pipe.init(mm, cfg, text_stage=_TextStage(), audio_decoder=dec.float().eval(), vocoder=voc.float().eval())
    img = torch.rand(80, 100, 3) * 255
    frames, wav, rate = pipe("a tiny test", input_image=img, seed=3, height=128, width=128, num_frames=9, num_inference_steps=2,
                             tiled=False, video_stg_blocks=[0], audio_stg_blocks=[0])  # fmt: skip
    assert len(frames) == 9 and frames[0].size == (128, 128) and rate == 24000
    assert wav.shape == (2, (9 * 4 - 3) * 8) and bool(torch.isfinite(wav).all())
    assert pipe.stage1_denoise_stage.forward_calls == 2 and pipe.stage2_denoise_stage.forward_calls == 3  # four guidance passes per batched call
    lat_v, lat_a = pipe("a tiny test", seed=3, height=128, width=128, num_frames=9, num_inference_steps=1, video_cfg_scale=1.0,
                        audio_cfg_scale=1.0, video_stg_scale=0.0, audio_stg_scale=0.0, video_modality_scale=1.0, audio_modality_scale=1.0,
                        return_latents=True)  # fmt: skip
    assert lat_v.shape == (1, 128, 2, 4, 4) and lat_a.shape == (1, 8, 9, 16)
    with pytest.raises(ValueError):
        assert_resolution(96, 128, True)
    cond = VAEStage("vae", mm, rc())
    packed = cond.encode_image(img, 64, 64, frame_idx=8, strength=0.8)
    assert packed.shape == (1, 129, 2, 2, 2) and torch.allclose(packed[:, 0, 1], torch.tensor(0.2)) and bool((packed[:, 0, 0] == 1).all())
    assert cond.encode_image(None, 64, 64) is None and cond.encode_image(img, 64, 64, strength=0.0) is None


def test_batched_guidance_equals_sequential_passes():
    ctx = (torch.randn(1, 8, 32), torch.randn(1, 8, 16))
    neg = (torch.randn(1, 8, 32), torch.randn(1, 8, 16))
    nv, na = torch.randn(1, 8, 128), torch.randn(1, 9, 128)
    full = DD.MultiModalGuiderParams(cfg_scale=3.0, stg_scale=1.0, stg_blocks=[1], rescale_scale=0.7, modality_scale=3.0)
    kw = dict(height=64, width=64, num_frames=9, frame_rate=24.0, conditionings=None, positive_context=ctx, negative_context=neg,
              num_inference_steps=2, video_guider_params=full, audio_guider_params=full, video_noise=nv, audio_noise=na)  # fmt: skip
    outs = []
    for batched in (False, True):
        stage = DD.DitDenoisingStage("denoise", None, ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32), dit=_dit(), batched_guidance=batched)
        stage.onload_models_flag = True
        outs.append(stage.process(**kw))
        assert stage.forward_calls == (2 if batched else 8)
    (v0, a0), (v1, a1) = outs
    assert torch.allclose(v0.latent, v1.latent, atol=2e-5) and torch.allclose(a0.latent, a1.latent, atol=2e-5)
