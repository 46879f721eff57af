"""FLUX.2 transformer, 2-D KL autoencoder and the klein pipeline: rope tables, checkpoint key names, batch and
reference-token handling, latent (un)packing, an end-to-end image on CPU; bf16 forward on GPUs against fp32."""

import pytest
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.autoencoder_kl import AutoencoderKL, AutoencoderKLConfig
from telefuser_b200.models.flux2_dit import Flux2DiT, Flux2DiTConfig, rope_tables
from telefuser_b200.pipelines.flux2_klein import Flux2KleinPipeline, Flux2KleinPipelineConfig
from telefuser_b200.pipelines.flux2_klein import pipeline as P


def small(dtype=torch.float32, device="cpu", head_dim=32, heads=2, text_dim=48, in_channels=128):
    torch.manual_seed(0)
    cfg = Flux2DiTConfig(in_channels=in_channels, num_layers=2, num_single_layers=2, attention_head_dim=head_dim,
                         num_attention_heads=heads, joint_attention_dim=text_dim, axes_dims_rope=(head_dim // 4,) * 4)  # fmt: skip
    m = Flux2DiT(cfg)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    m = m.to(dtype).to(device).eval()
    m.dtype = dtype
    return m


def small_vae():
    torch.manual_seed(1)
    cfg = AutoencoderKLConfig(latent_channels=32, block_out_channels=(8, 8, 16, 16), layers_per_block=1, norm_num_groups=4,
                              use_quant_conv=True, use_post_quant_conv=True, batch_norm=True)  # fmt: skip
    vae = AutoencoderKL(cfg).eval()
    vae.bn.running_mean.normal_()
    vae.bn.running_var.uniform_(0.5, 2.0)
    return vae


def test_rope_tables_and_ids():
    ids = P.latent_ids(2, 3)
    assert ids.tolist()[4] == [0, 1, 1, 0] and P.text_ids(3)[2].tolist() == [0, 0, 0, 2]
    assert P.reference_image_ids([(1, 2), (1, 1)])[:, 0].tolist() == [10, 10, 20]
    cos, sin = rope_tables(ids, (8, 8, 8, 8), 2000.0)
    assert cos.shape == (6, 16) and torch.allclose(cos**2 + sin**2, torch.ones_like(cos), atol=1e-6)
    assert torch.allclose(sin[4, :4], torch.zeros(4)) and torch.allclose(sin[4, 4], torch.sin(torch.tensor(1.0)))
    assert torch.allclose(sin[4, 9], torch.sin(torch.tensor(2000.0 ** (-2 / 8))), atol=1e-6)


def test_key_names_shapes_and_forward_variants():
    with torch.device("meta"):
        full = Flux2DiT(Flux2DiTConfig(num_layers=1, num_single_layers=1))
    sd = full.state_dict()
    assert sd["single_transformer_blocks.0.attn.to_qkv_mlp_proj.weight"].shape == (3 * 4096 + 2 * 12288, 4096)
    assert sd["single_transformer_blocks.0.attn.to_out.weight"].shape == (4096, 4096 + 12288)
    assert sd["double_stream_modulation_img.linear.weight"].shape == (6 * 4096, 4096)
    for k in ("time_guidance_embed.timestep_embedder.linear_1.weight", "context_embedder.weight", "x_embedder.weight",
              "transformer_blocks.0.attn.norm_added_k.weight", "transformer_blocks.0.attn.to_add_out.weight",
              "transformer_blocks.0.ff_context.linear_in.weight", "transformer_blocks.0.attn.to_out.0.weight",
              "single_stream_modulation.linear.weight", "norm_out.linear.weight", "proj_out.weight"):  # fmt: skip
        assert k in sd, k
    assert not any(k.endswith(".bias") for k in sd)
    conv = Flux2DiT.state_dict_converter()
    renamed, _ = conv.from_official({"double_blocks.0.x": 1, "final_layer.linear.weight": 2, "img_in.weight": 3})
    assert set(renamed) == {"transformer_blocks.0.x", "norm_out.linear.weight", "x_embedder.weight"}
    m = small(in_channels=16)
    x, e, t = torch.randn(2, 12, 16), torch.randn(2, 5, 48), torch.tensor([0.6, 0.6])
    ids, tids = P.latent_ids(3, 4), P.text_ids(5)
    both = m(x, e, t, ids, tids)
    one = m(x[1:], e[1:], t[1:], ids, tids)
    assert both.shape == (2, 12, 16) and (both[1:] - one).abs().max() <= 1e-5
    ref_tokens = torch.randn(1, 4, 16)
    ext = m(torch.cat([x[1:], ref_tokens], 1), e[1:], t[1:], torch.cat([ids, P.reference_image_ids([(2, 2)])]), tids)
    assert ext.shape == (1, 16, 16) and not torch.allclose(ext[:, :12], one, atol=1e-4)


def test_latent_packing_round_trips_and_vae_shapes():
    z = torch.randn(2, 32, 8, 12)
    p = P.patchify_latents(z)
    assert p.shape == (2, 128, 4, 6) and torch.equal(P.unpatchify_latents(p), z)
    assert p[0, 5, 1, 2] == z[0, 1, 2, 5]  # channel 1, patch offset (0, 1)
    tokens = P.pack_latents(p)
    perm = torch.randperm(24)
    assert torch.equal(P.unpack_latents_with_ids(tokens[:, perm], P.latent_ids(4, 6)[perm]), p)
    vae = small_vae()
    img = torch.rand(1, 3, 32, 48) * 2 - 1
    lat = vae.encode(img).mode()
    assert lat.shape == (1, 32, 4, 6) and vae.decode(lat).shape == img.shape and vae.spatial_factor == 8
    keys = set(vae.state_dict())
    for k in ("encoder.down_blocks.0.downsamplers.0.conv.weight", "encoder.mid_block.attentions.0.to_q.weight",
              "decoder.up_blocks.0.upsamplers.0.conv.bias", "decoder.up_blocks.2.resnets.0.conv_shortcut.weight",
              "decoder.mid_block.attentions.0.to_out.0.bias", "quant_conv.weight", "post_quant_conv.bias",
              "bn.running_mean", "encoder.conv_norm_out.weight"):  # fmt: skip
        assert k in keys, k


def test_pipeline_generates_and_edits_on_cpu():
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(small(), "flux2_dit")
    mm.add_module(small_vae(), "vae")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = Flux2KleinPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, Flux2KleinPipelineConfig(dit_config=rc(), text_encoding_config=rc(), vae_config=rc()))
    pos, neg = torch.randn(1, 6, 48), torch.randn(1, 6, 48)
    kw = dict(prompt_embeds=pos, negative_prompt_embeds=neg, cfg_scale=3.0, num_inference_steps=3, seed=2, height=64, width=96)
    a = pipe(output_type="pt", **kw)
    b = pipe(output_type="pt", **kw)
    assert a.shape == (1, 3, 64, 96) and torch.isfinite(a).all() and torch.equal(a, b)
    lat = pipe(output_type="latent", **kw)
    assert lat.shape == (1, 24, 128)
    imgs = pipe(reference_images=[torch.rand(1, 3, 32, 32) * 2 - 1], **{**kw, "cfg_scale": 1.0})
    assert len(imgs) == 1 and imgs[0].size == (96, 64)


@pytest.mark.gpu
def test_gpu_bf16_forward_tracks_cpu_fp32():
    ref_m = small(head_dim=128, in_channels=64)
    x, e, t = torch.randn(1, 24 * 24, 64), torch.randn(1, 32, 48), torch.tensor([0.7])
    ids, tids = P.latent_ids(24, 24), P.text_ids(32)
    ref = ref_m(x, e, t, ids, tids)
    gpu_m = small(torch.bfloat16, "cuda", head_dim=128, in_channels=64)
    got = gpu_m(x.cuda().bfloat16(), e.cuda().bfloat16(), t.cuda(), ids.cuda(), tids.cuda()).float().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err
