"""Z-Image DiT and pipeline, the discrete flow-matching and LCM schedulers."""

import math

import pytest
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.autoencoder_kl import AutoencoderKL, AutoencoderKLConfig
from telefuser_b200.models.z_image_dit import ZImageTransformer2DModel
from telefuser_b200.pipelines.z_image import ZImagePipeline, ZImagePipelineConfig, guided_prediction, tiled_decode
from telefuser_b200.schedulers.flow_match_discrete import FlowMatchDiscreteScheduler, linear_mu
from telefuser_b200.schedulers.lcm import LCMScheduler


def small(dtype=torch.float32, device="cpu", head_dim=32, axes=(8, 12, 12), in_channels=16, heads=2):
    torch.manual_seed(0)
    m = ZImageTransformer2DModel(in_channels=in_channels, dim=heads * head_dim, n_layers=2, n_refiner_layers=1, n_heads=heads,
                                 n_kv_heads=heads, cap_feat_dim=24, axes_dims=axes)  # fmt: skip
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    m = m.to(dtype).to(device).eval()
    m.dtype = dtype
    return m


def test_schedulers():
    s = FlowMatchDiscreteScheduler(shift=3.0)
    s.set_timesteps(4)
    assert len(s.timesteps) == 4 and len(s.sigmas) == 5 and s.sigmas[-1] == 0
    assert math.isclose(float(s.sigmas[2]), 3 * 0.5 / (1 + 2 * 0.5), rel_tol=1e-6)
    x = torch.ones(2)
    for t in s.timesteps:
        x = s.step(torch.ones(2), t, x, return_dict=False)[0]
    assert torch.allclose(x, torch.zeros(2), atol=1e-6)  # dt sums to -1
    with pytest.raises(ValueError):
        s.step(x, 3, x)
    f = FlowMatchDiscreteScheduler(use_flux_shift=True)
    f.set_timesteps(4, n_tokens=4096)
    mu = linear_mu(4096)
    assert math.isclose(mu, 1.15, rel_tol=1e-6)
    assert math.isclose(float(f.sigmas[2]), math.exp(mu) / (math.exp(mu) + 1), rel_tol=1e-6)
    f.set_timesteps_mu(5, 0.8)
    assert len(f.timesteps) == 5 and f.sigmas[0] == 1 and f.sigmas[4] == 0 and f.sigmas[5] == 0
    l = LCMScheduler(1000, 5.0)
    l.set_timesteps(4, "cpu", seed=3)
    assert l.denoising_step_list == [1000, 750, 500, 250] and math.isclose(float(l.sigmas[0]), 1.0)
    assert math.isclose(float(l.sigmas[2]), 5 * 0.5 / (1 + 4 * 0.5), rel_tol=1e-5)
    last = l.step(torch.ones(3), l.timesteps[3], torch.full((3,), 2.0))
    assert torch.allclose(last, torch.full((3,), 2.0 - float(l.sigmas[3])))
    assert l.step(torch.ones(3), l.timesteps[0], torch.ones(3)).shape == (3,)


def test_model_keys_lists_and_batches():
    m = small()
    keys = set(m.state_dict())
    for k in ("all_x_embedder.2-1.weight", "all_final_layer.2-1.adaLN_modulation.1.bias", "noise_refiner.0.adaLN_modulation.0.weight",
              "context_refiner.0.attention.to_out.0.weight", "layers.1.feed_forward.w3.weight", "layers.0.attention.norm_k.weight",
              "t_embedder.mlp.2.bias", "cap_embedder.0.weight", "cap_embedder.1.bias", "x_pad_token", "cap_pad_token",
              "layers.0.ffn_norm2.weight"):  # fmt: skip
        assert k in keys, k
    assert "context_refiner.0.adaLN_modulation.0.weight" not in keys
    with torch.device("meta"):
        full = ZImageTransformer2DModel(n_layers=1)
    assert full.state_dict()["layers.0.feed_forward.w1.weight"].shape == (10240, 3840)
    x = [torch.randn(16, 1, 6, 10), torch.randn(16, 1, 8, 8)]
    caps = [torch.randn(7, 24), torch.randn(40, 24)]
    t = torch.tensor([0.3, 0.3])
    out = m(x, t, caps)
    assert [o.shape for o in out] == [v.shape for v in x]
    alone = m(x[1:], t[1:], caps[1:])[0]
    assert (out[1] - alone).abs().max() <= 1e-5
    same = m([x[0], 2 * x[0]], t, [caps[0], caps[0] + 1])  # equal sizes: one batch
    assert (same[0] - out[0]).abs().max() <= 1e-5


def test_guidance_and_pipeline():
    p, n = torch.randn(1, 4, 8, 8), torch.randn(1, 4, 8, 8)
    assert torch.allclose(guided_prediction(p, n, 2.0), p + 2 * (p - n))
    capped = guided_prediction(p, n, 5.0, normalization=1.0)
    assert torch.linalg.vector_norm(capped) <= torch.linalg.vector_norm(p) * (1 + 1e-5)
    torch.manual_seed(1)
    vae = AutoencoderKL(AutoencoderKLConfig(block_out_channels=(8, 8, 16, 16), layers_per_block=1, norm_num_groups=4)).eval()
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(small(), "zimage_dit")
    mm.add_module(vae, "z_image_vae")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = ZImagePipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, ZImagePipelineConfig(dit_config=rc(), text_encoding_config=rc(), vae_config=rc()))
    kw = dict(prompt_embeds=[torch.randn(9, 24)], negative_prompt_embeds=[torch.randn(5, 24)], cfg_scale=3.0,
              num_inference_steps=3, seed=4, height=64, width=96)  # fmt: skip
    a = pipe(output_type="pt", **kw)
    assert a.shape == (1, 3, 64, 96) and torch.isfinite(a).all() and torch.equal(a, pipe(output_type="pt", **kw))
    trunc = pipe(output_type="pt", cfg_truncation=-0.1, **kw)  # guidance off for the whole trajectory
    nocfg = pipe(output_type="pt", **{**kw, "cfg_scale": 1.0})
    assert torch.allclose(trunc, nocfg, atol=1e-5) and not torch.allclose(trunc, a, atol=1e-3)
    imgs = pipe(**kw)
    assert imgs[0].size == (96, 64)
    z = torch.randn(1, 16, 20, 24)
    assert (tiled_decode(vae, z, tile=12, overlap=4) - vae.decode(z)).abs().mean() < 0.1  # seams blend, interiors agree
    assert tiled_decode(vae, z, tile=64).shape == (1, 3, 160, 192)


@pytest.mark.gpu
def test_gpu_bf16_forward_tracks_cpu_fp32():
    ref_m = small(head_dim=128, axes=(32, 48, 48), heads=3)  # width 384: the MLP width 1024 suits the tensor-core GEMM
    x, caps, t = [torch.randn(16, 1, 32, 48)], [torch.randn(21, 24)], torch.tensor([0.4])
    ref = ref_m(x, t, caps)[0]
    gpu_m = small(torch.bfloat16, "cuda", head_dim=128, axes=(32, 48, 48), heads=3)
    got = gpu_m([x[0].cuda().bfloat16()], t.cuda(), [caps[0].cuda().bfloat16()])[0].float().cpu()
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err
