"""LingBot-World streaming pipeline on CPU with tiny random-init models: chunks flow through the
encode -> denoise -> decode actor graph in order, the rolling cache evicts, sessions are isolated."""
import torch

from telefuser_b200.cache.rolling_kv import RollingKVCache
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.lingbot_world_dit import LingBotWorldFastDiT
from telefuser_b200.models.wan_vae import WanVideoVAE
from telefuser_b200.pipelines.lingbot_world.control import (LingBotWorldFastControlBuilder,
                                                              LingBotWorldFastControlContext, integrate_keys,
                                                              pinhole_intrinsics, random_walk_trajectory)
from telefuser_b200.pipelines.lingbot_world.pipeline import LingBotWorldFastPipeline, LingBotWorldFastPipelineConfig
from telefuser_b200.testing.synthetic import random_init_


def tiny_pipeline(local_attn=3, sink=1, chunk=2):
    torch.manual_seed(0)
    dit = random_init_(LingBotWorldFastDiT(in_dim=36, dim=64, ffn_dim=128, text_dim=32, num_heads=2, num_layers=2,
                                           local_attn_size=local_attn, sink_size=sink).float())
    dit.dtype = torch.float32
    vae = random_init_(WanVideoVAE(dim=8).float(), std=0.05)
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(dit.eval(), "lingbot_world_fast_dit")
    mm.add_module(vae.eval(), "wan_video_vae")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    cfg = LingBotWorldFastPipelineConfig(dit_config=rc(), vae_encode_config=rc(), vae_decode_config=rc(),
                                         text_encoding_config=rc(), chunk_size=chunk, local_attn_size=local_attn,
                                         sink_size=sink, timestep_indices=(0, 500), max_sequence_length=8)
    pipe = LingBotWorldFastPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, cfg)
    return pipe


def test_generate_video_through_actor_graph():
    pipe = tiny_pipeline()
    emb = torch.randn(1, 8, 32)
    img = torch.rand(3, 32, 32) * 2 - 1
    seen = []
    video, metrics = pipe.generate_video("", img, num_frames=29, height=32, width=32, seed=1, prompt_emb=emb,
                                         on_chunk=lambda i, f: seen.append(i))
    assert video.shape == (1, 3, 29, 32, 32) and torch.isfinite(video).all()
    assert seen == [0, 1, 2, 3] and metrics["chunks"] == 4
    assert len(metrics["stage_busy_s"]["denoise"]) == 4
    video2, _ = pipe.generate_video("", img, num_frames=29, height=32, width=32, seed=1, prompt_emb=emb)
    assert torch.equal(video, video2)  # sessions do not leak state into each other
    pipe.close()


def test_rolling_cache_eviction_keeps_sink():
    c = RollingKVCache(1, 6, 1, 2, "cpu", torch.float32, sink_tokens=2)
    for step in range(5):
        k = torch.full((1, 2, 1, 2), float(step))
        for _ in range(2):  # same chunk written twice (denoise pass + commit pass)
            c.append(k, k, step * 2)
    kw, _ = c.window(100)
    assert kw[0, :, 0, 0].tolist() == [0.0, 0.0, 3.0, 3.0, 4.0, 4.0]
    assert c.global_end == 10 and c.local_end == 6
    kw3, _ = c.window(3)
    assert kw3.shape[1] == 3


def test_control_builder_and_key_integration():
    ctx = LingBotWorldFastControlContext("cam", "cpu", torch.float32, 32, 48, 32, 48, 4, 6, 4, 2, pinhole_intrinsics(32, 48))
    b = LingBotWorldFastControlBuilder(ctx)
    seq = b.build_sequence(random_walk_trajectory(4, seed=3), ctx.intrinsics)
    assert len(seq) == 2 and seq[0].shape == (1, 6 * 64, 2, 4, 6)
    one = b.build({"poses": integrate_keys(torch.eye(4), ["w", "l"], 2)})
    assert one.shape == (1, 384, 2, 4, 6) and torch.isfinite(one).all()
    moved = integrate_keys(torch.eye(4), ["w"], 3)
    assert moved[-1, 2, 3] > moved[0, 2, 3] > 0
