"""LingBot-World streaming pipeline on CPU with tiny random-init models: chunks flow through the
encode -> denoise -> decode actor graph in order, the rolling cache evicts, sessions are isolated."""
import pytest
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


def test_interactive_service_session():
    import asyncio

    import numpy as np

    from telefuser_b200.pipelines.lingbot_world.service import (LingBotWorldFastService, LingBotWorldFastSessionConfig,
                                                                  frame_num_for_duration, keys_from_chunk, load_image,
                                                                  overlay_control_hud)

    assert frame_num_for_duration(1.0, 16, 2) == 13 and frame_num_for_duration(0.1, 16, 2) == 5 and frame_num_for_duration(2.0, 16, 3) == 33
    assert keys_from_chunk({"keys": ["W", "x", "j"]}) == {"w", "j"} and keys_from_chunk({"directions": ["left", "nope"]}) == {"a"}
    assert keys_from_chunk({"type": "ping"}) is None
    hud = overlay_control_hud(np.zeros((2, 48, 64, 3), np.uint8), ["w"])
    assert hud.max() == 255 and (hud == 40).any() and hud.shape == (2, 48, 64, 3)
    import pytest
    with pytest.raises(ValueError):
        load_image({"image_data_url": "http://x"})
    pipe = tiny_pipeline()
    svc = LingBotWorldFastService(pipe, LingBotWorldFastSessionConfig(height=32, width=32, fps=16, max_duration_seconds=2.0, hud=True))
    svc.start()
    emb, img = torch.randn(1, 8, 32), torch.rand(3, 32, 32) * 2 - 1
    sid = svc.create_session({"image": img, "prompt_emb": emb, "seed": 1})
    assert svc.has_session(sid)
    svc.push_chunk(sid, {"type": "key_down", "key": "w"})
    svc.push_chunk(sid, {"keys": ["w", "l"]})

    async def collect():
        return [m async for m in svc.pull_chunks(sid)]

    msgs = asyncio.run(collect())
    kinds = [m["type"] for m in msgs]
    assert kinds[0] == "status" and kinds[-1] == "done" and kinds.count("frames") == 4  # 2 s at 16 fps -> 29 frames -> 4 chunks
    frames = [m for m in msgs if m["type"] == "frames"]
    assert [m["chunk_index"] for m in frames] == [0, 1, 2, 3] and frames[0]["frames"].shape == (5, 32, 32, 3) and frames[1]["frames"].shape == (8, 32, 32, 3)
    assert frames[0]["frames"].dtype == np.uint8 and msgs[-1]["chunks"] == 4 and not msgs[-1]["cancelled"]
    # progress travels with every chunk; the final message carries the session's measurement snapshot
    assert frames[-1]["progress"]["completed_chunks"] == 4 and frames[-1]["progress"]["total_chunks"] == 4
    assert frames[-1]["progress"]["generated_frames"] == frames[-1]["progress"]["target_frames"] == 29
    assert frames[0]["progress"]["generated_frames"] == 5 and frames[-1]["progress"]["generated_duration_s"] == 1.75
    snap = msgs[-1]["metrics"]["session"]
    assert snap["chunks_emitted"] == 4 and snap["controls_received"] == 2 and snap["first_chunk_s"] >= snap["worker_start_s"] >= 0
    assert snap["output_queue_high_watermark"] >= 1 and "control_to_output_p50_s" in snap
    svc.close_session(sid)
    assert not svc.has_session(sid)
    # control revisions: acknowledged at once, newest snapshot wins, the applied revision is reported with the chunk,
    # and with `benchmark_metrics` a status message with the snapshot follows every chunk
    sid3 = svc.create_session({"image": img, "prompt_emb": emb, "seed": 1, "benchmark_metrics": True})
    for rev, keys in ((1, ["w"]), (2, ["a"]), (3, ["d"])):
        svc.push_chunk(sid3, {"keys": keys, "revision": rev})
    svc.push_chunk(sid3, {"poses": random_walk_trajectory(2, seed=1), "relative": True})
    svc.push_chunk(sid3, {"poses": random_walk_trajectory(2, seed=2), "relative": True, "revision": 4})  # replaces the first
    msgs3 = svc.drain(sid3, timeout=120.0)
    acks = [m["revision"] for m in msgs3 if m["type"] == "control_ack"]
    assert acks == [1, 2, 3, 4]
    fr3 = [m for m in msgs3 if m["type"] == "frames"]
    assert len(fr3) == 4 and fr3[-1]["control_revision"] == 4
    stat3 = [m for m in msgs3 if m["type"] == "status" and m.get("stage") == "chunk"]
    assert len(stat3) == 4 and stat3[-1]["metrics"]["chunks_emitted"] == 4
    m3 = svc.session_metrics(sid3)
    assert m3["explicit_controls_overwritten"] == 1 and m3["control_revision_received"] == 4 and m3["controls_received"] == 5
    assert m3["controls_superseded"] >= 1  # of three snapshots pushed back to back at most two could each steer a chunk
    svc.close_session(sid3)
    # explicit pose chunks and an early stop
    poses = random_walk_trajectory(2, seed=3)
    sid2 = svc.create_session({"image": img, "prompt_emb": emb, "seed": 1, "max_duration_seconds": 3.0, "hud": False,
                               "controls": [{"poses": poses, "relative": True}]})
    first = None
    for _ in range(2000):
        got = svc.drain(sid2, timeout=0.05)
        first = next((m for m in got if m["type"] == "frames"), first)
        if first is not None:
            break
    assert first is not None and first["controls"] is None
    svc.push_chunk(sid2, {"type": "stop"})
    tail = svc.drain(sid2, timeout=30.0)
    assert tail[-1]["type"] == "done" and tail[-1]["cancelled"]
    svc.stop()
    pipe.close()


def test_denoising_session_snapshot_resumes_with_identical_chunks():
    """Two chunks, snapshot, two more chunks; a fresh stage restored from the snapshot produces the same last two
    chunks (K/V history, both generators and the chunk counter are carried over)."""
    import pickle

    pipe = tiny_pipeline()
    stage = pipe.denoise_stage
    emb = torch.randn(1, 8, 32)
    g = torch.Generator().manual_seed(0)
    conds = [torch.randn(1, 20, 2, 4, 4, generator=g) for _ in range(4)]
    frame_tokens, kv = 4, 4 * 3
    init = lambda st, h: st.initialize_cache(h, 1, kv, 8, 10.0, 11, 12, (1, 16, 2, 4, 4), (0, 500), frame_tokens)  # noqa: E731
    step = lambda st, h, i: st.denoise_and_update_cache(h, conds[i], emb, None, i * 2 * frame_tokens, kv)  # noqa: E731
    init(stage, 1)
    first = [step(stage, 1, i) for i in range(2)]
    snap = pickle.loads(pickle.dumps(stage.snapshot_cache(1)))  # what a worker restart would ship
    assert snap["chunks_done"] == 2 and snap["model_cache"]["kv"][0]["local_end"] > 0
    want = [step(stage, 1, i) for i in (2, 3)]

    other = tiny_pipeline().denoise_stage  # same seed: same weights
    init(other, 7)
    assert other.restore_cache(7, snap)
    got = [step(other, 7, i) for i in (2, 3)]
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert other._state(7).chunks_done == 4 and torch.isfinite(first[0]).all()
    bad = dict(snap, noise_shape=[1, 16, 2, 8, 8])
    with pytest.raises(ValueError, match="another resolution"):
        other.restore_cache(7, bad)
    pipe.close()


def test_rolling_cache_against_a_list_model_over_random_chunk_streams():
    """Chunks of random length, each written one to three times (the denoising steps and the clean commit of one chunk
    land on the same slot), against a plain list model: the sink tokens stay, the oldest of the rest leave first, a
    re-run overwrites in place, and the window view is the newest `max_attention_size` entries."""
    import random

    for seed in range(8):
        rng = random.Random(seed)
        n = rng.choice([2, 3, 4])
        sink = rng.choice([0, n, 2 * n])
        cap = sink + n * rng.choice([2, 3, 4])
        cache = RollingKVCache(1, cap, 1, 2, "cpu", torch.float32, sink_tokens=sink)
        model: list[tuple[int, int]] = []  # (absolute position, version written)
        for chunk in range(rng.randrange(6, 14)):
            start = chunk * n
            for version in range(rng.randrange(1, 4)):
                k = torch.tensor([[[[float(start + i), float(version)]] for i in range(n)]])  # [1, n, 1, 2]
                end = cache.append(k, -k, start)
                if version == 0:  # a new chunk: make room among the non-sink entries, then append
                    overflow = len(model) + n - cap
                    if overflow > 0:
                        del model[sink : sink + overflow]
                    model.extend((start + i, 0) for i in range(n))
                else:  # a re-run of the newest chunk overwrites it
                    model[-n:] = [(start + i, version) for i in range(n)]
                assert end == len(model) == cache.local_end and cache.global_end == start + n
                want = torch.tensor([[p, ver] for p, ver in model], dtype=torch.float32)
                assert torch.equal(cache.k[0, :end, 0], want) and torch.equal(cache.v[0, :end, 0], -want), (seed, chunk, version)
                win = rng.randrange(1, cap + 1)
                wk, wv = cache.window(win)
                assert torch.equal(wk[0, :, 0], want[-win:]) and torch.equal(wv, -wk)
        assert [p for p, _ in model[:sink]] == list(range(sink))  # the first tokens ever written are still pinned
