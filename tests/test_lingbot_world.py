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
    # output size from the reference image, calibration from the client
    pipe.config.max_area = 32 * 48
    wide = torch.rand(3, 64, 96) * 2 - 1
    sid4 = svc.create_session({"image": wide, "prompt_emb": emb, "fit_image": True, "max_duration_seconds": 0.5,
                               "intrinsics": [[80.0, 80.0, 48.0, 32.0]], "intrinsics_width": 96, "intrinsics_height": 64})  # fmt: skip
    ctx4 = svc._state(sid4).generation.control_builder.context
    assert ctx4.intrinsics.tolist() == [80.0, 80.0, 48.0, 32.0] and (ctx4.orig_width, ctx4.orig_height) == (96, 64)
    msgs4 = svc.drain(sid4, timeout=120.0)
    assert msgs4[0]["height"] == 32 and msgs4[0]["width"] == 48
    assert next(m for m in msgs4 if m["type"] == "frames")["frames"].shape[1:] == (32, 48, 3)
    svc.close_session(sid4)
    # browser key names, press / release events, resets, the preview picture, the duration cap
    from telefuser_b200.pipelines.lingbot_world.service import canonical_key

    assert [canonical_key(n) for n in ("ArrowUp", "KeyA", "forward", "turn_left", "L", "PageUp", "F13")] == ["w", "a", "w", "j", "l", "e", None]
    sid5 = svc.create_session({"image": img, "prompt_emb": emb, "seed": 1, "max_duration_seconds": 20.0, "preview": True, "hud": True})
    st5 = svc._state(sid5)
    svc.push_chunk(sid5, {"key": "ArrowUp", "event": "press"})
    svc.push_chunk(sid5, {"control": "KeyL", "event": "press"})
    svc.push_chunk(sid5, {"direction": "forward", "event": "release"})
    assert st5.held_keys == {"l"}
    svc.push_chunk(sid5, {"keys": ["ArrowLeft", "KeyI", "F13"]})
    assert st5.held_keys == {"a", "i"}
    svc.push_chunk(sid5, {"type": "control_state", "controls": ["w", "KeyJ"]})  # the browser's canonical keyboard state
    assert st5.held_keys == {"w", "j"}
    svc.push_chunk(sid5, {"type": "control_state", "controls": ["w", "F13"]})  # an unknown name voids the whole message
    assert st5.held_keys == {"w", "j"}
    svc.push_chunk(sid5, {"keys": ["ArrowLeft", "KeyI"]})
    svc.push_chunk(sid5, {"poses": random_walk_trajectory(2, seed=5), "relative": True})
    svc.push_chunk(sid5, {"key": "w", "event": "hold"})  # unknown event: ignored
    assert st5.held_keys == {"a", "i"} and len(st5.explicit_chunks) <= 1
    st5.pose = torch.eye(4) * 2
    svc.push_chunk(sid5, {"type": "reset"})
    assert st5.held_keys == set() and not st5.explicit_chunks and st5.pose[0, 0] == 2  # the pose survives a control reset
    svc.push_chunk(sid5, {"key": "d", "event": "reset_pose"})
    assert torch.equal(st5.pose, torch.eye(4)) or st5.submitted > 0  # (a chunk bound in between may have moved it again)
    svc.push_chunk(sid5, {"type": "stop"})
    msgs5 = svc.drain(sid5, timeout=60.0)
    prev = [m for m in msgs5 if m["type"] == "preview"]
    assert len(prev) == 1 and prev[0]["frames"].shape == (1, 32, 32, 3) and prev[0]["frames"].dtype == np.uint8 and prev[0]["chunk_index"] == -1
    states = [m["controls"] for m in msgs5 if m["type"] == "status" and m.get("stage") == "control_state"]
    assert states[:3] == [["w"], ["l", "w"], ["l"]] and ["j", "w"] in states and states[-2:] == [[], []]
    svc.close_session(sid5)
    with pytest.raises(ValueError, match="at most 20 s"):
        svc.create_session({"image": img, "prompt_emb": emb, "max_duration_seconds": 30.0})
    # an operator who configures two-minute sessions gets two-minute sessions; an explicit limit wins over both
    assert LingBotWorldFastService(pipe, LingBotWorldFastSessionConfig(max_duration_seconds=120.0)).max_generation_seconds == 120.0
    assert LingBotWorldFastService(pipe, LingBotWorldFastSessionConfig(max_duration_seconds=120.0), max_generation_seconds=60).max_generation_seconds == 60.0
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


def test_frame_count_rule_and_session_record():
    from telefuser_b200.pipelines.lingbot_world.session import LingBotWorldFastSessionConfig, resolve_lingbot_frame_count

    assert resolve_lingbot_frame_count(81, 3) == (81, 21)  # 21 latent frames = 7 whole chunks
    assert resolve_lingbot_frame_count(81, 4, "truncate") == (77, 20)  # 21 -> 20 latent frames
    assert resolve_lingbot_frame_count(77, 4, "strict") == (77, 20)
    for args, msg in (((81, 4, "strict"), "whole number of chunks"), ((5, 3, "truncate"), "shorter than the first chunk"),
                      ((80, 3, "truncate"), "4n\\+1"), ((81, 0, "truncate"), "positive integer"), ((81, True, "strict"), "positive integer"),
                      ((81.0, 3, "strict"), "must be an integer"), ((81, 3, "round"), "frame_policy")):  # fmt: skip
        with pytest.raises(ValueError, match=msg):
            resolve_lingbot_frame_count(*args)
    img = torch.zeros(3, 32, 32)
    cfg = LingBotWorldFastSessionConfig("p", img, chunk_size=4, frame_num=81).validate("cam")
    assert cfg.frame_num == 77
    with pytest.raises(ValueError, match="control mode 'act'"):
        LingBotWorldFastSessionConfig("p", img, control_mode="act").validate("cam")
    with pytest.raises(ValueError, match="both or neither"):
        LingBotWorldFastSessionConfig("p", img, intrinsics=[1, 1, 1, 1], intrinsics_width=10).validate()
    with pytest.raises(ValueError, match="nothing to apply to"):
        LingBotWorldFastSessionConfig("p", img, intrinsics_width=10, intrinsics_height=10).validate()
    with pytest.raises(ValueError, match="positive integer"):
        LingBotWorldFastSessionConfig("p", img, intrinsics=[1, 1, 1, 1], intrinsics_width=0, intrinsics_height=10).validate()


def test_pose_resampling_and_recorded_windows():
    import numpy as np

    from telefuser_b200.pipelines.lingbot_world import control as C

    def rot_y(a):
        return np.array([[np.cos(a), 0, np.sin(a)], [0, 1, 0], [-np.sin(a), 0, np.cos(a)]])

    src = np.array([0.0, 4.0, 8.0])
    rots = np.stack([rot_y(0.0), rot_y(1.0), rot_y(3.0)])  # 0 -> 1 rad -> 3 rad about y
    trans = np.array([[0.0, 0, 0], [4.0, 0, 0], [4.0, 8, 0]])
    out = C.interpolate_camera_poses(src, rots, trans, np.arange(-1, 11))
    assert out.shape == (12, 4, 4) and out.dtype == torch.float32 and (out[:, 3] == torch.tensor([0.0, 0, 0, 1])).all()
    for frame, angle in ((2, 0.5), (4, 1.0), (6, 2.0), (8, 3.0)):  # constant angular speed inside each segment
        assert torch.allclose(out[frame + 1, :3, :3], torch.from_numpy(rot_y(angle)).float(), atol=1e-6)
    assert torch.allclose(out[0, :3, :3], torch.eye(3), atol=1e-6)  # rotation is held outside the key frames ...
    assert torch.allclose(out[:, :3, 3][0], torch.tensor([-1.0, 0, 0]), atol=1e-6)  # ... translation is extrapolated
    assert torch.allclose(out[:, :3, 3][11], torch.tensor([4.0, 12, 0]), atol=1e-6)
    det = torch.linalg.det(out[:, :3, :3].double())
    assert torch.allclose(det, torch.ones_like(det), atol=1e-6)
    with pytest.raises(ValueError, match="strictly ascending"):
        C.interpolate_camera_poses([0, 0, 1], rots, trans, [0])

    poses, ks, act = np.zeros((40, 4, 4)), np.arange(12.0).reshape(3, 4), np.ones((40, 4))
    p, k, a = C.truncate_control_sequence(poses, ks, act, 29)
    assert p.shape[0] == 29 and a.shape[0] == 29 and k.tolist() == [0.0, 1.0, 2.0, 3.0]  # the first row is the calibration
    assert C.truncate_control_sequence(poses, ks[1], None, 29)[1].tolist() == [4.0, 5.0, 6.0, 7.0]
    for args, msg in (((poses, ks, act, 41), "pose recording has 40"), ((poses, ks, act[:10], 29), "action recording has 10"),
                      ((poses, np.zeros((0, 4)), None, 29), "intrinsics are"), ((poses, np.zeros(3), None, 29), "intrinsics are"),
                      ((poses, ks, None, 30), "4n\\+1")):  # fmt: skip
        with pytest.raises(ValueError, match=msg):
            C.truncate_control_sequence(*args)


def test_recorded_trajectory_drives_a_session_from_files(tmp_path):
    import numpy as np

    from telefuser_b200.pipelines.lingbot_world.control import random_walk_trajectory
    from telefuser_b200.pipelines.lingbot_world.session import LingBotWorldFastSessionConfig

    pipe = tiny_pipeline()
    assert pipe.best_output_size(832, 480, 480 * 832) == (832, 464)  # floating-point floor: the published 480p runs are 832 x 464
    assert pipe.best_output_size(1000, 1000, 480 * 832) == (624, 624)
    pipe.config.max_area = 32 * 32
    img = torch.rand(3, 64, 64) * 2 - 1
    record = LingBotWorldFastSessionConfig("", img, chunk_size=2, frame_num=33, seed=1)  # 9 latent frames -> 8 -> 29 frames
    ctx = pipe.control_context(record)
    assert record.frame_num == 29 and (ctx.height, ctx.width, ctx.latent_frames, ctx.chunk_size) == (32, 32, 8, 2)
    assert ctx.intrinsics.tolist() == [64.0, 64.0, 32.0, 32.0] and (ctx.orig_width, ctx.orig_height) == (64, 64)
    given = LingBotWorldFastSessionConfig("", img, chunk_size=2, frame_num=29, intrinsics=[[50.0, 50, 20, 20], [1, 1, 1, 1]])
    assert pipe.control_context(given).intrinsics.tolist() == [50.0, 50.0, 20.0, 20.0]
    assert (pipe.control_context(given).orig_width, pipe.control_context(given).orig_height) == (832, 480)  # configured calibration size
    with pytest.raises(ValueError, match="control mode"):
        pipe.control_context(LingBotWorldFastSessionConfig("", img, control_mode="act", chunk_size=2, frame_num=29))

    video_rate = random_walk_trajectory(40, seed=3).numpy()
    np.save(tmp_path / "poses.npy", video_rate)
    np.save(tmp_path / "intrinsics.npy", np.array([[40.0, 40.0, 32.0, 32.0]] * 40))
    with pytest.raises(ValueError, match="both or neither"):
        pipe.prepare_offline_controls(record, tmp_path, tmp_path / "intrinsics.npy", intrinsics_width=64)
    controls = pipe.prepare_offline_controls(record, tmp_path, tmp_path / "intrinsics.npy", intrinsics_width=64, intrinsics_height=64)
    assert len(controls) == 4 and all(callable(c) for c in controls)
    source = controls[0].source
    assert all(c.source is source for c in controls)
    assert source.materialize_count == 0  # nothing is converted until a chunk asks
    first = controls[0]()
    assert first.shape == (1, 6 * 64, 2, 4, 4) and source.materialize_count == 1 and controls[3]().shape == first.shape
    assert source.materialize_count == 1
    emb = torch.randn(1, 8, 32)
    video, metrics = pipe.generate_video("", img, prompt_emb=emb, controls=controls, session_config=record)
    assert video.shape == (1, 3, 29, 32, 32) and torch.isfinite(video).all() and metrics["chunks"] == 4
    # the same trajectory given as latent-rate poses with the same calibration produces the same video
    rt, ctx2 = pipe.create_session(LingBotWorldFastSessionConfig("", img, chunk_size=2, frame_num=29, seed=1, intrinsics=[40.0, 40, 32, 32],
                                                                 intrinsics_width=64, intrinsics_height=64), emb)  # fmt: skip
    pipe.validate_control(rt, first)
    with pytest.raises(ValueError, match="this session takes"):
        pipe.validate_control(rt, first[:, :6])
    direct = rt.control_builder.build_sequence(video_rate[:29], ctx2.intrinsics)
    assert all(torch.allclose(d, c(), atol=1e-6) for d, c in zip(direct, controls))
    pipe.denoise_stage.release_cache(rt.cache_handle)
    with pytest.raises(ValueError, match="controls were given"):
        pipe.generate_video("", img, prompt_emb=emb, controls=controls[:2], session_config=record)
    v2, _ = pipe.generate_video("", img, num_frames=33, height=32, width=32, seed=1, prompt_emb=emb, controls=[c() for c in controls],
                                frame_policy="truncate")  # fmt: skip
    assert torch.equal(v2, video)
    with pytest.raises(ValueError, match="whole number of chunks"):
        pipe.generate_video("", img, num_frames=33, height=32, width=32, prompt_emb=emb)
    pipe.close()


def test_world_cache_replays_matching_chunks_and_diverges_exactly():
    from telefuser_b200.cache.world_kv import WorldKVBinding, WorldKVStore, tensor_digest, world_key

    # the store on its own: one control sequence per world, truncation on divergence, LRU by bytes
    store = WorldKVStore(max_bytes=3 * 4 * 16)
    lat = [torch.full((4, 4), float(i)) for i in range(4)]
    a = WorldKVBinding(store, "world-a")
    assert a.lookup(0, "c0") is None and a.misses == 1  # empty store; from now on this session only records
    for i in range(3):
        a.finalize(i, f"c{i}", lat[i])
    b = WorldKVBinding(store, "world-a")
    assert torch.equal(b.lookup(0, "c0"), lat[0]) and torch.equal(b.lookup(1, "c1"), lat[1]) and b.lookup(2, "other") is None
    assert b.lookup(2, "c2") is None and (b.hits, b.misses) == (2, 2)  # after a divergence nothing matches any more
    b.finalize(2, "other", lat[3])
    assert store.get("world-a").control_digests == ["c0", "c1", "other"] and torch.equal(store.get("world-a").latents[2], lat[3])
    store.record_chunk("world-a", 5, "gap", lat[0])  # not contiguous: ignored
    assert len(store.get("world-a")) == 3
    store.record_chunk("world-b", 0, "x", lat[0])  # over budget: the older world goes
    assert store.get("world-a") is None and store.stats()["worlds"] == 1 and store.stats()["evictions"] == 1
    assert tensor_digest(torch.zeros(3)) != tensor_digest(torch.zeros(3, 1)) and tensor_digest(torch.zeros(2)) != tensor_digest(torch.zeros(2).half())
    assert world_key(lat[0], lat[1], 1, h=2) == world_key(lat[0].clone(), lat[1], 1, h=2) != world_key(lat[0], lat[1], 2, h=2)

    # through the pipeline
    def run(pipe, controls, **kw):
        calls = {"n": 0}
        hook = pipe.denoise_stage.dit.register_forward_pre_hook(lambda *_: calls.__setitem__("n", calls["n"] + 1))
        video, metrics = pipe.generate_video("", img, num_frames=29, height=32, width=32, seed=1, prompt_emb=emb, controls=controls, **kw)
        hook.remove()
        return video, metrics, calls["n"]

    emb, img = torch.randn(1, 8, 32), torch.rand(3, 32, 32) * 2 - 1
    plain = tiny_pipeline()
    rt = plain._create_initialized_session("", img, 29, 32, 32, 1, emb)
    walk, other = (rt.control_builder.build_sequence(random_walk_trajectory(8, seed=s), rt.control_builder.context.intrinsics) for s in (1, 2))
    for stage in (plain.denoise_stage, plain.vae_encode_stage, plain.vae_decode_stage):
        stage.release_cache(rt.cache_handle)
    mixed = walk[:2] + other[2:]  # the same first two chunks, then another way
    cold_walk, m0, n0 = run(plain, walk)
    cold_mixed, _, _ = run(plain, mixed)
    assert n0 == 4 * 3 and "world_cache_hits" not in m0  # two denoising steps + the commit pass per chunk
    plain.close()

    pipe = tiny_pipeline()
    pipe.world_store = WorldKVStore(1 << 20)
    first, m1, n1 = run(pipe, walk)
    assert torch.equal(first, cold_walk) and (m1["world_cache_hits"], m1["world_cache_misses"], n1) == (0, 4, 12)
    again, m2, n2 = run(pipe, walk)
    assert torch.equal(again, cold_walk) and (m2["world_cache_hits"], n2) == (4, 4)  # one forward (the commit) per chunk
    forked, m3, n3 = run(pipe, mixed)
    assert (m3["world_cache_hits"], m3["world_cache_misses"], n3) == (2, 2, 2 * 1 + 2 * 3)
    assert torch.equal(forked, cold_mixed)  # the replayed prefix left cache and generators exactly as a cold run does
    _, m4, _ = run(pipe, mixed)
    assert m4["world_cache_hits"] == 4  # the record now follows the newer path ...
    _, m5, _ = run(pipe, walk)
    assert m5["world_cache_hits"] == 2  # ... so the older one matches only up to the fork
    other_seed, m7 = pipe.generate_video("", img, num_frames=29, height=32, width=32, seed=2, prompt_emb=emb, controls=walk)
    assert m7["world_cache_hits"] == 0 and not torch.equal(other_seed, cold_walk)
    assert pipe.world_store.stats()["worlds"] == 2
    pipe.close()
