"""Serving layer on CPU: task manager, contract, security validator, files/artefacts, latent cache,
HTTP API end to end against a fake pipeline file, OpenAI-style routes, streaming over WebSocket,
replica pool with eviction, CLI validate/scan."""

import json
import textwrap
import threading
import time

import pytest
import torch
from fastapi.testclient import TestClient

from telefuser_b200.service.api import ApiServer, RateLimiter
from telefuser_b200.service.contract import apply_task_contract_defaults, validate_required_task_parameters
from telefuser_b200.service.files import ArtifactStore, FileService, MediaError, MediaType, handler_for
from telefuser_b200.service.pipeline_service import (PipelinePool, PipelineService, ServerConfig,
                                                     resolve_replica_device_ids)  # fmt: skip
from telefuser_b200.service.security import PipelineSecurityValidator, SecurityError
from telefuser_b200.service.stream_service import StreamPipelineService
from telefuser_b200.service.task_manager import QueueFullError, TaskManager, TaskStatus
from telefuser_b200.service.task_processor import LatentCache

PNG = (b"\x89PNG\r\n\x1a\n" + b"\x00" * 64)

FAKE_PIPELINE = textwrap.dedent('''
    import time
    import torch

    PIPELINE_MANIFEST = {
        "pipeline_name": "fake_t2v",
        "supported_tasks": ["t2v", "t2i"],
        "task_contracts": {
            "t2v": {"required_inputs": ["prompt"],
                    "parameters": {"num_inference_steps": {"type": "integer", "default": 4},
                                   "mode": {"type": "string", "default": "fast", "enum": ["fast", "slow"]}}},
            "t2i": {"required_inputs": ["prompt"], "media_type": "image"},
        },
    }

    class FakePipe:
        def __init__(self, parallelism):
            self.parallelism = parallelism
            self.calls = 0

    def get_pipeline(parallelism=1):
        return FakePipe(parallelism)

    def run_with_file(pipeline, prompt, output_path, seed=42, num_inference_steps=4, mode="fast", stop_event=None,
                      latent_data=None, sleep_s=0.0):
        pipeline.calls += 1
        if prompt == "boom":
            raise RuntimeError("pipeline exploded")
        t_end = time.time() + float(sleep_s)
        while time.time() < t_end:
            if stop_event is not None and stop_event.is_set():
                return None
            time.sleep(0.01)
        start = 0 if latent_data is None else latent_data["resume_step"]
        x = torch.full((4,), float(seed))
        saved = {}
        for i in range(start, num_inference_steps):
            x = x + 1
            saved[i + 1] = x.clone()
        with open(output_path, "wb") as f:
            f.write(b"\\x00\\x00\\x00\\x18ftypmp42" + f"{prompt}|{seed}|{num_inference_steps}|{mode}|{start}".encode())
        return {"output_path": output_path, "latent_payload": {"steps": saved}}
''')

FAKE_STREAM = textwrap.dedent('''
    import asyncio
    import torch

    class Bidi:
        def __init__(self):
            self.q = {}
        def start(self): pass
        def stop(self): pass
        def create_session(self, config):
            sid = config.get("session_id", "s0")
            self.q[sid] = asyncio.Queue()
            return sid
        def push_chunk(self, sid, chunk):
            self.q[sid].put_nowait(chunk)
        async def pull_chunks(self, sid):
            while True:
                c = await self.q[sid].get()
                frames = torch.zeros(2, 8, 8, 3, dtype=torch.uint8)
                out = {"frames": frames, "echo": c.get("key"), "done": c.get("key") == "end"}
                if c.get("key") == "sound":  # a chunk with half a second of stereo sound
                    out.update(audio=torch.zeros(8000, 2), audio_sample_rate=16000)
                yield out
        def close_session(self, sid):
            self.q.pop(sid, None)

    def get_service(gpu_num=1):
        return Bidi()
''')


@pytest.fixture
def ppl_file(tmp_path):
    p = tmp_path / "fake_pipeline.py"
    p.write_text(FAKE_PIPELINE)
    return str(p)


def make_api(tmp_path, ppl_file, **cfg):
    config = ServerConfig(cache_dir=str(tmp_path / "cache"), metrics_enabled=True, **cfg)
    svc = PipelineService(config)
    svc.start_pipeline(ppl_file, "t2v", parallelism=1)
    return ApiServer(config, svc)


def wait_done(client, tid, timeout=10.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        st = client.get(f"/v1/tasks/{tid}/status").json()
        if st["status"] in ("completed", "failed", "cancelled"):
            return st
        time.sleep(0.02)
    raise AssertionError("task did not finish")


# ---------------------------------------------------------------------------
def test_task_manager_lifecycle_and_capacity():
    tm = TaskManager(max_queue_size=2, max_concurrent_processing=1)
    a = tm.create_task({"prompt": "a"})
    b = tm.create_task({"prompt": "b"})
    with pytest.raises(QueueFullError):
        tm.create_task({"prompt": "c"})
    t = tm.claim_next_pending_task()
    assert t.task_id == a and t.status == TaskStatus.PROCESSING
    assert tm.claim_next_pending_task() is None  # single slot
    tm.complete_task(a, output_path="x.mp4", inference_time_s=1.0)
    assert tm.get_status(a)["status"] == "completed"
    assert tm.cancel_task(b) and tm.get_status(b)["status"] == "cancelled"
    assert not tm.cancel_task(b)
    tm.set_max_concurrent_processing(0)
    with pytest.raises(RuntimeError):
        tm.create_task({"prompt": "d"})


def test_contract_defaults_and_validation(ppl_file):
    svc = PipelineService(ServerConfig())
    svc.start_pipeline(ppl_file, "t2v")
    c = svc.contract
    assert c.pipeline_name == "fake_t2v" and c.supported_tasks == ("t2v", "t2i")
    d = apply_task_contract_defaults(c, "t2v", {"prompt": "x"})
    assert d["num_inference_steps"] == 4 and d["mode"] == "fast"
    with pytest.raises(ValueError):
        validate_required_task_parameters(c, "t2v", {"prompt": ""})
    with pytest.raises(ValueError):
        validate_required_task_parameters(c, "t2v", {"prompt": "x", "mode": "warp"})
    with pytest.raises(ValueError):
        apply_task_contract_defaults(c, "i2v", {})
    assert c.to_metadata()["tasks"]["t2i"]["media_type"] == "image"


def test_legacy_contract_from_signature(tmp_path):
    p = tmp_path / "legacy.py"
    p.write_text("def get_pipeline(parallelism=1):\n    return object()\n"
                 "def run_with_file(pipeline, prompt, first_image_path, output_path, steps=8, cfg=5.0):\n    return output_path\n")
    svc = PipelineService(ServerConfig())
    svc.start_pipeline(str(p), "i2v")
    tc = svc.contract.task_contracts["i2v"]
    assert tc.required_inputs == ("prompt", "first_image_path")
    assert tc.parameters["steps"].type == "integer" and tc.parameters["cfg"].default == 5.0


def test_security_validator_levels(tmp_path):
    bad = "import os\nos.system('rm -rf /')\n"
    sneaky = "import socket\ns = socket.socket()\n"
    main_only = "def get_pipeline():\n    return 1\nif __name__ == '__main__':\n    import os\n    os.system('ls')\n"
    v = PipelineSecurityValidator("strict")
    assert not v.validate_source(bad).passed
    assert not v.validate_source(sneaky).passed
    assert PipelineSecurityValidator("basic").validate_source(sneaky).passed
    assert v.validate_source(main_only).passed
    assert not v.validate_source("eval('1+1')").passed
    assert not v.validate_source("import subprocess\nsubprocess.run('ls', shell=True)").passed
    assert PipelineSecurityValidator("none").validate_source(bad).passed
    f = tmp_path / "bad.py"
    f.write_text(bad)
    with pytest.raises(SecurityError):
        v.check_file(str(f))
    sb = PipelineSecurityValidator("sandbox")
    mod = sb.loader.load_module("import math\nx = math.sqrt(4)\n")
    assert mod.x == 2.0
    with pytest.raises(SecurityError):
        sb.loader.load_module("import http.client\n")


def test_files_and_artifacts(tmp_path):
    fs = FileService(str(tmp_path / "c"), max_upload_mb=1)
    p = fs.save_bytes(PNG, MediaType.IMAGE)
    assert p.endswith(".png")
    with pytest.raises(MediaError):
        fs.save_bytes(b"not an image at all", MediaType.IMAGE)
    with pytest.raises(MediaError):
        fs.save_bytes(PNG + b"\x00" * (2 << 20), MediaType.IMAGE)
    import base64

    assert fs.save_base64("data:image/png;base64," + base64.b64encode(PNG).decode(), MediaType.IMAGE).endswith(".png")
    assert handler_for("video").sniff(b"\x00\x00\x00\x18ftypmp42....") == "mp4"
    with pytest.raises(PermissionError):
        fs.resolve_inside("../../etc/passwd", fs.output_dir)
    store = ArtifactStore(str(tmp_path / "a"), retention_hours=1.0, max_gb=1e-6)  # ~1 KB cap
    paths = []
    for i in range(3):
        f = tmp_path / f"o{i}.bin"
        f.write_bytes(b"x" * 600)
        paths.append(f)
        store.register(str(f), f"t{i}", "t2v", "video")
        time.sleep(0.01)
    assert store.get("t0") is None and not paths[0].exists()  # size cap evicts the oldest
    assert store.get("t2") is not None
    again = ArtifactStore(str(tmp_path / "a"), 1.0, 1e-6)
    assert again.get("t2") is not None  # index persisted
    assert again.enforce_retention(now=time.time() + 7200) and again.get("t2") is None


def test_latent_cache_resume(tmp_path):
    c = LatentCache(str(tmp_path / "lc"), mode="readwrite", min_similarity=0.6)
    req = {"task": "t2v", "prompt": "a red fox runs over snow", "seed": 1, "resolution": "720p"}
    q = c.build_query(req)
    assert c.lookup(q) is None
    c.save(q, {"steps": {2: torch.ones(3), 4: torch.ones(3) * 2}})
    hit = c.lookup(c.build_query(req))
    assert hit["similarity"] == 1.0 and c.apply_resume(hit)["resume_step"] == 4
    near = c.lookup(c.build_query({**req, "prompt": "a red fox runs over fresh snow"}))
    assert near is not None and near["similarity"] < 1.0 and c.apply_resume(near)["resume_step"] == 2
    assert c.lookup(c.build_query({**req, "prompt": "city at night"})) is None
    assert c.lookup(c.build_query({**req, "resolution": "480p"})) is None
    ro = LatentCache(str(tmp_path / "lc"), mode="read")
    assert ro.save(q, {"steps": {1: torch.ones(1)}}) is None


def test_rate_limiter_window():
    rl = RateLimiter(2, 10.0)
    assert rl.allow("a", 0.0)[0] and rl.allow("a", 1.0)[0]
    ok, retry = rl.allow("a", 2.0)
    assert not ok and 7.9 < retry <= 8.0
    assert rl.allow("b", 2.0)[0] and rl.allow("a", 10.5)[0]


# ---------------------------------------------------------------------------
def test_http_task_flow(tmp_path, ppl_file):
    api = make_api(tmp_path, ppl_file)
    with TestClient(api.app) as client:
        health = client.get("/v1/service/health").json()
        assert health["status"] == "healthy" and health["pipeline_ready"] is True and health["version"] and health["timestamp"].endswith("+00:00")
        assert client.get("/v1/service/ready").status_code == 200
        meta = client.get("/v1/service/metadata").json()
        assert meta["pipeline_name"] == "fake_t2v" and "t2v" in meta["tasks"] and meta["task_contracts"] == meta["tasks"]
        assert meta["pipeline_file"] == ppl_file and meta["parallelism"] == 1 and meta["task"] == "t2v" and meta["runner"] == "PipelineRunner"
        assert isinstance(meta["declared_pipeline_contract"], bool) and meta["entrypoints"] == {"get_pipeline": "get_pipeline", "run_with_file": "run_with_file"}
        assert meta["max_queue_size"] == 100 and meta["service_configured_max_concurrent_tasks"] == 1 and meta["security_level"]
        assert set(meta["task_contracts"]["t2v"]) == {"media_type", "required_inputs", "optional_inputs", "parameters"}
        r = client.post("/v1/tasks/create", json={"task": "t2v", "prompt": "hello", "seed": 7, "mode": "slow"})
        assert r.status_code == 200, r.text
        tid = r.json()["task_id"]
        st = wait_done(client, tid)
        assert st["status"] == "completed" and st["inference_time_s"] >= 0
        body = client.get(f"/v1/tasks/{tid}/result").content
        assert body.endswith(b"hello|7|4|slow|0")
        name = st["output_path"].rsplit("/", 1)[1]
        assert client.get(f"/v1/files/download/{name}").status_code == 200
        assert client.get("/v1/files/download/../../../etc/passwd").status_code in (403, 404)
        # validation errors
        assert client.post("/v1/tasks/create", json={"task": "t2v", "prompt": ""}).status_code == 400
        assert client.post("/v1/tasks/create", json={"task": "i2v", "prompt": "x"}).status_code == 400
        assert client.post("/v1/tasks/create", json={"task": "t2v", "prompt": "x", "aspect_ratio": "5:1"}).status_code == 422
        assert client.get("/v1/tasks/nope/status").status_code == 404
        # failure is reported
        tid2 = client.post("/v1/tasks/create", json={"task": "t2v", "prompt": "boom"}).json()["task_id"]
        st2 = wait_done(client, tid2)
        assert st2["status"] == "failed" and "exploded" in st2["error"]
        # cancellation of a running task (cooperative stop event)
        tid3 = client.post("/v1/tasks/create", json={"task": "t2v", "prompt": "slow", "sleep_s": 5.0}).json()["task_id"]
        time.sleep(0.2)
        assert client.delete(f"/v1/tasks/{tid3}").json()["stop_status"] == "success"
        assert wait_done(client, tid3)["status"] == "cancelled"
        assert client.delete(f"/v1/tasks/{tid3}").json()["stop_status"] == "do_nothing"
        # form route with an upload
        r = client.post("/v1/tasks/form", data={"task": "t2v", "prompt": "123", "seed": "9", "num_inference_steps": "2"},
                        files={"first_image_file": ("a.png", PNG, "image/png")})
        assert r.status_code == 200, r.text
        assert client.get(f"/v1/tasks/{r.json()['task_id']}/result") is not None
        st4 = wait_done(client, r.json()["task_id"])
        assert st4["status"] == "completed"
        q = client.get("/v1/tasks/queue/status").json()
        assert q["active_count"] == 0 and q["queue_size"] == 100
        prom = client.get("/v1/service/metrics").text
        assert "telefuser" in prom and "tasks" in prom
        otlp = client.get("/v1/service/metrics", params={"format": "opentelemetry"})
        assert otlp.headers["content-type"].startswith("application/json") and otlp.json()["resourceMetrics"][0]["scopeMetrics"][0]["metrics"]
        assert "|g" in client.get("/v1/service/metrics", params={"format": "statsd"}).text
        assert client.get("/v1/service/metrics", params={"format": "graphite"}).status_code == 400
        assert client.get("/v1/service/status").json()["pipeline_ready"] is True


def test_latent_cache_through_http(tmp_path, ppl_file):
    api = make_api(tmp_path, ppl_file, enable_latent_cache=True)
    with TestClient(api.app) as client:
        body = {"task": "t2v", "prompt": "same prompt", "seed": 3}
        t1 = client.post("/v1/tasks/create", json=body).json()["task_id"]
        wait_done(client, t1)
        assert client.get(f"/v1/tasks/{t1}/result").content.endswith(b"|0")
        t2 = client.post("/v1/tasks/create", json=body).json()["task_id"]
        wait_done(client, t2)
        assert client.get(f"/v1/tasks/{t2}/result").content.endswith(b"|4")  # resumed at the last saved step
        assert client.get("/v1/service/status").json()["latent_cache"]["hits"] == 1


def test_openai_routes(tmp_path, ppl_file):
    api = make_api(tmp_path, ppl_file)
    with TestClient(api.app) as client:
        r = client.post("/v1/images/generations", json={"prompt": "a cat", "size": "1024x768", "n": 2,
                                                        "response_format": "b64_json"})  # fmt: skip
        assert r.status_code == 200, r.text
        data = r.json()["data"]
        assert len(data) == 2 and data[0]["b64_json"]
        r = client.post("/v1/images/generations", json={"prompt": "a cat"})
        url = r.json()["data"][0]["url"]
        assert client.get(url.replace("http://testserver", "")).status_code == 200
        facts = r.json()["data"][0]["artifact_metadata"]
        assert facts["backend"] == "local" and facts["media_type"] == "image" and facts["filename"].endswith(".png") and facts["size_bytes"] > 0
        assert facts["task_id"] == r.json()["data"][0]["artifact_id"] and not facts["relative_path"].startswith("/")
        v = client.post("/v1/videos", json={"prompt": "waves", "seconds": 2, "size": "1280x720"}).json()
        assert v["object"] == "video" and v["status"] in ("queued", "generating", "completed") and v["size"] == "1280x720"
        for _ in range(200):
            v = client.get(f"/v1/videos/{v['id']}").json()
            if v["status"] == "completed":
                break
            time.sleep(0.02)
        assert v["status"] == "completed" and v["progress"] == 100
        assert v["artifact_metadata"]["media_type"] == "video" and v["artifact_metadata"]["task_id"] == v["id"]
        assert client.get(f"/v1/videos/{v['id']}/content").content.startswith(b"\x00\x00\x00\x18ftyp")
        lst = client.get("/v1/videos").json()
        assert lst["object"] == "list" and lst["data"][0]["id"] == v["id"]
        assert client.delete(f"/v1/videos/{v['id']}").json()["status"] == "deleted"
        assert client.get(f"/v1/videos/{v['id']}/content").status_code == 404
        assert client.get("/v1/videos/video_missing").status_code == 404


def test_rate_limit_middleware(tmp_path, ppl_file):
    api = make_api(tmp_path, ppl_file, rate_limit_enabled=True, rate_limit_requests=3, rate_limit_window_s=60.0)
    with TestClient(api.app) as client:
        codes = [client.get("/v1/tasks/queue/status").status_code for _ in range(5)]
        assert codes == [200, 200, 200, 429, 429]
        assert client.get("/v1/service/health").status_code == 200  # exempt


def test_stream_websocket_bidirectional(tmp_path):
    p = tmp_path / "fake_stream.py"
    p.write_text(FAKE_STREAM)
    config = ServerConfig(cache_dir=str(tmp_path / "cache"))
    svc = StreamPipelineService(config)
    svc.start_service(str(p))
    assert svc.stream_mode == "bidirectional"
    api = ApiServer(config, None, svc)
    with TestClient(api.app) as client:
        assert client.get("/v1/service/ready").status_code == 200
        with client.websocket_connect("/v1/stream/ws") as ws:
            ws.send_text(json.dumps({"session_id": "abc"}))
            hello = json.loads(ws.receive_text())
            assert hello == {"type": "session", "session_id": "abc", "stream_mode": "bidirectional"}
            assert client.get("/v1/stream/sessions/abc/status").json()["status"] == "active"
            ws.send_text(json.dumps({"key": "w"}))
            msg = json.loads(ws.receive_text())
            assert msg["type"] == "chunk" and msg["index"] == 0 and msg["num_frames"] == 2 and msg["data"]["echo"] == "w"
            jpegs = [ws.receive_bytes() for _ in range(2)]
            assert all(j[:3] == b"\xff\xd8\xff" for j in jpegs)
            ws.send_text(json.dumps({"key": "sound"}))
            msg = json.loads(ws.receive_text())
            assert msg["num_frames"] == 2 and msg["audio"] == {"sample_rate": 16000, "channels": 2, "num_samples": 8000, "format": "pcm_s16le"}
            assert "audio" not in msg["data"]
            [ws.receive_bytes() for _ in range(2)]
            assert len(ws.receive_bytes()) == 8000 * 2 * 2  # interleaved PCM16 after the pictures
            ws.send_text(json.dumps({"key": "end"}))
            msg = json.loads(ws.receive_text())
            assert msg["data"]["done"] is True
            [ws.receive_bytes() for _ in range(2)]
            assert json.loads(ws.receive_text())["type"] == "done"
        assert client.get("/v1/stream/sessions/abc/status").json()["status"] == "unknown"
        assert client.post("/v1/stream/webrtc/offer", json={"sdp": "x", "task": "t2v"}).status_code == 501
        # a second session under a live id is a conflict; beyond the configured number of sessions the server is busy
        api.sessions.max_sessions = 1
        with client.websocket_connect("/v1/stream/ws") as first:
            first.send_text(json.dumps({"session_id": "only"}))
            assert json.loads(first.receive_text())["type"] == "session"
            with client.websocket_connect("/v1/stream/ws") as second:
                second.send_text(json.dumps({"session_id": "other"}))
                assert "limit 1" in json.loads(second.receive_text())["error"]
            api.sessions.max_sessions = 0
            with client.websocket_connect("/v1/stream/ws") as again:
                again.send_text(json.dumps({"session_id": "only"}))
                assert "already exists" in json.loads(again.receive_text())["error"]
        assert client.delete("/v1/stream/webrtc/abc").status_code == 404 and client.delete("/v1/stream/sessions/abc").status_code == 404

        class FakeConnections:  # a peer connection without a pipeline session behind it still counts as found
            def __init__(self):
                self.connections, self.closed = {"rtc-1": object(), "rtc-2": object()}, []

            async def close_connection(self, sid):
                self.connections.pop(sid)
                self.closed.append(sid)
                if sid == "rtc-2":
                    raise RuntimeError("peer already gone")

        api.webrtc = FakeConnections()
        assert client.delete("/v1/stream/webrtc/rtc-1").json() == {"session_id": "rtc-1", "status": "closed"}
        assert client.delete("/v1/stream/sessions/rtc-2").status_code == 200 and api.webrtc.closed == ["rtc-1", "rtc-2"]
        ui = client.get("/ui")  # the browser front end: one static page that talks to the WebSocket transport
        assert ui.status_code == 200 and "text/html" in ui.headers["content-type"] and "/v1/stream/ws" in ui.text


# ---------------------------------------------------------------------------
def _fake_replica(conn, index_file, die_on):
    """Replica stand-in: answers tasks, exits abruptly when the prompt equals `die_on`."""
    import os

    conn.send(("ready", {"pipeline_name": "fake", "supported_tasks": ["t2v"]}))
    while True:
        msg = conn.recv()
        if msg[0] == "shutdown":
            return
        if msg[0] == "task":
            _, tid, data = msg
            if data.get("prompt") == die_on:
                os._exit(3)
            conn.send(("ok", tid, (f"{data['prompt']}@{os.getpid()}", None, 0.01)))


def test_replica_pool_dispatch_and_eviction():
    from telefuser_b200.service.pipeline_service import ReplicaDeadError, ReplicaHandle
    import multiprocessing as mp

    assert resolve_replica_device_ids(2, 2, [0, 1, 2, 3]) == [[0, 1], [2, 3]]
    with pytest.raises(ValueError):
        resolve_replica_device_ids(2, 4, [0, 1, 2, 3])
    tm = TaskManager()
    pool = PipelinePool(ServerConfig(task_timeout=20.0, replica_start_timeout=60.0), tm)
    ctx = mp.get_context("spawn")
    for i in range(2):
        pool.replicas.append(ReplicaHandle(i, [i], ctx, _fake_replica, ("", "die")))
    for r in pool.replicas:
        r.wait_ready(60.0)
    tm.set_max_concurrent_processing(2)
    try:
        outs = []
        ths = [threading.Thread(target=lambda k=k: outs.append(pool.run_task_with_stop_event({"prompt": f"p{k}"})))
               for k in range(4)]  # fmt: skip
        [t.start() for t in ths]
        [t.join() for t in ths]
        assert sorted(o.output_path.split("@")[0] for o in outs) == ["p0", "p1", "p2", "p3"]
        with pytest.raises(ReplicaDeadError):
            pool.run_task_with_stop_event({"prompt": "die"})
        assert len(pool.replicas) == 1 and tm.queue_status()["processing_slots"] == 1
        assert pool.run_task_with_stop_event({"prompt": "after"}).output_path.startswith("after@")
        pending = tm.create_task({"prompt": "queued"})
        with pytest.raises(ReplicaDeadError):
            pool.run_task_with_stop_event({"prompt": "die"})
        assert not pool.ready and tm.get_status(pending)["status"] == "failed"
        with pytest.raises(RuntimeError):
            tm.create_task({"prompt": "no capacity"})
    finally:
        pool.stop()


def test_cli_validate_and_scan(tmp_path, ppl_file):
    from click.testing import CliRunner

    from telefuser_b200.entrypoints.cli import main

    runner = CliRunner()
    res = runner.invoke(main, ["validate", ppl_file, "--json"])
    assert res.exit_code == 0 and json.loads(res.output)["passed"] is True
    bad = tmp_path / "bad.py"
    bad.write_text("import os\nos.system('x')\n")
    res = runner.invoke(main, ["validate", str(bad)])
    assert res.exit_code == 1 and "FORBIDDEN_CALL" in res.output
    res = runner.invoke(main, ["scan", str(tmp_path)])
    assert res.exit_code == 1 and "1 failed" in res.output
    res = runner.invoke(main, ["serve", ppl_file, "--validate-only"])
    assert res.exit_code == 0 and "PASSED" in res.output


def test_clients_against_live_server(tmp_path, ppl_file):
    import socket

    import uvicorn

    from telefuser_b200.client import OpenAICompatibleClient, TaskFailedError, TFClient

    api = make_api(tmp_path, ppl_file)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(api.app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    url = f"http://127.0.0.1:{port}"
    try:
        c = TFClient(url, timeout=20)
        for _ in range(200):
            if c.health_check():
                break
            time.sleep(0.05)
        assert c.health_check()
        t = c.create_t2v_task("from client", seed=5)
        st = c.wait_for_completion(t["task_id"], poll_interval=0.02)
        assert st["status"] == "completed"
        out = tmp_path / "dl" / "r.mp4"
        assert c.download_result(t["task_id"], str(out)) and out.read_bytes().endswith(b"from client|5|4|fast|0")
        bad = c.create_t2v_task("boom")
        with pytest.raises(TaskFailedError):
            c.wait_for_completion(bad["task_id"], poll_interval=0.02)
        assert c.get_service_metadata()["pipeline_name"] == "fake_t2v"
        assert c.get_queue_status()["active_count"] == 0
        oc = OpenAICompatibleClient(url)
        imgs = oc.images.generate("a dog", size="512x512")
        assert len(imgs) == 1 and imgs[0].bytes()
        v = oc.videos.create("surf", seconds=1).wait(poll_interval=0.02, timeout=20)
        assert v.is_success and v.download().startswith(b"\x00\x00\x00\x18ftyp")
        assert len(oc.videos.list()) == 1 and oc.videos.delete(v.id).status == "deleted"
    finally:
        server.should_exit = True
        th.join(10)


def test_compact_manifest_expands_to_a_full_contract():
    import types

    from telefuser_b200.service.contract import expand_short_manifest, load_contract

    def run_with_file(pipeline, prompt, output_path, first_image_path=None, seed=3, steps=20, resolution="720p", stop_event=None):
        return output_path

    mod = types.SimpleNamespace(PPL_CONFIG={"name": "demo"}, run_with_file=run_with_file, get_pipeline=lambda parallelism=1: None,
                                PIPELINE_MANIFEST={"tasks": ["t2v", "i2v", "t2i"], "media_type": "video",
                                                   "required_inputs": {"t2v": ["prompt"], "i2v": ["prompt", "first_image_path"]},
                                                   "parameters": {"t2i": {"resolution": {"default": "1024x1024", "enum": ["1024x1024"]}}},
                                                   "effective_max_concurrent_tasks": 2})  # fmt: skip
    c = load_contract(mod, None, "file_stem")
    assert c.pipeline_name == "demo" and c.supported_tasks == ("t2v", "i2v", "t2i") and c.effective_max_concurrent_tasks == 2
    assert c.task_contracts["i2v"].required_inputs == ("prompt", "first_image_path") and c.task_contracts["t2i"].required_inputs == ("prompt",)
    assert c.task_contracts["t2i"].media_type == "image" and c.task_contracts["t2v"].media_type == "video"
    params = c.task_contracts["t2v"].parameters
    assert set(params) == {"seed", "steps", "resolution"} and params["steps"].default == 20 and params["steps"].type == "integer"
    assert c.task_contracts["t2i"].parameters["resolution"].default == "1024x1024" and c.task_contracts["t2i"].parameters["resolution"].enum == ("1024x1024",)
    full = {"supported_tasks": ["t2v"], "tasks": ["ignored"]}
    assert expand_short_manifest(full, mod, "x") is full  # a complete mapping is left as it is
    single = expand_short_manifest({"tasks": ["vsr"], "media_type": "video"}, None, "upscaler")
    assert single["pipeline_name"] == "upscaler" and single["task_contracts"]["vsr"]["required_inputs"] == ["ref_video_path"]


def test_pipeline_file_cache_config_and_cli_precedence(tmp_path, monkeypatch):
    from pathlib import Path

    from click.testing import CliRunner

    from telefuser_b200.entrypoints import cli
    from telefuser_b200.service import main as service_main
    from telefuser_b200.service.contract import load_cache_config, resolve_latent_cache_settings

    example = str(Path(__file__).resolve().parents[1] / "examples" / "wan_video" / "wan22_14b_text_to_video_service.py")
    monkeypatch.delenv("TELEFUSER_LATENT_CACHE_DIR", raising=False)
    monkeypatch.setenv("TELEFUSER_CACHE_MODE", "write_only")
    declared = load_cache_config(example)  # read from the source text: nothing of the file is imported or run
    assert declared == {"enable_latent_cache": True, "latent_cache_dir": "./latent_cache/wan22_t2v", "cache_mode": "write_only"}
    got = resolve_latent_cache_settings(example, None, None)
    assert (got["enabled"], got["mode"], got["directory"], got["source"]) == (True, "write", "./latent_cache/wan22_t2v", "pipeline file")
    assert resolve_latent_cache_settings(example, False, None)["enabled"] is False  # the command line wins
    assert resolve_latent_cache_settings(example, None, "read_only")["mode"] == "read"
    with pytest.raises(ValueError, match="not one of"):
        resolve_latent_cache_settings(example, None, "sometimes")

    f = tmp_path / "ppl.py"
    f.write_text("import os\nROOT = os.path.join('/data', 'cache')\nTHRESH = float(os.getenv('NO_SUCH_VAR_FOR_TEST', '0.9'))\n"
                 "CACHE_CONFIG = {'enable_latent_cache': True, 'latent_cache_dir': ROOT, 'rerank_score_threshold': THRESH,\n"
                 "                'key_steps': [5, 10], 'odd': open('/etc/hostname').read(), 'neg': -1}\n")
    declared = load_cache_config(str(f))
    assert declared == {"enable_latent_cache": True, "latent_cache_dir": "/data/cache", "rerank_score_threshold": 0.9, "key_steps": [5, 10], "neg": -1}
    assert resolve_latent_cache_settings(str(f), None, None)["min_similarity"] == 0.9
    plain = tmp_path / "plain.py"
    plain.write_text("PPL_CONFIG = {}\n")
    assert load_cache_config(str(plain)) is None and resolve_latent_cache_settings(str(plain), None, None)["enabled"] is False
    bad = tmp_path / "bad.py"
    bad.write_text("CACHE_CONFIG = dict(enable_latent_cache=True, cache_mode='sometimes')\n")
    with pytest.raises(ValueError, match="cache_mode 'sometimes'"):
        resolve_latent_cache_settings(str(bad), None, None)

    seen = {}

    class FakeContainer:
        def __init__(self, cfg):
            seen["cfg"] = cfg

        def initialize_all(self, *a, **k):
            return True

    monkeypatch.setattr(service_main, "ServiceContainer", FakeContainer)
    monkeypatch.setattr(service_main, "_run", lambda *a, **k: None)
    runner = CliRunner()
    assert runner.invoke(cli.main, ["serve", str(f), "-t", "t2v"]).exit_code == 0
    cfg = seen["cfg"]
    assert cfg.enable_latent_cache and cfg.latent_cache_dir == "/data/cache" and cfg.latent_cache_min_similarity == 0.9 and cfg.latent_cache_mode == "readwrite"
    assert runner.invoke(cli.main, ["serve", str(f), "-t", "t2v", "--disable-latent-cache", "--cache-mode", "read_only"]).exit_code == 0
    assert not seen["cfg"].enable_latent_cache and seen["cfg"].latent_cache_mode == "read"
    assert runner.invoke(cli.main, ["serve", str(plain), "-t", "t2v"]).exit_code == 0 and not seen["cfg"].enable_latent_cache


def test_webrtc_offer_status_codes(tmp_path, monkeypatch):
    import telefuser_b200.service.api as api_mod
    import telefuser_b200.service.webrtc as webrtc_mod
    from telefuser_b200.service.stream_service import SessionConflict, SessionLimitReached

    p = tmp_path / "fake_stream.py"
    p.write_text(FAKE_STREAM)
    config = ServerConfig(cache_dir=str(tmp_path / "cache"))
    svc = StreamPipelineService(config)
    svc.start_service(str(p))
    api = ApiServer(config, None, svc)
    monkeypatch.setattr(api_mod, "webrtc_available", lambda: True)
    outcome = {}

    async def fake_answer(server, body):
        if isinstance(outcome["value"], Exception):
            raise outcome["value"]
        return outcome["value"]

    monkeypatch.setattr(webrtc_mod, "answer_offer", fake_answer)
    with TestClient(api.app) as client:
        for value, status in (({"session_id": "s", "sdp": "v=0", "type": "answer"}, 200), (SessionLimitReached("4 open (limit 4)"), 503),
                              (SessionConflict("session 's' already exists"), 409), (KeyError("sdp"), 400), (ValueError("bad SDP"), 400)):  # fmt: skip
            outcome["value"] = value
            r = client.post("/v1/stream/webrtc/offer", json={"sdp": "x", "type": "offer", "task": "bidirectional"})
            assert r.status_code == status, (value, r.text)
