"""The client-side load generators under benchmarks/ against live local servers with stand-in pipelines."""
import importlib.util
import json
import socket
import sys
import threading
import time
from pathlib import Path

import pytest

from telefuser_b200.service.api import ApiServer
from telefuser_b200.service.pipeline_service import ServerConfig
from telefuser_b200.service.stream_service import StreamPipelineService

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(Path(__file__).resolve().parent))
from test_service import FAKE_PIPELINE, FAKE_STREAM, make_api  # noqa: E402


def load(name: str):
    spec = importlib.util.spec_from_file_location(name, ROOT / "benchmarks" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class LiveServer:
    def __init__(self, app):
        import uvicorn

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            self.port = s.getsockname()[1]
        self.server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=self.port, log_level="error"))
        self.thread = threading.Thread(target=self.server.run, daemon=True)
        self.url = f"http://127.0.0.1:{self.port}"

    def __enter__(self):
        self.thread.start()
        import requests

        for _ in range(200):
            try:
                if requests.get(self.url + "/v1/service/health", timeout=1).status_code == 200:
                    return self
            except requests.RequestException:
                pass
            time.sleep(0.05)
        raise RuntimeError("server did not come up")

    def __exit__(self, *exc):
        self.server.should_exit = True
        self.thread.join(10)


def test_committed_configs_parse_and_plans_are_reproducible():
    vb, sb = load("video_generation_bench"), load("stream_session_bench")
    for name in ("video_generation_quick", "video_generation_e2e", "video_generation_rate"):
        cfg = vb.load_config(str(ROOT / "benchmarks" / "configs" / f"{name}.json"))
        plan = vb.arrival_times(cfg)
        assert len(plan) == cfg["profiling"]["requests"] and plan == sorted(plan) and plan == vb.arrival_times(cfg)
    rate = vb.load_config(str(ROOT / "benchmarks" / "configs" / "video_generation_rate.json"))
    gaps = [b - a for a, b in zip(vb.arrival_times(rate), vb.arrival_times(rate)[1:])]
    assert len(set(round(g, 6) for g in gaps)) > 1  # poisson arrivals, not a fixed spacing
    assert len(vb.load_prompts(str(ROOT / "benchmarks" / "data" / "video_prompts.jsonl"))) >= 4
    for name in ("stream_lingbot_world_quick", "stream_lingbot_world_compare"):
        cfg = sb.load_config(str(ROOT / "benchmarks" / "configs" / f"{name}.json"))
        trace = sb.load_control_trace(str(ROOT / cfg["control_trace_path"]))
        assert trace and [e["t"] for e in trace] == sorted(e["t"] for e in trace)
    with pytest.raises(ValueError):
        vb.load_config(None, {"type": "poisson", "rate": 0.0})
    assert sb.percentile([1.0, 2.0, 3.0, 100.0], 50) in (2.0, 3.0) and sb.percentile([], 99) is None


def test_video_generation_bench_against_a_live_task_service(tmp_path):
    vb = load("video_generation_bench")
    ppl = tmp_path / "fake_pipeline.py"
    ppl.write_text(FAKE_PIPELINE)
    prompts = tmp_path / "p.jsonl"
    prompts.write_text('{"text": "one"}\n{"text": "boom"}\n{"text": "three"}\n')
    with LiveServer(make_api(tmp_path, str(ppl)).app) as srv:
        cfg = vb.load_config(None, {"server_url": srv.url, "type": "constant", "rate": 50.0, "concurrency": 2, "requests": 5,
                                    "artifacts_dir": str(tmp_path / "art")})  # fmt: skip
        cfg["dataset"]["path"] = str(prompts)
        cfg["poll_interval_s"] = 0.02
        cfg["extra"] = {"num_inference_steps": 3}
        summary = vb.run(cfg)
    assert summary["requests"] == 5 and summary["failed"] == 2 and summary["completed"] == 3  # "boom" raises in the pipeline
    assert summary["latency_s"]["p50"] > 0 and summary["throughput_rps"] > 0
    rows = [json.loads(line) for line in (tmp_path / "art" / "records.jsonl").read_text().splitlines()]
    assert len(rows) == 5 and sum(r["status"] == "completed" for r in rows) == 3
    assert json.loads((tmp_path / "art" / "summary.json").read_text())["completed"] == 3


def test_stream_session_bench_against_a_live_stream_service(tmp_path):
    sb = load("stream_session_bench")
    p = tmp_path / "fake_stream.py"
    p.write_text(FAKE_STREAM)
    config = ServerConfig(cache_dir=str(tmp_path / "cache"))
    svc = StreamPipelineService(config)
    svc.start_service(str(p))
    trace = tmp_path / "trace.json"
    trace.write_text(json.dumps({"events": [{"t": 0.05 + 0.1 * i, "message": {"key": f"k{i}"}} for i in range(6)]}))
    with LiveServer(ApiServer(config, None, svc).app) as srv:
        cfg = sb.load_config(None, {"server_url": srv.url, "session_count": 2, "session_duration_s": 1.2, "warmup_sessions": 1,
                                    "artifacts_dir": str(tmp_path / "art")})  # fmt: skip
        cfg["control_trace_path"] = str(trace)
        cfg["server_metrics"] = {"enabled": True, "urls": [srv.url + "/v1/service/health"], "collection_interval_s": 0.2}
        import asyncio

        summary = asyncio.run(sb.run(cfg))
    assert summary["sessions"] == 2 and summary["success_rate"] == 1.0
    assert summary["chunks_received"] == 12 and summary["frames_received"] == 24  # every control echoes one 2-frame chunk
    assert summary["first_chunk_ms"]["p50"] > 0 and summary["control_to_next_chunk_ms_p50"]["p50"] >= 0
    rows = [json.loads(line) for line in (tmp_path / "art" / "sessions.jsonl").read_text().splitlines()]
    assert len(rows) == 2 and all(r["controls_sent"] == 6 and r["ok"] for r in rows)
    ev = [json.loads(line) for line in (tmp_path / "art" / "events_0.jsonl").read_text().splitlines()]
    assert [e["event"] for e in ev].count("control") == 6 and [e["event"] for e in ev].count("chunk") == 6
    assert (tmp_path / "art" / "server_metrics.jsonl").read_text().count('"status": 200') >= 2


def test_feature_cache_bench_reports_skipped_steps_and_similarity(capsys):
    import torch

    from telefuser_b200.utils.quality import psnr, ssim

    x = torch.rand(3, 2, 16, 16) * 2 - 1
    assert psnr(x, x) == float("inf") and ssim(x, x) == pytest.approx(1.0)
    y = (x + 0.05 * torch.randn_like(x)).clamp(-1, 1)
    assert 20 < psnr(y, x) < 45 and 0.5 < ssim(y, x) < 1.0 and ssim(y[:, 0], x[:, 0]) > 0.5  # single images too
    fb = load("feature_cache_bench")
    assert fb.main(["--random-init", "--preset", "tiny", "--device", "cpu", "--steps", "12", "--frames", "5", "--height", "32",
                    "--width", "32", "--orders", "0,1"]) == 0  # fmt: skip
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    summary = lines[-1]["summary"]
    assert [r["config"] for r in summary] == ["no cache", "adaptive Taylor cache, order 0", "adaptive Taylor cache, order 1"]
    assert summary[0]["computed_steps"] == 12 and all(r["computed_steps"] < 12 and r["finite"] for r in summary[1:])
    assert all(r["psnr_db"] > 25 and r["ssim"] > 0.85 for r in summary[1:])


def test_stream_session_bench_against_the_world_model_example(tmp_path, monkeypatch):
    """Full stack on CPU: the LingBot-World example file (tiny random-init model) behind the stream API, driven by the
    load generator over a real socket; acknowledgements and applied revisions give the two control latencies."""
    import asyncio

    monkeypatch.setenv("TFB_RANDOM_INIT", "1")
    monkeypatch.setenv("TFB_TINY", "1")
    sb = load("stream_session_bench")
    config = ServerConfig(cache_dir=str(tmp_path / "cache"), security_level="strict")
    svc = StreamPipelineService(config)
    assert svc.start_service(str(ROOT / "examples" / "lingbot" / "lingbot_world_v2_image_to_video.py"), gpu_num=1)
    trace = tmp_path / "trace.json"
    trace.write_text(json.dumps({"events": [{"t": 0.05, "message": {"keys": ["w"]}}, {"t": 0.4, "message": {"keys": ["a"]}}]}))
    try:
        with LiveServer(ApiServer(config, None, svc).app) as srv:
            cfg = sb.load_config(None, {"server_url": srv.url, "session_count": 1, "session_duration_s": 60.0,
                                        "warmup_sessions": 0, "artifacts_dir": str(tmp_path / "art")})  # fmt: skip
            cfg["control_trace_path"] = str(trace)
            from PIL import Image

            Image.new("RGB", (64, 64), (90, 120, 150)).save(tmp_path / "first.png")
            cfg["image_path"] = str(tmp_path / "first.png")
            cfg["request_extra"] = {"height": 64, "width": 64, "max_duration_seconds": 2.0, "benchmark_metrics": True}
            summary = asyncio.run(sb.run(cfg))
    finally:
        svc.service.stop()
    assert summary["success_rate"] == 1.0 and summary["chunks_received"] >= 2 and summary["frames_received"] >= 9
    assert summary["control_ack_ms_p50"] is not None and summary["control_applied_ms_p50"] is not None
    assert summary["control_ack_ms_p50"]["p50"] <= summary["control_applied_ms_p50"]["p50"]
