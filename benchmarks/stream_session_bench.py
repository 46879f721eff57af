"""Client-side load generator for the streaming service (`telefuser stream-serve`): interactive sessions over the
WebSocket transport `/v1/stream/ws`, measured from the client's side of the wire.

    python benchmarks/stream_session_bench.py --config benchmarks/configs/stream_lingbot_world_quick.json

One session = connect, send the session config, replay a timed control trace (key / camera events) while receiving
chunk messages and their JPEG frames, close after `session_duration_s`. `warmup_sessions` run first and are not
counted. Per session the harness records: connect and session-open latency, time to the first chunk and first frame,
frames and chunks received, stream fps over the session, chunk inter-arrival p50 / p99, and for every control event
the time until the next media chunk that arrives after it (`control_to_next_chunk_ms`); every control is sent with a
`revision`, and a service that acknowledges revisions and reports the revision each chunk was steered by (the
LingBot-World service does) also yields `control_ack_ms` and `control_applied_ms`. With `server_metrics` the
service's Prometheus text (`/v1/service/metrics`) is sampled beside the run. Output: `sessions.jsonl`, one
`events_<n>.jsonl` trace per session, `server_metrics.jsonl`, and `summary.json` in `artifacts_dir`; the summary is also
printed as one JSON line.

Role: the reference drives its stream service with an external load tool configured by
benchmarks/telefuser_aiperf/configs/stream_lingbot_world_fast_{quick,compare}.json and
benchmarks/telefuser_aiperf/stream_benchmark_contract.yaml (WebRTC transport); this is the in-tree equivalent on the
WebSocket transport, with the same workload fields (fps, session_count, warmup_sessions, session_duration_s,
stagger_s, control trace, request_extra) and the same client-side metrics.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import statistics
import time
import uuid
from pathlib import Path

DEFAULTS = {
    "server_url": "http://127.0.0.1:8088", "prompt": "", "image_path": None, "fps": 16, "session_count": 1,
    "warmup_sessions": 1, "session_duration_s": 90.0, "stagger_s": 0.0, "control_trace_path": None,
    "request_extra": {}, "transport": {"connect_timeout_s": 60.0, "frame_timeout_s": 180.0},
    "server_metrics": {"enabled": False, "urls": [], "collection_interval_s": 1.0},
    "artifacts_dir": "artifacts/stream_session_bench",
}  # fmt: skip


def load_config(path: str | None, overrides: dict | None = None) -> dict:
    cfg = json.loads(json.dumps(DEFAULTS))
    if path:
        user = json.loads(Path(path).read_text())
        for k, v in user.items():
            if isinstance(v, dict) and isinstance(cfg.get(k), dict):
                cfg[k].update(v)
            else:
                cfg[k] = v
    for k, v in (overrides or {}).items():
        if v is not None:
            cfg[k] = v
    if cfg["session_count"] < 1 or cfg["session_duration_s"] <= 0:
        raise ValueError("session_count must be >= 1 and session_duration_s > 0")
    return cfg


def load_control_trace(path: str | None) -> list[dict]:
    """[{"t": seconds from session start, "message": {...sent as is...}}, ...] sorted by time."""
    if not path:
        return []
    events = json.loads(Path(path).read_text())
    events = events["events"] if isinstance(events, dict) else events
    out = [{"t": float(e["t"]), "message": e["message"]} for e in events]
    return sorted(out, key=lambda e: e["t"])


def percentile(xs: list[float], q: float) -> float | None:
    if not xs:
        return None
    xs = sorted(xs)
    k = min(len(xs) - 1, max(0, int(round(q / 100.0 * (len(xs) - 1)))))
    return xs[k]


async def run_session(cfg: dict, index: int, trace: list[dict], events_path: Path | None) -> dict:
    import aiohttp

    ws_url = cfg["server_url"].replace("http://", "ws://").replace("https://", "wss://").rstrip("/") + "/v1/stream/ws"
    tr = cfg["transport"]
    rec: dict = {"index": index, "ok": False, "frames": 0, "chunks": 0}
    events: list[dict] = []
    t_start = time.perf_counter()

    def mark(kind: str, **kw) -> float:
        t = time.perf_counter() - t_start
        events.append({"t": round(t, 6), "event": kind, **kw})
        return t

    session_cfg = {"session_id": f"bench-{index}-{uuid.uuid4().hex[:8]}", "prompt": cfg["prompt"], "fps": cfg["fps"],
                   **cfg["request_extra"]}  # fmt: skip
    if cfg.get("image_path"):
        session_cfg["image_path"] = cfg["image_path"]
    chunk_times: list[float] = []
    control_sent: list[float] = []  # send times of controls not yet followed by a media chunk
    control_lat: list[float] = []
    sent_by_revision: dict[int, float] = {}
    ack_lat: list[float] = []
    applied_lat: list[float] = []  # control sent -> first media chunk that reports its revision (or a later one) as applied
    unapplied: dict[int, float] = {}
    pending_frames = 0
    try:
        timeout = aiohttp.ClientTimeout(total=None, sock_connect=tr["connect_timeout_s"])
        async with aiohttp.ClientSession(timeout=timeout) as http:
            async with http.ws_connect(ws_url, max_msg_size=0, heartbeat=None) as ws:
                rec["connect_ms"] = round(mark("connected") * 1e3, 3)
                await ws.send_str(json.dumps(session_cfg))
                hello = json.loads((await ws.receive(timeout=tr["connect_timeout_s"])).data)
                if hello.get("type") != "session":
                    raise RuntimeError(f"session refused: {hello}")
                rec["session_id"] = hello["session_id"]
                rec["session_open_ms"] = round(mark("session", session_id=hello["session_id"]) * 1e3, 3)
                t_open = time.perf_counter()

                async def controls() -> None:
                    for ev in trace:
                        delay = ev["t"] - (time.perf_counter() - t_open)
                        if delay > 0:
                            await asyncio.sleep(delay)
                        if time.perf_counter() - t_open >= cfg["session_duration_s"]:
                            return
                        message = dict(ev["message"])
                        revision = message.setdefault("revision", len(sent_by_revision) + 1)
                        await ws.send_str(json.dumps(message))
                        now = time.perf_counter()
                        control_sent.append(now)
                        sent_by_revision[revision] = unapplied[revision] = now
                        mark("control", message=message)

                ctl = asyncio.create_task(controls())
                try:
                    while time.perf_counter() - t_open < cfg["session_duration_s"]:
                        left = cfg["session_duration_s"] - (time.perf_counter() - t_open)
                        try:
                            msg = await ws.receive(timeout=min(tr["frame_timeout_s"], max(left, 0.05)))
                        except asyncio.TimeoutError:
                            continue
                        if msg.type == aiohttp.WSMsgType.BINARY:
                            rec["frames"] += 1
                            pending_frames = max(0, pending_frames - 1)
                            if "first_frame_ms" not in rec:
                                rec["first_frame_ms"] = round(mark("first_frame") * 1e3, 3)
                        elif msg.type == aiohttp.WSMsgType.TEXT:
                            body = json.loads(msg.data)
                            data = body.get("data") if isinstance(body.get("data"), dict) else {}
                            if body.get("type") == "chunk" and int(body.get("num_frames", 0)) == 0 and not body.get("error"):
                                # a service message without media (status, control acknowledgement)
                                now = time.perf_counter()
                                if data.get("type") == "control_ack" and data.get("revision") in sent_by_revision:
                                    ack_lat.append((now - sent_by_revision[data["revision"]]) * 1e3)
                                mark("message", message_type=data.get("type"), revision=data.get("revision"))
                                if data.get("type") in ("done", "error") or data.get("done"):
                                    break
                            elif body.get("type") == "chunk":
                                now = time.perf_counter()
                                chunk_times.append(now)
                                rec["chunks"] += 1
                                pending_frames = int(body.get("num_frames", 0))
                                if "first_chunk_ms" not in rec:
                                    rec["first_chunk_ms"] = round((now - t_start) * 1e3, 3)
                                while control_sent and control_sent[0] <= now:  # controls answered by this chunk
                                    control_lat.append((now - control_sent.pop(0)) * 1e3)
                                applied = data.get("control_revision")
                                if isinstance(applied, int):
                                    for rev in [r for r in unapplied if r <= applied]:
                                        applied_lat.append((now - unapplied.pop(rev)) * 1e3)
                                mark("chunk", chunk=body.get("index"), num_frames=body.get("num_frames"), control_revision=applied)
                                if data.get("done"):
                                    break
                            elif body.get("type") in ("done", "error"):
                                mark(body["type"], detail=body.get("error"))
                                if body.get("type") == "error":
                                    rec["error"] = str(body.get("error"))
                                break
                        elif msg.type in (aiohttp.WSMsgType.CLOSE, aiohttp.WSMsgType.CLOSED, aiohttp.WSMsgType.ERROR):
                            break
                finally:
                    ctl.cancel()
                    try:
                        await ws.send_str(json.dumps({"type": "close"}))
                    except Exception:  # noqa: BLE001 - the server may have closed first
                        pass
        rec["ok"] = "error" not in rec
    except Exception as e:  # noqa: BLE001 - a failed session is a data point, not a crash of the run
        rec["error"] = f"{type(e).__name__}: {e}"
    runtime = time.perf_counter() - t_start
    gaps = [(b - a) * 1e3 for a, b in zip(chunk_times, chunk_times[1:])]
    span = (chunk_times[-1] - chunk_times[0]) if len(chunk_times) > 1 else 0.0
    rec.update(session_runtime_s=round(runtime, 3),
               stream_fps=round((rec["frames"] - rec["frames"] / max(rec["chunks"], 1)) / span, 3) if span > 0 else None,
               chunk_gap_ms_p50=percentile(gaps, 50), chunk_gap_ms_p99=percentile(gaps, 99),
               control_to_next_chunk_ms_p50=percentile(control_lat, 50),
               control_to_next_chunk_ms_p99=percentile(control_lat, 99), controls_sent=len(control_lat) + len(control_sent),
               control_ack_ms_p50=percentile(ack_lat, 50), control_ack_ms_p99=percentile(ack_lat, 99),
               control_applied_ms_p50=percentile(applied_lat, 50), control_applied_ms_p99=percentile(applied_lat, 99))  # fmt: skip
    if events_path is not None:
        events_path.write_text("".join(json.dumps(e) + "\n" for e in events))
    return rec


async def sample_server_metrics(cfg: dict, out_path: Path, stop: asyncio.Event) -> None:
    import aiohttp

    sm = cfg["server_metrics"]
    async with aiohttp.ClientSession() as http:
        with out_path.open("w") as f:
            while not stop.is_set():
                for url in sm["urls"]:
                    try:
                        async with http.get(url, timeout=aiohttp.ClientTimeout(total=5)) as r:
                            f.write(json.dumps({"t": time.time(), "url": url, "status": r.status, "body": await r.text()}) + "\n")
                    except Exception as e:  # noqa: BLE001
                        f.write(json.dumps({"t": time.time(), "url": url, "error": str(e)}) + "\n")
                try:
                    await asyncio.wait_for(stop.wait(), timeout=sm["collection_interval_s"])
                except asyncio.TimeoutError:
                    pass


async def run(cfg: dict) -> dict:
    art = Path(cfg["artifacts_dir"])
    art.mkdir(parents=True, exist_ok=True)
    trace = load_control_trace(cfg["control_trace_path"])
    stop = asyncio.Event()
    sampler = None
    if cfg["server_metrics"]["enabled"] and cfg["server_metrics"]["urls"]:
        sampler = asyncio.create_task(sample_server_metrics(cfg, art / "server_metrics.jsonl", stop))
    for w in range(cfg["warmup_sessions"]):
        await run_session(cfg, -1 - w, trace, None)

    async def staggered(i: int) -> dict:
        await asyncio.sleep(i * cfg["stagger_s"])
        return await run_session(cfg, i, trace, art / f"events_{i}.jsonl")

    t0 = time.perf_counter()
    sessions = await asyncio.gather(*(staggered(i) for i in range(cfg["session_count"])))
    wall = time.perf_counter() - t0
    stop.set()
    if sampler is not None:
        await sampler
    (art / "sessions.jsonl").write_text("".join(json.dumps(s) + "\n" for s in sessions))
    good = [s for s in sessions if s["ok"]]

    def agg(key: str) -> dict | None:
        xs = [s[key] for s in good if s.get(key) is not None]
        return {"mean": round(statistics.fmean(xs), 3), "p50": percentile(xs, 50), "p99": percentile(xs, 99)} if xs else None

    summary = {"sessions": len(sessions), "success_rate": round(len(good) / len(sessions), 4), "wall_s": round(wall, 3),
               "frames_received": sum(s["frames"] for s in sessions), "chunks_received": sum(s["chunks"] for s in sessions),
               **{k: agg(k) for k in ("connect_ms", "session_open_ms", "first_chunk_ms", "first_frame_ms", "stream_fps",
                                      "chunk_gap_ms_p50", "chunk_gap_ms_p99", "control_to_next_chunk_ms_p50",
                                      "control_to_next_chunk_ms_p99", "control_ack_ms_p50", "control_applied_ms_p50",
                                      "session_runtime_s")},
               "config": {k: cfg[k] for k in ("server_url", "fps", "session_count", "warmup_sessions", "session_duration_s",
                                              "stagger_s", "control_trace_path", "request_extra")}}  # fmt: skip
    (art / "summary.json").write_text(json.dumps(summary, indent=1))
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config")
    ap.add_argument("--server-url")
    ap.add_argument("--session-count", type=int)
    ap.add_argument("--session-duration-s", type=float)
    ap.add_argument("--warmup-sessions", type=int)
    ap.add_argument("--artifacts-dir")
    a = ap.parse_args(argv)
    cfg = load_config(a.config, {"server_url": a.server_url, "session_count": a.session_count,
                                 "session_duration_s": a.session_duration_s, "warmup_sessions": a.warmup_sessions,
                                 "artifacts_dir": a.artifacts_dir})  # fmt: skip
    summary = asyncio.run(run(cfg))
    print(json.dumps(summary))
    return 0 if summary["success_rate"] == 1.0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
