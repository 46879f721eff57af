"""Client-side load generator for the batch generation service (`telefuser serve`): submits generation tasks over
the HTTP task API, waits for each result, and reports end-to-end latency and throughput.

    python benchmarks/video_generation_bench.py --config benchmarks/configs/video_generation_quick.json

Workload (`profiling`): `type` "e2e" sends `requests` tasks with at most `concurrency` in flight, each as soon as a
slot frees; "poisson" draws exponential gaps for an average arrival `rate` (requests per second) and still caps the
number in flight at `concurrency`; "constant" spaces arrivals 1 / rate apart. Prompts come from a JSONL file (one
`{"text": ..., "image": optional path}` per line, used in order, cycled). For every request the harness records the
submit time, queue wait and run time as the service reports them, the client-side end-to-end latency, and the final
status; the summary holds request throughput, latency mean / p50 / p90 / p99 and the failure count. Output:
`records.jsonl` and `summary.json` in `artifacts_dir`, the summary also printed as one JSON line.

Role: the reference measures its service with an external load tool configured by
benchmarks/telefuser_aiperf/configs/video_generation_{quick,e2e,rate}.yaml; this is the in-tree equivalent on the
task API (`POST /v1/tasks/create`, `GET /v1/tasks/{id}/status`), with the same workload fields.
"""

from __future__ import annotations

import argparse
import json
import random
import statistics
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

DEFAULTS = {
    "server_url": "http://127.0.0.1:8000", "task": "t2v", "timeout_s": 3600.0, "poll_interval_s": 0.5, "random_seed": 42,
    "extra": {}, "dataset": {"path": "benchmarks/data/video_prompts.jsonl"},
    "profiling": {"type": "e2e", "rate": 0.2, "concurrency": 1, "requests": 4},
    "artifacts_dir": "artifacts/video_generation_bench",
}  # fmt: skip


def load_config(path: str | None, overrides: dict | None = None) -> dict:
    cfg = json.loads(json.dumps(DEFAULTS))
    if path:
        for k, v in json.loads(Path(path).read_text()).items():
            if isinstance(v, dict) and isinstance(cfg.get(k), dict):
                cfg[k].update(v)
            else:
                cfg[k] = v
    for k, v in (overrides or {}).items():
        if v is not None:
            if k in ("rate", "concurrency", "requests", "type"):
                cfg["profiling"][k] = v
            else:
                cfg[k] = v
    p = cfg["profiling"]
    if p["type"] not in ("e2e", "poisson", "constant") or p["requests"] < 1 or p["concurrency"] < 1:
        raise ValueError(f"bad profiling section: {p}")
    if p["type"] != "e2e" and not p["rate"] > 0:
        raise ValueError("rate must be positive for poisson / constant arrivals")
    return cfg


def load_prompts(path: str) -> list[dict]:
    rows = [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]
    if not rows:
        raise ValueError(f"{path} holds no prompt")
    return rows


def arrival_times(cfg: dict) -> list[float]:
    """Planned submit times (seconds from the start) of every request."""
    p = cfg["profiling"]
    if p["type"] == "e2e":
        return [0.0] * p["requests"]
    rng = random.Random(cfg["random_seed"])
    t, out = 0.0, []
    for _ in range(p["requests"]):
        out.append(t)
        t += rng.expovariate(p["rate"]) if p["type"] == "poisson" else 1.0 / p["rate"]
    return out


def percentile(xs: list[float], q: float) -> float | None:
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, max(0, int(round(q / 100.0 * (len(xs) - 1)))))]


def one_request(cfg: dict, index: int, prompt: dict, planned: float, t0: float, slots: threading.Semaphore) -> dict:
    from telefuser_b200.client.tf_client import TFClient

    delay = planned - (time.perf_counter() - t0)
    if delay > 0:
        time.sleep(delay)
    rec: dict = {"index": index, "planned_s": round(planned, 3), "status": "error"}
    with slots:
        t_submit = time.perf_counter()
        rec["submit_s"] = round(t_submit - t0, 3)
        try:
            with TFClient(cfg["server_url"], timeout=int(cfg["timeout_s"])) as c:
                params = {"prompt": prompt.get("text", ""), **cfg["extra"]}
                if prompt.get("image") and cfg["task"] != "t2v":
                    params["first_image_path"] = prompt["image"]
                task = c.create_task(cfg["task"], **params)
                rec["task_id"] = task["task_id"]
                final = c.wait_for_completion(task["task_id"], poll_interval=cfg["poll_interval_s"], timeout=cfg["timeout_s"])
                rec["status"] = final.get("status", "unknown")
                for k in ("queue_time", "processing_time", "error"):
                    if final.get(k) is not None:
                        rec[k] = final[k]
        except Exception as e:  # noqa: BLE001 - a failed request is a data point
            rec["error"] = f"{type(e).__name__}: {e}"
        rec["latency_s"] = round(time.perf_counter() - t_submit, 4)
    return rec


def run(cfg: dict) -> dict:
    art = Path(cfg["artifacts_dir"])
    art.mkdir(parents=True, exist_ok=True)
    prompts = load_prompts(cfg["dataset"]["path"])
    plan = arrival_times(cfg)
    slots = threading.Semaphore(cfg["profiling"]["concurrency"])
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=max(cfg["profiling"]["concurrency"] * 2, 4)) as pool:
        futs = [pool.submit(one_request, cfg, i, prompts[i % len(prompts)], plan[i], t0, slots) for i in range(len(plan))]
        records = [f.result() for f in futs]
    wall = time.perf_counter() - t0
    (art / "records.jsonl").write_text("".join(json.dumps(r) + "\n" for r in records))
    ok = [r for r in records if r["status"] == "completed"]
    lat = [r["latency_s"] for r in ok]
    summary = {"requests": len(records), "completed": len(ok), "failed": len(records) - len(ok), "wall_s": round(wall, 3),
               "throughput_rps": round(len(ok) / wall, 5) if wall > 0 else None,
               "latency_s": {"mean": round(statistics.fmean(lat), 4) if lat else None, "p50": percentile(lat, 50),
                             "p90": percentile(lat, 90), "p99": percentile(lat, 99)},
               "config": {"server_url": cfg["server_url"], "task": cfg["task"], "profiling": cfg["profiling"], "extra": cfg["extra"]}}  # fmt: skip
    (art / "summary.json").write_text(json.dumps(summary, indent=1))
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config")
    ap.add_argument("--server-url")
    ap.add_argument("--type", choices=["e2e", "poisson", "constant"])
    ap.add_argument("--rate", type=float)
    ap.add_argument("--concurrency", type=int)
    ap.add_argument("--requests", type=int)
    ap.add_argument("--artifacts-dir")
    a = ap.parse_args(argv)
    cfg = load_config(a.config, {"server_url": a.server_url, "type": a.type, "rate": a.rate, "concurrency": a.concurrency,
                                 "requests": a.requests, "artifacts_dir": a.artifacts_dir})  # fmt: skip
    summary = run(cfg)
    print(json.dumps(summary))
    return 0 if summary["failed"] == 0 else 1


if __name__ == "__main__":
    import sys

    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    raise SystemExit(main())
