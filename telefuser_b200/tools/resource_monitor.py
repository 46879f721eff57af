"""Resource monitor for a serving deployment: samples GPU memory / utilisation (NVML, read-only) and the memory of the
service's processes over hours, and tells a leak from a plateau.

    python -m telefuser_b200.tools.resource_monitor record --match "telefuser serve" -i 5 -m 3600 -o run.csv
    python -m telefuser_b200.tools.resource_monitor report run.csv --warmup-s 600 --leak-mb-per-hour 50

`record` writes one CSV row per interval: wall time, per-GPU used memory and utilisation, and the summed RSS / thread
count / open files of every process whose command line contains `--match` (or the given `--pid` and its children).
`report` fits a line through every series after the warm-up window and prints, per series, first / last / min / max,
the slope per hour and whether the growth is a leak: slope above the threshold AND the last quarter of the run still
rising (a cache that fills and plateaus is not flagged), OR the local maxima of the series rise faster than the threshold:
a serving process breathes with its requests, and the trend of its peaks shows what each request leaves behind.
`--plot` also draws every series (smoothed) as one line of characters.

Role: tools/deploy/docker_monitor.py (sampling a running deployment into a CSV) and tools/deploy/show_stat.py
(moving average, peak trend, leak-trend summary) of the reference, for processes instead of containers and with a textual
verdict and terminal plots instead of matplotlib figures.
"""

from __future__ import annotations

import argparse
import csv
import json
import sys
import time


# ---------------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------------
def process_sample(match: str | None, pid: int | None, psutil_mod=None) -> dict:
    """Summed memory / threads / open files of the watched processes (matching command lines, or a pid with its children)."""
    ps = psutil_mod
    if ps is None:
        import psutil as ps
    procs = []
    if pid is not None:
        try:
            root = ps.Process(pid)
            procs = [root] + root.children(recursive=True)
        except ps.Error:
            procs = []
    elif match:
        me = ps.Process().pid
        for p in ps.process_iter(["pid", "cmdline"]):
            try:
                if p.info["pid"] != me and match in " ".join(p.info["cmdline"] or []):
                    procs.append(p)
            except ps.Error:
                continue
    rss = threads = files = 0
    alive = 0
    for p in procs:
        try:
            with p.oneshot():
                rss += p.memory_info().rss
                threads += p.num_threads()
                try:
                    files += p.num_fds()
                except (ps.Error, AttributeError):
                    pass
            alive += 1
        except ps.Error:
            continue
    return {"processes": alive, "rss_mb": round(rss / 2**20, 2), "threads": threads, "open_files": files}


def gpu_sample(collector=None) -> dict:
    if collector is None:
        from telefuser_b200.metrics.service_metrics import GPUCollector

        collector = GPUCollector()
    out = {}
    for g in collector.sample():
        out[f"gpu{g['index']}_mem_mb"] = round(g["mem_used_mb"], 1)
        out[f"gpu{g['index']}_util"] = g["util"]
    return out


def record(path: str, interval_s: float, max_seconds: float, match: str | None, pid: int | None, collector=None,
           psutil_mod=None, clock=time.time, sleep=time.sleep) -> int:  # fmt: skip
    """Appends one row per interval until `max_seconds` have passed (or the watched pid is gone). Returns the row count."""
    t0, rows, writer = clock(), 0, None
    with open(path, "w", newline="") as f:
        while True:
            now = clock()
            row = {"t": round(now - t0, 3), **gpu_sample(collector), **process_sample(match, pid, psutil_mod)}
            if writer is None:
                writer = csv.DictWriter(f, fieldnames=list(row))
                writer.writeheader()
            writer.writerow({k: row.get(k, "") for k in writer.fieldnames})
            f.flush()
            rows += 1
            if now - t0 + interval_s > max_seconds or (pid is not None and row["processes"] == 0):
                return rows
            sleep(interval_s)


# ---------------------------------------------------------------------------------------------------
# report
# ---------------------------------------------------------------------------------------------------
def fit_slope(ts: list[float], ys: list[float]) -> float:
    """Least-squares slope (units of y per second)."""
    n = len(ts)
    if n < 2:
        return 0.0
    mt, my = sum(ts) / n, sum(ys) / n
    den = sum((t - mt) ** 2 for t in ts)
    return 0.0 if den == 0 else sum((t - mt) * (y - my) for t, y in zip(ts, ys)) / den


def local_maxima(ys: list[float], window: int = 5) -> list[int]:
    """Indices whose value exceeds every sample up to `window` places before them and is not exceeded by any up to
    `window` places after them (so a plateau counts once, at its start)."""
    out = []
    for i, y in enumerate(ys):
        left, right = ys[max(0, i - window) : i], ys[i + 1 : i + window + 1]
        if (not left or y > max(left)) and (not right or y >= max(right)):
            out.append(i)
    return out


def moving_average(ys: list[float], window: int) -> list[float]:
    out, acc = [], 0.0
    for i, y in enumerate(ys):
        acc += y
        if i >= window:
            acc -= ys[i - window]
        out.append(acc / min(i + 1, window))
    return out


def sparkline(ys: list[float], width: int = 72) -> str:
    """One line of block characters for a series (resampled to `width` points by averaging)."""
    if not ys:
        return ""
    bars = " .:-=+*#%@"
    step = max(1, len(ys) // width)
    pts = [sum(ys[i : i + step]) / len(ys[i : i + step]) for i in range(0, len(ys), step)]
    lo, hi = min(pts), max(pts)
    return "".join(bars[int((p - lo) / (hi - lo) * (len(bars) - 1))] if hi > lo else bars[0] for p in pts)


def analyse(rows: list[dict], warmup_s: float = 0.0, leak_per_hour: float = 50.0) -> dict:
    """Per numeric series: summary statistics, slope per hour after the warm-up, and the leak verdict for memory series."""
    if not rows:
        return {}
    keys = [k for k in rows[0] if k != "t"]
    out = {}
    for k in keys:
        pts = [(float(r["t"]), float(r[k])) for r in rows if r.get(k) not in ("", None) and float(r["t"]) >= warmup_s]
        if len(pts) < 2:
            continue
        ts, ys = [p[0] for p in pts], [p[1] for p in pts]
        slope_h = fit_slope(ts, ys) * 3600.0
        tail = pts[len(pts) * 3 // 4 :]
        tail_slope_h = fit_slope([p[0] for p in tail], [p[1] for p in tail]) * 3600.0 if len(tail) >= 2 else 0.0
        entry = {"first": ys[0], "last": ys[-1], "min": min(ys), "max": max(ys), "mean": round(sum(ys) / len(ys), 3),
                 "slope_per_hour": round(slope_h, 3), "tail_slope_per_hour": round(tail_slope_h, 3)}  # fmt: skip
        # a serving process breathes with its requests: the trend of its PEAKS says more about a leak than the mean does
        peaks = local_maxima(ys, max(2, len(ys) // 40))
        peak_slope_h = fit_slope([ts[i] for i in peaks], [ys[i] for i in peaks]) * 3600.0 if len(peaks) >= 3 else None
        entry["peaks"] = len(peaks)
        entry["peak_slope_per_hour"] = None if peak_slope_h is None else round(peak_slope_h, 3)
        if k.endswith("_mb"):
            by_mean = slope_h > leak_per_hour and tail_slope_h > leak_per_hour / 2
            by_peaks = peak_slope_h is not None and peak_slope_h > leak_per_hour and slope_h > 0
            entry["leak"] = bool(by_mean or by_peaks)
        out[k] = entry
    return out


def report(path: str, warmup_s: float, leak_per_hour: float) -> dict:
    with open(path, newline="") as f:
        rows = list(csv.DictReader(f))
    series = analyse(rows, warmup_s, leak_per_hour)
    leaks = sorted(k for k, v in series.items() if v.get("leak"))
    return {"file": path, "samples": len(rows), "duration_s": float(rows[-1]["t"]) if rows else 0.0, "warmup_s": warmup_s,
            "leak_threshold_mb_per_hour": leak_per_hour, "leaking_series": leaks, "series": series}  # fmt: skip


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("record")
    r.add_argument("--match", default=None, help="substring of the command lines to watch")
    r.add_argument("--pid", type=int, default=None, help="watch this process and its children instead")
    r.add_argument("-i", "--interval", type=float, default=5.0)
    r.add_argument("-m", "--max-seconds", type=float, default=3600.0)
    r.add_argument("-o", "--output", default="resource_monitor.csv")
    p = sub.add_parser("report")
    p.add_argument("csv")
    p.add_argument("--warmup-s", type=float, default=0.0)
    p.add_argument("--leak-mb-per-hour", type=float, default=50.0)
    p.add_argument("--plot", action="store_true", help="also draw every series as a line of characters (smoothed)")
    a = ap.parse_args(argv)
    if a.cmd == "record":
        n = record(a.output, a.interval, a.max_seconds, a.match, a.pid)
        print(json.dumps({"rows": n, "output": a.output}))
        return 0
    rep = report(a.csv, a.warmup_s, a.leak_mb_per_hour)
    print(json.dumps(rep, indent=1))
    if a.plot:
        with open(a.csv, newline="") as f:
            rows = [r for r in csv.DictReader(f) if float(r["t"]) >= a.warmup_s]
        for k in rep["series"]:
            ys = [float(r[k]) for r in rows if r.get(k) not in ("", None)]
            print(f"{k:>24} {sparkline(moving_average(ys, max(1, len(ys) // 50)))}")
    return 1 if rep["leaking_series"] else 0


if __name__ == "__main__":
    sys.exit(main())
