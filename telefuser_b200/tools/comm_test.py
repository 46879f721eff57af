"""Node communication check: host <-> device copies, collectives and this package's peer-memory kernels.

`python -m telefuser_b200.tools.comm_test` (one GPU: pinned H2D / D2H bandwidth), or under
`torchrun --nproc-per-node N --master-addr 127.0.0.1 -m telefuser_b200.tools.comm_test [--sizes-mb 16 256]`
(all-reduce, all-gather, all-to-all, ring send/recv through NCCL, and the peer-store row all-gather used by the
fused paths), each timed with CUDA events after warm-up, maximum over ranks, reported as algorithm and bus
bandwidth. With `--backend gloo` the same plan runs on CPU with wall-clock timing (plumbing check only).
Role parity: tools/deploy/multi_device_communication_test.py:18-429.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def environment() -> dict:
    info = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(), "nccl": None, "devices": []}
    if torch.cuda.is_available():
        info["nccl"] = ".".join(str(x) for x in torch.cuda.nccl.version()) if hasattr(torch.cuda, "nccl") else None
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "memory_gb": round(p.total_memory / 2**30, 1),
                                    "sms": p.multi_processor_count})  # fmt: skip
        n = torch.cuda.device_count()
        info["peer_access"] = [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
    return info


class _Timer:
    """CUDA events on the current stream when on a GPU, wall clock otherwise."""

    def __init__(self, device: torch.device) -> None:
        self.cuda = device.type == "cuda"

    def run(self, fn, warmup: int, iters: int) -> float:
        for _ in range(warmup):
            fn()
        if self.cuda:
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / 1e3 / iters
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        return (time.perf_counter() - t0) / iters


def host_device_bandwidth(device: torch.device, size_mb: int, warmup: int = 3, iters: int = 10) -> dict:
    n = size_mb << 20
    host = torch.empty(n, dtype=torch.uint8, pin_memory=device.type == "cuda")
    dev = torch.empty(n, dtype=torch.uint8, device=device)
    t = _Timer(device)
    h2d = t.run(lambda: dev.copy_(host, non_blocking=True), warmup, iters)
    d2h = t.run(lambda: host.copy_(dev, non_blocking=True), warmup, iters)
    return {"size_mb": size_mb, "h2d_gbs": n / h2d / 1e9, "d2h_gbs": n / d2h / 1e9}


def _max_over_ranks(seconds: float, device: torch.device, group) -> float:
    t = torch.tensor([seconds], dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def collective_bandwidth(device: torch.device, size_mb: int, group=None, warmup: int = 3, iters: int = 10, peer: bool = True) -> dict:
    """Per-collective seconds (max over ranks), algorithm bandwidth (payload / time) and bus bandwidth (NCCL convention)."""
    P, rank = dist.get_world_size(group), dist.get_rank(group)
    dt = torch.bfloat16 if device.type == "cuda" else torch.float32
    n = (size_mb << 20) // torch.empty(0, dtype=dt).element_size() // P * P
    x = torch.ones(n, dtype=dt, device=device)
    shard = torch.ones(n // P, dtype=dt, device=device)
    gathered = torch.empty(n, dtype=dt, device=device)
    a2a_out = torch.empty_like(x)
    nbytes = n * x.element_size()
    timer = _Timer(device)
    plan = {
        "all_reduce": (lambda: dist.all_reduce(x, group=group), 2 * (P - 1) / P),
        "all_gather": (lambda: dist.all_gather_into_tensor(gathered, shard, group=group), (P - 1) / P),
        "all_to_all": (lambda: dist.all_to_all_single(a2a_out, x, group=group), (P - 1) / P),
    }
    if device.type != "cuda":  # gloo: list-form all-gather, no all-to-all
        parts = [torch.empty_like(shard) for _ in range(P)]
        plan["all_gather"] = (lambda: dist.all_gather(parts, shard, group=group), (P - 1) / P)
        plan.pop("all_to_all")
    if P > 1:
        nxt, prv = (rank + 1) % P, (rank - 1) % P
        recv = torch.empty_like(shard)

        def ring_step():
            for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, shard, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]):
                w.wait()

        plan["send_recv_ring"] = (ring_step, 1 / P)
    out = {"size_mb": size_mb, "world": P}
    for name, (fn, bus_factor) in plan.items():
        sec = _max_over_ranks(timer.run(fn, warmup, iters), device, group)
        out[name] = {"ms": sec * 1e3, "alg_gbs": nbytes / sec / 1e9, "bus_gbs": nbytes * bus_factor / sec / 1e9}
    if peer and device.type == "cuda" and P > 1:
        from telefuser_b200.parallel import symm

        rows, cols = n // P // 4096, 4096
        if rows > 0:
            ws = symm.PeerWorkspace(group, rows * P * cols * 2 + (1 << 20))
            xl = torch.ones(rows, cols, dtype=torch.bfloat16, device=device)
            sec = _max_over_ranks(timer.run(lambda: symm.all_gather_rows_fused(xl, ws), warmup, iters), device, group)
            b = rows * P * cols * 2
            out["peer_store_all_gather"] = {"ms": sec * 1e3, "alg_gbs": b / sec / 1e9, "bus_gbs": b * (P - 1) / P / sec / 1e9}
            ws.close()
    return out


def format_report(report: dict) -> str:
    lines = [f"torch {report['environment']['torch']}  NCCL {report['environment'].get('nccl')}  world {report.get('world', 1)}"]
    for d in report["environment"]["devices"]:
        lines.append(f"  GPU {d['index']}: {d['name']} sm_{d['sm']} {d['memory_gb']} GB, {d['sms']} SMs")
    for r in report.get("host_device", []):
        lines.append(f"host<->device {r['size_mb']:>5} MB: H2D {r['h2d_gbs']:.1f} GB/s, D2H {r['d2h_gbs']:.1f} GB/s")
    for r in report.get("collectives", []):
        for name, v in r.items():
            if isinstance(v, dict):
                lines.append(f"{name:<22} {r['size_mb']:>5} MB: {v['ms']:.3f} ms, alg {v['alg_gbs']:.1f} GB/s, bus {v['bus_gbs']:.1f} GB/s")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Communication bandwidth check for one node")
    ap.add_argument("--sizes-mb", type=int, nargs="+", default=[16, 256])
    ap.add_argument("--backend", default=None, help="nccl (default on GPUs) or gloo")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", type=str, help="write the report to this file (rank 0)")
    ap.add_argument("--no-peer", action="store_true", help="skip the peer-memory kernels")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    backend = args.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    use_cuda = backend == "nccl" and torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    report = {"environment": environment(), "world": world, "backend": backend}
    if use_cuda or world == 1:
        report["host_device"] = [host_device_bandwidth(device, s, iters=args.iters) for s in args.sizes_mb]
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29555")
        dist.init_process_group(backend, device_id=device if use_cuda else None)
        try:
            report["collectives"] = [collective_bandwidth(device, s, iters=args.iters, peer=not args.no_peer) for s in args.sizes_mb]
        finally:
            dist.destroy_process_group()
    if int(os.environ.get("RANK", "0")) == 0:
        print(format_report(report))
        if args.json:
            with open(args.json, "w") as f:
                json.dump(report, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
