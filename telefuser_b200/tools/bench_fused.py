"""Micro-benchmarks of the peer-memory (fused) collectives against their NCCL compositions.

Run under `python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P
-m telefuser_b200.tools.bench_fused [--seq 75600 --heads 40 --dim 5120 --ffn 13824]`. Every case is timed on
the device with CUDA events after warm-up, an L2 flush between iterations, and the maximum over ranks is
reported; rank 0 prints one JSON line per case with both times, the bytes this rank must move over NVLink, and the
fraction of the measured per-direction link bandwidth (770 GB/s) or of the measured GEMM peak that the fused
form reaches.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import ring, symm, tp_fused, ulysses

LINK_GBS = 770.0  # measured peer copy, per direction per GPU


def _peak_tflops() -> float:
    try:
        here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:  # noqa: BLE001 - fall back to the earlier measurement on this class of machine
        return 1590.0


class Bench:
    def __init__(self, group, device, iters: int = 5, warmup: int = 3) -> None:
        self.group, self.device, self.iters, self.warmup = group, device, iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def time(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            self.flush.zero_()
            dist.barrier(group=self.group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        t = torch.tensor([total / self.iters], device=self.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t)

    def report(self, name: str, fused_ms: float, nccl_ms: float, link_bytes: float = 0.0, flops: float = 0.0, **cfg) -> None:
        if dist.get_rank(self.group) != 0:
            return
        row = {"case": name, "fused_ms": round(fused_ms, 4), "nccl_ms": round(nccl_ms, 4), "speedup": round(nccl_ms / fused_ms, 3),
               "world": dist.get_world_size(self.group), **cfg}  # fmt: skip
        floor_ms = max(link_bytes / (LINK_GBS * 1e6), flops / (_peak_tflops() * 1e9))
        if floor_ms > 0:
            row.update(roofline_ms=round(floor_ms, 4), frac_of_roofline=round(floor_ms / fused_ms, 3), peaks="of measured")
        print(json.dumps(row), flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=75600)
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--dim", type=int, default=5120)
    ap.add_argument("--ffn", type=int, default=13824)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    P, rank = dist.get_world_size(), dist.get_rank()
    b = Bench(group, dev, args.iters)
    H, D, C = args.heads, 128, args.dim
    S = args.seq // (8 * P) * 8 * P
    S_loc = S // P
    torch.manual_seed(rank)
    try:
        q, k, v = (torch.randn(1, S_loc, H, D, device=dev).bfloat16() for _ in range(3))
        attn_flops = 4.0 * S_loc * S * H * D  # this rank's share of the full attention
        # Ulysses: sequence shards -> head shards by peer stores, attention, output rows stored back to their owners
        if H % P == 0:
            ws = symm.PeerWorkspace(group, 4 * (S_loc * H * D * 2 + 256) + 4096)
            fused = b.time(lambda: symm.ulysses_attention_fused(q, k, v, ws))
            nccl = b.time(lambda: ulysses.gather_heads(TF.attention(*(ulysses.scatter_heads(t, group) for t in (q, k, v))), group))
            b.report("ulysses_attention", fused, nccl, link_bytes=4 * S_loc * H * D * 2 * (P - 1) / P, flops=attn_flops, seq=S, heads=H)
            ws.close()
        # context parallel: K / V all-gathered once by peer stores vs NCCL ring steps
        ws = symm.PeerWorkspace(group, symm.ring_workspace_bytes(S_loc, H, D, P))
        fused = b.time(lambda: symm.ring_attention_fused(q, k, v, ws))
        nccl = b.time(lambda: ring.ring_attention(q, k, v, group))
        b.report("ring_attention", fused, nccl, link_bytes=2 * S_loc * H * D * 2 * (P - 1), flops=attn_flops, seq=S, heads=H)
        ws.close()
        del q, k, v
        # tensor-parallel MLP: column-parallel up (all-gather -> GEMM), row-parallel down (GEMM -> all-reduce)
        M = S // P * P
        ws = symm.PeerWorkspace(group, 3 * M * C * 2 + (64 << 20))
        x_rows = torch.randn(M // P, C, device=dev).bfloat16()
        w_up = (torch.randn(args.ffn // P // 8 * 8, C, device=dev) / C**0.5).bfloat16()
        h = torch.randn(M, w_up.shape[0], device=dev).bfloat16()
        w_down = (torch.randn(C, w_up.shape[0], device=dev) / C**0.5).bfloat16()
        res = torch.randn(M, C, device=dev).bfloat16()
        fused = b.time(lambda: tp_fused.all_gather_gemm(x_rows, w_up, None, "gelu_tanh", group, ws))
        nccl = b.time(lambda: tp_fused.all_gather_gemm(x_rows, w_up, None, "gelu_tanh", group, None))
        b.report("all_gather_gemm", fused, nccl, link_bytes=(P - 1) * x_rows.numel() * 2, flops=2.0 * M * w_up.shape[0] * C, m=M, n=w_up.shape[0], k=C)
        fused = b.time(lambda: tp_fused.gemm_all_reduce(h, w_down, None, res, None, group, ws))
        nccl = b.time(lambda: tp_fused.gemm_all_reduce(h, w_down, None, res, None, group, None))
        b.report("gemm_all_reduce", fused, nccl, link_bytes=2 * (P - 1) / P * M * C * 2, flops=2.0 * M * C * w_up.shape[0], m=M, n=C, k=w_up.shape[0])
        ws.close()
        # row all-gather of the head output
        ws = symm.PeerWorkspace(group, M * 64 * 2 + (1 << 20))
        y = torch.randn(M // P, 64, device=dev).bfloat16()
        parts = torch.empty(M, 64, device=dev, dtype=torch.bfloat16)
        fused = b.time(lambda: symm.all_gather_rows_fused(y, ws))
        nccl = b.time(lambda: dist.all_gather_into_tensor(parts, y, group=group))
        b.report("all_gather_rows", fused, nccl, link_bytes=(P - 1) * y.numel() * 2, rows=M // P, cols=64)
        ws.close()
    finally:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
