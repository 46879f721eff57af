"""SPMD check of the peer-memory paths against the collective-library paths on real GPUs.

Run as `world_size` NCCL ranks (one per GPU). Every rank builds the same random q/k/v, shards them
over the sequence, and compares, for several "layers" in a row (slab reuse, barrier epochs):
fused Ulysses attention vs scatter_heads -> attention -> gather_heads; the CFG combine + Euler step
over peer memory vs all-gather + local kernel; the row all-gather vs `dist.all_gather`.
Rank 0 writes the maximum errors to `out_path`.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import native
from telefuser_b200.parallel import symm, ulysses


def tp_fused_errors(group, dev, ws, M: int = 1400, K: int = 1024, N: int = 768, rounds: int = 2) -> dict:
    """Relative errors of the fused tensor-parallel linears (peer workspace `ws`, or None for the collective
    composition) against the unsharded fp32 product; every rank builds the same full operands."""
    from telefuser_b200.parallel import tp_fused

    rank, P = dist.get_rank(group), dist.get_world_size(group)
    out = {"tp_rs": 0.0, "tp_ar": 0.0, "tp_ag": 0.0}
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()  # noqa: E731
    for it in range(rounds):
        g = torch.Generator().manual_seed(300 + it)
        x = (torch.randn(M, K, generator=g) / 4).to(dt)
        w = (torch.randn(N, K, generator=g) / K**0.5).to(dt)
        bias = torch.randn(N, generator=g).to(dt)
        res = torch.randn(M, N, generator=g).to(dt)
        gate = torch.randn(1, N, generator=g)
        full = res.float() + gate * (x.float() @ w.float().t() + bias.float())
        kc, seg = K // P, M // P
        xs, wsh = x[:, rank * kc : (rank + 1) * kc].to(dev), w[:, rank * kc : (rank + 1) * kc].to(dev)
        b = bias.to(dev) if rank == 0 else None
        mine = slice(rank * seg, (rank + 1) * seg)
        got = tp_fused.gemm_reduce_scatter(xs, wsh, b, res[mine].to(dev), gate.to(dev), group, ws)
        out["tp_rs"] = max(out["tp_rs"], rel(got.cpu(), full[mine]))
        got = tp_fused.gemm_all_reduce(xs, wsh, b, res.to(dev), gate.to(dev), group, ws)
        out["tp_ar"] = max(out["tp_ar"], rel(got.cpu(), full))
        nc = N // P  # column-parallel weight shard on row-sharded activations
        want = torch.nn.functional.gelu(x.float() @ w[rank * nc : (rank + 1) * nc].float().t() + bias[rank * nc : (rank + 1) * nc].float(),
                                        approximate="tanh")  # fmt: skip
        got = tp_fused.all_gather_gemm(x[mine].to(dev), w[rank * nc : (rank + 1) * nc].to(dev), bias[rank * nc : (rank + 1) * nc].to(dev),
                                       "gelu_tanh", group, ws, n_copiers=4)  # fmt: skip
        out["tp_ag"] = max(out["tp_ag"], rel(got.cpu(), want))
    return out


def rank_main(rank: int, world_size: int, port: int, out_path: str, seq: int = 512, heads: int = 8, layers: int = 3):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0")  # fmt: skip
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world_size, device_id=dev)
    errs = {}
    try:
        group = dist.group.WORLD
        P, D, B = world_size, 128, 1
        S_loc = seq // P
        ws = symm.PeerWorkspace(group, 4 * (B * S_loc * heads * D * 2 + 256) + (32 << 20))
        worst = 0.0
        for layer in range(layers):
            g = torch.Generator(device="cpu").manual_seed(100 + layer)
            qkv = torch.randn(B, seq, 3 * heads * D, generator=g).bfloat16()
            mine = qkv[:, rank * S_loc : (rank + 1) * S_loc].to(dev)  # fused projection output of this rank
            q, k, v = (mine[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)) for i in range(3))
            hq, hk, hv = (ulysses.scatter_heads(t.contiguous(), group) for t in (q, k, v))
            want = ulysses.gather_heads(TF.attention(hq, hk, hv), group)
            got = symm.ulysses_attention_fused(q, k, v, ws)
            worst = max(worst, (got.float() - want.float()).abs().max().item())
        errs["ulysses"] = worst
        # row all-gather, twice (region reuse)
        worst = 0.0
        for it in range(2):
            x = torch.full((37, 256), float(rank + 1 + 10 * it), device=dev).bfloat16()
            parts = [torch.empty_like(x) for _ in range(P)]
            dist.all_gather(parts, x, group=group)
            got = symm.all_gather_rows_fused(x, ws)
            worst = max(worst, (got.float() - torch.cat(parts).float()).abs().max().item())
        errs["gather"] = worst
        # context-parallel attention: K / V exchanged by peer stores vs the NCCL ring and vs attention over the full sequence
        from telefuser_b200.parallel import ring

        rws = symm.PeerWorkspace(group, symm.ring_workspace_bytes(S_loc, heads, D, P))
        worst = 0.0
        for it in range(2):  # twice: the gather buffers are reused
            g = torch.Generator(device="cpu").manual_seed(200 + it)
            qkv = torch.randn(B, seq, 3 * heads * D, generator=g).bfloat16()
            mine = qkv[:, rank * S_loc : (rank + 1) * S_loc].to(dev)
            q, k, v = (mine[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)) for i in range(3))
            got = symm.ring_attention_fused(q, k, v, rws)
            want = ring.ring_attention(q.contiguous(), k.contiguous(), v.contiguous(), group)
            full_k, full_v = (qkv[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)).to(dev) for i in (1, 2))
            oracle = TF.attention(q.contiguous(), full_k.contiguous(), full_v.contiguous())
            worst = max(worst, (got.float() - want.float()).abs().max().item(), (got.float() - oracle.float()).abs().max().item())
        errs["ring"] = worst
        rws.close()
        if world_size == 2:
            torch.manual_seed(7)
            lat = torch.randn(1, 16, 3, 8, 8, device=dev)
            preds = [torch.randn(1, 16, 3, 8, 8, generator=torch.Generator().manual_seed(50 + r)).bfloat16().to(dev)
                     for r in range(2)]  # fmt: skip
            worst = 0.0
            for it in range(2):
                want = TF.cfg_euler_step(lat, preds[0], preds[1], 5.0, -0.02)
                got = symm.cfg_combine_step_fused(lat, preds[rank], ws, 5.0, -0.02)
                worst = max(worst, (got - want).abs().max().item())
            errs["cfg"] = worst
        errs.update(tp_fused_errors(group, dev, ws))
        torch.cuda.synchronize()
        errs["status"] = native.last_status()
        gathered = [None] * world_size
        dist.all_gather_object(gathered, errs, group=group)
        if rank == 0:
            torch.save(gathered, out_path)
        ws.close()
    finally:
        dist.destroy_process_group()


def spawn(world_size: int, **kw):
    import tempfile

    import torch.multiprocessing as mp

    from telefuser_b200.utils.system import find_free_port

    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "errs.pt")
        mp.spawn(rank_main, nprocs=world_size, join=True, args=(world_size, find_free_port(), path),
                 daemon=False)  # fmt: skip
        return torch.load(path)
