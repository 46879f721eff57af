"""One-launch correctness sweep of every multi-GPU path on N ranks (N = 2, 4 or 8 GPUs of one node).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 \\
        -m telefuser_b200.testing.multi_gpu_suite --out mgpu_N.json

All checks run inside ONE process-group lifetime (process start-up and NCCL initialisation dominate the cost of a
multi-GPU test, so they are paid once):
 1. denoising layouts: the small Wan DiT (8 heads x 128) denoises the same latents under every layout that fits N
    (CFG2 x Ulysses, Ulysses-N, ring-N, Ulysses x ring, TP-N, PP2 x Ulysses, sharded weights), once with the
    peer-memory kernels and once with the collective-library path, each compared with the one-GPU result;
 2. peer-memory kernels against their collective compositions and against unsharded oracles at P = N: Ulysses
    attention at two different sequence lengths back to back (workspace re-carving), row all-gather,
    context-parallel attention, CFG combine (pairs), GEMM -> reduce-scatter / all-reduce, all-gather -> GEMM;
 3. expert parallelism at EP = N on the LingBot-Video MoE block (8 experts) against the one-GPU forward;
 4. VAE 2-D split decode on N GPUs against the one-GPU decode;
 5. the device status word of every rank is zero at the end.
Rank 0 writes a JSON report; the exit code is 0 only when every check is inside its tolerance on every rank.
With `--backend gloo` the layout sweep (1) and the VAE check (4) run on CPU ranks (host-side logic only).
"""

from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def layouts_for(n: int) -> list[dict]:
    out = [dict(sp_ulysses_degree=n), dict(sp_ring_degree=n), dict(tp_degree=n)]
    if n % 2 == 0:
        out.insert(0, dict(cfg_degree=2, sp_ulysses_degree=n // 2) if n > 2 else dict(cfg_degree=2))
    if n >= 4:
        out.append(dict(sp_ulysses_degree=n // 2, sp_ring_degree=2))
        out.append(dict(pp_degree=2, sp_ulysses_degree=n // 2))
        out.append(dict(cfg_degree=2, sp_ulysses_degree=n // 4, sp_ring_degree=2) if n >= 8 else dict(cfg_degree=2, sp_ring_degree=n // 2))
    out.append(dict(sp_ulysses_degree=n, enable_fsdp=True))
    return out


def name_of(layout: dict) -> str:
    short = {"cfg_degree": "cfg", "sp_ulysses_degree": "u", "sp_ring_degree": "r", "tp_degree": "tp", "pp_degree": "pp"}
    return "x".join(f"{short[k]}{v}" for k, v in layout.items() if k in short) + ("+fsdp" if layout.get("enable_fsdp") else "")


def wide_model(dtype, device):
    """8 heads x 128 so that every degree up to 8 divides heads, tokens (48) and the FFN width."""
    from telefuser_b200.models.wan_dit import WanModel

    torch.manual_seed(0)
    m = WanModel(dim=1024, ffn_dim=2048, num_heads=8, num_layers=2, text_dim=256).to(dtype)
    m.dtype = dtype
    return m.eval().to(device)


def denoise(layout: dict | None, device: str, dtype, world: int):
    from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig
    from telefuser_b200.parallel import mesh as pmesh
    from telefuser_b200.pipelines.wan.denoising import WanDenoisingStage
    from telefuser_b200.schedulers.flow_match import FlowMatchScheduler
    from telefuser_b200.testing.distributed_checks import make_tiny_inputs

    par = ParallelConfig(device_ids=list(range(world)), **layout) if layout else ParallelConfig()
    dev = torch.device(device)
    cfg = ModelRuntimeConfig(torch_dtype=dtype, parallel_config=par, device_type=dev.type, device_id=dev.index or 0)
    stage = WanDenoisingStage("denoise", None, cfg, FlowMatchScheduler("Wan"), dit=wide_model(dtype, device))
    if layout:
        stage.parallel_models()
    else:
        pmesh.set_mesh(None)
        stage.mesh = pmesh.get_mesh()
    stage.onload_models_flag = True
    lat, ctx, neg = make_tiny_inputs()
    out = stage.process(lat.to(device), 3, None, ctx.to(device, dtype), neg.to(device, dtype), None, 5.0, 5.0)
    return out.float().cpu()


def rel(a, b) -> float:
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def check_layouts(rank: int, world: int, device: str, dtype, gpu: bool) -> dict:
    from telefuser_b200.parallel import symm

    report = {}
    ref = denoise(None, device, dtype, world) if rank == 0 else None
    for layout in layouts_for(world):
        for fused in (("1", "0") if gpu else ("0",)):
            os.environ["TFB_FUSED_COLLECTIVES"] = fused
            key = f"{name_of(layout)}/{'peer' if fused == '1' else 'collectives'}"
            t0 = time.time()
            try:
                out = denoise(layout, device, dtype, world)
                err = rel(out, ref) if rank == 0 else 0.0
                report[key] = {"rel_err": err, "seconds": round(time.time() - t0, 2)}
            except Exception as e:  # noqa: BLE001 - reported, the sweep goes on
                report[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
            if gpu:
                torch.cuda.synchronize()
                symm.release_workspaces()
            dist.barrier()
    os.environ.pop("TFB_FUSED_COLLECTIVES", None)
    return report


def check_peer_kernels(rank: int, world: int, dev) -> dict:
    from telefuser_b200.ops import functional as TF
    from telefuser_b200.parallel import ring, symm, ulysses
    from telefuser_b200.testing.peer_checks import tp_fused_errors

    group, P, D, B, heads = dist.group.WORLD, world, 128, 1, 8
    errs: dict = {}
    os.environ["TFB_PEER_CANARY"] = "1"
    ws = symm.get_workspace(group, 4 * (B * 1024 * heads * D * 2 + 4096) + (48 << 20), tag="suite")
    worst = 0.0
    for layer, seq in enumerate((1024, 512, 1024, 768)):  # a smaller, a larger and a new shape: regions are re-carved
        S_loc = seq // P
        g = torch.Generator(device="cpu").manual_seed(100 + layer)
        qkv = torch.randn(B, seq, 3 * heads * D, generator=g).bfloat16()
        mine = qkv[:, rank * S_loc : (rank + 1) * S_loc].to(dev)
        q, k, v = (mine[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)) for i in range(3))
        hq, hk, hv = (ulysses.scatter_heads(t.contiguous(), group) for t in (q, k, v))
        want = ulysses.gather_heads(TF.attention(hq, hk, hv), group)
        got = symm.ulysses_attention_fused(q, k, v, ws)
        full = [qkv[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)).to(dev) for i in range(3)]
        oracle = TF.attention_reference(full[0][:, rank * S_loc : (rank + 1) * S_loc], full[1], full[2])
        worst = max(worst, (got.float() - want.float()).abs().max().item(), (got.float() - oracle.float()).abs().max().item())
    errs["ulysses_vs_collectives_and_oracle"] = worst
    worst = 0.0
    for it in range(2):
        x = torch.full((37, 256), float(rank + 1 + 10 * it), device=dev).bfloat16()
        parts = [torch.empty_like(x) for _ in range(P)]
        dist.all_gather(parts, x, group=group)
        worst = max(worst, (symm.all_gather_rows_fused(x, ws).float() - torch.cat(parts).float()).abs().max().item())
    errs["row_all_gather"] = worst
    seq, S_loc = 1024, 1024 // P
    rws = symm.get_workspace(group, symm.ring_workspace_bytes(S_loc, heads, D, P), tag="suite-ring")
    worst = 0.0
    for it in range(2):
        g = torch.Generator(device="cpu").manual_seed(200 + it)
        qkv = torch.randn(B, seq, 3 * heads * D, generator=g).bfloat16()
        mine = qkv[:, rank * S_loc : (rank + 1) * S_loc].to(dev)
        q, k, v = (mine[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)) for i in range(3))
        got = symm.ring_attention_fused(q, k, v, rws)
        want = ring.ring_attention(q.contiguous(), k.contiguous(), v.contiguous(), group)
        fk, fv = (qkv[..., i * heads * D : (i + 1) * heads * D].unflatten(-1, (heads, D)).to(dev) for i in (1, 2))
        oracle = TF.attention_reference(q.contiguous(), fk, fv)
        worst = max(worst, (got.float() - want.float()).abs().max().item(), (got.float() - oracle.float()).abs().max().item())
    errs["context_parallel_vs_ring_and_oracle"] = worst
    # CFG combine on pairs (rank 2i holds the conditional branch, 2i+1 the unconditional one)
    if P % 2 == 0:
        pairs = [dist.new_group([2 * i, 2 * i + 1]) for i in range(P // 2)]
        pg = pairs[rank // 2]
        cws = symm.get_workspace(pg, 1 << 20, tag="suite-cfg")
        lat = torch.randn(1, 16, 3, 8, 8, generator=torch.Generator().manual_seed(7)).to(dev)
        preds = [torch.randn(1, 16, 3, 8, 8, generator=torch.Generator().manual_seed(50 + r)).bfloat16().to(dev) for r in range(2)]
        worst = 0.0
        for _ in range(2):
            want = TF.cfg_euler_step(lat, preds[0], preds[1], 5.0, -0.02)
            got = symm.cfg_combine_step_fused(lat, preds[rank % 2], cws, 5.0, -0.02)
            worst = max(worst, (got - want).abs().max().item())
        errs["cfg_combine"] = worst
    errs.update(tp_fused_errors(group, dev, ws, M=128 * P * 2, K=128 * P, N=64 * P))
    torch.cuda.synchronize()
    for w in (ws, rws):
        w.check_canaries()
    errs["canaries"] = 0
    os.environ.pop("TFB_PEER_CANARY", None)
    symm.release_workspaces()
    return errs


def check_expert_parallel(rank: int, world: int, device: str) -> dict:
    from telefuser_b200.parallel import expert
    from telefuser_b200.testing.lingbot_video_checks import make_inputs, make_model

    if 8 % world:
        return {"skipped": "8 experts are not divisible by the world size"}
    heads = max(2, world)  # the Ulysses + EP case splits the heads over all ranks
    over = dict(hidden_size=128 * heads, num_attention_heads=heads, axes_dims=(32, 48, 48), moe_intermediate_size=128)
    kw = dict(frames=2, size=16, text_len=8)  # 520 tokens: divisible by 8
    out = {}
    single = make_model("tiny-moe", torch.bfloat16, device, **over)
    x, t, txt = make_inputs(text_dim=single.config.text_dim, **kw)
    args = (x.to(device, torch.bfloat16), t.to(device), txt.to(device, torch.bfloat16))
    ref = single(*args).float().cpu()
    for mode in ("ep", "both"):
        m = make_model("tiny-moe", torch.bfloat16, device, **over)
        if mode == "both":
            m.set_ulysses_group(dist.group.WORLD)
        m.enable_expert_parallel(dist.group.WORLD)
        out[f"expert_parallel_{mode}"] = rel(m(*args).float().cpu(), ref)
        torch.cuda.synchronize()
        dist.barrier()
    expert.release()
    return out


def check_vae(rank: int, world: int, device: str, dtype) -> dict:
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.testing.synthetic import random_init_

    torch.manual_seed(0)
    vae = random_init_(WanVideoVAE(dim=16).to(dtype), 0, std=0.05).eval().to(device)
    vae.parallelism = world
    lat = torch.randn(1, 16, 3, 16, 24, generator=torch.Generator().manual_seed(1)).to(device, dtype)
    with torch.no_grad():
        plain = vae.model.decode(lat, vae.scale).clamp(-1, 1).float().cpu()
        split = vae.decode_dist_2d(lat, halo=24).float().cpu()
        tiled = vae.tiled_decode(lat, tile_size=(8, 8), tile_stride=(4, 4)).float().cpu()
        vae.parallelism = 1
        tiled_one = vae.tiled_decode(lat, tile_size=(8, 8), tile_stride=(4, 4)).float().cpu()
    return {"vae_2d_split_vs_plain": (split - plain).abs().max().item(),
            "vae_tiled_ranks_vs_one": (tiled - tiled_one).abs().max().item()}  # fmt: skip


TOLERANCES = {"layout": 2.5e-2, "ulysses_vs_collectives_and_oracle": 3e-2, "row_all_gather": 0.0,
              "context_parallel_vs_ring_and_oracle": 3e-2, "cfg_combine": 1e-6, "tp_rs": 1e-2, "tp_ar": 1e-2, "tp_ag": 1e-2,
              "expert_parallel_ep": 2e-2, "expert_parallel_both": 2e-2, "vae_2d_split_vs_plain": 2e-2,
              "vae_tiled_ranks_vs_one": 2e-2, "canaries": 0}  # fmt: skip


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--skip", default="", help="comma list of: layouts, peer, ep, vae")
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    gpu = a.backend == "nccl"
    skip = set(filter(None, a.skip.split(",")))
    if gpu:
        torch.cuda.set_device(local)
        device, dtype = f"cuda:{local}", torch.bfloat16
        dist.init_process_group("nccl", device_id=torch.device(device))
    else:
        torch.set_num_threads(1)
        device, dtype = "cpu", torch.float32
        dist.init_process_group("gloo")
    report: dict = {"world": world, "backend": a.backend}
    failures: list[str] = []
    try:
        def section(name: str, fn) -> None:
            """One part of the sweep: an exception is recorded as that part's failure (the other parts still run), and
            rank 0 rewrites the report file after every part so that a later crash does not lose what was measured."""
            try:
                report[name] = fn()
            except Exception as e:  # noqa: BLE001
                report[name] = {"error": f"{type(e).__name__}: {e}"[:400]}
                failures.append(f"{name}: {report[name]['error']}")
            if rank == 0 and a.out:
                with open(a.out, "w") as f:
                    json.dump({"world": world, "backend": a.backend, "partial": True, "rank0": report,
                               "failures_so_far": failures}, f, indent=1)  # fmt: skip

        if "layouts" not in skip:
            section("layouts", lambda: check_layouts(rank, world, device, dtype, gpu))
            tol = TOLERANCES["layout"] if gpu else 1e-4
            for k, v in report["layouts"].items():
                if isinstance(v, dict) and ("error" in v or v.get("rel_err", 0.0) > tol):
                    failures.append(f"layout {k}: {v}")
        if gpu and "peer" not in skip:
            section("peer", lambda: check_peer_kernels(rank, world, torch.device(device)))
        if gpu and "ep" not in skip:
            section("ep", lambda: check_expert_parallel(rank, world, device))
        if "vae" not in skip:
            section("vae", lambda: check_vae(rank, world, device, dtype))
        for part in ("peer", "ep", "vae"):
            for k, v in report.get(part, {}).items():
                if isinstance(v, (int, float)) and k in TOLERANCES and v > (TOLERANCES[k] if gpu else 1e-4):
                    failures.append(f"{part}.{k} = {v}")
        if gpu:
            from telefuser_b200.ops import native

            torch.cuda.synchronize()
            report["status_word"] = native.last_status()
            if report["status_word"]:
                failures.append(f"status word {report['status_word']}")
        report["failures"] = failures
        gathered = [None] * world
        dist.all_gather_object(gathered, report)
        all_failures = [f"rank {r}: {f}" for r, rep in enumerate(gathered) for f in rep["failures"]]
        if rank == 0:
            summary = {"world": world, "backend": a.backend, "passed": not all_failures, "failures": all_failures,
                       "rank0": report, "other_ranks": [{k: v for k, v in rep.items() if k in ("peer", "ep", "vae", "status_word")}
                                                        for rep in gathered[1:]]}  # fmt: skip
            text = json.dumps(summary, indent=1)
            if a.out:
                os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
                with open(a.out, "w") as f:
                    f.write(text)
            print(text if len(text) < 20000 else json.dumps({k: summary[k] for k in ("world", "passed", "failures")}))
        return 1 if all_failures else 0
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    raise SystemExit(main())
