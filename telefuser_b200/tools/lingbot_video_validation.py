"""Validation and benchmark tool for the LingBot-Video transformer (dense 1.3B and MoE 30B-A3B forms).

    python -m telefuser_b200.tools.lingbot_video_validation inspect /models/lingbot-video/transformer
    python -m telefuser_b200.tools.lingbot_video_validation capture --preset tiny-moe --out single.pt
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m telefuser_b200.tools.lingbot_video_validation \\
        capture --preset tiny-moe --layout u2 --expert-parallel --out sp.pt
    python -m telefuser_b200.tools.lingbot_video_validation compare single.pt sp.pt --tol 2e-2
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m telefuser_b200.tools.lingbot_video_validation \\
        bench --preset moe-30b-a3b --layout cfg2u4 --expert-parallel --frames 81 --height 480 --width 832 --steps 2

* `inspect`: what a checkpoint (file, sharded folder or index) holds: dense or MoE, depth, expert count and shapes,
  parameter totals per group, and every difference against the preset it resolves to.
* `capture`: one seeded denoising run (random-init weights of a preset, or a checkpoint) that records the output of
  every transformer block at the first step and the latent after every step; under `torchrun` the model runs with
  the given layout (`cfg2`, `u<N>`, `--expert-parallel`, `--fsdp`) and rank 0 writes the file.
* `compare`: two captures tensor by tensor (max abs, relative L2, cosine); non-zero exit above the tolerance.
* `refiner-handoff`: the base-model -> refiner hand-off on a tiny random-init model: frame budget, sigma tail, the starting
  mix of encoded video and noise, clean-first-frame conditioning, seed determinism; non-zero exit if a check fails.
* `bench`: device-timed denoising steps of the full-size model on N GPUs (CUDA events, max over ranks, warm-up
  first), one JSON line: ms per step, per-stage breakdown of the first timed step, layout, tokens.

Role: tools/validation/ of the reference (checkpoint inspection, reference capture and replay, dense / MoE /
sequence-parallel parity runs, distributed run, refiner hand-off validation, benchmark), folded into one entry point.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys
import time
from collections import defaultdict

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------------------------------
# inspect
# ---------------------------------------------------------------------------------------------------
def read_checkpoint_shapes(path: str) -> dict[str, tuple]:
    """{tensor name: shape} of a safetensors file, a folder of shards or an index json, without loading data."""
    from safetensors import safe_open

    files: list[str] = []
    if os.path.isdir(path):
        files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
    elif path.endswith(".json"):
        idx = json.load(open(path))
        files = sorted({os.path.join(os.path.dirname(path), f) for f in idx["weight_map"].values()})
    else:
        files = [path]
    if not files:
        raise FileNotFoundError(f"no safetensors file under {path}")
    shapes: dict[str, tuple] = {}
    for f in files:
        with safe_open(f, framework="pt") as sf:
            for k in sf.keys():
                shapes[k] = tuple(sf.get_slice(k).get_shape())
    return shapes


def inspect_shapes(shapes: dict[str, tuple]) -> dict:
    from telefuser_b200.models.lingbot_video import LingBotVideoConfig, LingBotVideoTransformer3DModel

    depth = 1 + max((int(m.group(1)) for k in shapes if (m := re.match(r"(?:.*\.)?blocks\.(\d+)\.", k))), default=-1)
    expert_keys = [k for k in shapes if ".experts." in k]
    num_experts = 0
    for k in expert_keys:
        if (m := re.search(r"\.experts\.(\d+)\.", k)) is not None:
            num_experts = max(num_experts, int(m.group(1)) + 1)
        elif k.endswith(("experts.w1", "experts.w2", "experts.w3")):
            num_experts = max(num_experts, shapes[k][0])
    groups: dict[str, int] = defaultdict(int)
    for k, s in shapes.items():
        n = 1
        for d in s:
            n *= d
        part = "experts" if ".experts." in k else "router" if "router" in k or ".gate." in k else \
            "attention" if ".attn." in k else "ffn" if ".ffn." in k or ".mlp." in k else \
            "embedders" if "embed" in k else "other"  # fmt: skip
        groups[part] += n
    preset = "moe-30b-a3b" if num_experts else "dense-1.3b"
    cfg = LingBotVideoConfig.preset(preset)
    with torch.device("meta"):
        want = {k: tuple(v.shape) for k, v in LingBotVideoTransformer3DModel(cfg).state_dict().items()}
    report = {"kind": "moe" if num_experts else "dense", "depth": depth, "num_experts": num_experts, "tensors": len(shapes),
              "parameters": sum(groups.values()), "parameters_by_group": dict(groups), "resolved_preset": preset,
              "preset_depth": cfg.depth, "preset_num_experts": cfg.num_experts}  # fmt: skip
    # names may carry the exporter's prefix and per-expert layout; compare the ones that exist under both names
    common = set(shapes) & set(want)
    report["names_in_both"] = len(common)
    report["shape_mismatches"] = {k: [list(shapes[k]), list(want[k])] for k in sorted(common) if shapes[k] != want[k]}
    report["only_in_checkpoint"] = sorted(set(shapes) - set(want))[:20]
    report["only_in_model"] = sorted(set(want) - set(shapes))[:20]
    return report


# ---------------------------------------------------------------------------------------------------
# model / layout helpers
# ---------------------------------------------------------------------------------------------------
def parse_layout(spec: str, world: int) -> dict:
    out = {"cfg_degree": 1, "sp_ulysses_degree": 1}
    for tok in re.findall(r"cfg\d+|u\d+", spec or ""):
        if tok.startswith("cfg"):
            out["cfg_degree"] = int(tok[3:])
        else:
            out["sp_ulysses_degree"] = int(tok[1:])
    if spec in ("", "auto", None):
        out = {"cfg_degree": 2 if world % 2 == 0 and world > 1 else 1, "sp_ulysses_degree": max(1, world // (2 if world % 2 == 0 and world > 1 else 1))}
    if out["cfg_degree"] * out["sp_ulysses_degree"] != world:
        raise SystemExit(f"layout {spec!r} needs {out['cfg_degree'] * out['sp_ulysses_degree']} ranks, the launch has {world}")
    return out


def init_distributed() -> tuple[int, int, str]:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    gpu = torch.cuda.is_available()
    device = f"cuda:{local}" if gpu else "cpu"
    if gpu:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {"device_id": torch.device(device)} if gpu else {}
        dist.init_process_group("nccl" if gpu else "gloo", **kw)
    return rank, world, device


def build_stage(args, world: int, device: str, dtype):
    """The denoising stage of the pipeline around a random-init (or loaded) transformer, wired for the layout."""
    from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig
    from telefuser_b200.models.lingbot_video import LingBotVideoConfig, LingBotVideoTransformer3DModel
    from telefuser_b200.pipelines.lingbot_video.pipeline import LingBotVideoDenoisingStage
    from telefuser_b200.testing.synthetic import random_init_

    cfg = LingBotVideoConfig.preset(args.preset)
    if getattr(args, "depth", 0):
        cfg.depth = args.depth
    if device.startswith("cuda") and args.preset not in ("tiny", "tiny-moe"):
        with torch.device("meta"):
            model = LingBotVideoTransformer3DModel(cfg)
        model = model.to_empty(device=device).to(dtype)
    else:
        model = LingBotVideoTransformer3DModel(cfg).to(dtype).to(device)
    random_init_(model, seed=args.seed, std=0.03)
    if args.checkpoint:
        from telefuser_b200.utils.model_weight import load_state_dict

        model.load_state_dict(load_state_dict(args.checkpoint), strict=False)
    model.eval()
    model.promote_stability_layers_to_fp32()
    model.dtype = dtype
    layout = parse_layout(args.layout, world)
    pc = ParallelConfig(device_ids=list(range(world)) if world > 1 else None, cfg_degree=layout["cfg_degree"],
                        sp_ulysses_degree=layout["sp_ulysses_degree"], enable_fsdp=bool(args.fsdp))  # fmt: skip
    dev = torch.device(device)
    rc = ModelRuntimeConfig(torch_dtype=dtype, parallel_config=pc, device_type=dev.type, device_id=dev.index or 0)
    stage = LingBotVideoDenoisingStage("denoise", None, rc, dit=model, expert_parallel=bool(args.expert_parallel) and world > 1)
    stage.device = dev
    if world > 1:
        stage.parallel_models()
    stage.onload_models_flag = True
    return stage, cfg, layout


def synthetic_inputs(cfg, frames: int, height: int, width: int, text_len: int, seed: int, device: str, dtype):
    from telefuser_b200.pipelines.lingbot_video.pipeline import latent_shape

    g = torch.Generator().manual_seed(seed)
    f, h, w = latent_shape(frames, height, width)
    latent = torch.randn(1, cfg.in_channels, f, h, w, generator=g)
    pos = torch.randn(1, text_len, cfg.text_dim, generator=g).to(device, dtype)
    neg = torch.randn(1, text_len, cfg.text_dim, generator=g).to(device, dtype)
    mask = torch.ones(1, text_len, dtype=torch.bool, device=device)
    tokens = f * (h // cfg.patch_size[1]) * (w // cfg.patch_size[2])
    return latent.to(device), pos, neg, mask, tokens


# ---------------------------------------------------------------------------------------------------
# capture / compare
# ---------------------------------------------------------------------------------------------------
def capture(args) -> int:
    rank, world, device = init_distributed()
    dtype = torch.bfloat16 if device.startswith("cuda") and not args.fp32 else torch.float32
    stage, cfg, layout = build_stage(args, world, device, dtype)
    latent, pos, neg, mask, tokens = synthetic_inputs(cfg, args.frames, args.height, args.width, args.text_len, args.seed + 1,
                                                      device, dtype)  # fmt: skip
    record: dict[str, torch.Tensor] = {}
    first_step = {"on": True}
    hooks = []
    for i, blk in enumerate(stage.dit.blocks):
        def hook(_m, _inp, out, i=i):
            if first_step["on"] and f"block{i:02d}" not in record:
                record[f"block{i:02d}"] = (out[0] if isinstance(out, tuple) else out).detach().float().cpu()
        hooks.append(blk.register_forward_hook(hook))
    from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

    sched = FlowMatchScheduler("Wan")
    sched.set_timesteps(args.steps, shift=args.shift)
    sig = sched.sigmas.tolist()
    sig = sig + [0.0] if len(sig) == args.steps else sig
    x = latent.float()
    with torch.no_grad():
        for s in range(args.steps):
            x = _one_step(stage, x, pos, neg, mask, args.guidance, sig[s], sig[s + 1])
            first_step["on"] = False
            record[f"latent_step{s:02d}"] = x.detach().float().cpu()
    for h in hooks:
        h.remove()
    if world > 1:
        dist.barrier()
    if rank == 0:
        meta = {"preset": args.preset, "layout": layout, "world": world, "expert_parallel": bool(args.expert_parallel),
                "fsdp": bool(args.fsdp), "dtype": str(dtype), "tokens": tokens, "steps": args.steps}  # fmt: skip
        torch.save({"meta": meta, "tensors": record}, args.out)
        print(json.dumps({"captured": len(record), "out": args.out, **meta}))
    _finish(world)
    return 0


def _one_step(stage, x, pos, neg, mask, guidance, s0, s1):
    from telefuser_b200.ops import functional as TF

    t = torch.full((x.shape[0],), s0 * 1000.0, device=x.device)
    cond, uncond = stage.predict_noise_with_cfg(x, t, pos, neg, mask, mask, guidance)
    return TF.cfg_euler_step(x, cond, uncond, guidance, s1 - s0)


def _finish(world: int) -> None:
    if world > 1 and dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            try:
                from telefuser_b200.parallel import expert

                expert.release()
            except Exception:  # noqa: BLE001
                pass
        dist.barrier()
        dist.destroy_process_group()


def compare_captures(a: dict, b: dict) -> list[dict]:
    rows = []
    for k in sorted(set(a["tensors"]) & set(b["tensors"])):
        x, y = a["tensors"][k].double(), b["tensors"][k].double()
        if x.shape != y.shape:  # block outputs of a sequence-parallel run hold this rank's token shard only
            rows.append({"tensor": k, "skipped": f"shapes {tuple(x.shape)} vs {tuple(y.shape)}"})
            continue
        diff = (x - y)
        rows.append({"tensor": k, "max_abs": float(diff.abs().max()), "rel_l2": float(diff.norm() / (y.norm() + 1e-30)),
                     "cosine": float((x.flatten() @ y.flatten()) / (x.norm() * y.norm() + 1e-30))})  # fmt: skip
    return rows


def compare(args) -> int:
    a, b = torch.load(args.a, weights_only=False), torch.load(args.b, weights_only=False)
    rows = compare_captures(a, b)
    worst = max((r["rel_l2"] for r in rows if "rel_l2" in r), default=float("nan"))
    for r in rows:
        print(json.dumps(r))
    ok = bool(rows) and worst <= args.tol
    print(json.dumps({"compared": sum("rel_l2" in r for r in rows), "skipped": sum("skipped" in r for r in rows),
                      "worst_rel_l2": worst, "tolerance": args.tol, "passed": ok, "a": a["meta"], "b": b["meta"]}))  # fmt: skip
    return 0 if ok else 1


# ---------------------------------------------------------------------------------------------------
# bench
# ---------------------------------------------------------------------------------------------------
def bench(args) -> int:
    rank, world, device = init_distributed()
    gpu = device.startswith("cuda")
    dtype = torch.bfloat16 if gpu else torch.float32
    stage, cfg, layout = build_stage(args, world, device, dtype)
    latent, pos, neg, mask, tokens = synthetic_inputs(cfg, args.frames, args.height, args.width, args.text_len, args.seed + 1,
                                                      device, dtype)  # fmt: skip
    x = latent.float()

    def step():
        return _one_step(stage, x, pos, neg, mask, args.guidance, 0.9, 0.85)

    def sync():
        if gpu:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    with torch.no_grad():
        for _ in range(args.warmup):
            step()
        sync()
        if gpu:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            out = step()
        if gpu:
            e1.record()
        sync()
        ms = (e0.elapsed_time(e1) if gpu else (time.perf_counter() - t0) * 1e3) / args.steps
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    finite = bool(torch.isfinite(out).all())
    if rank == 0:
        active = cfg.num_experts_per_tok + cfg.n_shared_experts if cfg.num_experts else 0
        from telefuser_b200.ops import native

        print(json.dumps({"metric": "lingbot_video_ms_per_denoising_step", "value": round(float(t.item()), 3), "unit": "ms",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": False,
                          "dtype": str(dtype).split(".")[-1], "data": "synthetic (random-init weights)", "finite_output": finite,
                          "gpu_launches": native.launch_count() if gpu else 0,
                          "config": {"model": f"lingbot-video {args.preset}", "depth": cfg.depth, "experts": cfg.num_experts,
                                     "experts_per_token": active, "tokens": tokens, "frames": args.frames, "height": args.height,
                                     "width": args.width, "parallelism": f"cfg{layout['cfg_degree']} x ulysses{layout['sp_ulysses_degree']}"
                                     + (f" x ep{world}" if args.expert_parallel and world > 1 else "") + (" + sharded weights" if args.fsdp else ""),
                                     "step": "cond + uncond forward + guidance + Euler update"}}))  # fmt: skip
    _finish(world)
    return 0


# ---------------------------------------------------------------------------------------------------
# refiner hand-off
# ---------------------------------------------------------------------------------------------------
def refiner_handoff(args) -> int:
    """Checks the base-model -> refiner hand-off on a tiny random-init model: frame selection and resize facts, the
    low-noise sigma schedule, that the latent the refiner starts from is the stated mix of encoded video and noise,
    that an image-conditioned run keeps its clean first frame, and that the same seed gives the same video."""
    import numpy as np

    from telefuser_b200.core.config import ModelRuntimeConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.lingbot_video import LingBotVideoPipeline, LingBotVideoPipelineConfig, compute_refiner_sigmas
    from telefuser_b200.pipelines.lingbot_video import refiner as R
    from telefuser_b200.testing.lingbot_video_checks import make_model
    from telefuser_b200.testing.synthetic import random_init_

    sample, fps, lat = R.compute_training_frame_budget(args.source_frames, args.source_fps, args.sample_fps)
    sig = compute_refiner_sigmas(1.0, 0.0, args.steps, args.shift, args.t_thresh, args.tail_steps)
    report = {"source": {"frames": args.source_frames, "fps": args.source_fps}, "sampled_frames": sample, "represented_fps": round(fps, 4),
              "latent_frames": lat, "sigmas": [round(float(v), 6) for v in sig], "denoising_steps": len(sig), "checks": {}}  # fmt: skip
    dev, dt = "cpu", torch.float32
    mm = ModuleManager(torch_dtype=dt, device=dev)
    mm.add_module(make_model("tiny-moe" if args.moe else "tiny"), "lingbot_video_moe_transformer" if args.moe else "lingbot_video_transformer")
    mm.add_module(random_init_(WanVideoVAE(dim=8).float(), std=0.05).eval(), "wan_video_vae")
    rc = lambda: ModelRuntimeConfig(device_type=dev, torch_dtype=dt)  # noqa: E731
    pipe = LingBotVideoPipeline(device=dev, torch_dtype=dt)
    pipe.init(mm, LingBotVideoPipelineConfig(text_encoding_config=rc(), dit_config=rc(), vae_config=rc(), num_inference_steps=1))
    stage = R.LingBotVideoRefinerStage(pipe.denoising_stage, pipe.vae_stage, device=dev, torch_dtype=dt)
    g = torch.Generator().manual_seed(args.seed)
    low = torch.rand(1, 3, min(args.source_frames, 9), 16, 16, generator=g) * 2 - 1
    video, facts = R.prepare_refiner_video(low, args.source_fps, 32, 32, args.sample_fps, max_frames=9)
    report["tiny_run"] = facts
    pos, neg = torch.randn(1, 6, 32, generator=g), torch.randn(1, 4, 32, generator=g)
    kw = dict(num_inference_steps=args.steps, shift=args.shift, t_thresh=args.t_thresh, tail_steps=args.tail_steps, seed=args.seed)
    enc = pipe.vae_stage.process("encode_video", video).float()
    noise = torch.randn(enc.shape, generator=torch.Generator().manual_seed(args.seed))
    start = R.prepare_refiner_latent(enc, noise, float(sig[0]))
    checks = report["checks"]
    checks["start_is_the_stated_mix"] = bool(torch.allclose(start, (1 - float(sig[0])) * enc + float(sig[0]) * noise, atol=1e-6))
    lat_a = stage.refine(video, pos, neg, decode=False, **kw)
    checks["finite"] = bool(torch.isfinite(lat_a).all())
    checks["same_seed_same_result"] = bool(torch.equal(lat_a, stage.refine(video, pos, neg, decode=False, **kw)))
    checks["other_seed_other_result"] = not torch.equal(lat_a, stage.refine(video, pos, neg, decode=False, **{**kw, "seed": args.seed + 1}))
    clean = torch.rand(1, 3, 32, 32, generator=g) * 2 - 1
    lat_c = stage.refine(video, pos, neg, decode=False, clean_first_frame=clean, **kw)
    first = pipe.vae_stage.process("encode_video", clean.unsqueeze(2)).float()[:, :, :1]
    checks["clean_first_frame_kept"] = bool(torch.allclose(lat_c[:, :, :1], first, atol=1e-6))
    out = stage.refine(video, pos, neg, **kw)
    checks["decoded_shape"] = list(out.shape)
    checks["schedule_descends_from_threshold"] = bool(abs(float(sig[0]) - args.t_thresh) < 1e-6 and np.all(np.diff(sig) < 0))
    report["passed"] = all(v for k, v in checks.items() if isinstance(v, bool))
    print(json.dumps(report, indent=1))
    return 0 if report["passed"] else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("inspect")
    p.add_argument("path")
    for name in ("capture", "bench"):
        p = sub.add_parser(name)
        p.add_argument("--preset", default="tiny-moe", choices=["dense-1.3b", "moe-30b-a3b", "tiny", "tiny-moe"])
        p.add_argument("--checkpoint", default="")
        p.add_argument("--depth", type=int, default=0, help="override the number of blocks (0: the preset's)")
        p.add_argument("--layout", default="auto", help="auto | cfg2 | u<N> | cfg2u<N>")
        p.add_argument("--expert-parallel", action="store_true")
        p.add_argument("--fsdp", action="store_true")
        p.add_argument("--frames", type=int, default=5)
        p.add_argument("--height", type=int, default=64)
        p.add_argument("--width", type=int, default=64)
        p.add_argument("--text-len", type=int, default=16)
        p.add_argument("--steps", type=int, default=2)
        p.add_argument("--warmup", type=int, default=1)
        p.add_argument("--guidance", type=float, default=3.0)
        p.add_argument("--shift", type=float, default=5.0)
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--fp32", action="store_true")
        if name == "capture":
            p.add_argument("--out", required=True)
    p = sub.add_parser("compare")
    p.add_argument("a")
    p.add_argument("b")
    p.add_argument("--tol", type=float, default=2e-2)
    p = sub.add_parser("refiner-handoff")
    p.add_argument("--source-frames", type=int, default=81)
    p.add_argument("--source-fps", type=float, default=24.0)
    p.add_argument("--sample-fps", type=int, default=24)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--shift", type=float, default=3.0)
    p.add_argument("--t-thresh", type=float, default=0.85)
    p.add_argument("--tail-steps", type=int, default=2)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--moe", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "refiner-handoff":
        return refiner_handoff(a)
    if a.cmd == "inspect":
        print(json.dumps(inspect_shapes(read_checkpoint_shapes(a.path)), indent=1))
        return 0
    return {"capture": capture, "compare": compare, "bench": bench}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
