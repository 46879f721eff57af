"""Streaming benchmark: chunk period / latency and frames per second of the LingBot-World-Fast style
causal 14B DiT + Wan VAE running on the streaming actor graph (encode -> denoise -> decode).

    python bench_stream.py --chunks 8 --warmup-chunks 2            # one GPU, all stages on it
    python bench_stream.py --gpus 4 --chunks 8                     # denoise on 4 GPUs (Ulysses), VAE on GPU 0

`--impl reference` would run the reference's own streaming denoising stage on the same shapes; its stage imports
the reference's UniPC scheduler, which needs the `diffusers` package, and its pipeline needs the UMT5 tokenizer
files - neither is on this machine, so that arm prints an `unavailable` line with the import error.
`--session-seconds T` sizes the timed session by duration (chunks = T x fps / frames per chunk) instead of `--chunks`;
`--lookahead N` is the number of chunks the client may submit ahead of the newest output (1 = interactive use:
a control takes effect at most one chunk period after the chunk in flight).

Workload (the reference's published setting, examples/lingbot/README.md:181-193): 832x464, chunks of
4 latent frames (16 video frames), 4 denoising steps + the clean-latent commit per chunk, attention
window 18 latent frames with 6 sink frames, bf16 DiT, random-init weights, synthetic image / prompt
embedding / camera path. One warm-up session, then one timed session; per-chunk times come from the
orchestrator's own timestamps (host clock around device-synchronous stage calls). Prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import statistics
import time

import torch


def build_pipeline(args, device: str):
    from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.lingbot_world_dit import LingBotWorldFastDiT
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.lingbot_world.pipeline import LingBotWorldFastPipeline, LingBotWorldFastPipelineConfig
    from telefuser_b200.testing.synthetic import random_init_

    dtype = torch.bfloat16
    small = args.model == "small"
    kw = dict(in_dim=36, local_attn_size=args.window, sink_size=args.sink)
    if small:
        kw.update(dim=1536, ffn_dim=8960, num_heads=12, num_layers=30)
    with torch.device(device):
        dit = LingBotWorldFastDiT(**kw).to(dtype)
        vae = WanVideoVAE().to(dtype)
    random_init_(dit)
    random_init_(vae, std=0.02)
    dit.dtype = dtype
    mm = ModuleManager(torch_dtype=dtype, device=device)
    mm.add_module(dit.eval(), "lingbot_world_fast_dit")
    mm.add_module(vae.eval(), "wan_video_vae")

    def rc(parallel=None):
        return ModelRuntimeConfig(device_type="cuda", device_id=0, torch_dtype=dtype,
                                  parallel_config=parallel or ParallelConfig())  # fmt: skip

    from telefuser_b200.pipelines.lingbot_world_v2 import resolve_stage_devices

    dit_devices, enc_dev, dec_dev = resolve_stage_devices(args.gpus)
    par = None
    if len(dit_devices) > 1:
        par = ParallelConfig(device_ids=dit_devices, sp_ulysses_degree=len(dit_devices))
    args.placement = {"dit": dit_devices, "vae_encode": enc_dev, "vae_decode": dec_dev}

    def rcd(dev_id):
        c = rc()
        c.device_id = dev_id
        return c

    cfg = LingBotWorldFastPipelineConfig(
        dit_config=rc(par), vae_encode_config=rcd(enc_dev), vae_decode_config=rcd(dec_dev), text_encoding_config=rc(),
        chunk_size=args.chunk_size, local_attn_size=args.window, sink_size=args.sink,
        timestep_indices=tuple(int(i * 1000 / args.steps) for i in range(args.steps)), max_sequence_length=512,
        enable_denoising_parallel=par is not None, edge_capacity=max(1, args.lookahead))  # fmt: skip
    pipe = LingBotWorldFastPipeline(device=device, torch_dtype=dtype)
    pipe.init(mm, cfg)
    return pipe


def run_session(pipe, args, chunks: int, seed: int):
    frames_per_chunk = args.chunk_size * 4
    n = (args.chunk_size * chunks - 1) * 4 + 1
    emb = torch.randn(1, 512, pipe.denoise_stage_text_dim(), device=pipe.device, dtype=pipe.torch_dtype)
    img = torch.rand(3, args.height, args.width) * 2 - 1
    arrivals = []
    t0 = time.perf_counter()
    video, metrics = pipe.generate_video("", img, n, args.height, args.width, seed=seed, prompt_emb=emb,
                                         on_chunk=lambda i, f: arrivals.append(time.perf_counter()),
                                         bind_controls_late=True)  # fmt: skip
    total = time.perf_counter() - t0
    periods = [b - a for a, b in zip(arrivals, arrivals[1:])]
    return dict(video_shape=list(video.shape), finite=bool(torch.isfinite(video.float()).all()), total_s=total,
                periods=periods, first_s=arrivals[0] - t0, metrics=metrics, frames_per_chunk=frames_per_chunk)  # fmt: skip


def pct(xs, q):
    xs = sorted(xs)
    if not xs:
        return None
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--chunks", type=int, default=8)
    ap.add_argument("--warmup-chunks", type=int, default=2)
    ap.add_argument("--height", type=int, default=464)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--chunk-size", type=int, default=4)
    ap.add_argument("--window", type=int, default=18)
    ap.add_argument("--sink", type=int, default=6)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--model", default="14b", choices=["14b", "small"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--session-seconds", type=float, default=0.0, help="size the timed session by duration")
    ap.add_argument("--lookahead", type=int, default=1, help="chunks submitted ahead of the newest output")
    args = ap.parse_args()
    if args.impl == "reference":
        import os
        import sys

        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
        try:
            from telefuser.pipelines.lingbot_world_fast.denoising import LingBotWorldFastDenoisingStage  # noqa: F401
            from telefuser.pipelines.lingbot_world_fast.pipeline import LingBotWorldFastPipeline  # noqa: F401

            why = "its pipeline needs the UMT5 tokenizer files (google/umt5-xxl), which are not on this machine"
        except Exception as e:  # noqa: BLE001
            why = f"{type(e).__name__}: {e}"[:240]
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return
    if args.session_seconds > 0:
        args.chunks = max(2, int(round(args.session_seconds * 16 / (args.chunk_size * 4))))
    device = "cuda:0"
    torch.cuda.set_device(0)
    from telefuser_b200.ops import native

    pipe = build_pipeline(args, device)
    try:
        run_session(pipe, args, args.warmup_chunks, seed=0)  # warm-up session
        native.reset_launch_count()
        r = run_session(pipe, args, args.chunks, seed=1)
    finally:
        pipe.close()
    busy = r["metrics"]["stage_busy_s"]
    steady = r["periods"][1:] if len(r["periods"]) > 2 else r["periods"]
    p50 = statistics.median(steady)
    out = {
        "metric": "lingbot_world_stream_chunk_period_p50_s", "value": round(p50, 4), "unit": "s/chunk",
        "higher_is_better": False, "n_gpus": args.gpus, "chunks": args.chunks, "warmup_chunks": args.warmup_chunks,
        "chunk_period_p99_s": round(pct(steady, 0.99), 4), "fps": round(r["frames_per_chunk"] / p50, 2),
        "first_chunk_latency_s": round(r["first_s"], 4),
        "dit_s_per_chunk_p50": round(statistics.median(busy["denoise"]), 4),
        "vae_decode_s_per_chunk_p50": round(statistics.median(busy["decode"]), 4),
        "vae_encode_s_per_chunk_p50": round(statistics.median(busy["encode"]), 4),
        "control_to_output_p50_s": r["metrics"]["control_to_output_p50_s"],
        "control_bound_to_output_p50_s": r["metrics"].get("control_bound_to_output_p50_s"),
        "control_bound_to_output_in_chunk_periods": (round(r["metrics"]["control_bound_to_output_p50_s"] / p50, 2)
                                                     if r["metrics"].get("control_bound_to_output_p50_s") else None),
        "session_s": round(r["total_s"], 2), "lookahead_chunks": args.lookahead,
        "stage_placement": getattr(args, "placement", None),
        "dtype": "bf16", "data": "synthetic (random-init weights, random image, prompt embedding and camera walk)",
        "finite_output": r["finite"], "gpu_launches": native.launch_count(),
        "config": {"model": f"lingbot-world-fast causal DiT ({args.model})", "height": args.height, "width": args.width,
                   "chunk_latent_frames": args.chunk_size, "frames_per_chunk": r["frames_per_chunk"],
                   "denoise_steps": args.steps, "window_frames": args.window, "sink_frames": args.sink,
                   "parallelism": "single" if args.gpus == 1 else f"ulysses{len(args.placement['dit'])} (denoise), VAE encode on GPU {args.placement['vae_encode']}, decode on GPU {args.placement['vae_decode']}"},
        "reference_published": {"2xH100_dit_s_per_chunk": 1.587, "2xH100_chunk_period_s": 2.096,
                                "4xH100_dit_s_per_chunk": 0.911, "4xH100_chunk_period_s": 1.615},
    }  # fmt: skip
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
