"""Headline benchmark: Wan2.1-T2V-14B, 81 frames, 720x1280 (75,600 tokens), seconds per video.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

A *step* is one full denoising step of the 50-step sampler: conditional and
unconditional DiT forward (40 blocks, dim 5120) + classifier-free guidance (5.0)
+ flow-matching Euler update. `value` is the time of the denoising loop of one
video: 50 x the measured step time. The one-off stages of the public pipeline
call (UMT5-XXL prompt encoding of the two prompts, 720p VAE decode of the
81 frames) are measured once each, on rank 0, after the timed region, and
reported beside it as `pipeline` (their sum with `value` is the time of
`pipeline(prompt, num_frames=81, height=720, width=1280)`). Weights are
random-init bf16 tensors of the real architectures; text embeddings and noise
latents are synthetic tensors of the real shapes.

Layouts (`--layout`, default by GPU count): 1 GPU plain; 2 GPUs CFG-parallel;
4 GPUs CFG2 x Ulysses2; 8 GPUs CFG2 x Ulysses4 (strong scaling: one video, more
GPUs). Others are spelled from `cfg2`, `u<N>` (Ulysses), `r<N>` (ring / context
parallel), `tp<N>` (tensor-parallel FFN): `u8`, `r8`, `u4r2`, `tp8`, `cfg2u4`.
`--quant fp8|mxfp8` runs the block projections in W8A8 (per-channel FP8 or
block-scaled MXFP8); such a line says so in `dtype` and is not the bf16 headline.

`--impl reference` runs the unmodified reference package installed under
baseline/_ref through its own stage API on the same shapes, with the fastest
attention setting among those it ships that work on this machine
(`--ref-attn auto` times TORCH_SDPA and TORCH_CUDNN on one layer's attention call
and keeps the winner, `--ref-attn fa2` selects its FLASH_ATTN_2 setting; the table
is printed in `ref_attention_ms`).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    "wan2.1-t2v-14b": dict(dim=5120, ffn_dim=13824, num_heads=40, num_layers=40),
    "wan2.1-t2v-1.3b": dict(dim=1536, ffn_dim=8960, num_heads=12, num_layers=30),
}
SAMPLER_STEPS = 50
CFG_SCALE = 5.0
SIGMA_SHIFT = 5.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="wan2.1-t2v-14b", choices=sorted(MODELS))
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--height", type=int, default=720)
    ap.add_argument("--width", type=int, default=1280)
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (pinned host <-> device) measurement")
    ap.add_argument("--layout", default="auto", help="auto | single | cfg2 | u8 | r8 | u4r2 | tp8 | cfg2u4 | ...")
    ap.add_argument("--quant", default="none", choices=["none", "fp8", "mxfp8"])
    ap.add_argument("--attn", default="bf16", choices=["bf16", "int8"], help="int8: Q.K^T scores on int8 operands")
    ap.add_argument("--ref-attn", default="auto", choices=["auto", "sdpa", "cudnn", "fa2"])
    ap.add_argument("--no-pipeline-stages", action="store_true", help="skip the text-encode / VAE-decode timings")
    return ap.parse_args()


def layout_for(n: int, spec: str = "auto") -> dict:
    """Parallel degrees for `n` GPUs. `spec` is a concatenation of cfg2 / u<N> / r<N> / tp<N> whose product is n."""
    import re

    if spec in ("auto", ""):
        spec = {1: "single", 2: "cfg2"}.get(n, f"cfg2xulysses{n // 2}")
    out = dict(cfg_degree=1, sp_ulysses_degree=1, sp_ring_degree=1, tp_degree=1, name=spec)
    if spec != "single":
        keys = {"cfg": "cfg_degree", "u": "sp_ulysses_degree", "ulysses": "sp_ulysses_degree", "r": "sp_ring_degree",
                "ring": "sp_ring_degree", "tp": "tp_degree", "x": None}  # fmt: skip
        for word, num in re.findall(r"(cfg|ulysses|ring|tp|u|r|x)(\d*)", spec.lower()):
            if keys[word] is not None:
                out[keys[word]] = int(num or 1)
    prod = out["cfg_degree"] * out["sp_ulysses_degree"] * out["sp_ring_degree"] * out["tp_degree"]
    if prod != n:
        raise SystemExit(f"layout {spec!r} needs {prod} GPUs, --gpus says {n}")
    return out


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)  # fmt: skip
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = self.proc.communicate()[0]
        clocks, maxc, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                clocks.append(float(f[1]))
                maxc = float(f[2])
                power.append(float(f[3]))
            except ValueError:
                continue
            for nme, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        load = [c for c, p in zip(clocks, power) if p > 300] or clocks
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": maxc,
                "power_w_median": statistics.median(power) if power else None, "samples": len(clocks),
                "reasons": sorted(reasons)}  # fmt: skip


def dist_setup(n: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if n > 1 and world != n:
        raise SystemExit(f"--gpus {n} needs torchrun with {n} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier_sync(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(v: float, world: int) -> float:
    if world == 1:
        return v
    t = torch.tensor([v], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def random_init_(model: torch.nn.Module, seed: int = 0) -> None:
    """Random-init weights of the real architecture, directly on the device."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    for name, p in model.named_parameters():
        if p.dim() >= 2 and "modulation" not in name:
            p.data.normal_(0.0, 0.02, generator=g)
        elif "modulation" in name:
            p.data.normal_(0.0, 1.0 / p.shape[-1] ** 0.5, generator=g)
        elif name.endswith("bias"):
            p.data.normal_(0.0, 0.01, generator=g)
        else:
            p.data.fill_(1.0)


def make_inputs(args, seed=1):
    """Pinned-host synthetic inputs of the real shapes."""
    g = torch.Generator().manual_seed(seed)
    lat_shape = (1, 16, (args.frames - 1) // 4 + 1, args.height // 8, args.width // 8)
    latents = torch.randn(lat_shape, generator=g).pin_memory()
    posi = torch.randn(1, 512, 4096, generator=g).to(torch.bfloat16).pin_memory()
    nega = torch.randn(1, 512, 4096, generator=g).to(torch.bfloat16).pin_memory()
    return latents, posi, nega


# ---------------------------------------------------------------------------
# Arms
# ---------------------------------------------------------------------------
def build_ours(args, layout, world, local):
    from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig
    from telefuser_b200.models.wan_dit import WanModel
    from telefuser_b200.ops import native
    from telefuser_b200.pipelines.wan.denoising import WanDenoisingStage
    from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

    native.load()
    with torch.device("meta"):
        model = WanModel(**MODELS[args.model])
    model = model.to_empty(device="cuda").to(torch.bfloat16)
    random_init_(model)
    model.eval()
    if args.quant != "none":
        n_q = model.enable_quant("mxfp8" if args.quant == "mxfp8" else "fp8")
        if local == 0:
            print(f"[bench] {n_q} linear layers quantised to {args.quant}", file=sys.stderr)
    pc = ParallelConfig(device_ids=list(range(world)) if world > 1 else None, cfg_degree=layout["cfg_degree"],
                        sp_ulysses_degree=layout["sp_ulysses_degree"], sp_ring_degree=layout["sp_ring_degree"],
                        tp_degree=layout["tp_degree"])  # fmt: skip
    cfg = ModelRuntimeConfig(torch_dtype=torch.bfloat16, parallel_config=pc, device_type="cuda", device_id=local)
    if args.attn == "int8":
        from telefuser_b200.core.config import AttentionConfig, AttnImplType

        cfg.attention_config = AttentionConfig(attn_impl=AttnImplType.TCGEN05_Q8)
    stage = WanDenoisingStage("dit_denoise", None, cfg, FlowMatchScheduler("Wan"), dit=model)
    if world > 1:
        stage.parallel_models()
    stage.onload_models_flag = True

    def run(latents, steps, posi, nega):
        return stage.process(latents, steps, None, posi, nega, None, CFG_SCALE, SIGMA_SHIFT)

    return run, native, {}


def pick_reference_attention(args, AttentionConfig, AttnImplType, attention, heads: int, tokens: int) -> tuple:
    """Times one layer's self-attention call of the real shape through the reference's own `attention()` for each
    stock setting that works here; returns (winning AttnImplType, {name: ms or reason})."""
    names = {"sdpa": "TORCH_SDPA", "cudnn": "TORCH_CUDNN", "fa2": "FLASH_ATTN_2"}
    # `auto` compares the two settings that run inside torch itself; the flash-attn package path is timed only when
    # asked for by name (its kernels are a separate binary build that this selection step has no way to vet first).
    todo = ["sdpa", "cudnn"] if args.ref_attn == "auto" else [args.ref_attn]
    q, k, v = (torch.randn(1, tokens, heads, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    table, best = {}, (None, float("inf"))
    for key in todo:
        impl = getattr(AttnImplType, names[key])
        cfg = AttentionConfig.dense_attention(impl)
        try:
            for _ in range(2):
                attention(q, k, v, attention_config=cfg, input_layout="BSND", output_layout="BSND")
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                attention(q, k, v, attention_config=cfg, input_layout="BSND", output_layout="BSND")
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 3
            table[names[key]] = round(ms, 3)
            if ms < best[1]:
                best = (impl, ms)
        except Exception as e:  # noqa: BLE001 - a setting that does not run on this machine is skipped
            table[names[key]] = f"failed: {type(e).__name__}: {e}"[:160]
    if best[0] is None:
        best = (AttnImplType.TORCH_SDPA, float("nan"))
    return best[0], table


def build_reference(args, layout, world, local):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "telefuser")):
        raise RuntimeError("reference is not installed under baseline/_ref")
    sys.path.insert(0, ref_root)
    os.environ.setdefault("TELEFUSER_LOG_LEVEL", "WARNING")
    from telefuser.core.config import AttentionConfig, AttnImplType, ModelRuntimeConfig, ParallelConfig
    from telefuser.core.module_manager import ModuleManager
    from telefuser.models.wan_video_dit import WanModel
    from telefuser.ops.attention.attention_impl import attention as ref_attention
    from telefuser.pipelines.wan_video.single_dit_denoising import SingleDitDenoisingStage

    if args.attn != "bf16":
        raise RuntimeError("the reference's SageAttention kernels come from its tf_kernel extension, which cannot be built "
                           "offline here")  # fmt: skip
    if args.quant != "none":
        raise RuntimeError("the reference's quantised linears need its tf_kernel extension or vLLM kernels, neither of "
                           "which can be built offline here")  # fmt: skip

    # The reference's `telefuser.schedulers` package imports its UniPC scheduler, which needs
    # `diffusers` (not installable offline). Its flow-matching scheduler file has no such
    # dependency, so that unmodified file is loaded by path instead of through the package.
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "telefuser_ref_flow_match", os.path.join(ref_root, "telefuser", "schedulers", "flow_match.py"))
    fm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fm)
    FlowMatchScheduler = fm.FlowMatchScheduler

    m = MODELS[args.model]
    with torch.device("meta"):
        model = WanModel(dim=m["dim"], in_dim=16, ffn_dim=m["ffn_dim"], out_dim=16, text_dim=4096, freq_dim=256,
                         eps=1e-6, patch_size=(1, 2, 2), num_heads=m["num_heads"], num_layers=m["num_layers"],
                         has_image_input=False)  # fmt: skip
    model = model.to_empty(device="cuda").to(torch.bfloat16)
    random_init_(model)
    # buffers created outside parameters (rope tables) are rebuilt by the reference itself
    from telefuser.models.wan_video_dit import precompute_freqs_cis_3d

    model.normal_freqs = precompute_freqs_cis_3d(model.head_dim)
    model.freqs = model.normal_freqs
    model.eval()
    mm = ModuleManager(torch_dtype=torch.bfloat16, device="cuda")
    mm.add_module(model, "wan_video_dit")
    pc = ParallelConfig(device_ids=list(range(world)) if world > 1 else None, cfg_degree=layout["cfg_degree"],
                        sp_ulysses_degree=layout["sp_ulysses_degree"], sp_ring_degree=layout["sp_ring_degree"],
                        tp_degree=layout["tp_degree"])  # fmt: skip
    sp = layout["sp_ulysses_degree"]
    tokens = ((args.frames - 1) // 4 + 1) * (args.height // 16) * (args.width // 16)
    try:
        impl, table = pick_reference_attention(args, AttentionConfig, AttnImplType, ref_attention, m["num_heads"] // sp,
                                               tokens)  # fmt: skip
    except Exception as e:  # noqa: BLE001 - the selection is an optimisation of the arm, never a reason to lose it
        impl, table = AttnImplType.TORCH_SDPA, {"selection_failed": f"{type(e).__name__}: {e}"[:200]}
    torch.cuda.empty_cache()
    cfg = ModelRuntimeConfig(torch_dtype=torch.bfloat16, parallel_config=pc, device_type="cuda", device_id=local,
                             attention_config=AttentionConfig.dense_attention(impl))  # fmt: skip
    stage = SingleDitDenoisingStage("dit_denoise", mm, cfg, FlowMatchScheduler("Wan"))
    if hasattr(model, "set_attention_config"):
        model.set_attention_config(cfg.attention_config)
    if world > 1:
        stage.parallel_models()
    stage.onload_models_flag = True

    def run(latents, steps, posi, nega):
        return stage.process(latents.to(torch.bfloat16), steps, None, posi, nega, None, CFG_SCALE, SIGMA_SHIFT)

    return run, None, {"ref_attn_impl": impl.name, "ref_attention_ms": table}


def time_pipeline_stages(args) -> dict:
    """The one-off stages of the public pipeline call at the headline shape, each timed once after one warm-up:
    UMT5-XXL encoding of the positive and the negative prompt (512 tokens each) and the VAE decode of the
    [1, 16, 21, 90, 160] latents to 81 frames of 720 x 1280. Random-init weights of the real architectures."""
    out: dict = {}
    lat = torch.randn(1, 16, (args.frames - 1) // 4 + 1, args.height // 8, args.width // 8, device="cuda")
    ids = torch.randint(1, 30000, (1, 512), device="cuda")
    mask = torch.ones(1, 512, dtype=torch.long, device="cuda")

    def timed(fn, warm: int = 1):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3

    if args.impl == "reference":
        from telefuser.models.wan_video_text_encoder import WanTextEncoder
        from telefuser.models.wan_video_vae import WanVideoVAE
    else:
        from telefuser_b200.models.umt5 import WanTextEncoder
        from telefuser_b200.models.wan_vae import WanVideoVAE
    try:
        with torch.device("meta"):
            te = WanTextEncoder()
        te = te.to_empty(device="cuda").to(torch.bfloat16).eval()
        random_init_(te, seed=5)
        with torch.no_grad():
            out["text_encode_s"] = round(timed(lambda: (te(ids, mask), te(ids, mask))), 4)
        del te
    except Exception as e:  # noqa: BLE001
        out["text_encode_s"], out["text_encode_error"] = None, f"{type(e).__name__}: {e}"[:200]
    torch.cuda.empty_cache()
    try:
        vae = WanVideoVAE().to("cuda").to(torch.bfloat16).eval()
        random_init_(vae, seed=6)
        dev = torch.device("cuda", torch.cuda.current_device())
        with torch.no_grad():
            out["vae_decode_s"] = round(timed(lambda: vae.decode(lat.to(torch.bfloat16), device=dev)), 4)
        del vae
    except Exception as e:  # noqa: BLE001
        out["vae_decode_s"], out["vae_decode_error"] = None, f"{type(e).__name__}: {e}"[:200]
    torch.cuda.empty_cache()
    return out


def main():
    args = parse_args()
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device on this machine"}))
            return
        raise SystemExit("bench.py needs a CUDA device")
    rank, world, local = dist_setup(args.gpus)
    layout = layout_for(world, args.layout)
    t_start = time.perf_counter()

    def progress(what: str) -> None:
        """Milestones on stderr (rank 0), so that a run cut short by a time limit still says how far it got."""
        if rank == 0:
            print(f"[bench {args.impl}] {what} at {time.perf_counter() - t_start:.1f} s", file=sys.stderr, flush=True)

    try:
        run, native, extra = (build_reference if args.impl == "reference" else build_ours)(args, layout, world, local)
        progress(f"arm built ({extra})" if extra else "arm built")
    except Exception as e:  # noqa: BLE001 - report why the arm cannot run
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
            return
        raise
    lat_h, posi_h, nega_h = make_inputs(args)
    lat = lat_h.cuda(non_blocking=True)
    posi = posi_h.cuda(non_blocking=True)
    nega = nega_h.cuda(non_blocking=True)
    tokens = lat.shape[2] * (lat.shape[3] // 2) * (lat.shape[4] // 2)

    # ---- device-timed K steps (inputs resident; activations >> L2 so no flush is needed) ----
    if args.warmup > 0:
        run(lat, args.warmup, posi, nega)
    barrier_sync(world)
    progress(f"{args.warmup} warm-up steps done")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    if native is not None:
        native.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = run(lat, args.steps, posi, nega)
    e1.record()
    barrier_sync(world)
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps, world)
    launches = native.launch_count() if native is not None else None
    clocks = sampler.stop() if rank == 0 else None
    finite = bool(torch.isfinite(out.float()).all().item())
    progress(f"{args.steps} timed steps done: {ms_step:.1f} ms/step, finite={finite}")

    # ---- end to end through the stage API: pinned host -> device -> step -> host, every step ----
    e2e = None
    if not args.no_e2e:
        res_h = torch.empty(lat_h.shape, dtype=torch.float32).pin_memory()
        barrier_sync(world)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            l_d = lat_h.cuda(non_blocking=True)
            p_d = posi_h.cuda(non_blocking=True)
            n_d = nega_h.cuda(non_blocking=True)
            o = run(l_d, 1, p_d, n_d)
            res_h.copy_(o.float(), non_blocking=True)
            torch.cuda.synchronize()
        barrier_sync(world)
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / args.steps, world)
        e2e = {"value": e2e_ms * SAMPLER_STEPS / 1e3, "unit": "s/video", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": lat_h.numel() * 4 + posi_h.numel() * 2 + nega_h.numel() * 2,
               "d2h_bytes_per_step": res_h.numel() * 4}  # fmt: skip

    progress("end-to-end steps done" if e2e is not None else "end-to-end steps skipped")
    stages = None
    if rank == 0 and not args.no_pipeline_stages:
        stages = time_pipeline_stages(args)
        progress(f"pipeline stages timed: {stages}")
    barrier_sync(world)

    if rank == 0:
        value = ms_step * SAMPLER_STEPS / 1e3
        if stages is not None:
            parts = [stages.get("text_encode_s"), stages.get("vae_decode_s")]
            stages["denoise_loop_s"] = value
            stages["total_s"] = None if None in parts else round(value + sum(parts), 3)
            stages["what"] = "text encode (2 prompts) + 50-step denoising loop + VAE decode = pipeline(prompt, 81, 720, 1280)"
        line = {
            "metric": "wan2.1_t2v_14b_81f_720p_seconds_per_video" if args.model.endswith("14b") else
                      f"{args.model}_seconds_per_video",  # fmt: skip
            "value": value, "unit": "s/video", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": ("bf16" if args.quant == "none" else f"bf16 activations, {args.quant} W8A8 block projections")
                     + ("" if args.attn == "bf16" else ", int8 attention scores"),  # fmt: skip
            "data": "synthetic (random-init weights, N(0,1) latents and text embeddings)",
            "impl": args.impl, "finite_output": finite,
            "config": {"model": args.model, "global_batch": 1, "seq_len": tokens, "frames": args.frames,
                       "height": args.height, "width": args.width, "sampler_steps": SAMPLER_STEPS,
                       "cfg_scale": CFG_SCALE, "parallelism": layout["name"],
                       "step": "cond+uncond DiT forward + guidance + Euler update",
                       "value_formula": "50 * ms_per_step / 1000 (DiT denoising loop; text encoder and VAE decode not in value)",
                       "l2": "activations per step (>700 MB per tensor) exceed the 126 MB L2; no flush needed"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "pipeline": stages, **extra,
        }  # fmt: skip
        if args.quant != "none":
            line["metric"] += f"_{args.quant}"
        if args.attn != "bf16":
            line["metric"] += f"_attn_{args.attn}"
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
