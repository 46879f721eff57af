"""End-to-end regression runner for the example pipelines.

Every case builds a small random-init pipeline of one family (same code path as the full model: text encoding,
denoising loop, VAE decode, streaming runtime) and is run twice in isolated subprocesses from the same seed:
once on the production path (bf16, native sm_100a kernels on a GPU) and once on the oracle path (fp32, plain
PyTorch evaluation of every op, `TFB_FORCE_REFERENCE=1`). The two videos are compared (PSNR, SSIM, NaN / Inf
check), wall time and peak device memory of the production run are checked against per-case limits, and summary
statistics of the oracle output are compared with the stored baseline (`examples/data/regression_baseline.json`)
so that a change of the maths itself is noticed too.

    python examples/run_examples.py --list
    python examples/run_examples.py                       # all cases, device auto
    python examples/run_examples.py --only wan21_t2v --device cpu
    python examples/run_examples.py --update-baseline     # after an intended numerical change

Exit code 0 when every case passes. Role parity: examples/run_examples.py of the reference (isolated subprocess
per example, PSNR >= 25 / SSIM >= 0.85 against a baseline, NaN check, time / memory thresholds).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
BASELINE_FILE = ROOT / "examples" / "data" / "regression_baseline.json"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


# ---------------------------------------------------------------------------------------------------
# cases (run inside the child process)
# ---------------------------------------------------------------------------------------------------
def case_wan21_t2v(device: str, dtype):
    import torch

    from telefuser_b200.models.wan_dit import WanModelConfig
    from telefuser_b200.pipelines.wan.wan21_video import Wan21VideoPipeline

    cfg = WanModelConfig(dim=256, ffn_dim=512, num_heads=2, num_layers=2, text_dim=256)
    pipe = Wan21VideoPipeline.from_random_init(cfg, device=device, torch_dtype=dtype, seed=0)
    out = pipe("a red fox trotting through fresh snow", negative_prompt="blurry", num_frames=9, height=64, width=64,
               num_inference_steps=4, seed=7, output_type="pt")  # fmt: skip
    return out[0].float().cpu()  # [3, T, H, W] in [-1, 1]


def case_lingbot_world_stream(device: str, dtype):
    import torch

    from telefuser_b200.core.config import ModelRuntimeConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.lingbot_world_dit import LingBotWorldFastDiT
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.lingbot_world_v2 import LingBotWorldV2Pipeline, LingBotWorldV2PipelineConfig
    from telefuser_b200.testing.synthetic import random_init_

    torch.manual_seed(0)
    dit = random_init_(LingBotWorldFastDiT(in_dim=36, dim=256, ffn_dim=512, text_dim=64, num_heads=2, num_layers=2,
                                           local_attn_size=3, sink_size=1).to(device).to(dtype))  # fmt: skip
    dit.dtype = dtype
    vae = random_init_(WanVideoVAE(dim=16).to(device).to(dtype), std=0.05)
    mm = ModuleManager(torch_dtype=dtype, device=device)
    mm.add_module(dit.eval(), "lingbot_world_fast_dit")
    mm.add_module(vae.eval(), "wan_video_vae")
    dev = torch.device(device)
    rc = lambda: ModelRuntimeConfig(device_type=dev.type, device_id=dev.index or 0, torch_dtype=dtype)  # noqa: E731
    cfg = LingBotWorldV2PipelineConfig(dit_config=rc(), vae_encode_config=rc(), vae_decode_config=rc(),
                                       text_encoding_config=rc(), chunk_size=2, local_attn_size=3, sink_size=1)  # fmt: skip
    pipe = LingBotWorldV2Pipeline(device=device, torch_dtype=dtype)
    pipe.init(mm, cfg)
    try:
        g = torch.Generator().manual_seed(3)
        emb = torch.randn(1, 8, 64, generator=g).to(device, dtype)
        img = torch.rand(3, 64, 64, generator=g) * 2 - 1
        video, _ = pipe.generate_video("", img, num_frames=21, height=64, width=64, seed=5, prompt_emb=emb)
    finally:
        pipe.close()
    video = video.float().cpu()
    return video[0] if video.dim() == 5 else video


CASES = {
    # name: (function, PSNR floor [dB], SSIM floor, seconds limit, peak device MiB limit)
    "wan21_t2v": (case_wan21_t2v, 25.0, 0.85, 600.0, 8192.0),
    "lingbot_world_stream": (case_lingbot_world_stream, 25.0, 0.85, 600.0, 8192.0),
}


# ---------------------------------------------------------------------------------------------------
# metrics
# ---------------------------------------------------------------------------------------------------
from telefuser_b200.utils.quality import psnr, ssim  # noqa: E402


def summary(video) -> dict:
    v = video.double()
    return {"shape": list(video.shape), "mean": round(float(v.mean()), 5), "std": round(float(v.std()), 5),
            "abs_mean": round(float(v.abs().mean()), 5)}  # fmt: skip


# ---------------------------------------------------------------------------------------------------
# child / parent
# ---------------------------------------------------------------------------------------------------
def run_child(name: str, mode: str, device: str, out_path: str) -> None:
    import torch

    fn = CASES[name][0]
    dtype = torch.float32 if (mode == "oracle" or device == "cpu") else torch.bfloat16
    if device.startswith("cuda"):
        torch.cuda.reset_peak_memory_stats()
    t0 = time.perf_counter()
    video = fn(device, dtype)
    if device.startswith("cuda"):
        torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    launches = 0
    if device.startswith("cuda"):
        from telefuser_b200.ops import native

        launches = native.launch_count()
    meta = {"seconds": seconds, "peak_mib": torch.cuda.max_memory_allocated() / 2**20 if device.startswith("cuda") else 0.0,
            "native_launches": launches, "finite": bool(torch.isfinite(video).all())}  # fmt: skip
    torch.save({"video": video, "meta": meta}, out_path)


def spawn(name: str, mode: str, device: str, out_path: str, timeout: float) -> None:
    env = dict(os.environ)
    env.pop("TFB_FORCE_REFERENCE", None)
    if mode == "oracle":
        env["TFB_FORCE_REFERENCE"] = "1"
    cmd = [sys.executable, str(Path(__file__).resolve()), "--run-case", name, "--mode", mode, "--device", device, "--out", out_path]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    if res.returncode != 0:
        raise RuntimeError(f"{name} [{mode}] exited with {res.returncode}:\n{res.stderr[-3000:]}")


def run_case(name: str, device: str, baseline: dict, update: bool) -> dict:
    import torch

    _, psnr_min, ssim_min, sec_max, mib_max = CASES[name]
    with tempfile.TemporaryDirectory() as tmp:
        outs = {}
        for mode in ("native", "oracle"):
            path = os.path.join(tmp, f"{mode}.pt")
            spawn(name, mode, device, path, sec_max * 2)
            outs[mode] = torch.load(path, weights_only=False)
    nat, ora = outs["native"], outs["oracle"]
    report = {"case": name, "device": device, "psnr_db": round(psnr(nat["video"], ora["video"]), 2),
              "ssim": round(ssim(nat["video"], ora["video"]), 4), "seconds": round(nat["meta"]["seconds"], 2),
              "peak_mib": round(nat["meta"]["peak_mib"], 1), "native_launches": nat["meta"]["native_launches"],
              "oracle": summary(ora["video"]), "failures": []}  # fmt: skip
    fail = report["failures"]
    if not (nat["meta"]["finite"] and ora["meta"]["finite"]):
        fail.append("NaN or Inf in the output")
    if report["psnr_db"] < psnr_min:
        fail.append(f"PSNR {report['psnr_db']} dB below {psnr_min}")
    if report["ssim"] < ssim_min:
        fail.append(f"SSIM {report['ssim']} below {ssim_min}")
    if report["seconds"] > sec_max:
        fail.append(f"{report['seconds']} s above the limit of {sec_max} s")
    if report["peak_mib"] > mib_max:
        fail.append(f"peak memory {report['peak_mib']} MiB above {mib_max}")
    if device.startswith("cuda") and report["native_launches"] == 0:
        fail.append("the production run launched no native kernel")
    kind = device.split(":")[0]
    base = baseline.get(name)
    if base is not None and base.get("device", "cpu") != kind and not update:
        report["baseline"] = f"recorded on {base.get('device', 'cpu')}: not compared on {kind}"
    elif update or base is None:
        baseline[name] = {**report["oracle"], "device": kind}
        report["baseline"] = "stored"
    else:
        drift = max(abs(report["oracle"][k] - base[k]) for k in ("mean", "std", "abs_mean"))
        report["baseline_drift"] = round(drift, 6)
        if report["oracle"]["shape"] != base["shape"] or drift > 5e-3:
            fail.append(f"oracle output moved away from the stored baseline (drift {drift:.4g})")
    report["passed"] = not fail
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--only", action="append", default=[])
    ap.add_argument("--device", default="auto")
    ap.add_argument("--update-baseline", action="store_true")
    ap.add_argument("--baseline", default=str(BASELINE_FILE))
    ap.add_argument("--run-case")
    ap.add_argument("--mode", default="native", choices=["native", "oracle"])
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    if a.list:
        print("\n".join(CASES))
        return 0
    device = a.device
    if device == "auto":
        import torch

        device = "cuda:0" if torch.cuda.is_available() else "cpu"
    if a.run_case:
        run_child(a.run_case, a.mode, device, a.out)
        return 0
    path = Path(a.baseline)
    baseline = json.loads(path.read_text()) if path.is_file() else {}
    names = a.only or list(CASES)
    ok = True
    for name in names:
        rep = run_case(name, device, baseline, a.update_baseline)
        ok &= rep["passed"]
        print(json.dumps(rep), flush=True)
    if a.update_baseline or not path.is_file():
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(baseline, indent=1, sort_keys=True) + "\n")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
