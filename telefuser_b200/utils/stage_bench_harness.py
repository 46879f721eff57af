"""Replay of one pipeline stage in isolation from a recorded I/O signature.

A timing report (`GlobalTimingRegistry.export`, written when `TELEFUSER_PROFILE_DEBUG=1`) stores for every profiled
stage call the shapes, dtypes and scalar values of its arguments. `StageBenchHarness` rebuilds arguments of the
same signature from random data, calls the stage's method on them, and times it with CUDA events after warm-up,
optionally under `torch.profiler` for a per-kernel table. That lets one DiT denoising stage, VAE decode, or any
other stage of either a 1.3B or a 14B pipeline be measured and profiled without running the stages in front of it.

    python -m telefuser_b200.utils.stage_bench_harness --signature work_dirs/timing.json --stage dit_denoise \\
        --factory examples/wan_video/wan21_text_to_video.py:get_pipeline --attr denoise_stage --steps 3

For iterative stages (`process(latents, num_inference_steps, ...)`) `--override num_inference_steps=1` turns the
replay into a single denoising step. `generate_test_script()` writes a standalone script with the same inputs.
Role parity: telefuser/utils/stage_bench_harness.py:47-740.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch

_DTYPES = {str(d): d for d in (torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32,
                               torch.int16, torch.int8, torch.uint8, torch.bool, torch.float8_e4m3fn)}  # fmt: skip


@dataclass
class HarnessConfig:
    warmup: int = 1
    profile_steps: int = 1
    output_dir: str = "work_dirs/stage_bench"
    with_torch_profiler: bool = False
    seed: int = 0
    device: str | None = None  # None: where the signature says (cuda tensors land on the current device)


@dataclass
class StageIOSignature:
    stage: str
    args: list = field(default_factory=list)
    kwargs: dict = field(default_factory=dict)

    @classmethod
    def from_report(cls, report: dict, stage: str, call_index: int = 0) -> "StageIOSignature":
        """Picks the `call_index`-th recorded call whose name contains `stage`."""
        hits = [r for r in report.get("records", []) if stage in r.get("name", "") and r.get("io_signature")]
        if not hits:
            names = sorted({r.get("name", "") for r in report.get("records", [])})
            raise KeyError(f"no recorded call of a stage matching {stage!r}; recorded: {names}")
        io = hits[min(call_index, len(hits) - 1)]["io_signature"]
        return cls(hits[0]["name"], list(io.get("args", [])), dict(io.get("kwargs", {})))


def materialise(sig: Any, gen: torch.Generator, device: str | None):
    """Signature node -> value: tensors are rebuilt with random contents (N(0, 1) for floats, small non-negative
    integers for integer types, alternating bits for bools), containers recursively, scalars as recorded."""
    if isinstance(sig, dict) and "tensor" in sig and "dtype" in sig:
        dtype = _DTYPES.get(sig["dtype"], torch.float32)
        dev = device or ("cuda" if sig.get("device") == "cuda" and torch.cuda.is_available() else "cpu")
        shape = tuple(sig["tensor"])
        if dtype.is_floating_point:
            base = torch.randn(shape, generator=gen, dtype=torch.float32)
            return base.to(dev).to(dtype)
        if dtype == torch.bool:
            return (torch.arange(max(1, int(torch.tensor(shape).prod()) if shape else 1)) % 2 == 0).reshape(shape or ()).to(dev)
        return torch.randint(0, 8, shape, generator=gen).to(dtype).to(dev)
    if isinstance(sig, dict):
        return {k: materialise(v, gen, device) for k, v in sig.items()}
    if isinstance(sig, list):
        return [materialise(v, gen, device) for v in sig]
    return sig


class StageBenchHarness:
    def __init__(self, stage_name: str, io_signature: StageIOSignature, stage_instance: Any = None,
                 method: str = "process", config: HarnessConfig | None = None) -> None:  # fmt: skip
        self.stage_name, self.signature, self.stage, self.method = stage_name, io_signature, stage_instance, method
        self.config = config or HarnessConfig()
        self.overrides: dict[str, Any] = {}
        self.inputs: tuple[list, dict] | None = None
        self.fn: Callable | None = None

    @classmethod
    def from_signature_file(cls, path: str, stage_name: str, stage_instance: Any = None, method: str = "process",
                            config: HarnessConfig | None = None, call_index: int = 0) -> "StageBenchHarness":  # fmt: skip
        report = json.loads(Path(path).read_text())
        return cls(stage_name, StageIOSignature.from_report(report, stage_name, call_index), stage_instance, method, config)

    # ---- set-up -------------------------------------------------------------------------------------
    def override(self, **values) -> "StageBenchHarness":
        """Replaces recorded keyword arguments (or positional ones by index: `arg1=...`)."""
        self.overrides.update(values)
        return self

    def setup(self) -> None:
        gen = torch.Generator().manual_seed(self.config.seed)
        args = [materialise(a, gen, self.config.device) for a in self.signature.args]
        kwargs = {k: materialise(v, gen, self.config.device) for k, v in self.signature.kwargs.items()}
        for k, v in self.overrides.items():
            if k.startswith("arg") and k[3:].isdigit():
                args[int(k[3:])] = v
            else:
                kwargs[k] = v
        self.inputs = (args, kwargs)
        if self.stage is not None:
            self.fn = getattr(self.stage, self.method)

    def run_single_step(self) -> Any:
        if self.inputs is None:
            self.setup()
        if self.fn is None:
            raise RuntimeError("no stage instance: pass `stage_instance` or use `generate_test_script()`")
        args, kwargs = self.inputs
        out = self.fn(*args, **kwargs)
        return out() if callable(out) else out  # asynchronous stages hand back a waiter

    # ---- measurement --------------------------------------------------------------------------------
    def profile(self, warmup: int | None = None, profile_steps: int | None = None) -> dict:
        warmup = self.config.warmup if warmup is None else warmup
        steps = self.config.profile_steps if profile_steps is None else profile_steps
        cuda = torch.cuda.is_available()
        for _ in range(warmup):
            self.run_single_step()
        if cuda:
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
        prof = None
        if self.config.with_torch_profiler:
            acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if cuda else [])
            prof = torch.profiler.profile(activities=acts)
            prof.__enter__()
        device_ms, wall_ms = [], []
        for _ in range(steps):
            t0 = time.perf_counter()
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            self.run_single_step()
            if cuda:
                e1.record()
                torch.cuda.synchronize()
                device_ms.append(e0.elapsed_time(e1))
            wall_ms.append((time.perf_counter() - t0) * 1e3)
        result = {"stage": self.stage_name, "method": self.method, "warmup": warmup, "steps": steps,
                  "wall_ms": wall_ms, "device_ms": device_ms or None,
                  "peak_allocated_mb": torch.cuda.max_memory_allocated() / 2**20 if cuda else None}  # fmt: skip
        out = Path(self.config.output_dir)
        out.mkdir(parents=True, exist_ok=True)
        if prof is not None:
            prof.__exit__(None, None, None)
            result["kernel_breakdown"] = self.kernel_breakdown(prof)
            (out / f"{self.stage_name}_kernels.txt").write_text(
                prof.key_averages().table(sort_by="cuda_time_total" if cuda else "cpu_time_total", row_limit=40))
        (out / f"{self.stage_name}_bench.json").write_text(json.dumps(result, indent=2))
        return result

    @staticmethod
    def kernel_breakdown(prof, top: int = 15) -> list[dict]:
        """Top device kernels (or host ops without a GPU) by total time, with their share."""
        rows = []
        for e in prof.key_averages():
            t = getattr(e, "device_time_total", 0) or getattr(e, "cuda_time_total", 0) or 0
            rows.append((e.key, float(t) or float(e.cpu_time_total), e.count))
        rows.sort(key=lambda r: -r[1])
        total = sum(r[1] for r in rows) or 1.0
        return [{"name": k, "total_us": round(t, 1), "calls": n, "share": round(t / total, 4)} for k, t, n in rows[:top]]

    # ---- standalone script --------------------------------------------------------------------------
    def generate_test_script(self, factory: str = "", attr: str = "") -> str:
        """A script that rebuilds the same inputs and calls the stage `--steps` times (factory given as
        `file.py:function`, `attr` the attribute of the returned pipeline that holds the stage)."""
        sig = {"stage": self.signature.stage, "args": self.signature.args, "kwargs": self.signature.kwargs}
        return (
            '"""Isolated replay of stage ' + repr(self.stage_name) + ' from its recorded I/O signature."""\n'
            "import json, sys\n\nimport torch\n\n"
            "from telefuser_b200.utils.stage_bench_harness import HarnessConfig, StageBenchHarness, StageIOSignature, load_stage\n\n"
            f"SIGNATURE = json.loads({json.dumps(json.dumps(sig))})\n"
            f"FACTORY, ATTR, METHOD = {factory!r}, {attr!r}, {self.method!r}\n"
            f"OVERRIDES = {self.overrides!r}\n\n"
            "if __name__ == '__main__':\n"
            "    steps = int(sys.argv[1]) if len(sys.argv) > 1 else 1\n"
            "    stage = load_stage(FACTORY, ATTR)\n"
            "    sig = StageIOSignature(SIGNATURE['stage'], SIGNATURE['args'], SIGNATURE['kwargs'])\n"
            "    h = StageBenchHarness(sig.stage, sig, stage, METHOD, HarnessConfig(profile_steps=steps)).override(**OVERRIDES)\n"
            "    print(json.dumps(h.profile(), indent=2))\n"
        )


def load_stage(factory: str, attr: str = ""):
    """`path/to/file.py:function` -> function(); `attr` (dotted) selects the stage on the returned object."""
    path, _, fn = factory.partition(":")
    spec = importlib.util.spec_from_file_location("stage_bench_factory", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    obj = getattr(mod, fn or "get_pipeline")()
    for part in filter(None, attr.split(".")):
        obj = getattr(obj, part)
    return obj


def _parse_override(text: str):
    k, _, v = text.partition("=")
    try:
        return k, json.loads(v)
    except ValueError:
        return k, v


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--signature", required=True, help="timing report with recorded I/O signatures")
    ap.add_argument("--stage", required=True, help="(part of) the recorded stage name")
    ap.add_argument("--factory", default="", help="file.py:function building the pipeline or stage")
    ap.add_argument("--attr", default="", help="attribute path of the stage on the factory's result")
    ap.add_argument("--method", default="process")
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--call-index", type=int, default=0)
    ap.add_argument("--override", action="append", default=[], help="name=json value, repeatable")
    ap.add_argument("--torch-profiler", action="store_true")
    ap.add_argument("--output-dir", default="work_dirs/stage_bench")
    ap.add_argument("--write-script", default="", help="write a standalone replay script here and exit")
    a = ap.parse_args(argv)
    cfg = HarnessConfig(a.warmup, a.steps, a.output_dir, a.torch_profiler)
    stage = load_stage(a.factory, a.attr) if a.factory and not a.write_script else None
    h = StageBenchHarness.from_signature_file(a.signature, a.stage, stage, a.method, cfg, a.call_index)
    h.override(**dict(_parse_override(o) for o in a.override))
    if a.write_script:
        Path(a.write_script).write_text(h.generate_test_script(a.factory, a.attr))
        print(a.write_script)
        return
    print(json.dumps(h.profile(), indent=2))


if __name__ == "__main__":
    main()
