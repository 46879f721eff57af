"""Isolated stage replay: a profiled run of the tiny Wan pipeline records the denoising stage's I/O signature; the
harness rebuilds inputs of that signature, replays one denoising step and writes its report and a standalone script."""

import json

import torch

from telefuser_b200.utils import profiler
from telefuser_b200.utils.stage_bench_harness import HarnessConfig, StageBenchHarness, StageIOSignature, main, materialise


def test_materialise_rebuilds_tensors_containers_and_scalars():
    gen = torch.Generator().manual_seed(0)
    sig = {"x": {"tensor": [2, 3], "dtype": "torch.bfloat16", "device": "cpu"}, "ids": {"tensor": [4], "dtype": "torch.int64", "device": "cpu"},
           "flags": {"tensor": [3], "dtype": "torch.bool", "device": "cpu"}, "steps": 4, "name": "euler", "nest": [1.5, None, {"tensor": [1], "dtype": "torch.float32", "device": "cpu"}]}
    out = materialise(sig, gen, None)
    assert out["x"].shape == (2, 3) and out["x"].dtype == torch.bfloat16 and out["ids"].dtype == torch.int64
    assert out["flags"].tolist() == [True, False, True] and out["steps"] == 4 and out["name"] == "euler"
    assert out["nest"][0] == 1.5 and out["nest"][1] is None and out["nest"][2].shape == (1,)


class _Stage:
    def __init__(self):
        self.calls = []

    def process(self, latents, num_inference_steps, context=None, cfg_scale=5.0):
        self.calls.append((tuple(latents.shape), num_inference_steps, None if context is None else tuple(context.shape), cfg_scale))
        x = latents.float()
        for _ in range(num_inference_steps):
            x = x * 0.9 + (0 if context is None else context.float().mean())
        return x


def test_record_replay_and_script(tmp_path, monkeypatch):
    monkeypatch.setenv("TELEFUSER_PROFILE_DEBUG", "1")
    profiler.GlobalTimingRegistry.instance().reset()

    class Recorded(_Stage):  # decorate while profiling is on
        @profiler.ProfilingContext4Debug("toy_denoise")
        def process(self, *a, **k):
            return _Stage.process(self, *a, **k)

    Recorded().process(torch.zeros(1, 16, 3, 8, 8), 4, context=torch.zeros(1, 7, 32, dtype=torch.bfloat16), cfg_scale=3.0)
    report = tmp_path / "timing.json"
    profiler.GlobalTimingRegistry.instance().export(str(report))
    rec = json.loads(report.read_text())["records"][0]
    assert rec["io_signature"]["args"][0]["tensor"] == [1, 16, 3, 8, 8]

    stage = _Stage()
    h = StageBenchHarness.from_signature_file(str(report), "toy_denoise", stage, config=HarnessConfig(1, 2, str(tmp_path / "out")))
    h.override(arg1=1)  # a single denoising step instead of the recorded four
    res = h.profile()
    assert len(stage.calls) == 3 and stage.calls[0] == ((1, 16, 3, 8, 8), 1, (1, 7, 32), 3.0)
    assert res["steps"] == 2 and len(res["wall_ms"]) == 2 and (tmp_path / "out" / "toy_denoise_bench.json").is_file()
    script = h.generate_test_script("factory.py:make", "denoise_stage")
    compile(script, "replay.py", "exec")
    assert "factory.py:make" in script and "'arg1': 1" in script

    out_script = tmp_path / "replay.py"
    main(["--signature", str(report), "--stage", "toy", "--write-script", str(out_script), "--override", "cfg_scale=1.0"])
    assert "cfg_scale" in out_script.read_text()
    try:
        StageIOSignature.from_report(json.loads(report.read_text()), "vae")
    except KeyError as e:
        assert "toy_denoise" in str(e)
    else:
        raise AssertionError("a missing stage must be reported")


def test_memory_checkpoints_report_growth_peaks_and_pool_overhead():
    from telefuser_b200.utils import memory_snapshot as M

    readings = iter([(100 << 20, 128 << 20, 100 << 20, 128 << 20),      # baseline: weights
                     (150 << 20, 192 << 20, 400 << 20, 448 << 20),      # after the text encoder
                     (130 << 20, 512 << 20, 900 << 20, 1024 << 20),     # after denoising: highest peak
                     (140 << 20, 512 << 20, 300 << 20, 1024 << 20),     # a second denoising call reads lower
                     (120 << 20, 512 << 20, 600 << 20, 1024 << 20)])    # after the decode
    cp = M.MemoryCheckpoints(reader=lambda device: next(readings))
    base = cp.set_baseline()
    assert base.allocated_mb == 100 and base.pool_overhead_mb == 28 and round(base.pool_overhead_pct, 3) == 21.875
    cp.record("text")
    cp.record("denoise")
    cp.record("denoise")  # keeps the worse of the two readings per counter
    cp.record("decode")
    a = cp.analysis()
    rows = {r["checkpoint"]: r for r in a["checkpoints"]}
    assert list(rows) == ["text", "denoise", "decode"]
    assert rows["text"]["allocated_over_baseline_mb"] == 50 and rows["denoise"]["allocated_over_previous_mb"] == -10
    assert rows["denoise"]["allocated_mb"] == 140 and rows["denoise"]["peak_allocated_mb"] == 900
    assert a["highest_peak_checkpoint"] == "denoise" and a["highest_peak_reserved_mb"] == 1024
    assert "highest peak: 900.0 MiB at 'denoise'" in cp.summary()
    assert (cp.points["denoise"] - base).allocated_mb == 40
    M.reset_memory_registry()
    M.set_memory_baseline()
    snap = M.record_memory_snapshot("anything")  # without a GPU every counter is zero; with one they are non-negative
    assert snap.allocated_mb >= 0 and "anything" in M.get_memory_snapshots() and M.get_memory_analysis()["checkpoints"]
