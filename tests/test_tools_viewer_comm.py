"""Checkpoint viewer and the communication check tool (CPU / gloo forms)."""

import json
import os
import subprocess
import sys

import pytest
import torch
from safetensors.torch import save_file

from telefuser_b200.tools import comm_test, weight_viewer
from telefuser_b200.utils.system import find_free_port


def test_weight_viewer_tree_merge_and_export(tmp_path, capsys):
    sd1 = {f"blocks.{i}.attn.q.weight": torch.zeros(8, 8, dtype=torch.bfloat16) for i in range(3)}
    sd1.update({f"blocks.{i}.attn.q.bias": torch.zeros(8, dtype=torch.bfloat16) for i in range(3)})
    sd2 = {"blocks.3.attn.q.weight": torch.zeros(8, 4), "head.weight": torch.zeros(4, 8), "patch.proj.weight": torch.zeros(2, 3, 1, 2, 2)}
    save_file(sd1, str(tmp_path / "m-00001-of-00002.safetensors"))
    save_file(sd2, str(tmp_path / "m-00002-of-00002.safetensors"))
    assert [os.path.basename(f) for f in weight_viewer.expand_file_pattern(str(tmp_path / "m-*.safetensors"))] == [
        "m-00001-of-00002.safetensors", "m-00002-of-00002.safetensors"]  # fmt: skip
    v = weight_viewer.WeightViewer().load_weights(str(tmp_path / "m-*.safetensors"))
    s = v.get_summary()
    assert s["files"] == 2 and s["tensors"] == 9 and s["parameters"] == 3 * 72 + 32 + 32 + 24
    assert s["dtypes"]["BF16"] == 216 and s["bytes"] == 216 * 2 + 88 * 4 and s["top_level"]["blocks"] == 248
    assert set(s["fingerprint"]) >= {"keys", "keys_and_shapes", "registered_as"} and s["fingerprint"]["registered_as"] is None
    lines = v.render(max_depth=5)
    assert any("0..2 (x3, identical)" in line for line in lines) and any(line.strip().startswith("3/") for line in lines)
    assert len(v.render(merge_similar=False)) > len(lines) and len(v.render(max_depth=1)) == 3
    assert weight_viewer.WeightViewer.format_number(1_500_000) == "1.50M"
    torch.save({"state_dict": {"a": {"w": torch.zeros(2, 2)}}}, tmp_path / "x.pt")
    assert weight_viewer.read_torch_checkpoint(str(tmp_path / "x.pt")) == {"a.w": ("float32", (2, 2))}
    assert weight_viewer.main([str(tmp_path / "m-*.safetensors"), "--quiet", "--export", str(tmp_path / "o.json")]) == 0
    assert "9 tensors" in capsys.readouterr().out and json.load(open(tmp_path / "o.json"))["tensors"]["head.weight"]["shape"] == [4, 8]


def test_comm_test_single_process_and_gloo(tmp_path):
    env = comm_test.environment()
    assert env["torch"] == torch.__version__ and isinstance(env["devices"], list)
    r = comm_test.host_device_bandwidth(torch.device("cpu"), 1, warmup=1, iters=2)
    assert r["h2d_gbs"] > 0 and r["d2h_gbs"] > 0
    text = comm_test.format_report({"environment": env, "world": 1, "host_device": [r]})
    assert "host<->device" in text
    out = tmp_path / "report.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(find_free_port()), "-m", "telefuser_b200.tools.comm_test", "--backend", "gloo", "--sizes-mb", "1",
           "--iters", "2", "--json", str(out)]  # fmt: skip
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env={**os.environ, "OMP_NUM_THREADS": "1"})
    assert res.returncode == 0, res.stderr[-2000:]
    rep = json.load(open(out))
    col = rep["collectives"][0]
    assert rep["world"] == 2 and col["world"] == 2 and {"all_reduce", "all_gather", "send_recv_ring"} <= set(col)
    assert col["all_reduce"]["bus_gbs"] > 0 and abs(col["all_reduce"]["bus_gbs"] / col["all_reduce"]["alg_gbs"] - 1.0) < 1e-6  # 2(P-1)/P = 1 at P = 2


def test_lingbot_video_validation_tool_inspect_capture_compare_bench(tmp_path):
    """Checkpoint inspection, a single-process capture against a 2-rank (Ulysses + expert-parallel) capture of the
    same seeded run, and the benchmark line, all on CPU ranks."""
    import json
    import subprocess
    import sys

    import torch
    from safetensors.torch import save_file

    from telefuser_b200.models.lingbot_video import LingBotVideoConfig, LingBotVideoTransformer3DModel
    from telefuser_b200.tools import lingbot_video_validation as V

    model = LingBotVideoTransformer3DModel(LingBotVideoConfig.preset("tiny-moe"))
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, str(tmp_path / "m.safetensors"))
    rep = V.inspect_shapes(V.read_checkpoint_shapes(str(tmp_path / "m.safetensors")))
    assert rep["kind"] == "moe" and rep["depth"] == 2 and rep["num_experts"] == 8 and rep["resolved_preset"] == "moe-30b-a3b"
    assert rep["parameters"] == sum(p.numel() for p in model.state_dict().values()) and rep["shape_mismatches"]  # tiny vs 30B
    single, sp = str(tmp_path / "single.pt"), str(tmp_path / "sp.pt")
    assert V.main(["capture", "--preset", "tiny-moe", "--out", single]) == 0
    env = {**__import__("os").environ, "PYTHONPATH": str(__import__("pathlib").Path(__file__).resolve().parents[1])}
    run = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(find_free_port()), "-m", "telefuser_b200.tools.lingbot_video_validation"]  # fmt: skip
    r = subprocess.run(run + ["capture", "--preset", "tiny-moe", "--layout", "u2", "--expert-parallel", "--out", sp],
                       capture_output=True, text=True, timeout=300, env=env)  # fmt: skip
    assert r.returncode == 0, r.stderr[-2000:]
    assert V.main(["compare", single, sp, "--tol", "1e-4"]) == 0
    a = torch.load(single, weights_only=False)
    a["tensors"]["latent_step01"] += 0.1
    torch.save(a, single)
    assert V.main(["compare", single, sp, "--tol", "1e-4"]) == 1
    r = subprocess.run(run + ["bench", "--preset", "tiny-moe", "--layout", "cfg2", "--steps", "1"], capture_output=True, text=True,
                       timeout=300, env=env)  # fmt: skip
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([x for x in r.stdout.splitlines() if x.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["finite_output"] and line["config"]["parallelism"] == "cfg2 x ulysses1"


def test_resource_monitor_records_and_tells_a_leak_from_a_plateau(tmp_path):
    import os

    from telefuser_b200.tools import resource_monitor as M

    class FakeGPU:
        def __init__(self):
            self.n = 0

        def sample(self):
            self.n += 1
            # gpu0 leaks 1 MB per sample, gpu1 fills a cache for 10 samples and then stays flat
            return [{"index": 0, "util": 50.0, "mem_used_mb": 1000.0 + self.n, "mem_total_mb": 180000.0},
                    {"index": 1, "util": 10.0, "mem_used_mb": 2000.0 + min(self.n, 10) * 5, "mem_total_mb": 180000.0}]

    now = [0.0]
    path = str(tmp_path / "run.csv")
    rows = M.record(path, 10.0, 600.0, None, os.getpid(), collector=FakeGPU(), clock=lambda: now[0],
                    sleep=lambda s: now.__setitem__(0, now[0] + s))  # fmt: skip
    assert rows == 61
    rep = M.report(path, warmup_s=120.0, leak_per_hour=50.0)
    assert rep["samples"] == 61 and rep["leaking_series"] == ["gpu0_mem_mb"]
    assert rep["series"]["gpu0_mem_mb"]["slope_per_hour"] == pytest.approx(360.0, rel=1e-3)
    assert rep["series"]["gpu1_mem_mb"]["leak"] is False and rep["series"]["rss_mb"]["min"] > 0
    assert rep["series"]["processes"]["min"] >= 1
    assert M.main(["report", path, "--warmup-s", "120"]) == 1  # non-zero exit when something leaks
    assert M.fit_slope([0, 1, 2], [1, 3, 5]) == pytest.approx(2.0) and M.analyse([]) == {}


def test_resource_monitor_reads_a_leak_from_the_peaks_of_a_breathing_process(tmp_path, capsys):
    import csv
    import math

    from telefuser_b200.tools import resource_monitor as M

    assert M.local_maxima([0, 1, 0, 2, 0, 3, 0], window=1) == [1, 3, 5] and M.local_maxima([5, 5, 5, 5], window=1) == [0]
    assert M.moving_average([1, 3, 5, 7], 2) == [1.0, 2.0, 4.0, 6.0] and len(M.sparkline(list(range(200)), 50)) == 50
    assert M.sparkline([]) == "" and set(M.sparkline([2.0, 2.0])) == {" "}

    def write(name, drift_mb_per_sample):
        # every request allocates ~400 MB of working memory and frees it again; `drift` is what each one leaves behind
        path = tmp_path / name
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["t", "rss_mb", "gpu0_util"])
            for i in range(400):
                w.writerow([i * 10.0, round(3000 + 400 * max(0.0, math.sin(i * 2 * math.pi / 20)) + drift_mb_per_sample * i, 3), 50])
        return str(path)

    steady, leaking = M.report(write("steady.csv", 0.0), 0.0, 50.0), M.report(write("leaking.csv", 0.2), 0.0, 50.0)
    assert steady["leaking_series"] == [] and steady["series"]["rss_mb"]["peaks"] >= 10
    assert abs(steady["series"]["rss_mb"]["peak_slope_per_hour"]) < 5
    assert leaking["leaking_series"] == ["rss_mb"] and leaking["series"]["rss_mb"]["peak_slope_per_hour"] == pytest.approx(72.0, rel=0.05)
    assert "leak" not in leaking["series"]["gpu0_util"]
    assert M.main(["report", str(tmp_path / "steady.csv"), "--plot"]) == 0
    out = capsys.readouterr().out
    assert "rss_mb" in out.splitlines()[-2] and len(out.splitlines()[-2].split(" ", 1)[1].strip()) > 20


def test_lingbot_video_validation_tool_refiner_handoff(capsys):
    import json

    from telefuser_b200.tools import lingbot_video_validation as V

    assert V.main(["refiner-handoff", "--source-frames", "121", "--source-fps", "30", "--steps", "6", "--t-thresh", "0.5", "--tail-steps", "1",
                   "--moe"]) == 0  # fmt: skip
    rep = json.loads(capsys.readouterr().out)
    assert rep["passed"] and rep["sampled_frames"] == 93 and rep["latent_frames"] == 24  # 121 frames at 30 fps thinned to 24 fps
    assert rep["sigmas"][0] == 0.5 and rep["denoising_steps"] == len(rep["sigmas"]) and all(rep["checks"][k] for k in (
        "start_is_the_stated_mix", "finite", "same_seed_same_result", "other_seed_other_result", "clean_first_frame_kept"))
