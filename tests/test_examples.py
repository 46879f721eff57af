"""The pipeline files under `examples/`: they pass the service's security validation, expose the entry points the
servers load, and two of them boot with random-init weights (a request through `PipelineService`, a streamed
session through the world-model service)."""

import os
import time
from pathlib import Path

import pytest
import torch

from telefuser_b200.service.pipeline_service import PipelineService, ServerConfig

EXAMPLES = Path(__file__).resolve().parents[1] / "examples"
REQUEST_FILES = sorted(str(p) for p in EXAMPLES.glob("*/*.py") if "lingbot_world" not in p.name)
STREAM_FILE = str(EXAMPLES / "lingbot" / "lingbot_world_v2_image_to_video.py")


@pytest.mark.parametrize("path", REQUEST_FILES + [STREAM_FILE], ids=lambda p: Path(p).stem)
def test_example_passes_strict_validation(path):
    res = PipelineService(ServerConfig(security_level="strict")).validate_only(path)
    assert res["passed"], res["violations"]


def test_stage_placement_rules():
    from telefuser_b200.pipelines.lingbot_world_v2 import resolve_stage_devices

    assert resolve_stage_devices(1) == ([0], 0, 0)
    assert resolve_stage_devices(2) == ([0, 1], 0, 1)
    assert resolve_stage_devices(4) == ([0, 1, 2, 3], 0, 1)
    assert resolve_stage_devices(5) == ([0, 1, 2, 3], 4, 4)
    assert resolve_stage_devices(6) == ([0, 1, 2, 3, 4], 5, 5)
    assert resolve_stage_devices(8, 0, 0) == (list(range(8)), 0, 0)
    with pytest.raises(ValueError):
        resolve_stage_devices(0)


def test_v2_facade_rejects_other_control_types():
    from telefuser_b200.pipelines.lingbot_world_v2 import LingBotWorldV2Pipeline, LingBotWorldV2PipelineConfig

    cfg = LingBotWorldV2PipelineConfig(control_type="act")
    with pytest.raises(ValueError, match="camera"):
        LingBotWorldV2Pipeline(device="cpu").init(None, cfg)
    assert LingBotWorldV2PipelineConfig().timestep_indices == (0, 250, 500, 750)


def test_streaming_example_serves_a_session_with_random_weights(monkeypatch):
    monkeypatch.setenv("TFB_RANDOM_INIT", "1")
    monkeypatch.setenv("TFB_TINY", "1")
    from telefuser_b200.service.stream_service import StreamPipelineService

    svc = StreamPipelineService(ServerConfig(security_level="strict"))
    assert svc.start_service(STREAM_FILE, gpu_num=1)
    try:
        inner = svc.service
        emb = torch.randn(1, 8, 64)
        sid = inner.create_session({"height": 64, "width": 64, "max_duration_seconds": 2.0, "prompt_emb": emb,
                                    "image": torch.zeros(3, 64, 64)})
        inner.push_chunk(sid, {"keys": ["w"]})
        msgs = inner.drain(sid, timeout=120.0)
        kinds = [m.get("type") for m in msgs]
        assert "frames" in kinds or "chunk" in kinds, kinds
        inner.close_session(sid)
    finally:
        inner.stop()


def _run_regression(*extra):
    import json
    import subprocess
    import sys

    cmd = [sys.executable, str(EXAMPLES / "run_examples.py"), *extra]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    reports = [json.loads(line) for line in res.stdout.splitlines() if line.startswith("{")]
    return res, reports


def test_regression_runner_on_the_oracle_path(tmp_path):
    """CPU: both runs take the fp32 evaluation, so the videos agree exactly and the stored baseline is matched."""
    res, reports = _run_regression("--only", "wan21_t2v", "--device", "cpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert reports[0]["passed"] and reports[0]["ssim"] == 1.0 and reports[0]["baseline_drift"] <= 5e-3


@pytest.mark.gpu
def test_regression_runner_bf16_kernels_against_the_fp32_oracle():
    """GPU: the whole pipelines (text encoder -> denoising -> VAE decode; streaming runtime) in bf16 on the native
    kernels against their fp32 evaluation from the same seed: PSNR >= 25 dB, SSIM >= 0.85, no NaN, native launches."""
    res, reports = _run_regression("--device", "cuda:0")
    assert len(reports) == 2, res.stdout + res.stderr
    for rep in reports:
        assert rep["passed"], rep
        assert rep["native_launches"] > 0 and rep["psnr_db"] >= 25.0
