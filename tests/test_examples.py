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


def test_frame_replay_service_streams_paced_chunks():
    """The model-free server-push example: loaded by the stream service under strict validation, it pushes the test
    card as paced chunks whose frame counts add up to the clip."""
    import asyncio

    from telefuser_b200.service.stream_service import StreamPipelineService

    svc = StreamPipelineService(ServerConfig(security_level="strict"))
    assert svc.start_service(str(EXAMPLES / "stream_server" / "stream_frame_replay.py"))
    assert svc.stream_mode == "server_push"

    async def collect():
        t0 = time.perf_counter()
        chunks = [c async for c in svc.stream_task({"fps": 400})]
        return chunks, time.perf_counter() - t0

    try:
        chunks, seconds = asyncio.run(collect())
    finally:
        svc.service.stop()
    assert [c["chunk_index"] for c in chunks] == list(range(6)) and sum(c["frames"].shape[0] for c in chunks) == 96
    assert chunks[0]["frames"].dtype == torch.uint8 and chunks[0]["frames"].shape[1:] == (240, 416, 3)
    assert 0.15 < seconds < 5.0  # 96 frames at 400 fps: paced, not dumped at once


@pytest.mark.parametrize("path", REQUEST_FILES + [STREAM_FILE], ids=lambda p: Path(p).stem)
def test_example_imports_and_exposes_the_service_entry_points(path):
    """Importing a pipeline file must not load weights; the names the servers look up exist and every keyword that
    `run_with_file` / `get_pipeline` use resolves (their local imports are executed here too)."""
    import importlib.util
    import inspect

    import sys

    spec = importlib.util.spec_from_file_location("example_" + Path(path).stem, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod  # as the service's loader does (dataclasses look their module up there)
    spec.loader.exec_module(mod)
    if hasattr(mod, "get_service"):
        assert callable(mod.get_service)
        return
    assert callable(mod.get_pipeline) and callable(mod.run_with_file)
    assert isinstance(mod.PIPELINE_MANIFEST["tasks"], list) and mod.PPL_CONFIG["name"]
    params = inspect.signature(mod.run_with_file).parameters
    assert "pipeline" in params and "output_path" in params
    for task, needed in mod.PIPELINE_MANIFEST["required_inputs"].items():
        assert task in mod.PIPELINE_MANIFEST["tasks"] and all(n in params for n in needed), (task, needed)
    # the imports inside get_pipeline / run_with_file must resolve (names that do not exist would only fail with weights)
    import ast
    import importlib
    import textwrap

    for fn in (mod.get_pipeline, mod.run_with_file):
        for node in ast.walk(ast.parse(textwrap.dedent(inspect.getsource(fn)))):
            if isinstance(node, ast.ImportFrom) and node.module and node.module.startswith("telefuser_b200"):
                target = importlib.import_module(node.module)
                for alias in node.names:
                    assert hasattr(target, alias.name), f"{node.module} has no {alias.name}"


def test_lingbot_video_example_request_handling(tmp_path, monkeypatch):
    """The LingBot-Video pipeline files on a tiny random-init model: a rewriter prompt file sets caption and length, a
    one-frame request is saved as a PNG, an image request conditions frame 0, `refine` goes through the refiner stage."""
    import importlib.util
    import json

    import numpy as np
    from PIL import Image

    from telefuser_b200.core.config import ModelRuntimeConfig
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.lingbot_video import LingBotVideoPipeline, LingBotVideoPipelineConfig
    from telefuser_b200.pipelines.lingbot_video.refiner import LingBotVideoRefinerStage
    from telefuser_b200.testing.lingbot_video_checks import make_model
    from telefuser_b200.testing.synthetic import random_init_

    def load(name):
        spec = importlib.util.spec_from_file_location(f"_example_{name}", EXAMPLES / "lingbot_video" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    moe, dense = load("lingbot_video_moe_text_to_video"), load("lingbot_video_dense_text_to_video")
    assert moe.PPL_CONFIG["supports_refiner"] and not dense.PPL_CONFIG["supports_refiner"]
    m = make_model("tiny")
    captions = []

    def text_stage(caption):
        captions.append(caption)
        return torch.randn(1, 5, m.config.text_dim, generator=torch.Generator().manual_seed(len(caption)))

    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(m, "lingbot_video_transformer")
    mm.add_module(random_init_(WanVideoVAE(dim=8).float(), std=0.05).eval(), "wan_video_vae")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = LingBotVideoPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, LingBotVideoPipelineConfig(text_encoding_config=rc(), dit_config=rc(), vae_config=rc(), num_inference_steps=1), text_stage=text_stage)
    monkeypatch.setitem(moe.PPL_CONFIG, "refiner_height", 32)
    monkeypatch.setitem(moe.PPL_CONFIG, "refiner_width", 48)
    monkeypatch.setitem(moe.PPL_CONFIG, "refiner_steps", 2)

    prompt_file = tmp_path / "rewritten.json"
    prompt_file.write_text(json.dumps({"caption": {"subject": "a fox"}, "duration": 0.3, "fps": 24}))
    out = moe.run_with_file(pipe, str(prompt_file), str(tmp_path / "a.mp4"), height=16, width=32)
    assert out["num_frames"] == 9 and os.path.getsize(out["output_path"]) > 0 and captions[0] == '{"subject":"a fox"}'

    still = dense.run_with_file(pipe, "a fox", str(tmp_path / "b.mp4"), num_frames=1, height=16, width=32)
    assert still["output_path"].endswith("b.png") and Image.open(still["output_path"]).size == (32, 16)
    assert json.loads(captions[-1])["universal_negative"] and "temporal_and_motion_stability" not in captions[-1]  # still-image negative

    Image.fromarray(np.random.default_rng(0).integers(0, 255, (40, 50, 3), dtype=np.uint8)).save(tmp_path / "first.png")
    built = []

    def fake_refiner(pipeline):
        built.append(1)
        return LingBotVideoRefinerStage(pipeline.denoising_stage, pipeline.vae_stage, device="cpu", torch_dtype=torch.float32)

    monkeypatch.setattr(moe, "build_refiner", fake_refiner)
    ref = moe.run_with_file(pipe, "a fox", str(tmp_path / "c.mp4"), num_frames=5, height=16, width=32, first_image_path=str(tmp_path / "first.png"),
                            negative_prompt="bad", refine=True)  # fmt: skip
    assert ref["refined"] and built == [1] and captions[-1] == "bad"
    import cv2

    cap = cv2.VideoCapture(ref["output_path"])
    assert (int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)), int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT))) == (48, 32)  # the refiner's size
    cap.release()
    with pytest.raises(FileNotFoundError, match="separate download"):
        load("lingbot_video_moe_text_to_video").build_refiner(pipe)


def test_template_example_runs_quantises_and_its_checkpoints_are_recognised(tmp_path):
    import importlib.util

    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.utils.model_weight import save_state_dict

    import sys

    spec = importlib.util.spec_from_file_location("_example_custom", EXAMPLES / "custom" / "minimal_custom_pipeline.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    pipe = mod.get_pipeline()
    out = mod.run_with_file(pipe, "a template", str(tmp_path / "img" / "a.png"))
    from PIL import Image

    assert Image.open(out["output_path"]).size == (32, 32)
    a = pipe("a template", seed=1)
    assert a.shape == (1, 3, 32, 32) and torch.isfinite(a).all() and torch.equal(a, pipe("a template", seed=1))
    assert not torch.equal(a, pipe("another prompt", seed=1))
    dit = pipe.denoise_stage.dit
    assert dit.enable_quant("int8") == 8 and dit.blocks[0].qkv.weight.dtype == torch.int8 and dit.head.weight.dtype == torch.float32
    b = pipe("a template", seed=1)
    assert ((b - a).norm() / a.norm()).item() < 0.1
    # a checkpoint written from the class is identified by its key fingerprint
    fresh = mod.TinyDiT(mod.PPL_CONFIG["dim"], mod.PPL_CONFIG["heads"], mod.PPL_CONFIG["depth"])
    save_state_dict(fresh.state_dict(), str(tmp_path / "tiny.safetensors"))
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    assert mm.load_model(str(tmp_path / "tiny.safetensors"))
    loaded = mm.fetch_module("tiny_custom_dit")
    assert type(loaded).__name__ == "TinyDiT" and torch.equal(loaded.head.weight, fresh.head.weight)  # (the class of whichever import registered first)
    svc = PipelineService(ServerConfig(security_level="strict"))
    meta = svc.start_pipeline(str(EXAMPLES / "custom" / "minimal_custom_pipeline.py"), "t2i")
    assert meta["supported_tasks"] == ["t2i"] and meta["declared_pipeline_contract"] is True
    res = svc.run_task_with_stop_event({"task": "t2i", "prompt": "served", "output_path": str(tmp_path / "served.png")})
    assert os.path.getsize(res.output_path) > 0


@pytest.mark.parametrize("path", REQUEST_FILES, ids=lambda p: Path(p).stem)
def test_example_manifest_becomes_a_service_contract(path):
    """What `telefuser serve FILE` does before it builds the pipeline: the file's manifest (all examples use the compact form)
    must turn into a contract whose tasks, required inputs and parameter defaults match `run_with_file`."""
    import inspect
    import sys

    from telefuser_b200.service.contract import apply_task_contract_defaults, load_contract, validate_required_task_parameters
    from telefuser_b200.service.pipeline_service import load_pipeline_module

    mod = load_pipeline_module(path)
    if hasattr(mod, "get_service"):
        pytest.skip("a streaming service file")
    contract = load_contract(mod, None, Path(path).stem)
    assert list(contract.supported_tasks) == list(mod.PIPELINE_MANIFEST["tasks"]) and contract.pipeline_name == mod.PPL_CONFIG["name"]
    sig = inspect.signature(mod.run_with_file).parameters
    for task, tc in contract.task_contracts.items():
        assert list(tc.required_inputs) == list(mod.PIPELINE_MANIFEST["required_inputs"][task])
        assert tc.media_type == ("image" if task in ("t2i", "i2i", "edit") else "video")
        for name, pc in tc.parameters.items():
            assert name in sig and sig[name].default == pc.default, (task, name)
        request = {k: "x" for k in tc.required_inputs}
        filled = apply_task_contract_defaults(contract, task, request)
        validate_required_task_parameters(contract, task, filled)
        with pytest.raises(ValueError, match="missing required"):
            validate_required_task_parameters(contract, task, {})
    meta = contract.to_metadata()
    assert meta["task_contracts"].keys() == set(contract.supported_tasks)
    assert sys.modules  # (the loader registers the module; nothing else to check here)


def test_wan21_example_serves_a_request_over_http(tmp_path, monkeypatch):
    """`telefuser serve examples/wan_video/wan21_text_to_video.py -t t2v`, with a tiny random-init model: metadata built from
    the file's compact manifest, a task through the queue, parameter defaults from `run_with_file`, the video download."""
    from fastapi.testclient import TestClient

    from telefuser_b200.service.api import ApiServer

    monkeypatch.setenv("TFB_RANDOM_INIT", "1")
    monkeypatch.setenv("TFB_TINY", "1")
    config = ServerConfig(cache_dir=str(tmp_path / "cache"), security_level="strict")
    svc = PipelineService(config)
    svc.start_pipeline(str(EXAMPLES / "wan_video" / "wan21_text_to_video.py"), "t2v")
    with TestClient(ApiServer(config, svc).app) as client:
        meta = client.get("/v1/service/metadata").json()
        assert meta["pipeline_name"] == "wan21_t2v" and meta["supported_tasks"] == ["t2v"] and meta["declared_pipeline_contract"]
        params = meta["task_contracts"]["t2v"]["parameters"]
        assert params["num_inference_steps"]["default"] == 50 and params["resolution"]["default"] == "480p" and "prompt" not in params
        assert client.post("/v1/tasks/create", json={"task": "i2v", "prompt": "x"}).status_code == 400  # not a task of this pipeline
        r = client.post("/v1/tasks/create", json={"task": "t2v", "prompt": "a fox in snow", "num_frames": 5, "num_inference_steps": 2,
                                                  "resolution": "64x48", "seed": 3})  # fmt: skip
        assert r.status_code == 200, r.text
        tid = r.json()["task_id"]
        for _ in range(600):
            st = client.get(f"/v1/tasks/{tid}/status").json()
            if st["status"] in ("completed", "failed"):
                break
            time.sleep(0.05)
        assert st["status"] == "completed", st
        video = client.get(f"/v1/tasks/{tid}/result").content
        assert len(video) > 500 and b"ftyp" in video[:32]
    svc.stop()
