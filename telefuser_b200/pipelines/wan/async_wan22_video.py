"""Wan2.2 A14B pipeline driven by the request-level orchestrator: stage events while a video is generated.

The same stages as `Wan22VideoPipeline` are described as a DAG (`StageConfig`): text encoding and reference-image
VAE encoding run concurrently (group "init"), then denoising, VAE decoding (the two VAE stages share a lock: one
model) and saving the artefact. `agenerate` yields one `stage_end` event per finished stage, an `error` event if a
stage fails, and a `final` event with the saved artefact and a snapshot of the request parameters.
Role parity: telefuser/pipelines/wan_video/async_wan22_video.py:30-467.
"""

from __future__ import annotations

import asyncio
import os
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from telefuser_b200.orchestrator.artifact_save import ArtifactSaveConfig, ArtifactSaveStage
from telefuser_b200.orchestrator.flexible import FlexiblePipelineOrchestrator, StageConfig

from .wan22_video import Wan22VideoPipeline, Wan22VideoPipelineConfig, _round_frames

EVENT_VERSION = "teleai.v2.event.v1"


@dataclass
class AsyncWan22VideoPipelineConfig(Wan22VideoPipelineConfig):
    name: str = ""
    output_root: str = ""


class AsyncWan22VideoPipeline(Wan22VideoPipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.run_name = "wan22_video"
        self.default_artifact_fps, self.default_artifact_quality = 16, 6
        self._orchestrator: FlexiblePipelineOrchestrator | None = None
        self._orchestrator_lock = asyncio.Lock()
        self.artifact_save_stage = ArtifactSaveStage()

    def init(self, module_manager, config, text_stage=None):
        super().init(module_manager, config, text_stage=text_stage)
        if getattr(config, "name", ""):
            self.run_name = config.name

    def _artifact_root(self) -> Path:
        root = getattr(self.config, "output_root", "") or os.getenv("TELEFUSER_OUTPUT_DIR", "outputs")
        return Path(root).expanduser().resolve()

    def normalize_request(self, *, prompt: str, input_image=None, negative_prompt: str = "", end_image=None, seed=None,
                          rand_device=None, height: int = 480, width: int = 832, num_frames: int = 81,
                          num_inference_steps: int = 50, sigma_shift: float = 5.0, tiled: bool = False, tile_size=(30, 52),
                          tile_stride=(15, 26), cfg_scale_high: float = 5.0, cfg_scale_low: float = 5.0,
                          boundary: float = 0.875, artifact_fps=None, artifact_quality=None, file_ext: str = ".mp4") -> dict:  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        return dict(prompt=prompt, negative_prompt=negative_prompt, input_image=input_image, end_image=end_image, seed=seed,
                    rand_device=rand_device, height=height, width=width, num_frames=_round_frames(num_frames),
                    num_inference_steps=num_inference_steps, sigma_shift=sigma_shift, tiled=tiled, tile_size=tile_size,
                    tile_stride=tile_stride, cfg_scale_high=cfg_scale_high, cfg_scale_low=cfg_scale_low, boundary=boundary,
                    artifact_fps=int(artifact_fps or self.default_artifact_fps), file_ext=file_ext,
                    artifact_quality=int(artifact_quality or self.default_artifact_quality))  # fmt: skip

    def get_orchestrator_stage_configs(self, with_image: bool = True) -> list[StageConfig]:
        tiler = lambda c: dict(tiled=bool(c.get("tiled", False)), tile_size=c.get("tile_size", (30, 52)),  # noqa: E731
                               tile_stride=c.get("tile_stride", (15, 26)))  # fmt: skip

        def text(ctx, _prev):
            prompts = [ctx.get("prompt", "")]
            if float(ctx.get("cfg_scale_high", 1.0)) != 1.0:
                prompts.append(ctx.get("negative_prompt", ""))
            return (prompts,), {}

        def vae_encode(ctx, _prev):
            img = ctx.get("input_image")
            if img is None:
                return ("noop",), {}
            h, w = int(ctx["height"]), int(ctx["width"])
            first = img if isinstance(img, torch.Tensor) else self.preprocess_image(img, h, w)
            end = ctx.get("end_image")
            end = None if end is None else (end if isinstance(end, torch.Tensor) else self.preprocess_image(end, h, w))
            return ("encode_image", first, end, int(ctx["num_frames"])), tiler(ctx)

        def denoise(ctx, _prev):
            h, w, n = int(ctx["height"]), int(ctx["width"]), int(ctx["num_frames"])
            noise = self.generate_noise((1, 16, (n - 1) // 4 + 1, h // 8, w // 8), seed=ctx.get("seed"),
                                        device=ctx.get("rand_device") or "cpu", dtype=torch.float32)  # fmt: skip
            embs = ctx["results"]["text_encoding"]
            hi = float(ctx.get("cfg_scale_high", 1.0))
            args = (noise.to(self.device), int(ctx.get("num_inference_steps", 50)), ctx["results"].get("vae_encode"), embs[0],
                    embs[1] if hi != 1.0 else None, hi, float(ctx.get("cfg_scale_low", 1.0)), float(ctx.get("sigma_shift", 5.0)),
                    float(ctx.get("boundary", 0.875)))  # fmt: skip
            return args, {}

        def vae_decode(ctx, _prev):
            return ("decode_video", ctx["results"]["denoise"]), tiler(ctx)

        def save(ctx, _prev):
            cfg = ArtifactSaveConfig(output_root=self._artifact_root(), run_name=self.run_name, fps=int(ctx["artifact_fps"]),
                                     quality=int(ctx["artifact_quality"]))  # fmt: skip
            return (ctx["results"]["vae_decode"],), {"request_id": str(ctx.get("request_id", "req")), "config": cfg,
                                                      "file_ext": ctx.get("file_ext", ".mp4")}  # fmt: skip

        stages = [StageConfig(0, "text_encoding", "text_encoding_stage", text, parallel_group="init",
                              metadata={"role": "encode_text", "output_key": "prompt_emb_list"})]  # fmt: skip
        if with_image:
            stages.append(StageConfig(1, "vae_encode", "_vae_encode_or_skip", vae_encode, shared_lock_group="vae",
                                      parallel_group="init", metadata={"role": "encode_ref", "output_key": "ref_latent"}))  # fmt: skip
        stages += [
            StageConfig(2, "denoise", "denoise_stage", denoise, metadata={"role": "denoise", "output_key": "denoised_latents"}),
            StageConfig(3, "vae_decode", "vae_stage", vae_decode, result_processor=lambda out: self.tensor2video(out[0]),
                        shared_lock_group="vae", metadata={"role": "decode", "output_key": "frames"}),
            StageConfig(4, "artifact_save", "artifact_save_stage", save,
                        metadata={"role": "artifact_save", "output_key": "video_artifact"}),
        ]  # fmt: skip
        return stages

    def _vae_encode_or_skip(self, method: str, *args, **kwargs):
        """Text-to-video requests pass through the reference-image stage without touching the VAE."""
        if method == "noop":
            return None
        out = self.vae_stage.process(method, *args, **kwargs)
        return out() if callable(out) else out

    async def astart(self) -> None:
        async with self._orchestrator_lock:
            if self._orchestrator is None:
                self._orchestrator = FlexiblePipelineOrchestrator(self, self.get_orchestrator_stage_configs())
                await self._orchestrator.start()

    async def astop(self) -> None:
        async with self._orchestrator_lock:
            if self._orchestrator is not None:
                await self._orchestrator.stop()
                self._orchestrator = None

    async def agenerate(self, *, request_id: str, include_raw: bool = False, **kwargs: Any):
        await self.astart()
        inputs = self.normalize_request(**kwargs)
        inputs["request_id"] = request_id
        by_id = {c.stage_id: c for c in self._orchestrator.stage_configs}
        head = {"v": EVENT_VERSION, "request_id": request_id, "pipeline": {"pipeline": "wan22_video", "run_name": self.run_name}}
        seq, t0 = 0, time.time()
        async for raw in self._orchestrator.generate(inputs, request_id=request_id):
            seq += 1
            evt = dict(head, seq=seq, ts_ms=int(time.time() * 1000))
            cfg = by_id.get(raw.get("stage_id", -1))
            stage = None if cfg is None else {"id": cfg.stage_id, "name": cfg.stage_name, "role": cfg.metadata.get("role"),
                                              "group": cfg.parallel_group}  # fmt: skip
            if raw.get("error"):
                evt.update(type="error", error={"message": raw["error"], "stage": stage})
            elif not raw.get("finished", False):
                key = cfg.metadata.get("output_key") if cfg else None
                evt.update(type="stage_end", stage=stage, timing={"duration_ms": 1000 * float(raw.get("metrics", {}).get("seconds", 0))},
                           payload={"output_key": key, "output_ref": f"context.{key}" if key else None})  # fmt: skip
            else:
                artifact = raw.get("results", {}).get("artifact_save", raw.get("outputs"))
                snap = {k: inputs.get(k) for k in ("seed", "num_inference_steps", "num_frames", "height", "width", "sigma_shift",
                                                    "cfg_scale_high", "cfg_scale_low", "boundary")}  # fmt: skip
                evt.update(type="final", timing={"total_ms": int(1000 * (time.time() - t0))},
                           payload={"artifacts": [artifact] if artifact is not None else [], "params_snapshot": snap})  # fmt: skip
            if include_raw:
                evt["raw"] = raw
            yield evt
            if evt["type"] == "error":
                return
