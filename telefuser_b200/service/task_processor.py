"""Task execution: input materialisation -> latent-cache lookup -> pipeline run -> artefact registration.

* `LatentCache`: on-disk store of intermediate latents keyed by the request (prompt, seed, geometry,
  steps). A lookup returns an exact hit or, if allowed, the most similar prompt (token Jaccard) with
  the same geometry, so the run can resume from a saved denoising step. Modes: read / write / readwrite.
  Every cache step is best effort: a failure degrades to "no cache".
* `MediaGenerationService`: turns a request into the kwargs of the pipeline's `run_with_file`.
* `AsyncTaskProcessor`: N asyncio workers (one per processing slot) that claim pending tasks and run
  them in threads, with a per-task timeout and cooperative cancellation.
Role parity: telefuser/service/core/task_service.py:42-189, core/task_processor.py:18-167 (the
reference delegates the cache to an external package; here it is in-tree).
"""

from __future__ import annotations

import asyncio
import hashlib
import json
import os
import re
import threading
import time
from pathlib import Path
from typing import Any

import torch

from telefuser_b200.utils.logging import logger

from .contract import apply_task_contract_defaults, infer_media_type_for_task, validate_required_task_parameters
from .files import ArtifactStore, FileService, MediaType
from .task_manager import TaskManager, TaskStatus

_GEOMETRY_KEYS = ("task", "resolution", "aspect_ratio", "target_video_length", "num_inference_steps", "height", "width",
                  "num_frames")  # fmt: skip


class LatentCache:
    def __init__(self, root: str, mode: str = "readwrite", min_similarity: float = 0.85, max_entries: int = 256) -> None:
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.mode, self.min_similarity, self.max_entries = mode, min_similarity, max_entries
        self._lock = threading.Lock()
        self.hits = self.misses = 0

    @staticmethod
    def _tokens(prompt: str) -> frozenset:
        return frozenset(re.findall(r"\w+", prompt.lower()))

    def build_query(self, data: dict) -> dict:
        geom = {k: data.get(k) for k in _GEOMETRY_KEYS if data.get(k) is not None}
        gkey = hashlib.sha1(json.dumps(geom, sort_keys=True, default=str).encode()).hexdigest()[:16]
        prompt = str(data.get("prompt") or "")
        pkey = hashlib.sha1(f"{prompt}|{data.get('negative_prompt') or ''}|{data.get('seed')}".encode()).hexdigest()[:16]
        return {"geometry": gkey, "key": pkey, "prompt": prompt, "seed": data.get("seed")}

    def _entries(self, gkey: str) -> list[dict]:
        d = self.root / gkey
        out = []
        if d.is_dir():
            for meta in d.glob("*.json"):
                try:
                    out.append(json.loads(meta.read_text()))
                except json.JSONDecodeError:
                    continue
        return out

    def lookup(self, query: dict) -> dict | None:
        if self.mode not in ("read", "readwrite"):
            return None
        best, best_sim = None, 0.0
        qt = self._tokens(query["prompt"])
        for e in self._entries(query["geometry"]):
            if e["key"] == query["key"]:
                best, best_sim = e, 1.0
                break
            if e.get("seed") != query.get("seed"):
                continue
            et = frozenset(e.get("tokens", ()))
            sim = len(qt & et) / max(1, len(qt | et))
            if sim > best_sim:
                best, best_sim = e, sim
        if best is None or best_sim < self.min_similarity:
            self.misses += 1
            return None
        self.hits += 1
        return {**best, "similarity": best_sim}

    def apply_resume(self, hit: dict) -> dict | None:
        """Loads the saved latents; an exact hit resumes at the saved step, a similar prompt earlier."""
        path = hit.get("path")
        if not path or not os.path.isfile(path):
            return None
        payload = torch.load(path, map_location="cpu", weights_only=True)
        steps = sorted(payload["steps"])
        step = steps[-1] if hit["similarity"] >= 1.0 else steps[0]
        return {"latents": payload["steps"][step], "resume_step": int(step), "similarity": hit["similarity"]}

    def save(self, query: dict, latent_payload: dict) -> str | None:
        """`latent_payload`: {"steps": {step_index: latent tensor}}."""
        if self.mode not in ("write", "readwrite") or not latent_payload or not latent_payload.get("steps"):
            return None
        d = self.root / query["geometry"]
        d.mkdir(parents=True, exist_ok=True)
        path = d / f"{query['key']}.pt"
        steps = {int(k): v.detach().to("cpu") for k, v in latent_payload["steps"].items()}
        with self._lock:
            torch.save({"steps": steps}, path)
            meta = {"key": query["key"], "geometry": query["geometry"], "seed": query.get("seed"), "path": str(path),
                    "tokens": sorted(self._tokens(query["prompt"])), "created": time.time()}  # fmt: skip
            (d / f"{query['key']}.json").write_text(json.dumps(meta))
            self._evict()
        return str(path)

    def _evict(self) -> None:
        metas = sorted(self.root.glob("*/*.json"), key=lambda p: p.stat().st_mtime)
        for m in metas[: max(0, len(metas) - self.max_entries)]:
            m.with_suffix(".pt").unlink(missing_ok=True)
            m.unlink(missing_ok=True)


class MediaGenerationService:
    def __init__(self, file_service: FileService, inference_service, artifact_store: ArtifactStore | None = None,
                 latent_cache: LatentCache | None = None) -> None:  # fmt: skip
        self.file_service, self.inference_service = file_service, inference_service
        self.artifact_store, self.latent_cache = artifact_store, latent_cache

    async def prepare(self, message: dict) -> dict:
        data = dict(message)
        fs = self.file_service
        for name, mt in (("first_image_path", MediaType.IMAGE), ("last_image_path", MediaType.IMAGE),
                         ("mask_path", MediaType.IMAGE), ("ref_video_path", MediaType.VIDEO),
                         ("audio_path", MediaType.AUDIO)):  # fmt: skip
            if data.get(name):
                data[name] = await fs.materialise_input(str(data[name]), mt, prefix=data.get("task_id", "input"))
        task = data.get("task", "t2v")
        ext = data.get("output_format", "png") if infer_media_type_for_task(task) == "image" else "mp4"
        name = data.get("output_path") or f"{data.get('task_id', 'out')}.{ext}"
        data["output_path"] = str(fs.output_path_for(str(name)))
        return data

    async def generate_media_with_stop_event(self, message: dict, stop_event: threading.Event) -> dict | None:
        data = await self.prepare(message)
        cache, query = self.latent_cache, None
        if cache is not None:
            try:
                query = cache.build_query(data)
                hit = cache.lookup(query)
                resume = cache.apply_resume(hit) if hit else None
                if resume is not None:
                    data["latent_data"] = resume
            except Exception as e:  # noqa: BLE001
                logger.warning(f"latent cache lookup failed, ignored: {e}")
        loop = asyncio.get_running_loop()
        res = await loop.run_in_executor(None, self.inference_service.run_task_with_stop_event, data, stop_event)
        if stop_event.is_set():
            return None
        if cache is not None and query is not None and res.extra and res.extra.get("latent_payload"):
            try:
                cache.save(query, res.extra["latent_payload"])
            except Exception as e:  # noqa: BLE001
                logger.warning(f"latent cache write-back failed, ignored: {e}")
        out = res.output_path or data["output_path"]
        task = data.get("task", "t2v")
        if self.artifact_store is not None and out and os.path.isfile(out):
            self.artifact_store.register(out, data.get("task_id", ""), task, infer_media_type_for_task(task),
                                         {"prompt": data.get("prompt", "")})  # fmt: skip
        return {"output_path": out, "peak_memory_mb": res.peak_memory_mb, "inference_time_s": res.inference_time_s}


class AsyncTaskProcessor:
    def __init__(self, task_manager: TaskManager, generation: MediaGenerationService, num_workers: int = 1,
                 task_timeout: float = 3600.0, poll_interval: float = 0.02, metrics=None) -> None:  # fmt: skip
        self.tm, self.generation = task_manager, generation
        self.num_workers, self.task_timeout, self.poll = max(1, num_workers), task_timeout, poll_interval
        self.metrics = metrics
        self._workers: list[asyncio.Task] = []
        self._stopping = False

    @property
    def is_running(self) -> bool:
        return any(not w.done() for w in self._workers)

    async def start(self) -> None:
        self._stopping = False
        self._workers = [asyncio.create_task(self._loop(i)) for i in range(self.num_workers)]

    async def stop(self) -> None:
        self._stopping = True
        for w in self._workers:
            w.cancel()
        await asyncio.gather(*self._workers, return_exceptions=True)
        self._workers = []

    async def _loop(self, idx: int) -> None:
        while not self._stopping:
            info = self.tm.claim_next_pending_task()
            if info is None:
                await asyncio.sleep(self.poll)
                continue
            await self._process(info)

    async def _process(self, info) -> None:
        tid, t0 = info.task_id, time.perf_counter()
        msg = info.message if isinstance(info.message, dict) else dict(info.message)
        try:
            res = await asyncio.wait_for(self.generation.generate_media_with_stop_event(msg, info.stop_event),
                                         timeout=self.task_timeout)  # fmt: skip
            if res is None or info.stop_event.is_set():
                self.tm.mark_cancelled(tid)
                status = TaskStatus.CANCELLED
            else:
                self.tm.complete_task(tid, **res)
                status = TaskStatus.COMPLETED
        except asyncio.TimeoutError:
            info.stop_event.set()
            self.tm.fail_task(tid, f"task timed out after {self.task_timeout} s")
            status = TaskStatus.FAILED
        except asyncio.CancelledError:
            info.stop_event.set()
            self.tm.fail_task(tid, "server shutting down")
            raise
        except Exception as e:  # noqa: BLE001
            logger.exception(f"task {tid} failed")
            self.tm.fail_task(tid, f"{type(e).__name__}: {e}")
            status = TaskStatus.FAILED
        finally:
            self.tm.release_processing_slot(tid)
        if self.metrics is not None:
            self.metrics.record_task(msg.get("task", "t2v"), status.value, time.perf_counter() - t0)


def validate_and_fill(contract, message: dict) -> dict:
    """Contract defaults + required-field check for one request (raises ValueError)."""
    task = message.get("task", "t2v")
    data = apply_task_contract_defaults(contract, task, message)
    validate_required_task_parameters(contract, task, data)
    return data


def task_message_defaults(message: dict) -> dict[str, Any]:
    out = dict(message)
    out.setdefault("task", "t2v")
    out.setdefault("seed", 42)
    return out
