"""HTTP API: task routes, service routes (health / ready / status / metadata / metrics), file download,
streaming (WebSocket transport + session routes, WebRTC signalling when `aiortc` exists), OpenAI-style
image / video routes, and middleware (request logging, metrics, sliding-window rate limit).

Route parity: telefuser/service/api/routers/{tasks,service,files,stream,webrtc}.py,
api/openai/{image_routes,video_routes,protocol,adapter}.py, api/middleware.py, api/api_server.py.
"""

from __future__ import annotations

import asyncio
import base64
import json
import time
import uuid
from collections import defaultdict, deque
from pathlib import Path
from typing import Any

from fastapi import APIRouter, FastAPI, File, HTTPException, Request, UploadFile, WebSocket, WebSocketDisconnect
from fastapi.responses import FileResponse, JSONResponse, PlainTextResponse
from pydantic import BaseModel, ConfigDict, Field, field_validator
from starlette.middleware.base import BaseHTTPMiddleware

from telefuser_b200.metrics.service_metrics import ServiceMetrics
from telefuser_b200.utils.logging import logger

from .contract import infer_media_type_for_task, validate_task_name_format
from .files import ArtifactStore, FileService, MediaError, MediaType
from .pipeline_service import ServerConfig
from .stream_service import AudioChunk, StreamPipelineService, StreamSessionManager, frame_to_jpeg, webrtc_available
from .task_manager import ACTIVE, NoCapacityError, QueueFullError, TaskManager, TaskStatus
from .task_processor import AsyncTaskProcessor, LatentCache, MediaGenerationService, validate_and_fill

ASPECT_RATIOS = ("16:9", "9:16", "4:3", "3:4", "1:1", "2:3", "3:2")


class TaskRequest(BaseModel):
    model_config = ConfigDict(extra="allow")

    task_id: str = Field(default_factory=lambda: uuid.uuid4().hex)
    task: str = "t2v"
    prompt: str = ""
    negative_prompt: str = ""
    first_image_path: str = ""
    last_image_path: str = ""
    ref_video_path: str = ""
    output_path: str = ""
    target_video_length: int = 5
    resolution: str = "720p"
    seed: int = 42
    aspect_ratio: str = "16:9"
    output_format: str = "png"

    @field_validator("aspect_ratio")
    @classmethod
    def _ratio(cls, v: str) -> str:
        if v not in ASPECT_RATIOS:
            raise ValueError(f"Invalid aspect ratio. Allowed values are: {', '.join(ASPECT_RATIOS)}")
        return v

    @field_validator("task")
    @classmethod
    def _task(cls, v: str) -> str:
        return validate_task_name_format(v)

    def payload(self) -> dict:
        d = self.model_dump()
        if not d["output_path"]:
            ext = d["output_format"] if infer_media_type_for_task(d["task"]) == "image" else "mp4"
            d["output_path"] = f"{d['task_id']}.{ext}"
        return d


class TaskResponse(BaseModel):
    task_id: str
    task_status: str
    output_path: str = ""
    peak_memory_mb: float | None = None
    inference_time_s: float | None = None


class StopTaskResponse(BaseModel):
    stop_status: str
    reason: str


# ---------------------------------------------------------------------------
# middleware
# ---------------------------------------------------------------------------
class RateLimiter:
    """Sliding window per client key."""

    def __init__(self, max_requests: int, window_s: float) -> None:
        self.max, self.window = max_requests, window_s
        self.hits: dict[str, deque] = defaultdict(deque)

    def allow(self, key: str, now: float | None = None) -> tuple[bool, float]:
        now = time.monotonic() if now is None else now
        q = self.hits[key]
        while q and now - q[0] > self.window:
            q.popleft()
        if len(q) >= self.max:
            return False, self.window - (now - q[0])
        q.append(now)
        return True, 0.0


class ServiceMiddleware(BaseHTTPMiddleware):
    EXEMPT = ("/v1/service/health", "/v1/service/ready", "/v1/service/metrics")

    def __init__(self, app, metrics: ServiceMetrics | None, limiter: RateLimiter | None) -> None:
        super().__init__(app)
        self.metrics, self.limiter = metrics, limiter

    async def dispatch(self, request: Request, call_next):
        path = request.url.path
        if self.limiter is not None and not path.startswith(self.EXEMPT):
            key = request.client.host if request.client else "unknown"
            ok, retry = self.limiter.allow(key)
            if not ok:
                return JSONResponse({"detail": "rate limit exceeded"}, status_code=429,
                                    headers={"Retry-After": str(int(retry) + 1)})  # fmt: skip
        t0 = time.perf_counter()
        rid = request.headers.get("x-request-id") or uuid.uuid4().hex[:12]
        try:
            response = await call_next(request)
        except Exception:
            if self.metrics is not None:
                self.metrics.record_request(request.method, path, 500, time.perf_counter() - t0)
            raise
        dt = time.perf_counter() - t0
        response.headers["x-request-id"] = rid
        response.headers["x-process-time"] = f"{dt:.4f}"
        if self.metrics is not None:
            self.metrics.record_request(request.method, path, response.status_code, dt)
        if not path.startswith(self.EXEMPT):
            logger.info(f"[{rid}] {request.method} {path} -> {response.status_code} in {dt * 1e3:.1f} ms")
        return response


# ---------------------------------------------------------------------------
# server object
# ---------------------------------------------------------------------------
class ApiServer:
    """Holds the services and builds the FastAPI app. `inference_service` is a PipelineService or a
    PipelinePool (anything with `run_task_with_stop_event`, `metadata()`, `ready`)."""

    def __init__(self, config: ServerConfig | None = None, inference_service=None,
                 stream_service: StreamPipelineService | None = None, num_workers: int = 1) -> None:  # fmt: skip
        self.config = config or ServerConfig()
        self.inference_service = inference_service
        self.stream_service = stream_service
        self.file_service = FileService(self.config.cache_dir, self.config.max_upload_mb)
        self.artifacts = ArtifactStore(str(Path(self.config.cache_dir) / "artifacts"), self.config.artifact_retention_hours,
                                       self.config.artifact_max_gb)  # fmt: skip
        self.metrics = ServiceMetrics() if self.config.metrics_enabled else None
        self.num_workers = num_workers
        self.task_manager = TaskManager(self.config.max_queue_size, self.config.cleanup_keep_count, num_workers)
        cache = None
        if self.config.enable_latent_cache:
            cache = LatentCache(self.config.latent_cache_dir or str(Path(self.config.cache_dir) / "latent_cache"),
                                self.config.latent_cache_mode, self.config.latent_cache_min_similarity)  # fmt: skip
        self.latent_cache = cache
        self.generation = MediaGenerationService(self.file_service, inference_service, self.artifacts, cache)
        self.processor = AsyncTaskProcessor(self.task_manager, self.generation, num_workers, self.config.task_timeout,
                                            metrics=self.metrics)  # fmt: skip
        self.sessions = None
        if stream_service is not None:
            self.sessions = StreamSessionManager(stream_service, self.config.stream_fps,
                                                 disconnect_grace_s=self.config.webrtc_disconnect_grace_s,
                                                 max_sessions=self.config.stream_max_sessions)  # fmt: skip
        self.started = time.time()
        self.app = self._build_app()

    # ---- shared operations (used by the native and the OpenAI-style routes) ----
    def contract(self):
        svc = self.inference_service
        return getattr(svc, "contract", None)

    def submit(self, payload: dict) -> TaskResponse:
        if self.inference_service is None or not self.inference_service.ready:
            raise HTTPException(503, "pipeline is not ready")
        contract = self.contract()
        try:
            if contract is not None:
                payload = validate_and_fill(contract, payload)
            else:
                meta = self.inference_service.metadata() or {}
                tasks = meta.get("supported_tasks")
                if tasks and payload.get("task") not in tasks:
                    raise ValueError(f"task {payload.get('task')!r} is not supported (supported: {tasks})")
            tid = self.task_manager.create_task(payload)
        except QueueFullError as e:
            raise HTTPException(429, str(e)) from e
        except NoCapacityError as e:
            raise HTTPException(503, str(e)) from e
        except ValueError as e:
            raise HTTPException(400, str(e)) from e
        except RuntimeError as e:
            raise HTTPException(409, str(e)) from e
        self._update_queue_metrics()
        return TaskResponse(task_id=tid, task_status=TaskStatus.PENDING.value, output_path=payload.get("output_path", ""))

    async def wait_for_completion(self, task_id: str, timeout: float | None = None) -> dict:
        deadline = time.monotonic() + (timeout or self.config.task_timeout)
        while time.monotonic() < deadline:
            st = self.task_manager.get_task(task_id)
            if st is None:
                raise HTTPException(404, "Task not found")
            if st.status not in ACTIVE:
                return st.to_dict()
            await asyncio.sleep(0.02)
        raise HTTPException(504, "task did not finish in time")

    def cancel(self, task_id: str) -> StopTaskResponse:
        t = self.task_manager.get_task(task_id)
        if t is None:
            return StopTaskResponse(stop_status="do_nothing", reason="Task not found.")
        if t.status not in ACTIVE:
            return StopTaskResponse(stop_status="do_nothing", reason=f"Task already terminal: {t.status.value}.")
        self.task_manager.cancel_task(task_id)
        return StopTaskResponse(stop_status="success", reason="Task cancellation accepted.")

    def _update_queue_metrics(self) -> None:
        if self.metrics is not None:
            c = self.task_manager.queue_status()["counts"]
            self.metrics.set_queue(c["pending"], c["processing"])

    def base_url(self, request: Request | None = None) -> str:
        if request is not None:
            return str(request.base_url).rstrip("/")
        return f"http://{self.config.host}:{self.config.port}"

    # ---- app ----
    def _build_app(self) -> FastAPI:
        from contextlib import asynccontextmanager

        @asynccontextmanager
        async def lifespan(app: FastAPI):
            if self.inference_service is not None:
                await self.processor.start()
            if self.metrics is not None:
                self.metrics.start_gpu_polling()
            reaper = asyncio.create_task(self._reap_loop()) if self.sessions is not None else None
            yield
            if reaper is not None:
                reaper.cancel()
            await self.processor.stop()
            if self.sessions is not None:
                await self.sessions.close_all()
            if self.stream_service is not None:
                await self.stream_service.aclose()
            if self.metrics is not None:
                self.metrics.stop()

        app = FastAPI(title="telefuser-b200", version="0.1", lifespan=lifespan)
        limiter = None
        if self.config.rate_limit_enabled:
            limiter = RateLimiter(self.config.rate_limit_requests, self.config.rate_limit_window_s)
        app.add_middleware(ServiceMiddleware, metrics=self.metrics, limiter=limiter)
        app.include_router(self._tasks_router())
        app.include_router(self._service_router())
        app.include_router(self._files_router())
        if self.stream_service is not None:
            app.include_router(self._stream_router())

            @app.get("/ui", include_in_schema=False)
            async def stream_ui():
                """The browser front end of the streaming service (one static page; it talks to /v1/stream/ws).
                Role of the reference's webui/stream_app.py, without a UI framework on the server."""
                from fastapi.responses import HTMLResponse

                page = Path(__file__).resolve().parent / "webui" / "stream.html"
                return HTMLResponse(page.read_text(encoding="utf-8"))
        from .openai_api import build_openai_routers

        for r in build_openai_routers(self):
            app.include_router(r)
        return app

    async def _reap_loop(self) -> None:
        while True:
            await asyncio.sleep(1.0)
            await self.sessions.reap()

    # ---- /v1/tasks ----
    def _tasks_router(self) -> APIRouter:
        r = APIRouter(prefix="/v1/tasks", tags=["tasks"])

        @r.post("/create", response_model=TaskResponse)
        async def create(message: TaskRequest) -> TaskResponse:
            for name in ("first_image_path", "last_image_path"):
                v = getattr(message, name)
                if v.startswith("http") and not await self.file_service.url_is_reachable(v):
                    raise HTTPException(400, f"{name} URL is not accessible")
            return self.submit(message.payload())

        @r.post("/form", response_model=TaskResponse)
        async def create_form(request: Request, first_image_file: UploadFile | None = File(None),
                              last_image_file: UploadFile | None = File(None)) -> TaskResponse:  # fmt: skip
            form = await request.form()
            payload: dict[str, Any] = {}
            for k, v in form.items():
                if isinstance(v, str):  # declared fields are parsed by the schema; extras are typed by their text
                    payload[k] = v if k in TaskRequest.model_fields else _coerce_form_value(v)
            try:
                if first_image_file is not None and first_image_file.filename:
                    is_video = (first_image_file.content_type or "").startswith("video/")
                    key, mt = ("ref_video_path", MediaType.VIDEO) if is_video else ("first_image_path", MediaType.IMAGE)
                    payload[key] = await self.file_service.save_upload(first_image_file, mt)
                if last_image_file is not None and last_image_file.filename:
                    payload["last_image_path"] = await self.file_service.save_upload(last_image_file, MediaType.IMAGE)
            except MediaError as e:
                raise HTTPException(400, str(e)) from e
            if not payload.get("task"):
                payload["task"] = ("vc" if payload.get("ref_video_path") else "fl2v" if payload.get("last_image_path")
                                   else "i2v" if payload.get("first_image_path") else "t2v")  # fmt: skip
            try:
                msg = TaskRequest(**payload)
            except ValueError as e:
                raise HTTPException(422, str(e)) from e
            return self.submit(msg.payload())

        @r.get("/")
        async def list_tasks() -> dict:
            return {"tasks": [t.to_dict() for t in list(self.task_manager._tasks.values())]}

        @r.get("/queue/status")
        async def queue_status() -> dict:
            q = self.task_manager.queue_status()
            c = q["counts"]
            active = c["pending"] + c["processing"] + c["streaming"]
            return {"is_processing": c["processing"] > 0, "current_task": self.task_manager.current_task_id(),
                    "pending_count": c["pending"], "active_count": active,
                    "queue_size": q["max_queue_size"], "queue_available": q["max_queue_size"] - active, **q}  # fmt: skip

        @r.get("/{task_id}/status")
        async def status(task_id: str) -> dict:
            st = self.task_manager.get_status(task_id)
            if st is None:
                raise HTTPException(404, "Task not found")
            return st

        @r.get("/{task_id}/result")
        async def result(task_id: str):
            t = self.task_manager.get_task(task_id)
            if t is None:
                raise HTTPException(404, "Task not found")
            if t.status != TaskStatus.COMPLETED or not t.output_path or not Path(t.output_path).is_file():
                raise HTTPException(409, f"task is {t.status.value}")
            return FileResponse(t.output_path, filename=Path(t.output_path).name)

        @r.delete("/{task_id}", response_model=StopTaskResponse)
        async def stop(task_id: str) -> StopTaskResponse:
            return self.cancel(task_id)

        return r

    # ---- /v1/service ----
    def _service_router(self) -> APIRouter:
        r = APIRouter(prefix="/v1/service", tags=["service"])

        @r.get("/status")
        async def status() -> dict:
            out = {"uptime_s": time.time() - self.started, "queue": self.task_manager.queue_status(),
                   "pipeline_ready": bool(self.inference_service and self.inference_service.ready)}  # fmt: skip
            if hasattr(self.inference_service, "status"):
                out["pool"] = self.inference_service.status()
            if self.stream_service is not None:
                out["stream"] = self.stream_service.server_metadata()
            if self.latent_cache is not None:
                out["latent_cache"] = {"hits": self.latent_cache.hits, "misses": self.latent_cache.misses}
            return out

        @r.get("/metadata")
        async def metadata() -> dict:
            meta = dict(self.inference_service.metadata()) if self.inference_service is not None else {}
            if meta:
                meta.update(service_effective_max_concurrent_tasks=self.task_manager.queue_status().get("processing_slots", 1),
                            service_configured_max_concurrent_tasks=self.num_workers, max_queue_size=self.config.max_queue_size)  # fmt: skip
            if self.stream_service is not None:
                meta["stream"] = self.stream_service.server_metadata()
            meta["webrtc_available"] = webrtc_available()
            return meta

        @r.get("/health")
        async def health() -> dict:
            from datetime import datetime, timezone
            from importlib.metadata import PackageNotFoundError, version

            try:
                ver = version("telefuser-b200")
            except PackageNotFoundError:
                ver = "source"
            ready = bool((self.inference_service and self.inference_service.ready)
                         or (self.stream_service and self.stream_service.is_running))  # fmt: skip
            return {"status": "healthy", "timestamp": datetime.now(timezone.utc).isoformat(timespec="seconds"),
                    "version": ver, "pipeline_ready": ready}  # fmt: skip

        @r.get("/ready")
        async def ready():
            ok = bool((self.inference_service and self.inference_service.ready)
                      or (self.stream_service and self.stream_service.is_running))  # fmt: skip
            return JSONResponse({"ready": ok}, status_code=200 if ok else 503)

        @r.get("/metrics")
        async def metrics(format: str = "prometheus"):
            """Prometheus text by default; `?format=opentelemetry` (OTLP/JSON) or `?format=statsd` (lines)."""
            if self.metrics is None:
                raise HTTPException(404, "metrics are disabled")
            self._update_queue_metrics()
            if format == "prometheus":
                return PlainTextResponse(self.metrics.registry.to_prometheus(), media_type="text/plain; version=0.0.4")
            from telefuser_b200.metrics.exporters import get_exporter

            try:
                exporter = get_exporter(format)
            except ValueError as e:
                raise HTTPException(400, str(e)) from None
            return PlainTextResponse(exporter.export(self.metrics.registry), media_type=exporter.content_type)

        @r.get("/metrics/json")
        async def metrics_json() -> dict:
            if self.metrics is None:
                raise HTTPException(404, "metrics are disabled")
            self._update_queue_metrics()
            return self.metrics.registry.to_dict()

        return r

    # ---- /v1/files ----
    def _files_router(self) -> APIRouter:
        r = APIRouter(prefix="/v1/files", tags=["files"])

        @r.get("/download/{file_path:path}")
        async def download(file_path: str):
            try:
                p = self.file_service.resolve_inside(file_path, self.file_service.output_dir)
            except PermissionError as e:
                raise HTTPException(403, str(e)) from e
            if not p.is_file():
                raise HTTPException(404, "File not found")
            return FileResponse(str(p), filename=p.name)

        @r.get("/artifacts")
        async def artifacts(media_type: str | None = None, limit: int = 100) -> dict:
            return {"artifacts": [a.__dict__ for a in self.artifacts.list(media_type, limit)]}

        return r

    # ---- /v1/stream ----
    def _stream_router(self) -> APIRouter:
        r = APIRouter(prefix="/v1/stream", tags=["stream"])
        sessions = self.sessions

        def require():
            if self.stream_service is None or not self.stream_service.is_running:
                raise HTTPException(503, "Stream service is not running")
            return self.stream_service

        async def close_both(session_id: str, reason: str) -> bool:
            """A streaming session has two owners, the pipeline-side session and (over WebRTC) a peer connection: both
            are closed; either one being there counts as found, and a failure on one side does not keep the other open."""
            found = False
            mgr = getattr(self, "webrtc", None)
            if mgr is not None and session_id in mgr.connections:
                found = True
                try:
                    await mgr.close_connection(session_id)
                except Exception as e:  # noqa: BLE001 - the pipeline session is still closed below
                    logger.warning(f"closing the WebRTC connection of session {session_id} failed: {e}")
            try:
                found = await sessions.close(session_id, reason=reason) or found
            except Exception as e:  # noqa: BLE001
                logger.warning(f"closing the pipeline session {session_id} failed: {e}")
            return found

        @r.delete("/sessions/{session_id}")
        async def close_session(session_id: str) -> dict:
            require()
            if not await close_both(session_id, "stream_session_delete"):
                raise HTTPException(404, f"Session {session_id} not found")
            return {"session_id": session_id, "status": "closed"}

        @r.delete("/webrtc/{session_id}")
        async def close_webrtc(session_id: str) -> dict:
            require()
            if not await close_both(session_id, "webrtc_delete"):
                raise HTTPException(404, f"Session {session_id} not found")
            return {"session_id": session_id, "status": "closed"}

        @r.get("/sessions/{session_id}/status")
        async def session_status(session_id: str) -> dict:
            svc = require()
            s = sessions.sessions.get(session_id)
            if s is None:
                return {"session_id": session_id, "status": "unknown"}
            return {"session_id": session_id, "status": "active", "stream_mode": svc.stream_mode,
                    "chunks_sent": s.chunks_sent, "frames_dropped": s.frames_dropped}  # fmt: skip

        @r.post("/webrtc/offer")
        async def webrtc_offer(body: dict) -> dict:
            require()
            if not webrtc_available():
                raise HTTPException(501, "WebRTC transport needs the aiortc package; use the WebSocket transport /v1/stream/ws")
            from .stream_service import SessionConflict, SessionLimitReached
            from .webrtc import answer_offer

            try:
                return await answer_offer(self, body)
            except SessionLimitReached as e:
                raise HTTPException(503, str(e)) from None
            except SessionConflict as e:
                raise HTTPException(409, str(e)) from None
            except (KeyError, ValueError, TypeError) as e:  # no / malformed SDP, a config the service refuses
                raise HTTPException(400, f"offer rejected: {e}") from None

        @r.websocket("/ws")
        async def ws(websocket: WebSocket) -> None:
            """First client message: JSON session config. Server -> client: JSON chunk messages, each
            followed by `num_frames` binary JPEG messages and, when the message has an `audio` entry, one binary message of
            interleaved PCM16. Client -> server (bidirectional mode): JSON
            chunks (e.g. key controls); `{"type": "close"}` ends the session."""
            await websocket.accept()
            if self.stream_service is None or not self.stream_service.is_running:
                await websocket.close(code=1013, reason="stream service is not running")
                return
            try:
                config = json.loads(await websocket.receive_text())
                s = await sessions.open(config)
            except Exception as e:  # noqa: BLE001
                await websocket.send_text(json.dumps({"type": "error", "error": str(e)}))
                await websocket.close(code=1011)
                return
            await websocket.send_text(json.dumps({"type": "session", "session_id": s.session_id,
                                                  "stream_mode": self.stream_service.stream_mode}))  # fmt: skip

            async def sender() -> None:
                while True:
                    frames, msg = await s.outbound.get()
                    await websocket.send_text(json.dumps(msg))
                    for f in frames:  # video frames as JPEG; a chunk's audio (announced in msg["audio"]) last, as raw PCM16
                        if isinstance(f, AudioChunk):
                            await websocket.send_bytes(f.pcm16)
                        else:
                            await websocket.send_bytes(f if isinstance(f, (bytes, bytearray)) else frame_to_jpeg(f))
                    s.chunks_sent += 1
                    if msg.get("type") == "done" or msg.get("error"):
                        return

            async def receiver() -> None:
                while True:
                    raw = await websocket.receive_text()
                    msg = json.loads(raw)
                    if msg.get("type") == "close":
                        return
                    if self.stream_service.stream_mode == "bidirectional":
                        sessions.push(s.session_id, msg)

            tasks = [asyncio.create_task(sender()), asyncio.create_task(receiver())]
            try:
                done, pending = await asyncio.wait(tasks, return_when=asyncio.FIRST_COMPLETED)
                for t in pending:
                    t.cancel()
                await asyncio.gather(*tasks, return_exceptions=True)
            except WebSocketDisconnect:
                pass
            finally:
                await sessions.close(s.session_id, reason="websocket closed")
                try:
                    await websocket.close()
                except RuntimeError:
                    pass

        return r


def _coerce_form_value(v: str) -> Any:
    s = v.strip()
    if s.lower() in ("true", "false"):
        return s.lower() == "true"
    for cast in (int, float):
        try:
            return cast(s)
        except ValueError:
            continue
    return v


def b64_file(path: str) -> str:
    return base64.b64encode(Path(path).read_bytes()).decode()
