"""Streaming service: loads a pipeline file that exposes `get_service(gpu_num=...)` and bridges it to
network sessions.

Two service protocols (structural; detected from the methods the object has):
* server push:   `start() / stop() / serve(request) -> async generator of chunk dicts`
* bidirectional: `start() / stop() / create_session(config) -> id / push_chunk(id, chunk) /
                  pull_chunks(id) -> async generator / close_session(id)`
`StreamSessionManager` owns the per-connection state independent of the transport (WebSocket here;
WebRTC signalling is available only when `aiortc` is importable): a pull task that drains the
pipeline into an outbound queue with frame dropping under backpressure, idle / disconnect grace
timers and ordered tear-down. `ChunkRouter` splits pipeline chunks into media frames (for a video
track or binary WebSocket messages) and JSON side-channel messages.
Role parity: telefuser/service/core/stream_pipeline_service.py:64-332, webrtc/session_manager.py,
webrtc/chunk_router.py, api/stream_schema.py.
"""

from __future__ import annotations

import asyncio
import inspect
import json
import time
import uuid
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, AsyncGenerator, Protocol, runtime_checkable

import numpy as np
import torch

from telefuser_b200.utils.logging import logger

from .pipeline_service import ServerConfig, load_pipeline_module
from .security import PipelineSecurityValidator


@runtime_checkable
class ServerPushService(Protocol):
    def start(self) -> None: ...
    def stop(self) -> None: ...
    def serve(self, request: dict) -> AsyncGenerator[dict, None]: ...


@runtime_checkable
class BidirectionalService(Protocol):
    def start(self) -> None: ...
    def stop(self) -> None: ...
    def create_session(self, config: dict) -> str: ...
    def push_chunk(self, session_id: str, chunk: dict) -> None: ...
    def pull_chunks(self, session_id: str) -> AsyncGenerator[dict, None]: ...
    def close_session(self, session_id: str) -> None: ...


def serialisable_chunk(chunk: dict) -> dict:
    """JSON-safe view of a chunk: tensors and arrays are replaced by their shapes."""
    out = {}
    for k, v in chunk.items():
        if isinstance(v, (str, int, float, bool, type(None))):
            out[k] = v
        elif isinstance(v, torch.Tensor):
            out[k] = {"tensor": list(v.shape), "dtype": str(v.dtype)}
        elif hasattr(v, "shape") and hasattr(v, "dtype"):
            out[k] = {"array": list(v.shape), "dtype": str(v.dtype)}
        else:
            try:
                json.dumps(v)
                out[k] = v
            except (TypeError, ValueError):
                out[k] = str(v)
    return out


class StreamPipelineService:
    def __init__(self, config: ServerConfig | None = None) -> None:
        self.config = config or ServerConfig()
        self.validator = PipelineSecurityValidator(self.config.security_level)
        self.service: Any = None
        self.stream_mode = "unknown"
        self.module = None
        self.is_running = False
        self._sessions: set[str] = set()

    @staticmethod
    def detect_mode(service: Any) -> str:
        if all(callable(getattr(service, m, None)) for m in ("create_session", "push_chunk", "pull_chunks", "close_session")):
            return "bidirectional"
        if callable(getattr(service, "serve", None)):
            return "server_push"
        raise TypeError("get_service() returned an object that implements neither streaming protocol")

    def start_service(self, ppl_file: str, skip_validation: bool = False, gpu_num: int = 1) -> bool:
        self.module = load_pipeline_module(ppl_file, None if skip_validation else self.validator)
        get = getattr(self.module, "get_service", None)
        if not callable(get):
            raise AttributeError(f"{Path(ppl_file).name} does not define get_service(gpu_num=...)")
        kw = {"gpu_num": gpu_num} if "gpu_num" in inspect.signature(get).parameters else {}
        self.service = get(**kw)
        self.stream_mode = self.detect_mode(self.service)
        self.service.start()
        self.is_running = True
        logger.info(f"stream service started in {self.stream_mode} mode")
        return True

    async def aclose(self) -> None:
        if not self.is_running:
            return
        for sid in list(self._sessions):
            try:
                self.close_session(sid)
            except Exception:  # noqa: BLE001
                pass
        self.is_running = False
        await asyncio.to_thread(self.service.stop)

    def _ensure_running(self) -> None:
        if not self.is_running:
            raise RuntimeError("stream service is not running")

    # ---- server push ----
    async def stream_task(self, task_data: dict) -> AsyncGenerator[dict, None]:
        self._ensure_running()
        if self.stream_mode != "server_push":
            raise RuntimeError("stream_task needs a server-push service")
        gen = self.service.serve(task_data)
        if inspect.isasyncgen(gen):
            async for chunk in gen:
                yield chunk
            return
        # plain generator: iterate in a thread so the event loop stays responsive
        it = iter(gen)
        sentinel = object()
        while True:
            chunk = await asyncio.to_thread(next, it, sentinel)
            if chunk is sentinel:
                return
            yield chunk

    # ---- bidirectional ----
    def _bidi(self):
        self._ensure_running()
        if self.stream_mode != "bidirectional":
            raise RuntimeError("this operation needs a bidirectional service")
        return self.service

    def create_session(self, config: dict) -> str:
        sid = self._bidi().create_session(config)
        self._sessions.add(sid)
        return sid

    def push_chunk(self, session_id: str, chunk: dict) -> None:
        self._bidi().push_chunk(session_id, chunk)

    async def pull_chunks(self, session_id: str) -> AsyncGenerator[dict, None]:
        async for c in self._bidi().pull_chunks(session_id):
            yield c

    def close_session(self, session_id: str) -> None:
        self._sessions.discard(session_id)
        self._bidi().close_session(session_id)

    def has_session(self, session_id: str) -> bool:
        return session_id in self._sessions

    def server_metadata(self) -> dict:
        meta = {"stream_mode": self.stream_mode, "running": self.is_running, "sessions": len(self._sessions)}
        fn = getattr(self.service, "metadata", None)
        if callable(fn):
            meta.update(fn())
        return meta


# ---------------------------------------------------------------------------
# Transport-independent session plumbing
# ---------------------------------------------------------------------------
@dataclass
class AudioChunk:
    """Interleaved signed 16-bit PCM that belongs to one chunk. It rides at the end of the chunk's media list: the
    WebSocket transport sends it as one more binary message, the WebRTC transport feeds its audio track."""

    pcm16: bytes
    sample_rate: int = 48000
    channels: int = 1

    @property
    def num_samples(self) -> int:
        return len(self.pcm16) // (2 * max(1, self.channels))


def audio_from_chunk(chunk: dict) -> AudioChunk | None:
    """`audio_b64` (base64 PCM16, the wire form) or `audio` (int16 array, or float array / tensor in [-1, 1], shaped
    [samples] or [samples, channels]) with `audio_sample_rate` (48000) and `audio_channels` (1)."""
    rate, channels = int(chunk.get("audio_sample_rate") or 48000), int(chunk.get("audio_channels") or 1)
    if chunk.get("audio_b64"):
        import base64

        return AudioChunk(base64.b64decode(chunk["audio_b64"]), rate, channels)
    a = chunk.get("audio")
    if a is None or isinstance(a, (bool, int, float, str, dict)):  # a flag or a description under that name is ordinary data
        return None
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    a = np.asarray(a)
    if a.ndim not in (1, 2) or a.size == 0:
        return None
    if a.ndim == 2 and "audio_channels" not in chunk:
        channels = a.shape[1]
    if a.dtype != np.int16:
        a = (np.clip(a.astype(np.float32), -1.0, 1.0) * 32767.0).round().astype(np.int16)
    return AudioChunk(np.ascontiguousarray(a).tobytes(), rate, channels)


class ChunkRouter:
    """Splits a pipeline chunk into media (video frames, then at most one `AudioChunk`) and a JSON message."""

    FRAME_KEYS = ("frames", "video", "frame")
    AUDIO_KEYS = ("audio", "audio_b64")

    def __init__(self, fps: int = 16) -> None:
        self.fps = fps

    def route(self, chunk: dict, session_id: str, index: int) -> tuple[list, dict]:
        frames: list = []
        media_keys: set = set()
        if chunk.get("frames_b64"):  # base64 JPEG strings: what server-push services written for HTTP clients produce
            import base64

            frames.extend(base64.b64decode(f) for f in chunk["frames_b64"])
            media_keys.add("frames_b64")
        for k in self.FRAME_KEYS:
            v = chunk.get(k)
            if v is None:
                continue
            if isinstance(v, torch.Tensor):
                v = v.detach()
                if v.dim() == 3:
                    v = v[None]
                frames.extend(v.unbind(0))
                media_keys.add(k)
            elif isinstance(v, np.ndarray) and v.ndim in (3, 4):
                frames.extend(list(v) if v.ndim == 4 else [v])
                media_keys.add(k)
            elif isinstance(v, (list, tuple)):
                frames.extend(v)
                media_keys.add(k)
            elif isinstance(v, (bytes, bytearray)) or hasattr(v, "save"):  # an encoded image or a PIL image
                frames.append(v)
                media_keys.add(k)
            # anything else under these names (a frame count, a flag) is ordinary data and stays in the message
        audio = audio_from_chunk(chunk)
        if audio is not None:
            media_keys.update(self.AUDIO_KEYS)
        msg = {"type": "chunk", "session_id": session_id, "index": index, "num_frames": len(frames),
               "data": serialisable_chunk({k: v for k, v in chunk.items() if k not in media_keys}),
               "timestamp": time.time()}  # fmt: skip
        if audio is not None:
            msg["audio"] = {"sample_rate": audio.sample_rate, "channels": audio.channels, "num_samples": audio.num_samples,
                            "format": "pcm_s16le"}  # fmt: skip
            frames.append(audio)
        if chunk.get("error"):
            msg["error"] = str(chunk["error"])
        return frames, msg


def frame_to_jpeg(frame, quality: int = 85) -> bytes:
    """uint8 HWC (or float in [-1, 1] / [0, 1] CHW) frame -> JPEG bytes."""
    import io

    import numpy as np
    from PIL import Image

    if isinstance(frame, torch.Tensor):
        t = frame.detach().float().cpu()
        if t.dim() == 3 and t.shape[0] in (1, 3) and t.shape[-1] not in (1, 3):
            t = t.permute(1, 2, 0)
        if frame.dtype != torch.uint8:
            t = ((t + 1) * 127.5 if t.min() < 0 else t * 255.0).clamp(0, 255)
        frame = t.to(torch.uint8).numpy()
    arr = np.asarray(frame)
    if arr.ndim == 3 and arr.shape[2] == 1:
        arr = arr[..., 0]
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="JPEG", quality=quality)
    return buf.getvalue()


@dataclass
class StreamSession:
    session_id: str
    outbound: asyncio.Queue
    created: float = field(default_factory=time.time)
    last_active: float = field(default_factory=time.time)
    pull_task: asyncio.Task | None = None
    chunks_sent: int = 0
    frames_dropped: int = 0
    closed: bool = False
    disconnect_deadline: float | None = None


class SessionLimitReached(RuntimeError):
    """The server already runs as many streaming sessions as it is configured for."""


class SessionConflict(ValueError):
    """A session with the requested id exists."""


class StreamSessionManager:
    def __init__(self, service: StreamPipelineService, fps: int = 16, max_queue: int = 64, disconnect_grace_s: float = 10.0,
                 idle_timeout_s: float = 600.0, max_sessions: int = 0) -> None:  # fmt: skip
        self.max_sessions = max_sessions
        self.service, self.router = service, ChunkRouter(fps)
        self.max_queue, self.grace, self.idle = max_queue, disconnect_grace_s, idle_timeout_s
        self.sessions: dict[str, StreamSession] = {}

    def has_session(self, sid: str) -> bool:
        return sid in self.sessions

    async def open(self, config: dict) -> StreamSession:
        """Creates the pipeline session (bidirectional) or starts the generator (server push)."""
        if self.max_sessions and len(self.sessions) >= self.max_sessions:
            raise SessionLimitReached(f"{len(self.sessions)} streaming sessions are open (limit {self.max_sessions})")
        wanted = config.get("session_id")
        if wanted is not None and str(wanted) in self.sessions:
            raise SessionConflict(f"streaming session {wanted!r} already exists")
        if self.service.stream_mode == "bidirectional":
            try:
                sid = await asyncio.to_thread(self.service.create_session, config)
            except ValueError as e:
                if "already exists" in str(e):
                    raise SessionConflict(str(e)) from e
                raise
            source = self.service.pull_chunks(sid)
        else:
            sid = str(config.get("session_id") or uuid.uuid4())
            source = self.service.stream_task(config)
        s = StreamSession(sid, asyncio.Queue(maxsize=self.max_queue))
        self.sessions[sid] = s
        s.pull_task = asyncio.create_task(self._pull(s, source))
        return s

    async def _pull(self, s: StreamSession, source) -> None:
        idx = 0
        try:
            async for chunk in source:
                frames, msg = self.router.route(chunk, s.session_id, idx)
                idx += 1
                item = (frames, msg)
                if s.outbound.full():  # backpressure: drop the oldest media item, never the newest
                    try:
                        old = s.outbound.get_nowait()
                        s.frames_dropped += len(old[0])
                    except asyncio.QueueEmpty:
                        pass
                await s.outbound.put(item)
                if chunk.get("done") or chunk.get("error"):
                    break
            await s.outbound.put(([], {"type": "done", "session_id": s.session_id, "total_chunks": idx,
                                       "timestamp": time.time()}))  # fmt: skip
        except asyncio.CancelledError:
            raise
        except Exception as e:  # noqa: BLE001
            logger.exception(f"stream session {s.session_id} failed")
            await s.outbound.put(([], {"type": "chunk", "session_id": s.session_id, "index": idx, "error": str(e),
                                       "timestamp": time.time()}))  # fmt: skip

    def push(self, sid: str, chunk: dict) -> None:
        s = self.sessions.get(sid)
        if s is None or s.closed:
            raise KeyError(sid)
        s.last_active = time.time()
        self.service.push_chunk(sid, chunk)

    def mark_disconnected(self, sid: str) -> None:
        s = self.sessions.get(sid)
        if s is not None:
            s.disconnect_deadline = time.time() + self.grace

    def mark_reconnected(self, sid: str) -> bool:
        s = self.sessions.get(sid)
        if s is None or s.closed:
            return False
        s.disconnect_deadline = None
        return True

    async def reap(self, now: float | None = None) -> list[str]:
        """Closes sessions whose disconnect grace or idle time ran out."""
        now = time.time() if now is None else now
        dead = [sid for sid, s in self.sessions.items()
                if (s.disconnect_deadline is not None and now > s.disconnect_deadline) or now - s.last_active > self.idle]  # fmt: skip
        for sid in dead:
            await self.close(sid, reason="reaped")
        return dead

    async def close(self, sid: str, reason: str = "", notify_pipeline: bool = True) -> bool:
        s = self.sessions.pop(sid, None)
        if s is None:
            return False
        s.closed = True
        if s.pull_task is not None:
            s.pull_task.cancel()
            await asyncio.gather(s.pull_task, return_exceptions=True)
        if notify_pipeline and self.service.stream_mode == "bidirectional" and self.service.has_session(sid):
            try:
                await asyncio.to_thread(self.service.close_session, sid)
            except Exception as e:  # noqa: BLE001
                logger.warning(f"closing pipeline session {sid} failed: {e}")
        logger.info(f"stream session {sid} closed ({reason})")
        return True

    async def close_all(self) -> None:
        for sid in list(self.sessions):
            await self.close(sid, reason="shutdown")


def webrtc_available() -> bool:
    try:
        import aiortc  # noqa: F401

        return True
    except ImportError:
        return False
