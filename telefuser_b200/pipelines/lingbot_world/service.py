"""Interactive LingBot-World session service: keyboard / pose control in, video chunks out.

Implements the bidirectional streaming-service interface (`start / stop / create_session / push_chunk /
pull_chunks / close_session`) on top of the pipeline's streaming runtime. Each session owns a worker thread
that, chunk by chunk, snapshots the held direction keys (or takes an explicit pose chunk pushed by the client),
integrates the camera pose over the chunk's latent frames, builds the control tensor, feeds the runtime while it
has input capacity and forwards decoded frames to a bounded output queue (oldest frame chunks are dropped when a
slow client falls behind; status and terminal messages are never dropped). An optional HUD draws the held keys
into the frames.
Role parity: telefuser/pipelines/lingbot_world_fast/service.py:71-1207.
"""

from __future__ import annotations

import asyncio
import base64
import io
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncGenerator

import numpy as np
import torch

from telefuser_b200.utils.logging import logger

from .control import KEY_MOVES, KEY_TURNS, integrate_keys

DIRECTION_KEYS = {"forward": "w", "backward": "s", "left": "a", "right": "d", "rise": "e", "descend": "q", "turn_left": "j", "turn_right": "l",
                  "look_up": "i", "look_down": "k"}  # fmt: skip
_VALID_KEYS = set(KEY_MOVES) | set(KEY_TURNS)
# what a browser or a game pad may call a control: DOM `KeyboardEvent.code` / `.key` names, arrows (movement), words
KEY_ALIASES = {**{k: k for k in _VALID_KEYS}, **{f"key{k}": k for k in _VALID_KEYS}, **DIRECTION_KEYS,
               "arrowup": "w", "arrowdown": "s", "arrowleft": "a", "arrowright": "d", "up": "w", "down": "s", "left": "a", "right": "d",
               "pageup": "e", "pagedown": "q", "space": "e"}  # fmt: skip
MAX_GENERATION_SECONDS = 20.0  # longest session a client may ask for unless the operator configures longer ones (bounds occupancy)


def canonical_key(name) -> str | None:
    """The movement / turn key a client-side name stands for (`ArrowUp`, `KeyW`, `forward`, `w` -> "w"), else None."""
    return KEY_ALIASES.get(str(name).strip().lower().replace("_", "")) or KEY_ALIASES.get(str(name).strip().lower())


@dataclass
class LingBotWorldFastSessionConfig:
    prompt: str = ""
    height: int = 480
    width: int = 832
    seed: int = 0
    fps: int = 16
    max_duration_seconds: float = 10.0
    move_step: float = 0.05
    turn_step_deg: float = 1.5
    hud: bool = False
    output_queue_size: int = 8
    benchmark_metrics: bool = False  # a "status" message with the runtime snapshot follows every chunk


@dataclass
class LingBotWorldFastSessionState:
    session_id: str
    config: LingBotWorldFastSessionConfig
    generation: Any
    stream: Any
    outputs: "queue.Queue[dict]"
    lock: threading.Lock = field(default_factory=threading.Lock)
    held_keys: set = field(default_factory=set)
    explicit_chunks: list = field(default_factory=list)
    pose: torch.Tensor = field(default_factory=lambda: torch.eye(4))
    stop_event: threading.Event = field(default_factory=threading.Event)
    worker: threading.Thread | None = None
    dropped_chunks: int = 0
    submitted: int = 0
    emitted: int = 0
    created_at: float = field(default_factory=time.time)
    finished: bool = False
    control_bound_at: dict = field(default_factory=dict)  # chunk index -> monotonic time its control was sampled
    control_latency_s: list = field(default_factory=list)  # control sampled -> frames emitted, per chunk
    # measurements a client or a load generator reads through status messages / `session_metrics`
    created_mono: float = field(default_factory=time.monotonic)
    worker_started_mono: float | None = None
    first_chunk_mono: float | None = None
    queue_high_watermark: int = 0
    controls_received: int = 0
    controls_superseded: int = 0  # key snapshots replaced by a newer one before any chunk sampled them
    explicit_overwritten: int = 0  # pose chunks dropped because a newer one arrived first (latest wins)
    control_revision_received: int = 0
    control_revision_applied: int = 0
    unsampled_snapshot: bool = False


def frame_num_for_duration(max_duration_seconds: float, fps: int, chunk_size: int) -> int:
    """Largest 4n+1 frame count within the duration whose latent frames are a whole number of chunks (at least one)."""
    latent = max(1, int(max_duration_seconds * fps) // 4 + 1)
    latent = max(chunk_size, latent // chunk_size * chunk_size)
    return (latent - 1) * 4 + 1


def load_image(config: dict):
    """`image` (PIL / array / tensor), `image_path`, or `image_data_url` (data:image/...;base64,...) -> PIL image or tensor."""
    from PIL import Image

    if config.get("image") is not None:
        return config["image"]
    if config.get("image_path"):
        return Image.open(config["image_path"]).convert("RGB")
    url = config.get("image_data_url")
    if url:
        if not url.startswith("data:image/") or ";base64," not in url:
            raise ValueError("image_data_url must be a base64 data URL of an image")
        return Image.open(io.BytesIO(base64.b64decode(url.split(";base64,", 1)[1]))).convert("RGB")
    raise ValueError("a session needs an image, image_path or image_data_url")


def keys_from_chunk(chunk: dict) -> set | None:
    """Held-key snapshot carried by a control message, or None when the message is not a snapshot."""
    if "keys" in chunk:
        names = chunk["keys"]
    elif "directions" in chunk:
        names = chunk["directions"]
    elif isinstance(chunk.get("controls"), (list, tuple, set)):
        # the browser's canonical keyboard state, `{"type": "control_state", "controls": ["w", "j"]}`: taken whole or not
        # at all, so that a client with names this service does not know cannot half-steer the camera
        names = list(chunk["controls"])
        if not all(isinstance(n, str) and canonical_key(n) is not None for n in names):
            logger.warning(f"control state {names!r} holds names that are not controls; ignored")
            return None
    else:
        return None
    return {k for k in map(canonical_key, names) if k is not None}


def overlay_control_hud(frames: np.ndarray, keys) -> np.ndarray:
    """Draws one small square per movement key in the lower-left corner (filled when held). frames: [T, H, W, 3] uint8."""
    out = frames.copy()
    _, h, w, _ = out.shape
    cell = max(4, min(h, w) // 24)
    layout = {"w": (1, 0), "a": (0, 1), "s": (1, 1), "d": (2, 1), "j": (4, 1), "l": (6, 1), "i": (5, 0), "k": (5, 1), "q": (0, 0), "e": (2, 0)}
    keys = set(keys or ())
    for key, (cx, cy) in layout.items():
        x0, y0 = cell + cx * (cell + 2), h - 3 * cell - 2 + cy * (cell + 2)
        if x0 + cell > w or y0 + cell > h or y0 < 0:
            continue
        out[:, y0 : y0 + cell, x0 : x0 + cell] = (255, 255, 255) if key in keys else (40, 40, 40)
    return out


class LingBotWorldFastService:
    def __init__(self, pipeline, default_config: LingBotWorldFastSessionConfig | None = None, warmup: bool = False,
                 max_generation_seconds: float | None = None) -> None:  # fmt: skip
        self.pipeline, self.default_config, self._warmup = pipeline, default_config or LingBotWorldFastSessionConfig(), warmup
        # what a client may ask for: the operator's limit, else the larger of 20 s and the session length the operator
        # configured as the default (a service set up for two-minute sessions serves two-minute sessions)
        self.max_generation_seconds = (float(max_generation_seconds) if max_generation_seconds is not None
                                       else max(MAX_GENERATION_SECONDS, float(self.default_config.max_duration_seconds)))  # fmt: skip
        self._sessions: dict[str, LingBotWorldFastSessionState] = {}
        self._lock = threading.Lock()
        self._started = False

    # ---- lifecycle ------------------------------------------------------------------------------
    def start(self) -> None:
        if self._started:
            return
        if self._warmup:
            self.pipeline.warmup(self.default_config.height, self.default_config.width)
        self._started = True

    def stop(self) -> None:
        for sid in list(self._sessions):
            self.close_session(sid, timeout=10.0)
        self._started = False

    def has_session(self, session_id: str) -> bool:
        return session_id in self._sessions

    def _state(self, session_id: str) -> LingBotWorldFastSessionState:
        state = self._sessions.get(session_id)
        if state is None:
            raise KeyError(f"unknown session {session_id!r}")
        return state

    def create_session(self, config: dict) -> str:
        known = LingBotWorldFastSessionConfig.__dataclass_fields__
        cfg = LingBotWorldFastSessionConfig(**{**self.default_config.__dict__, **{k: v for k, v in config.items() if k in known}})
        for name in ("fps", "max_duration_seconds", "move_step", "turn_step_deg"):
            if not float(getattr(cfg, name)) > 0:
                raise ValueError(f"{name} must be positive")
        chunk_size = self.pipeline.config.chunk_size
        frames = frame_num_for_duration(cfg.max_duration_seconds, cfg.fps, chunk_size)
        if (frames - 1) / cfg.fps > self.max_generation_seconds:  # judged on what would be generated, after rounding to chunks
            raise ValueError(f"a session may generate at most {self.max_generation_seconds:g} s of video; "
                             f"{cfg.max_duration_seconds:g} s at {cfg.fps} fps was asked for")  # fmt: skip
        image = load_image(config)
        if config.get("fit_image"):  # output size from the reference image's aspect ratio at the pipeline's pixel budget
            w, h = self.pipeline.best_output_size(*self.pipeline._image_size(image), self.pipeline.config.max_area)
            cfg.height, cfg.width = self.pipeline.check_resize_height_width(h, w)
        generation = self.pipeline._create_initialized_session(cfg.prompt, image, frames, cfg.height, cfg.width, cfg.seed,
                                                               prompt_emb=config.get("prompt_emb"),
                                                               world_cache=config.get("world_cache", True))  # fmt: skip
        if config.get("intrinsics") is not None:  # the client's calibration (fx, fy, cx, cy) and the image size it refers to
            import dataclasses

            ks = torch.as_tensor(config["intrinsics"], dtype=torch.float32).reshape(-1, 4)[0]
            ctx = generation.control_builder.context
            generation.control_builder.context = dataclasses.replace(
                ctx, intrinsics=ks.to(ctx.intrinsics.device), orig_width=int(config.get("intrinsics_width") or ctx.orig_width),
                orig_height=int(config.get("intrinsics_height") or ctx.orig_height))  # fmt: skip
        stream = self.pipeline.runtime.create_session(generation)
        sid = config.get("session_id") or uuid.uuid4().hex
        state = LingBotWorldFastSessionState(sid, cfg, generation, stream, queue.Queue())
        state.explicit_chunks = list(config.get("controls", []))  # pose chunks known up front, used before any key snapshot
        with self._lock:
            if sid in self._sessions:
                raise ValueError(f"session {sid!r} already exists")
            self._sessions[sid] = state
        self._enqueue(state, {"type": "status", "stage": "created", "session_id": sid, "frames": frames, "chunks": generation.chunk_count,
                              "chunk_size": chunk_size, "height": cfg.height, "width": cfg.width, "fps": cfg.fps})  # fmt: skip
        if config.get("preview", False):
            self._emit_preview(state, image)
        state.worker = threading.Thread(target=self._worker_loop, args=(state,), name=f"lingbot-session-{sid[:8]}", daemon=True)
        state.worker.start()
        return sid

    def _emit_preview(self, state: LingBotWorldFastSessionState, image) -> None:
        """The reference image at the session's output size (with the idle HUD when enabled), so a client has a picture
        on screen while the first chunk is still being generated."""
        h, w = state.config.height, state.config.width
        if isinstance(image, torch.Tensor):
            t = image.detach().float().cpu().reshape(1, *image.shape[-3:])
            if tuple(t.shape[-2:]) != (h, w):
                t = torch.nn.functional.interpolate(t, size=(h, w), mode="bilinear", antialias=True, align_corners=False)
            arr = ((t[0].clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8).permute(1, 2, 0).numpy()[None]
        else:
            from PIL import Image

            pil = image if isinstance(image, Image.Image) else Image.fromarray(np.asarray(image))
            arr = np.asarray(pil.convert("RGB").resize((w, h), Image.BICUBIC))[None]
        if state.config.hud:
            arr = overlay_control_hud(arr, None)
        self._enqueue(state, {"type": "preview", "session_id": state.session_id, "chunk_index": -1, "frames": arr, "fps": state.config.fps})

    # ---- client -> service ---------------------------------------------------------------------
    def push_chunk(self, session_id: str, chunk: dict) -> None:
        """One client message. Key events edit the held-key set; a key snapshot or a direction replaces it; a pose /
        control-tensor chunk steers the next chunk directly. Only the newest pending control of each kind is kept
        (an interactive session wants the latest intent, not a backlog). A message that carries `revision` is
        acknowledged with a `control_ack`, and the revision of the control that a chunk finally used is reported with
        that chunk, so a client can measure both the acknowledgement and the control-to-picture latency.

        Keys may be named as a browser names them (`ArrowUp`, `KeyW`), by letter or by word (`forward`, `turn_left`).
        Event form: `{"key" | "control" | "direction": name, "event": "press" | "release"}` edits the held set like
        `key_down` / `key_up`; `{"type": "reset"}` (or `"event": "reset"`) drops held keys and pending controls,
        `reset_pose` also returns the camera to the origin. Event and reset messages are answered with a `status`
        message of stage `control_state` listing the keys now held."""
        state = self._state(session_id)
        kind = chunk.get("type", "control")
        ack, report_state = None, False
        with state.lock:
            if kind == "stop":
                state.stop_event.set()
            else:
                state.controls_received += 1
                if isinstance(chunk.get("revision"), int):
                    state.control_revision_received = max(state.control_revision_received, chunk["revision"])
                    ack = chunk["revision"]
                named = canonical_key(chunk.get("key") or chunk.get("control") or chunk.get("direction") or "")
                event = str(chunk["event"]).lower() if "event" in chunk else None
                if kind in ("reset", "reset_pose") or event in ("reset", "reset_pose"):
                    # drop every pending intent; `reset_pose` also puts the camera back at the origin
                    state.held_keys = set()
                    state.explicit_chunks.clear()
                    state.unsampled_snapshot = False
                    if "reset_pose" in (kind, event):
                        state.pose = torch.eye(4)
                    report_state = True
                elif kind == "key_down" or event == "press":
                    if named is not None:
                        state.held_keys.add(named)
                    report_state = event is not None
                elif kind == "key_up" or event in ("release", "keyup", "end"):
                    state.held_keys.discard(named)
                    report_state = event is not None
                elif event is not None:
                    logger.warning(f"LingBot session {session_id}: control event {event!r} is not one of press / release / reset / reset_pose")
                elif "poses" in chunk or "control_tensor" in chunk:
                    if state.explicit_chunks and not chunk.get("queue", False):
                        state.explicit_overwritten += len(state.explicit_chunks)
                        state.explicit_chunks.clear()
                    state.explicit_chunks.append(chunk)  # used for the next chunk instead of the key snapshot
                else:
                    keys = keys_from_chunk(chunk)
                    if keys is None and canonical_key(chunk.get("direction", "")) is not None:
                        keys = {canonical_key(chunk["direction"])}
                    if keys is not None:
                        if state.unsampled_snapshot:
                            state.controls_superseded += 1
                        state.held_keys, state.unsampled_snapshot = keys, True
                        report_state = kind == "control_state"
        if ack is not None:
            self._enqueue(state, {"type": "control_ack", "session_id": session_id, "revision": ack,
                                  "elapsed_s": time.monotonic() - state.created_mono})  # fmt: skip
        if report_state:
            self._enqueue(state, {"type": "status", "stage": "control_state", "session_id": session_id,
                                  "controls": sorted(state.held_keys), "revision": state.control_revision_received})  # fmt: skip

    # ---- measurements ---------------------------------------------------------------------------
    def session_metrics(self, session_id: str) -> dict:
        """Runtime snapshot of one session (also sent as `status` messages when `benchmark_metrics` is on)."""
        return self._snapshot(self._state(session_id))

    @staticmethod
    def _snapshot(state: LingBotWorldFastSessionState) -> dict:
        now = time.monotonic()
        with state.lock:
            lat = sorted(state.control_latency_s)
            out = {"session_age_s": round(now - state.created_mono, 6), "chunks_submitted": state.submitted,
                   "chunks_emitted": state.emitted, "dropped_chunks": state.dropped_chunks,
                   "output_queue_depth": state.outputs.qsize(), "output_queue_high_watermark": state.queue_high_watermark,
                   "controls_received": state.controls_received, "controls_superseded": state.controls_superseded,
                   "explicit_controls_overwritten": state.explicit_overwritten, "explicit_controls_pending": len(state.explicit_chunks),
                   "control_revision_received": state.control_revision_received,
                   "control_revision_applied": state.control_revision_applied}  # fmt: skip
            if state.worker_started_mono is not None:
                out["worker_start_s"] = round(state.worker_started_mono - state.created_mono, 6)
            if state.first_chunk_mono is not None:
                out["first_chunk_s"] = round(state.first_chunk_mono - state.created_mono, 6)
            if lat:
                out["control_to_output_p50_s"] = round(lat[len(lat) // 2], 6)
                out["control_to_output_max_s"] = round(lat[-1], 6)
        return out

    @staticmethod
    def _progress(state: LingBotWorldFastSessionState) -> dict:
        """How far the session is: frames and seconds of video generated out of the requested total."""
        g, fps = state.generation, state.config.fps
        total_frames = (g.chunk_count * g.chunk_size - 1) * 4 + 1
        done_latent = state.emitted * g.chunk_size
        done_frames = 0 if state.emitted == 0 else min(total_frames, (done_latent - 1) * 4 + 1)
        return {"total_chunks": g.chunk_count, "completed_chunks": state.emitted, "target_frames": total_frames,
                "generated_frames": done_frames, "fps": fps, "target_duration_s": round((total_frames - 1) / fps, 3),
                "generated_duration_s": round(max(done_frames - 1, 0) / fps, 3)}  # fmt: skip

    # ---- service -> client ---------------------------------------------------------------------
    @staticmethod
    def _enqueue(state: LingBotWorldFastSessionState, payload: dict) -> None:
        """Frame chunks beyond the queue bound push out the oldest queued frame chunk; other messages always fit."""
        q = state.outputs
        if payload.get("type") == "frames":
            with state.lock:
                queued = [p for p in list(q.queue) if p.get("type") == "frames"]
                if len(queued) >= state.config.output_queue_size:
                    with q.mutex:
                        for i, p in enumerate(q.queue):
                            if p.get("type") == "frames":
                                del q.queue[i]
                                state.dropped_chunks += 1
                                break
        q.put(payload)
        depth = q.qsize()
        if depth > state.queue_high_watermark:
            state.queue_high_watermark = depth

    async def pull_chunks(self, session_id: str) -> AsyncGenerator[dict, None]:
        state = self._state(session_id)
        loop = asyncio.get_running_loop()
        while True:
            try:
                item = state.outputs.get_nowait()
            except queue.Empty:
                if state.finished and state.outputs.empty():
                    return
                await asyncio.sleep(0.005) if loop else None
                continue
            yield item
            if item.get("type") in ("done", "error"):
                return

    def drain(self, session_id: str, timeout: float = 60.0) -> list:
        """Blocking variant of `pull_chunks` for synchronous callers: every message up to the terminal one."""
        state, out, deadline = self._state(session_id), [], time.time() + timeout
        while time.time() < deadline:
            try:
                item = state.outputs.get(timeout=0.05)
            except queue.Empty:
                if state.finished:
                    break
                continue
            out.append(item)
            if item.get("type") in ("done", "error"):
                break
        return out

    # ---- per-session worker -------------------------------------------------------------------
    def _next_control(self, state: LingBotWorldFastSessionState, chunk_index: int):
        """(control tensor, key list) for chunk `chunk_index`: an explicit pose chunk if one is pending, else the held keys."""
        builder, cs = state.generation.control_builder, state.generation.chunk_size
        with state.lock:
            explicit = state.explicit_chunks.pop(0) if state.explicit_chunks else None
            keys = sorted(state.held_keys)
            state.unsampled_snapshot = False
            state.control_revision_applied = state.control_revision_received
        if explicit is not None:
            if "poses" in explicit:
                state.pose = torch.as_tensor(np.asarray(explicit["poses"]), dtype=torch.float32)[-1].cpu()
            return builder.build(explicit), None
        steps = (cs - 1 if chunk_index == 0 else cs) * 4
        path = integrate_keys(state.pose, keys, steps, state.config.move_step, state.config.turn_step_deg) if steps else torch.zeros(0, 4, 4)
        latent = path[3::4]
        poses = torch.cat([state.pose[None], latent]) if chunk_index == 0 else latent
        if len(path):
            state.pose = path[-1]
        return builder.build({"poses": poses, "relative": True}), keys

    def _worker_loop(self, state: LingBotWorldFastSessionState) -> None:
        runtime, stream, total = self.pipeline.runtime, state.stream, state.generation.chunk_count
        pending: dict[int, list | None] = {}
        cancelled = False
        try:
            state.worker_started_mono = time.monotonic()
            self._enqueue(state, {"type": "status", "stage": "running", "session_id": state.session_id})
            while state.emitted < total:
                if state.stop_event.is_set():
                    cancelled = True
                    break
                progressed = False
                if state.submitted < total and runtime.can_submit_chunk(stream):
                    idx = state.submitted

                    def bind_control(idx=idx):
                        # Latest-wins: called when the denoiser admits the chunk, not when the slot was reserved, so
                        # the keys held at that moment steer the chunk (one chunk period closer to its output).
                        control, keys = self._next_control(state, idx)
                        pending[idx] = keys
                        state.control_bound_at[idx] = time.monotonic()
                        return control

                    if runtime.try_submit_chunk(stream, idx, bind_control):
                        state.submitted += 1
                        progressed = True
                for idx, frames in runtime.poll_frames(stream):
                    self._emit_frames(state, idx, frames, pending.pop(idx, None))
                    progressed = True
                err = runtime.error(stream)
                if err is not None:
                    raise RuntimeError(f"streaming runtime failed: {err}")
                if not progressed:
                    time.sleep(0.001)
            metrics = {}
            try:
                metrics = runtime.metrics(stream)
                lat = sorted(state.control_latency_s)
                if lat:
                    metrics["control_bound_to_output_p50_s"] = lat[len(lat) // 2]
                    metrics["control_bound_to_output_max_s"] = lat[-1]
                metrics["session"] = self._snapshot(state)
            except Exception:  # noqa: BLE001 - metrics are best effort
                pass
            self._enqueue(state, {"type": "done", "session_id": state.session_id, "cancelled": cancelled, "chunks": state.emitted,
                                  "dropped_chunks": state.dropped_chunks, "metrics": metrics})  # fmt: skip
        except Exception as exc:  # noqa: BLE001 - reported to the client, then the session ends
            logger.error(f"LingBot session {state.session_id} failed: {exc}")
            cancelled = True
            self._enqueue(state, {"type": "error", "session_id": state.session_id, "message": str(exc)})
        finally:
            try:
                self.pipeline.release_session(stream, cancel=cancelled or state.emitted < total)
            except Exception as exc:  # noqa: BLE001
                logger.warning(f"release of LingBot session {state.session_id} failed: {exc}")
            state.finished = True

    def _emit_frames(self, state: LingBotWorldFastSessionState, idx: int, frames: torch.Tensor, keys) -> None:
        """frames: [B, 3, T, H, W] in [-1, 1] -> uint8 [T, H, W, 3] with the HUD drawn in when enabled."""
        from telefuser_b200.ops.functional import frames_to_uint8

        arr = frames_to_uint8(frames[0] if frames.dim() == 5 else frames)
        arr = arr.cpu().numpy() if isinstance(arr, torch.Tensor) else np.asarray(arr)
        if state.config.hud:
            arr = overlay_control_hud(arr, keys)
        state.emitted += 1
        if state.first_chunk_mono is None:
            state.first_chunk_mono = time.monotonic()
        bound = state.control_bound_at.pop(idx, None)
        latency = None if bound is None else time.monotonic() - bound
        if latency is not None:
            state.control_latency_s.append(latency)
        self._enqueue(state, {"type": "frames", "session_id": state.session_id, "chunk_index": idx, "frames": arr, "controls": keys,
                              "fps": state.config.fps, "elapsed_s": time.time() - state.created_at,
                              "control_to_output_s": latency, "control_revision": state.control_revision_applied,
                              "progress": self._progress(state)})  # fmt: skip
        if state.config.benchmark_metrics:
            self._enqueue(state, {"type": "status", "stage": "chunk", "session_id": state.session_id, "chunk_index": idx,
                                  "metrics": self._snapshot(state)})  # fmt: skip

    def close_session(self, session_id: str, timeout: float | None = None) -> None:
        state = self._sessions.get(session_id)
        if state is None:
            return
        state.stop_event.set()
        if state.worker is not None and state.worker is not threading.current_thread():
            state.worker.join(timeout if timeout is not None else 30.0)
        with self._lock:
            self._sessions.pop(session_id, None)
