"""Per-connection state of the WebRTC transport.

One `WebRTCSessionManager` lives in the API server. For every SDP offer it opens a streaming session
(`StreamSessionManager.open`), builds a peer connection with one paced video track (plus a paced audio track when the
offer's config asks for `audio`) and answers the offer. A pump
task moves the session's outbound items to the track (frames) and to the "control" data channel (JSON chunk
messages); client messages on that channel are forwarded to the pipeline (bidirectional services) or close the
session. Connection-state changes map onto the session manager's disconnect grace / reconnect / close.

Video settings: the preferred codec (H264 by default: hardware decoders everywhere, better at the bitrates a
720p interactive stream needs) is moved to the front of the transceiver's codec list, and aiortc's encoder
bitrate defaults (1 - 3 Mbit/s, too low for video diffusion output) are raised to `video_bitrate`.
Role parity: telefuser/service/webrtc/session_manager.py.
"""

from __future__ import annotations

import asyncio
import importlib
import json
import time
import uuid
from dataclasses import dataclass, field

from telefuser_b200.utils.logging import logger

from ..stream_service import AudioChunk
from .track import AudioPacer, FramePacer, make_audio_track, make_track


def backend():
    """(aiortc, av) modules; raises ImportError with one message when either is missing."""
    try:
        return importlib.import_module("aiortc"), importlib.import_module("av")
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise ImportError("the WebRTC transport needs the `aiortc` and `av` packages") from e


@dataclass
class WebRTCConnection:
    session_id: str
    pc: object
    pacer: FramePacer
    channel: object | None = None
    pump_task: asyncio.Task | None = None
    created: float = field(default_factory=time.time)
    messages_sent: int = 0
    messages_received: int = 0
    state: str = "new"
    audio_pacer: AudioPacer | None = None
    audio_unsent_chunks: int = 0


class WebRTCSessionManager:
    def __init__(self, sessions=None, stream_service=None, fps: int = 16, video_codec: str = "H264",
                 video_bitrate: int = 8_000_000, max_buffer_seconds: float = 4.0, modules=None) -> None:  # fmt: skip
        self.sessions, self.stream_service = sessions, stream_service
        self.fps, self.video_codec, self.video_bitrate = fps, video_codec.upper(), int(video_bitrate)
        self.max_buffer_seconds = max_buffer_seconds
        self.connections: dict[str, WebRTCConnection] = {}
        self._modules = modules
        self._bitrate_applied = False

    # ---- library access ---------------------------------------------------------------------
    def modules(self):
        if self._modules is None:
            self._modules = backend()
        return self._modules

    def apply_video_bitrate(self) -> None:
        """Raises the encoders' default / maximum bitrate constants of aiortc (module-level, process-wide)."""
        if self._bitrate_applied:
            return
        for name in ("aiortc.codecs.h264", "aiortc.codecs.vpx"):
            try:
                mod = importlib.import_module(name)
            except ImportError:
                continue
            for attr in ("DEFAULT_BITRATE", "MAX_BITRATE"):
                if hasattr(mod, attr):
                    setattr(mod, attr, max(int(getattr(mod, attr)), self.video_bitrate))
        self._bitrate_applied = True

    def set_video_codec_preferences(self, pc) -> None:
        """Moves the preferred codec (and its retransmission companion) to the front for every video transceiver."""
        aiortc, _ = self.modules()
        caps = aiortc.RTCRtpSender.getCapabilities("video")
        want = f"video/{self.video_codec}".lower()
        first = [c for c in caps.codecs if c.mimeType.lower() == want]
        if not first:
            return
        rest = [c for c in caps.codecs if c.mimeType.lower() != want]
        for tr in pc.getTransceivers():
            if getattr(tr, "kind", None) == "video":
                tr.setCodecPreferences(first + rest)

    # ---- signalling ---------------------------------------------------------------------------
    async def answer(self, body: dict) -> dict:
        aiortc, av = self.modules()
        self.apply_video_bitrate()
        config = {**(body.get("config") or {}), **{k: v for k, v in body.items() if k not in ("sdp", "type", "config")}}
        config.setdefault("session_id", body.get("session_id") or str(uuid.uuid4()))
        fps = int(body.get("fps") or self.fps)
        s = await self.sessions.open(config)
        pc = aiortc.RTCPeerConnection()
        pacer = FramePacer(fps, self.max_buffer_seconds)
        conn = WebRTCConnection(s.session_id, pc, pacer)
        self.connections[s.session_id] = conn
        pc.addTrack(make_track(pacer, aiortc, av))
        audio = config.get("audio")
        if audio:  # tracks are fixed at negotiation time: a client that wants the service's sound asks for it in the offer
            opts = audio if isinstance(audio, dict) else {}
            conn.audio_pacer = AudioPacer(int(opts.get("sample_rate") or config.get("audio_sample_rate") or 48000),
                                          int(opts.get("channels") or config.get("audio_channels") or 1), self.max_buffer_seconds)  # fmt: skip
            pc.addTrack(make_audio_track(conn.audio_pacer, aiortc, av))
        self.set_video_codec_preferences(pc)

        @pc.on("datachannel")
        def on_channel(channel) -> None:
            conn.channel = channel

            @channel.on("message")
            def on_message(message) -> None:
                self.handle_client_message(conn, message)

        @pc.on("connectionstatechange")
        async def on_state() -> None:
            await self.handle_state(conn, pc.connectionState)

        await pc.setRemoteDescription(aiortc.RTCSessionDescription(sdp=body["sdp"], type=body.get("type", "offer")))
        await pc.setLocalDescription(await pc.createAnswer())
        conn.pump_task = asyncio.ensure_future(self.pump(conn, s))
        return {"session_id": s.session_id, "sdp": pc.localDescription.sdp, "type": pc.localDescription.type}

    # ---- events ---------------------------------------------------------------------------------
    def handle_client_message(self, conn: WebRTCConnection, message) -> None:
        try:
            msg = json.loads(message)
        except (TypeError, ValueError):
            return
        if not isinstance(msg, dict):
            return
        conn.messages_received += 1
        if msg.get("type") == "close":
            asyncio.ensure_future(self.sessions.close(conn.session_id, reason="client close"))
        elif getattr(self.stream_service, "stream_mode", None) == "bidirectional":
            self.sessions.push(conn.session_id, msg)

    async def handle_state(self, conn: WebRTCConnection, state: str) -> None:
        conn.state = state
        if state == "disconnected":
            self.sessions.mark_disconnected(conn.session_id)  # the grace period starts; the pipeline keeps running
        elif state == "connected":
            self.sessions.mark_reconnected(conn.session_id)
        elif state in ("failed", "closed"):
            await self.sessions.close(conn.session_id, reason=f"webrtc {state}")
            self.connections.pop(conn.session_id, None)

    async def pump(self, conn: WebRTCConnection, s) -> None:
        """Session outbound queue -> pacer (frames) + data channel (messages), until the stream is done."""
        try:
            while not s.closed:
                frames, msg = await s.outbound.get()
                conn.pacer.push_frames([f for f in frames if not isinstance(f, AudioChunk)])
                for a in (f for f in frames if isinstance(f, AudioChunk)):
                    if conn.audio_pacer is None:
                        conn.audio_unsent_chunks += 1  # the client did not ask for an audio track
                        continue
                    try:
                        conn.audio_pacer.push(a.pcm16, a.sample_rate, a.channels)
                    except ValueError as e:
                        conn.audio_unsent_chunks += 1
                        logger.warning(f"session {s.session_id}: {e}")
                ch = conn.channel
                if ch is not None and getattr(ch, "readyState", "open") == "open":
                    ch.send(json.dumps(msg))
                    conn.messages_sent += 1
                s.chunks_sent += 1
                if msg.get("type") == "done":
                    break
        finally:
            conn.pacer.finish()
            s.frames_dropped += conn.pacer.dropped_frames

    async def close_connection(self, session_id: str) -> None:
        conn = self.connections.pop(session_id, None)
        if conn is None:
            return
        if conn.pump_task is not None:
            conn.pump_task.cancel()
        await conn.pc.close()

    async def close_all(self) -> None:
        for sid in list(self.connections):
            await self.close_connection(sid)

    def stats(self) -> dict:
        return {sid: {"state": c.state, "age_s": round(time.time() - c.created, 3), "sent": c.messages_sent,
                      "received": c.messages_received, **c.pacer.stats(),
                      **({"audio": c.audio_pacer.stats()} if c.audio_pacer is not None else {}),
                      "audio_unsent_chunks": c.audio_unsent_chunks} for sid, c in self.connections.items()}  # fmt: skip


async def answer_offer(api, body: dict) -> dict:
    """Route handler of `POST /v1/stream/webrtc/offer`: one manager per API server, created on first use."""
    mgr = getattr(api, "webrtc", None)
    if mgr is None:
        mgr = api.webrtc = WebRTCSessionManager(api.sessions, api.stream_service, fps=api.config.stream_fps)
    return await mgr.answer(body)
