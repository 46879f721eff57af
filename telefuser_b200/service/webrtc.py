"""WebRTC transport for streaming sessions. Needs the optional `aiortc` (+ `av`) packages; every
import of them happens inside the functions so that the module imports without them.

Signalling: `POST /v1/stream/webrtc/offer` carries the browser's SDP offer plus the session config;
the answer carries the server's SDP. Media frames leave on one video track paced at the session's fps
(the newest frame is repeated while the pipeline has nothing new); JSON chunk messages and client
controls use a data channel named "control".
Role parity: telefuser/service/api/routers/webrtc.py, webrtc/track.py, webrtc/session_manager.py.
"""

from __future__ import annotations

import asyncio
import fractions
import json
import time
import uuid


def _frame_to_ndarray(frame):
    import numpy as np
    import torch

    if isinstance(frame, torch.Tensor):
        t = frame.detach().float().cpu()
        if t.dim() == 3 and t.shape[0] in (1, 3) and t.shape[-1] not in (1, 3):
            t = t.permute(1, 2, 0)
        if frame.dtype != torch.uint8:
            t = ((t + 1) * 127.5 if t.min() < 0 else t * 255.0).clamp(0, 255)
        return t.to(torch.uint8).numpy()
    return np.asarray(frame)


def make_video_track(session, fps: int):
    from aiortc import MediaStreamTrack
    from av import VideoFrame

    class PipelineVideoTrack(MediaStreamTrack):
        kind = "video"

        def __init__(self) -> None:
            super().__init__()
            self.frames: asyncio.Queue = asyncio.Queue(maxsize=4 * fps)
            self.last = None
            self.pts = 0
            self.t0 = None

        async def recv(self):
            if self.t0 is None:
                self.t0 = time.monotonic()
            wait = self.t0 + self.pts / fps - time.monotonic()
            if wait > 0:
                await asyncio.sleep(wait)
            try:
                self.last = self.frames.get_nowait()
            except asyncio.QueueEmpty:
                if self.last is None:
                    self.last = await self.frames.get()
            vf = VideoFrame.from_ndarray(_frame_to_ndarray(self.last), format="rgb24")
            vf.pts, vf.time_base = self.pts, fractions.Fraction(1, fps)
            self.pts += 1
            return vf

    return PipelineVideoTrack()


async def answer_offer(api, body: dict) -> dict:
    from aiortc import RTCPeerConnection, RTCSessionDescription

    sessions = api.sessions
    config = {**(body.get("config") or {}), **{k: v for k, v in body.items() if k not in ("sdp", "type", "config")}}
    config.setdefault("session_id", body.get("session_id") or str(uuid.uuid4()))
    fps = int(body.get("fps") or api.config.stream_fps)
    s = await sessions.open(config)
    pc = RTCPeerConnection()
    track = make_video_track(s, fps)
    pc.addTrack(track)
    channel_box: dict = {}

    @pc.on("datachannel")
    def on_channel(channel) -> None:
        channel_box["ch"] = channel

        @channel.on("message")
        def on_message(message) -> None:
            try:
                msg = json.loads(message)
            except (TypeError, ValueError):
                return
            if msg.get("type") == "close":
                asyncio.ensure_future(sessions.close(s.session_id, reason="client close"))
            elif api.stream_service.stream_mode == "bidirectional":
                sessions.push(s.session_id, msg)

    @pc.on("connectionstatechange")
    async def on_state() -> None:
        if pc.connectionState in ("disconnected",):
            sessions.mark_disconnected(s.session_id)
        elif pc.connectionState == "connected":
            sessions.mark_reconnected(s.session_id)
        elif pc.connectionState in ("failed", "closed"):
            await sessions.close(s.session_id, reason=f"webrtc {pc.connectionState}")

    async def pump() -> None:
        while not s.closed:
            frames, msg = await s.outbound.get()
            for f in frames:
                if track.frames.full():
                    track.frames.get_nowait()
                    s.frames_dropped += 1
                track.frames.put_nowait(f)
            ch = channel_box.get("ch")
            if ch is not None and ch.readyState == "open":
                ch.send(json.dumps(msg))
            s.chunks_sent += 1
            if msg.get("type") == "done":
                break
        await pc.close()

    await pc.setRemoteDescription(RTCSessionDescription(sdp=body["sdp"], type=body.get("type", "offer")))
    await pc.setLocalDescription(await pc.createAnswer())
    asyncio.ensure_future(pump())
    return {"session_id": s.session_id, "sdp": pc.localDescription.sdp, "type": pc.localDescription.type}
