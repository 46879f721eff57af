"""Frame pacing for the outgoing video track.

`FramePacer` is the buffer between the pipeline (bursts of 16 frames every chunk period) and the WebRTC
sender (one frame every 1 / fps seconds): a bounded FIFO that drops the oldest frame when the client falls behind,
repeats the newest frame while the pipeline has nothing new (also after the stream has finished, so the picture
stays up), and stamps presentation times on a fixed 1 / fps grid. It knows nothing about aiortc; `make_track`
wraps it in a `MediaStreamTrack` when the library is present.
Role parity: telefuser/service/webrtc/track.py (`FrameGeneratorTrack`).
"""

from __future__ import annotations

import asyncio
import fractions
import time
from collections import deque


def frame_to_rgb(frame):
    """Tensor (CHW or HWC; uint8, [0, 1] or [-1, 1]), PIL image or array -> uint8 HWC numpy array."""
    import numpy as np
    import torch

    if isinstance(frame, torch.Tensor):
        t = frame.detach().cpu()
        if t.dim() == 3 and t.shape[0] in (1, 3) and t.shape[-1] not in (1, 3):
            t = t.permute(1, 2, 0)
        if t.dtype != torch.uint8:
            t = t.float()
            t = ((t + 1) * 127.5 if t.min() < 0 else t * 255.0).round().clamp(0, 255).to(torch.uint8)
        if t.shape[-1] == 1:
            t = t.expand(*t.shape[:-1], 3)
        return np.ascontiguousarray(t.numpy())
    arr = np.asarray(frame)
    if arr.ndim == 2:
        arr = np.stack([arr] * 3, axis=-1)
    return np.ascontiguousarray(arr.astype(np.uint8, copy=False))


class FramePacer:
    def __init__(self, fps: int = 16, max_buffer_seconds: float = 4.0, clock=time.monotonic) -> None:
        if fps < 1:
            raise ValueError("fps must be positive")
        self.fps = fps
        self.capacity = max(1, int(round(fps * max_buffer_seconds)))
        self.queue: deque = deque()
        self.clock = clock
        self.last = None
        self.pts = 0
        self.t0: float | None = None
        self.dropped_frames = 0
        self.repeated_frames = 0
        self.finished = False
        self._wakeup: asyncio.Event | None = None

    # ---- producer side (pipeline) ---------------------------------------------------------
    def push_frame(self, frame) -> None:
        if len(self.queue) >= self.capacity:
            self.queue.popleft()  # the client is behind: the oldest picture is the least useful one
            self.dropped_frames += 1
        self.queue.append(frame)
        if self._wakeup is not None:
            self._wakeup.set()

    def push_frames(self, frames) -> None:
        for f in frames:
            self.push_frame(f)

    def finish(self) -> None:
        """No more frames will come; `next_frame` keeps returning the last one."""
        self.finished = True
        if self._wakeup is not None:
            self._wakeup.set()

    # ---- consumer side (sender) ----------------------------------------------------------
    async def next_frame(self):
        """-> (frame, pts, time_base). Sleeps until the frame's slot on the 1 / fps grid."""
        if self._wakeup is None:
            self._wakeup = asyncio.Event()
        if self.t0 is None:
            self.t0 = self.clock()
        delay = self.t0 + self.pts / self.fps - self.clock()
        if delay > 0:
            await asyncio.sleep(delay)
        while not self.queue and self.last is None and not self.finished:
            self._wakeup.clear()
            await self._wakeup.wait()  # nothing has ever been produced: wait for the first picture
        if self.queue:
            self.last = self.queue.popleft()
        elif self.last is not None:
            self.repeated_frames += 1
        pts = self.pts
        self.pts += 1
        return self.last, pts, fractions.Fraction(1, self.fps)

    def stats(self) -> dict:
        return {"queued": len(self.queue), "sent": self.pts, "dropped": self.dropped_frames,
                "repeated": self.repeated_frames, "finished": self.finished}  # fmt: skip


def make_track(pacer: FramePacer, aiortc, av):
    """A video `MediaStreamTrack` of the given aiortc module whose frames come from `pacer`."""

    class PipelineVideoTrack(aiortc.MediaStreamTrack):
        kind = "video"

        def __init__(self) -> None:
            super().__init__()
            self.pacer = pacer

        async def recv(self):
            frame, pts, time_base = await pacer.next_frame()
            if frame is None:  # the stream finished before its first picture: a black frame keeps the track alive
                import numpy as np

                frame = np.zeros((16, 16, 3), dtype="uint8")
            vf = frame if isinstance(frame, av.VideoFrame) else av.VideoFrame.from_ndarray(frame_to_rgb(frame), format="rgb24")
            vf.pts, vf.time_base = pts, time_base
            return vf

    return PipelineVideoTrack()
