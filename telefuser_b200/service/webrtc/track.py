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
    if isinstance(frame, (bytes, bytearray)):  # an encoded picture (JPEG / PNG)
        import io

        from PIL import Image

        frame = Image.open(io.BytesIO(bytes(frame))).convert("RGB")
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


class AudioPacer:
    """The audio counterpart of `FramePacer`: chunks of interleaved PCM16 go in, fixed 20 ms packets come out on a
    real-time grid. While nothing is queued the packets are silence, so the track never stalls the connection; when the
    client falls more than `max_buffer_seconds` behind, the oldest samples are dropped."""

    PACKET_SECONDS = 0.02

    def __init__(self, sample_rate: int = 48000, channels: int = 1, max_buffer_seconds: float = 4.0, clock=time.monotonic) -> None:
        if sample_rate < 8000 or channels not in (1, 2):
            raise ValueError(f"audio tracks carry mono or stereo at 8 kHz or more, got {channels} channel(s) at {sample_rate} Hz")
        self.sample_rate, self.channels, self.clock = sample_rate, channels, clock
        self.packet_samples = int(round(sample_rate * self.PACKET_SECONDS))
        self.capacity_bytes = int(sample_rate * max_buffer_seconds) * 2 * channels
        self.buffer = bytearray()
        self.pts = 0
        self.t0: float | None = None
        self.dropped_samples = self.silent_packets = 0

    def push(self, pcm16: bytes, sample_rate: int | None = None, channels: int | None = None) -> None:
        if (sample_rate or self.sample_rate) != self.sample_rate or (channels or self.channels) != self.channels:
            raise ValueError(f"this track was negotiated as {self.channels} channel(s) at {self.sample_rate} Hz; the chunk has "
                             f"{channels} at {sample_rate}")  # fmt: skip
        self.buffer.extend(pcm16)
        over = len(self.buffer) - self.capacity_bytes
        if over > 0:
            frame = 2 * self.channels
            over = -(-over // frame) * frame
            del self.buffer[:over]
            self.dropped_samples += over // frame

    async def next_packet(self):
        """-> (PCM16 bytes of one packet, pts in samples, time base). Sleeps until the packet's slot."""
        if self.t0 is None:
            self.t0 = self.clock()
        delay = self.t0 + self.pts / self.sample_rate - self.clock()
        if delay > 0:
            await asyncio.sleep(delay)
        need = self.packet_samples * 2 * self.channels
        if len(self.buffer) >= need:
            data = bytes(self.buffer[:need])
            del self.buffer[:need]
        else:  # not enough for a whole packet: play what there is, pad with silence
            data = bytes(self.buffer) + bytes(need - len(self.buffer))
            self.silent_packets += 1
            self.buffer.clear()
        pts = self.pts
        self.pts += self.packet_samples
        return data, pts, fractions.Fraction(1, self.sample_rate)

    def stats(self) -> dict:
        return {"queued_samples": len(self.buffer) // (2 * self.channels), "sent_samples": self.pts,
                "dropped_samples": self.dropped_samples, "silent_packets": self.silent_packets}  # fmt: skip


def make_audio_track(pacer: AudioPacer, aiortc, av):
    """An audio `MediaStreamTrack` of the given aiortc module whose packets come from `pacer`."""
    import numpy as np

    class PipelineAudioTrack(aiortc.MediaStreamTrack):
        kind = "audio"

        def __init__(self) -> None:
            super().__init__()
            self.pacer = pacer

        async def recv(self):
            data, pts, time_base = await pacer.next_packet()
            samples = np.frombuffer(data, dtype=np.int16).reshape(1, -1)  # packed layout: one plane, channels interleaved
            af = av.AudioFrame.from_ndarray(samples, format="s16", layout="stereo" if pacer.channels == 2 else "mono")
            af.sample_rate, af.pts, af.time_base = pacer.sample_rate, pts, time_base
            return af

    return PipelineAudioTrack()
