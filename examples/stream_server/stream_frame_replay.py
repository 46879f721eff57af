"""Server-push stream service that replays a clip (or a synthetic test card when no file is given) as paced frame
chunks: the smallest service `telefuser stream-serve` can load, for checking a deployment's transport, the browser
front end at `/ui` and the client-side stream benchmark without any model.

    telefuser stream-serve examples/stream_server/stream_frame_replay.py -p 8088
    TFB_REPLAY_VIDEO=clip.mp4 telefuser stream-serve examples/stream_server/stream_frame_replay.py -p 8088
"""

from __future__ import annotations

import asyncio
import os
import time

import torch

FRAMES_PER_CHUNK = int(os.environ.get("TFB_REPLAY_CHUNK", "16"))
OUTPUT_FPS = int(os.environ.get("TFB_REPLAY_FPS", "16"))
VIDEO_PATH = os.environ.get("TFB_REPLAY_VIDEO", "")


def test_card(num_frames: int = 96, height: int = 240, width: int = 416) -> torch.Tensor:
    """[T, H, W, 3] uint8: colour bars with a bar sweeping across, so dropped or reordered frames are visible."""
    bars = torch.tensor([[235, 235, 235], [235, 235, 16], [16, 235, 235], [16, 235, 16], [235, 16, 235], [235, 16, 16],
                         [16, 16, 235], [16, 16, 16]], dtype=torch.uint8)  # fmt: skip
    row = bars[(torch.arange(width) * len(bars) // width)]
    frames = row.expand(num_frames, height, width, 3).clone()
    for t in range(num_frames):
        x = (t * width) // num_frames
        frames[t, :, x : x + 6] = 255
    return frames


class FrameReplayService:
    """`serve(request)` yields {"frames": uint8 [n, H, W, 3], "chunk_index", "pts_s"} at the clip's frame rate."""

    def __init__(self, video_path: str = VIDEO_PATH, frames_per_chunk: int = FRAMES_PER_CHUNK, fps: int = OUTPUT_FPS):
        self.video_path, self.frames_per_chunk, self.fps = video_path, frames_per_chunk, fps
        self.frames: torch.Tensor | None = None

    def start(self) -> None:
        if self.video_path:
            from telefuser_b200.utils.video import VideoData, frames_to_uint8_array

            self.frames = torch.from_numpy(frames_to_uint8_array(VideoData(self.video_path).raw_data()))
        else:
            self.frames = test_card()

    def stop(self) -> None:
        self.frames = None

    async def serve(self, request: dict):
        loops = max(1, int(request.get("loops", 1)))
        fps = int(request.get("fps", self.fps))
        total = self.frames.shape[0]
        t0, sent, index = time.perf_counter(), 0, 0
        for _ in range(loops):
            for start in range(0, total, self.frames_per_chunk):
                chunk = self.frames[start : start + self.frames_per_chunk]
                due = t0 + sent / fps  # a chunk leaves when its first frame is due
                delay = due - time.perf_counter()
                if delay > 0:
                    await asyncio.sleep(delay)
                yield {"frames": chunk, "chunk_index": index, "pts_s": round(sent / fps, 4)}
                sent += chunk.shape[0]
                index += 1


def get_service(gpu_num: int = 1) -> FrameReplayService:
    return FrameReplayService()
