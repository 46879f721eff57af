"""Video / image / audio file helpers (OpenCV + PIL + the standard library; no ffmpeg binding needed).

`VideoData` reads frames lazily from a video file or an image folder with optional crop-and-resize;
`save_video` writes uint8 frames (list of PIL / numpy, a `[T, H, W, 3]` uint8 array or tensor, or a
`[3, T, H, W]` float tensor in [-1, 1], which is converted on the device first) to mp4 through
`cv2.VideoWriter`; `save_wav` writes PCM16 audio.
Role parity: telefuser/utils/video.py:38-464, utils/audio.py:12.
"""

from __future__ import annotations

import base64
import io
import os
import re
import wave
from typing import Sequence

import numpy as np
import torch
from PIL import Image

_IMAGE_EXT = (".png", ".jpg", ".jpeg", ".bmp", ".webp")
_RATIOS = {"16:9": (16, 9), "9:16": (9, 16), "4:3": (4, 3), "3:4": (3, 4), "1:1": (1, 1), "2:3": (2, 3), "3:2": (3, 2)}
_SHORT_SIDE = {"480p": 480, "540p": 540, "720p": 720, "1080p": 1080}


def get_target_video_size_from_ratio(resolution: str = "720p", aspect_ratio: str = "16:9", multiple: int = 16):
    """(height, width) with the short side given by `resolution` ("480p", "720p", any "<n>p", or an explicit
    "WIDTHxHEIGHT"), both rounded down to `multiple`."""
    res = resolution.lower().strip()
    if "x" in res:  # explicit "WIDTHxHEIGHT": taken as given (rounded down to the multiple), whatever the aspect ratio says
        try:
            w, h = (int(v) for v in res.split("x", 1))
        except ValueError:
            raise ValueError(f"unknown resolution {resolution!r}") from None
        if w < multiple or h < multiple:
            raise ValueError(f"resolution {resolution!r} is smaller than one {multiple}-pixel tile")
        return h // multiple * multiple, w // multiple * multiple
    short = _SHORT_SIDE.get(res) or (int(res[:-1]) if res.endswith("p") and res[:-1].isdigit() else None)
    if short is None:
        raise ValueError(f"unknown resolution {resolution!r}")
    a, b = _RATIOS[aspect_ratio]
    if a >= b:
        h, w = short, short * a / b
    else:
        h, w = short * b / a, short
    return int(h) // multiple * multiple, int(w) // multiple * multiple


def get_target_image_size(image: Image.Image, max_area: int, multiple: int = 16) -> tuple[int, int]:
    """(height, width) that keeps the aspect ratio within `max_area` pixels."""
    w, h = image.size
    scale = (max_area / (w * h)) ** 0.5
    return max(multiple, int(h * scale) // multiple * multiple), max(multiple, int(w * scale) // multiple * multiple)


def images_to_base_64(images: Sequence[Image.Image]) -> list[str]:
    out = []
    for im in images:
        buf = io.BytesIO()
        im.save(buf, format="PNG")
        out.append(base64.b64encode(buf.getvalue()).decode())
    return out


def crop_and_resize(image: Image.Image, height: int, width: int) -> Image.Image:
    """Scale to cover the target, then centre-crop."""
    w, h = image.size
    scale = max(width / w, height / h)
    nw, nh = max(width, round(w * scale)), max(height, round(h * scale))
    image = image.resize((nw, nh), Image.LANCZOS)
    left, top = (nw - width) // 2, (nh - height) // 2
    return image.crop((left, top, left + width, top + height))


def search_for_images(folder: str) -> list[str]:
    def key(name: str):
        return [int(t) if t.isdigit() else t for t in re.split(r"(\d+)", name)]

    return sorted((f for f in os.listdir(folder) if f.lower().endswith(_IMAGE_EXT)), key=key)


class LowMemoryVideo:
    def __init__(self, file_name: str) -> None:
        import cv2

        self._cv2 = cv2
        self.cap = cv2.VideoCapture(file_name)
        if not self.cap.isOpened():
            raise FileNotFoundError(f"cannot open video {file_name}")
        self._pos = 0

    def fps(self) -> float:
        return float(self.cap.get(self._cv2.CAP_PROP_FPS) or 0.0)

    def __len__(self) -> int:
        return int(self.cap.get(self._cv2.CAP_PROP_FRAME_COUNT))

    def __getitem__(self, item: int) -> Image.Image:
        if item != self._pos:
            self.cap.set(self._cv2.CAP_PROP_POS_FRAMES, item)
        ok, frame = self.cap.read()
        if not ok:
            raise IndexError(item)
        self._pos = item + 1
        return Image.fromarray(self._cv2.cvtColor(frame, self._cv2.COLOR_BGR2RGB))

    def __del__(self) -> None:
        cap = getattr(self, "cap", None)
        if cap is not None:
            cap.release()


class LowMemoryImageFolder:
    def __init__(self, folder: str, file_list: list[str] | None = None) -> None:
        names = file_list if file_list is not None else search_for_images(folder)
        self.files = [os.path.join(folder, n) for n in names]

    def __len__(self) -> int:
        return len(self.files)

    def __getitem__(self, item: int) -> Image.Image:
        return Image.open(self.files[item]).convert("RGB")


class VideoData:
    def __init__(self, video_file: str | None = None, image_folder: str | None = None, height: int | None = None,
                 width: int | None = None, length: int | None = None) -> None:  # fmt: skip
        if video_file is not None:
            self.data = LowMemoryVideo(video_file)
        elif image_folder is not None:
            self.data = LowMemoryImageFolder(image_folder)
        else:
            raise ValueError("VideoData needs a video file or an image folder")
        self.height, self.width, self.length = height, width, length

    def fps(self) -> float:
        return self.data.fps() if hasattr(self.data, "fps") else 0.0

    def raw_data(self) -> list[Image.Image]:
        return [self[i] for i in range(len(self))]

    def set_length(self, length: int) -> None:
        self.length = length

    def set_shape(self, height: int, width: int) -> None:
        self.height, self.width = height, width

    def __len__(self) -> int:
        return len(self.data) if self.length is None else min(self.length, len(self.data))

    def shape(self):
        if self.height is not None and self.width is not None:
            return self.height, self.width
        w, h = self[0].size
        return h, w

    def __getitem__(self, item: int) -> Image.Image:
        frame = self.data[item]
        if self.height is not None and self.width is not None and frame.size != (self.width, self.height):
            frame = crop_and_resize(frame, self.height, self.width)
        return frame

    def to_tensor(self) -> torch.Tensor:
        """[3, T, H, W] in [-1, 1]."""
        arr = np.stack([np.asarray(self[i], dtype=np.float32) for i in range(len(self))])
        return torch.from_numpy(arr).permute(3, 0, 1, 2) / 127.5 - 1.0

    def save_images(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        for i in range(len(self)):
            self[i].save(os.path.join(folder, f"{i}.png"))


def frames_to_uint8_array(frames) -> np.ndarray:
    """Anything frame-like -> uint8 [T, H, W, 3]."""
    if isinstance(frames, torch.Tensor):
        if frames.dtype != torch.uint8:
            from telefuser_b200.ops import functional as TF

            if frames.dim() == 5:
                frames = frames[0]
            frames = TF.frames_to_uint8(frames)  # [3, T, H, W] in [-1, 1] -> [T, H, W, 3]
        return frames.cpu().numpy()
    if isinstance(frames, np.ndarray):
        return frames.astype(np.uint8, copy=False)
    return np.stack([np.asarray(f.convert("RGB") if isinstance(f, Image.Image) else f, dtype=np.uint8) for f in frames])


def save_video(frames, save_path: str, fps: int = 16, quality: int = 6, codec: str = "mp4v") -> str:
    import cv2

    arr = frames_to_uint8_array(frames)
    t, h, w, _ = arr.shape
    os.makedirs(os.path.dirname(os.path.abspath(save_path)), exist_ok=True)
    writer = cv2.VideoWriter(save_path, cv2.VideoWriter_fourcc(*codec), float(fps), (w, h))
    if not writer.isOpened():
        raise RuntimeError(f"cannot open a video writer for {save_path} (codec {codec})")
    try:
        writer.set(cv2.VIDEOWRITER_PROP_QUALITY, min(100.0, quality * 10.0))
        for i in range(t):
            writer.write(cv2.cvtColor(arr[i], cv2.COLOR_RGB2BGR))
    finally:
        writer.release()
    return save_path


def save_frames(frames, save_path: str) -> None:
    os.makedirs(save_path, exist_ok=True)
    for i, f in enumerate(frames_to_uint8_array(frames)):
        Image.fromarray(f).save(os.path.join(save_path, f"{i}.png"))


def resize_video(frames: Sequence[Image.Image], height: int, width: int) -> list[Image.Image]:
    return [crop_and_resize(f, height, width) for f in frames]


def color_video_by_mask(frames: Sequence[Image.Image], masks: Sequence[Image.Image], color=(255, 0, 0), alpha=0.5):
    out = []
    for f, m in zip(frames, masks):
        a = np.asarray(f.convert("RGB"), dtype=np.float32)
        k = (np.asarray(m.convert("L").resize(f.size), dtype=np.float32) / 255.0)[..., None] * alpha
        out.append(Image.fromarray((a * (1 - k) + np.asarray(color, dtype=np.float32) * k).astype(np.uint8)))
    return out


def save_wav(audio, save_path: str, sample_rate: int = 16000) -> str:
    """audio: float tensor / array in [-1, 1], shape [samples] or [channels, samples]."""
    a = audio.detach().float().cpu().numpy() if isinstance(audio, torch.Tensor) else np.asarray(audio, dtype=np.float32)
    if a.ndim == 1:
        a = a[None]
    pcm = (np.clip(a, -1.0, 1.0) * 32767.0).astype("<i2").T.copy()  # [samples, channels]
    os.makedirs(os.path.dirname(os.path.abspath(save_path)), exist_ok=True)
    with wave.open(save_path, "wb") as w:
        w.setnchannels(pcm.shape[1])
        w.setsampwidth(2)
        w.setframerate(sample_rate)
        w.writeframes(pcm.tobytes())
    return save_path
