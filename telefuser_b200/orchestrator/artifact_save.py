"""Stage that writes generated frames to disk with a metadata record.

Output layout: `<output_root>/<run_name>/[YYYYMMDD/]<request_id>.mp4` plus `<request_id>.json` holding
the request id, path, frame count, size, fps and creation time. Names are sanitised so that a request
id can never escape the run directory.
Role parity: telefuser/orchestrator/artifact_save_stage.py:22-119.
"""

from __future__ import annotations

import json
import re
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from telefuser_b200.utils.video import frames_to_uint8_array, save_frames, save_video


def _safe_component(s: str, max_len: int = 48) -> str:
    s = re.sub(r"[^A-Za-z0-9._-]+", "_", str(s)).strip("._") or "item"
    return s[:max_len]


@dataclass
class ArtifactSaveConfig:
    output_root: Path
    run_name: str
    fps: int = 16
    quality: int = 6


class ArtifactSaveStage:
    def __init__(self, name: str = "artifact_save") -> None:
        self.name = name

    def process(self, frames, *, request_id: str, config: ArtifactSaveConfig, file_ext: str = ".mp4",
                make_date_subdir: bool = True) -> dict[str, Any]:  # fmt: skip
        root = Path(config.output_root).resolve() / _safe_component(config.run_name)
        if make_date_subdir:
            root = root / time.strftime("%Y%m%d")
        root.mkdir(parents=True, exist_ok=True)
        stem = _safe_component(request_id)
        arr = frames_to_uint8_array(frames)
        if file_ext.lower() in (".mp4", ".avi", ".mov"):
            path = root / f"{stem}{file_ext}"
            save_video(arr, str(path), fps=config.fps, quality=config.quality)
        else:  # a folder of PNG frames
            path = root / stem
            save_frames(arr, str(path))
        meta = {"request_id": request_id, "path": str(path), "num_frames": int(arr.shape[0]), "height": int(arr.shape[1]),
                "width": int(arr.shape[2]), "fps": config.fps, "created": time.time(), "stage": self.name}  # fmt: skip
        (root / f"{stem}.json").write_text(json.dumps(meta, indent=2))
        return meta
