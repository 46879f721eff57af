"""Input / output file handling for the server.

* `MediaHandler` family: sniff and validate uploaded bytes (magic numbers, size limit), decode base64
  or data-URL payloads, pick file extensions.
* `FileService`: cache directory layout (`inputs/`, `outputs/`), safe path resolution (no escape
  from the cache directory), async download of http(s) inputs with a size cap, upload saving.
* `ArtifactStore`: index of produced artefacts (id -> path, task, media type, created, size) persisted
  as JSON; retention by age and by total size; lookup for the download routes.
Role parity: telefuser/service/media/media_base.py, core/file_service.py, core/artifact_store.py.
"""

from __future__ import annotations

import base64
import binascii
import json
import os
import re
import threading
import time
import uuid
from dataclasses import asdict, dataclass
from enum import Enum
from pathlib import Path


class MediaType(str, Enum):
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"


_MAGIC = {
    MediaType.IMAGE: [(b"\x89PNG\r\n\x1a\n", "png"), (b"\xff\xd8\xff", "jpg"), (b"GIF8", "gif"), (b"BM", "bmp"),
                      (b"RIFF", "webp")],  # fmt: skip
    MediaType.VIDEO: [(b"\x1aE\xdf\xa3", "webm"), (b"RIFF", "avi")],
    MediaType.AUDIO: [(b"RIFF", "wav"), (b"ID3", "mp3"), (b"\xff\xfb", "mp3"), (b"fLaC", "flac"), (b"OggS", "ogg")],
}
_DATA_URL = re.compile(r"^data:(?P<mime>[\w/+.-]+)?;base64,(?P<data>.*)$", re.S)


class MediaError(ValueError):
    pass


class MediaHandler:
    def __init__(self, media_type: MediaType, max_bytes: int = 512 << 20) -> None:
        self.media_type, self.max_bytes = media_type, max_bytes

    def sniff(self, data: bytes) -> str | None:
        head = data[:16]
        if self.media_type == MediaType.VIDEO and len(data) >= 12 and data[4:8] == b"ftyp":
            return "mov" if data[8:10] == b"qt" else "mp4"
        for magic, ext in _MAGIC[self.media_type]:
            if head.startswith(magic):
                if magic == b"RIFF":
                    kind = data[8:12]
                    want = {"webp": b"WEBP", "avi": b"AVI ", "wav": b"WAVE"}[ext]
                    if kind != want:
                        continue
                return ext
        return None

    def validate(self, data: bytes) -> str:
        if not data:
            raise MediaError(f"empty {self.media_type.value} payload")
        if len(data) > self.max_bytes:
            raise MediaError(f"{self.media_type.value} payload of {len(data)} bytes exceeds the limit {self.max_bytes}")
        ext = self.sniff(data)
        if ext is None:
            raise MediaError(f"payload is not a recognised {self.media_type.value} format")
        return ext

    @staticmethod
    def is_base64(s: str) -> bool:
        if _DATA_URL.match(s):
            return True
        if len(s) < 64 or len(s) % 4 or re.search(r"[^A-Za-z0-9+/=\s]", s[:256]):
            return False
        try:
            base64.b64decode(s[:64], validate=True)
            return True
        except (binascii.Error, ValueError):
            return False

    def decode_base64(self, s: str) -> tuple[bytes, str]:
        m = _DATA_URL.match(s)
        payload = m.group("data") if m else s
        try:
            data = base64.b64decode(payload, validate=False)
        except (binascii.Error, ValueError) as e:
            raise MediaError(f"invalid base64 {self.media_type.value} payload") from e
        return data, self.validate(data)


def handler_for(media_type: MediaType | str, max_bytes: int = 512 << 20) -> MediaHandler:
    return MediaHandler(MediaType(media_type), max_bytes)


class FileService:
    def __init__(self, cache_dir: str, max_upload_mb: int = 512) -> None:
        self.root = Path(cache_dir).resolve()
        self.input_dir = self.root / "inputs"
        self.output_dir = self.root / "outputs"
        for d in (self.input_dir, self.output_dir):
            d.mkdir(parents=True, exist_ok=True)
        self.max_bytes = max_upload_mb << 20

    # ---- paths ----
    def resolve_inside(self, rel: str, base: Path | None = None) -> Path:
        base = base or self.root
        p = (base / rel).resolve()
        if base not in p.parents and p != base:
            raise PermissionError(f"path {rel!r} escapes the cache directory")
        return p

    def output_path_for(self, name: str) -> Path:
        name = os.path.basename(name) or f"{uuid.uuid4().hex}.bin"
        return self.output_dir / name

    # ---- saving ----
    def save_bytes(self, data: bytes, media_type: MediaType | str, prefix: str = "input") -> str:
        ext = handler_for(media_type, self.max_bytes).validate(data)
        path = self.input_dir / f"{prefix}_{uuid.uuid4().hex[:12]}.{ext}"
        path.write_bytes(data)
        return str(path)

    def save_base64(self, payload: str, media_type: MediaType | str, prefix: str = "input") -> str:
        data, _ = handler_for(media_type, self.max_bytes).decode_base64(payload)
        return self.save_bytes(data, media_type, prefix)

    async def save_upload(self, upload, media_type: MediaType | str, prefix: str = "input") -> str:
        data = await upload.read()
        return self.save_bytes(data, media_type, prefix)

    async def url_is_reachable(self, url: str, timeout: float = 5.0) -> bool:
        import httpx

        try:
            async with httpx.AsyncClient(timeout=timeout, follow_redirects=True) as c:
                r = await c.head(url)
                return r.status_code < 400
        except Exception:  # noqa: BLE001
            return False

    async def download(self, url: str, media_type: MediaType | str, prefix: str = "input", timeout: float = 60.0) -> str:
        import httpx

        if not url.startswith(("http://", "https://")):
            raise MediaError("only http(s) URLs can be downloaded")
        buf = bytearray()
        async with httpx.AsyncClient(timeout=timeout, follow_redirects=True) as c:
            async with c.stream("GET", url) as r:
                r.raise_for_status()
                async for chunk in r.aiter_bytes():
                    buf.extend(chunk)
                    if len(buf) > self.max_bytes:
                        raise MediaError(f"download exceeds {self.max_bytes} bytes")
        return self.save_bytes(bytes(buf), media_type, prefix)

    async def materialise_input(self, value: str, media_type: MediaType | str, prefix: str = "input") -> str:
        """URL -> downloaded file; base64 / data URL -> decoded file; anything else is taken as a local path."""
        if not value:
            return value
        if value.startswith(("http://", "https://")):
            return await self.download(value, media_type, prefix)
        if MediaHandler.is_base64(value):
            return self.save_base64(value, media_type, prefix)
        return value

    def cleanup_inputs(self, older_than_s: float) -> int:
        now, n = time.time(), 0
        for p in self.input_dir.iterdir():
            if p.is_file() and now - p.stat().st_mtime > older_than_s:
                p.unlink(missing_ok=True)
                n += 1
        return n


@dataclass
class ArtifactRecord:
    artifact_id: str
    path: str
    task_id: str
    task: str
    media_type: str
    created: float
    size: int
    meta: dict | None = None


class ArtifactStore:
    def __init__(self, root: str, retention_hours: float = 24.0, max_gb: float = 50.0) -> None:
        self.root = Path(root).resolve()
        self.root.mkdir(parents=True, exist_ok=True)
        self.index_path = self.root / "artifacts.json"
        self.retention_s = retention_hours * 3600.0
        self.max_bytes = int(max_gb * (1 << 30))
        self._lock = threading.RLock()
        self._records: dict[str, ArtifactRecord] = {}
        self._load()

    def _load(self) -> None:
        if self.index_path.is_file():
            try:
                for raw in json.loads(self.index_path.read_text()):
                    rec = ArtifactRecord(**raw)
                    if os.path.isfile(rec.path):
                        self._records[rec.artifact_id] = rec
            except (json.JSONDecodeError, TypeError):
                self._records = {}

    def _save(self) -> None:
        tmp = self.index_path.with_suffix(".tmp")
        tmp.write_text(json.dumps([asdict(r) for r in self._records.values()]))
        os.replace(tmp, self.index_path)

    def register(self, path: str, task_id: str, task: str, media_type: str, meta: dict | None = None,
                 artifact_id: str | None = None) -> ArtifactRecord:  # fmt: skip
        size = os.path.getsize(path) if os.path.isfile(path) else 0
        rec = ArtifactRecord(artifact_id or task_id or uuid.uuid4().hex, str(path), task_id, task, media_type, time.time(),
                             size, meta)  # fmt: skip
        with self._lock:
            self._records[rec.artifact_id] = rec
            self.enforce_retention()
            self._save()
        return rec

    def get(self, artifact_id: str) -> ArtifactRecord | None:
        with self._lock:
            return self._records.get(artifact_id)

    def list(self, media_type: str | None = None, limit: int = 100) -> list[ArtifactRecord]:
        with self._lock:
            recs = sorted(self._records.values(), key=lambda r: -r.created)
        return [r for r in recs if media_type is None or r.media_type == media_type][:limit]

    def delete(self, artifact_id: str) -> bool:
        with self._lock:
            rec = self._records.pop(artifact_id, None)
            if rec is None:
                return False
            Path(rec.path).unlink(missing_ok=True)
            self._save()
            return True

    def total_bytes(self) -> int:
        with self._lock:
            return sum(r.size for r in self._records.values())

    def enforce_retention(self, now: float | None = None) -> list[str]:
        """Drops artefacts older than the retention window, then the oldest until under the size cap."""
        now = time.time() if now is None else now
        removed = []
        with self._lock:
            for aid, rec in list(self._records.items()):
                if now - rec.created > self.retention_s:
                    removed.append(aid)
            total = sum(r.size for a, r in self._records.items() if a not in removed)
            for rec in sorted(self._records.values(), key=lambda r: r.created):
                if total <= self.max_bytes:
                    break
                if rec.artifact_id not in removed:
                    removed.append(rec.artifact_id)
                    total -= rec.size
            for aid in removed:
                rec = self._records.pop(aid)
                Path(rec.path).unlink(missing_ok=True)
            if removed:
                self._save()
        return removed
