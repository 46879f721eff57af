"""Client of the OpenAI-style routes: `client.images.generate / edit`, `client.videos.create /
retrieve / list / delete`, with `Video.wait()` / `Video.download()` helpers.

Role parity: telefuser/client/openai/{client,images,videos}.py.
"""

from __future__ import annotations

import base64
import os
import time
from pathlib import Path

import requests


class OpenAIClientError(Exception):
    def __init__(self, status: int, message: str) -> None:
        super().__init__(f"HTTP {status}: {message}")
        self.status = status


class Image:
    def __init__(self, data: dict, client: "OpenAICompatibleClient") -> None:
        self.url, self.b64_json = data.get("url"), data.get("b64_json")
        self.revised_prompt, self.file_path = data.get("revised_prompt"), data.get("file_path")
        self.artifact_id = data.get("artifact_id")
        self._client = client

    def bytes(self) -> bytes:
        if self.b64_json:
            return base64.b64decode(self.b64_json)
        if self.url:
            return self._client.fetch(self.url)
        raise ValueError("image has neither url nor b64_json")

    def save(self, path: str | Path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_bytes(self.bytes())


class ImagesResponse:
    def __init__(self, data: dict, client: "OpenAICompatibleClient") -> None:
        self.created = data.get("created")
        self.data = [Image(d, client) for d in data.get("data", [])]
        self.peak_memory_mb, self.inference_time_s = data.get("peak_memory_mb"), data.get("inference_time_s")

    def __getitem__(self, i: int) -> Image:
        return self.data[i]

    def __len__(self) -> int:
        return len(self.data)


class ImagesAPI:
    def __init__(self, client: "OpenAICompatibleClient") -> None:
        self._c = client

    def generate(self, prompt: str, *, model: str | None = None, n: int = 1, size: str = "1024x1024",
                 response_format: str = "url", seed: int | None = 42, negative_prompt: str | None = None,
                 **extra) -> ImagesResponse:  # fmt: skip
        body = {"prompt": prompt, "model": model, "n": n, "size": size, "response_format": response_format, "seed": seed,
                "negative_prompt": negative_prompt, **extra}  # fmt: skip
        return ImagesResponse(self._c.post("/v1/images/generations", json=_drop_none(body)), self._c)

    def edit(self, prompt: str, image: str, *, mask: str | None = None, model: str | None = None, n: int = 1,
             size: str = "1024x1024", response_format: str = "url", seed: int | None = 42, **extra) -> ImagesResponse:  # fmt: skip
        body = {"prompt": prompt, "model": model, "n": n, "size": size, "response_format": response_format, "seed": seed, **extra}
        if image.startswith(("http://", "https://")):
            body["image_url"] = image
        else:
            body["image"] = _b64_if_file(image)
        if mask:
            body["mask"] = _b64_if_file(mask)
        return ImagesResponse(self._c.post("/v1/images/edits", json=_drop_none(body)), self._c)


class Video:
    def __init__(self, data: dict, client: "OpenAICompatibleClient") -> None:
        self._client = client
        self._update(data)

    def _update(self, data: dict) -> None:
        self.raw = data
        for k in ("id", "status", "progress", "url", "error", "size", "seconds", "file_path", "model", "created_at",
                  "completed_at", "peak_memory_mb", "inference_time_s"):  # fmt: skip
            setattr(self, k, data.get(k))

    @property
    def is_done(self) -> bool:
        return self.status in ("completed", "failed", "cancelled", "deleted")

    @property
    def is_success(self) -> bool:
        return self.status == "completed"

    def refresh(self) -> "Video":
        self._update(self._client.get(f"/v1/videos/{self.id}"))
        return self

    def wait(self, poll_interval: float = 1.0, timeout: float = 3600.0) -> "Video":
        deadline = time.monotonic() + timeout
        while not self.refresh().is_done:
            if time.monotonic() > deadline:
                raise TimeoutError(f"video {self.id} still {self.status}")
            time.sleep(poll_interval)
        return self

    def download(self, path: str | Path | None = None) -> bytes:
        data = self._client.fetch(f"{self._client.base_url}/v1/videos/{self.id}/content")
        if path is not None:
            Path(path).parent.mkdir(parents=True, exist_ok=True)
            Path(path).write_bytes(data)
        return data

    def cancel(self) -> bool:
        self._update(self._client.delete(f"/v1/videos/{self.id}"))
        return self.status == "deleted"


class VideosList:
    def __init__(self, data: dict, client: "OpenAICompatibleClient") -> None:
        self.data = [Video(d, client) for d in data.get("data", [])]
        self.has_more, self.first_id, self.last_id = data.get("has_more"), data.get("first_id"), data.get("last_id")

    def __getitem__(self, i: int) -> Video:
        return self.data[i]

    def __len__(self) -> int:
        return len(self.data)


class VideosAPI:
    def __init__(self, client: "OpenAICompatibleClient") -> None:
        self._c = client

    def create(self, prompt: str, *, input_reference: str | None = None, model: str | None = None, seconds: int = 4,
               size: str = "", seed: int | None = 1024, negative_prompt: str | None = None, **extra) -> Video:  # fmt: skip
        body = {"prompt": prompt, "model": model, "seconds": seconds, "size": size, "seed": seed,
                "negative_prompt": negative_prompt, **extra}  # fmt: skip
        if input_reference:
            if input_reference.startswith(("http://", "https://")):
                body["reference_url"] = input_reference
            else:
                body["input_reference"] = _b64_if_file(input_reference)
        return Video(self._c.post("/v1/videos", json=_drop_none(body)), self._c)

    def retrieve(self, video_id: str) -> Video:
        return Video(self._c.get(f"/v1/videos/{video_id}"), self._c)

    def list(self, limit: int = 20, order: str = "desc") -> VideosList:
        return VideosList(self._c.get("/v1/videos", params={"limit": limit, "order": order}), self._c)

    def delete(self, video_id: str) -> Video:
        return Video(self._c.delete(f"/v1/videos/{video_id}"), self._c)


class OpenAICompatibleClient:
    def __init__(self, base_url: str = "http://localhost:8000", api_key: str | None = None, timeout: float = 600.0,
                 session=None) -> None:  # fmt: skip
        self.base_url, self.timeout = base_url.rstrip("/"), timeout
        self.session = session or requests.Session()
        if api_key:
            self.session.headers["Authorization"] = f"Bearer {api_key}"
        self.images, self.videos = ImagesAPI(self), VideosAPI(self)

    def _request(self, method: str, path: str, **kw) -> dict:
        r = self.session.request(method, f"{self.base_url}{path}", timeout=self.timeout, **kw)
        if r.status_code >= 400:
            try:
                msg = r.json().get("detail", r.text)
            except ValueError:
                msg = r.text
            raise OpenAIClientError(r.status_code, str(msg))
        return r.json()

    def get(self, path: str, **kw) -> dict:
        return self._request("GET", path, **kw)

    def post(self, path: str, **kw) -> dict:
        return self._request("POST", path, **kw)

    def delete(self, path: str, **kw) -> dict:
        return self._request("DELETE", path, **kw)

    def fetch(self, url: str) -> bytes:
        if url.startswith("/"):
            url = self.base_url + url
        r = self.session.get(url, timeout=self.timeout)
        if r.status_code >= 400:
            raise OpenAIClientError(r.status_code, r.text)
        return r.content

    def close(self) -> None:
        self.session.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def _drop_none(d: dict) -> dict:
    return {k: v for k, v in d.items() if v is not None}


def _b64_if_file(path: str) -> str:
    if os.path.isfile(path):
        return base64.b64encode(Path(path).read_bytes()).decode()
    return path
