"""OpenAI-style image and video routes on top of the task queue.

`POST /v1/images/generations`, `POST /v1/images/edits` (synchronous: wait for the task, answer with a
URL or base64), `GET /v1/images/{id}/content`; `POST /v1/videos` (asynchronous job object),
`GET /v1/videos`, `GET /v1/videos/{id}`, `DELETE /v1/videos/{id}`, `GET /v1/videos/{id}/content`.
The adapter maps `size` / `seconds` onto the task request (resolution name + aspect ratio + length).
Role parity: telefuser/service/api/openai/{protocol,adapter,image_routes,video_routes}.py.
"""

from __future__ import annotations

import time
import uuid
from pathlib import Path
from typing import Any, Literal

from fastapi import APIRouter, HTTPException, Request
from fastapi.responses import FileResponse
from pydantic import BaseModel, Field

from .task_manager import TaskStatus

_RES_BY_SHORT_SIDE = ((480, "480p"), (720, "720p"), (1080, "1080p"))
_RATIOS = {"16:9": 16 / 9, "9:16": 9 / 16, "4:3": 4 / 3, "3:4": 3 / 4, "1:1": 1.0, "2:3": 2 / 3, "3:2": 3 / 2}


class ImageGenerationsRequest(BaseModel):
    prompt: str
    model: str | None = None
    n: int | None = Field(1, ge=1, le=10)
    quality: Literal["standard", "hd", "auto"] | None = None
    response_format: Literal["url", "b64_json"] | None = "url"
    size: str | None = "1024x1024"
    style: Literal["vivid", "natural"] | None = None
    user: str | None = None
    seed: int | None = Field(42, ge=0)
    negative_prompt: str | None = None


class ImageEditRequest(BaseModel):
    prompt: str
    image: str | None = None
    image_url: str | None = None
    mask: str | None = None
    model: str | None = None
    n: int | None = Field(1, ge=1, le=10)
    size: str | None = "1024x1024"
    response_format: Literal["url", "b64_json"] | None = "url"
    user: str | None = None
    seed: int | None = Field(42, ge=0)
    negative_prompt: str | None = None


class ImageResponseData(BaseModel):
    b64_json: str | None = None
    url: str | None = None
    revised_prompt: str | None = None
    file_path: str | None = None
    artifact_id: str | None = None
    artifact_metadata: dict[str, Any] | None = None


class ImageResponse(BaseModel):
    created: int = Field(default_factory=lambda: int(time.time()))
    data: list[ImageResponseData]
    peak_memory_mb: float | None = None
    inference_time_s: float | None = None


class VideoGenerationsRequest(BaseModel):
    prompt: str
    input_reference: str | None = None
    reference_url: str | None = None
    model: str | None = None
    seconds: int | None = Field(4, ge=1, le=60)
    size: str | None = ""
    seed: int | None = Field(1024, ge=0)
    negative_prompt: str | None = None
    output_path: str | None = None


class VideoResponse(BaseModel):
    id: str
    object: Literal["video"] = "video"
    model: str = "telefuser"
    status: Literal["queued", "generating", "completed", "failed", "cancelled", "deleted"] = "queued"
    progress: int = Field(0, ge=0, le=100)
    created_at: int = Field(default_factory=lambda: int(time.time()))
    size: str = ""
    seconds: str = "4"
    quality: str = "standard"
    url: str | None = None
    completed_at: int | None = None
    error: dict[str, Any] | None = None
    file_path: str | None = None
    artifact_id: str | None = None
    artifact_metadata: dict[str, Any] | None = None
    peak_memory_mb: float | None = None
    inference_time_s: float | None = None


class VideoListResponse(BaseModel):
    data: list[VideoResponse]
    object: Literal["list"] = "list"
    has_more: bool | None = False
    first_id: str | None = None
    last_id: str | None = None


def parse_size(size: str | None) -> dict:
    """'1280x720' -> width/height/resolution/aspect_ratio; '720p' -> resolution only."""
    if not size:
        return {}
    s = size.lower().strip()
    if "x" in s:
        try:
            w, h = (int(v) for v in s.split("x", 1))
        except ValueError as e:
            raise HTTPException(400, f"invalid size {size!r}") from e
        if w <= 0 or h <= 0:
            raise HTTPException(400, f"invalid size {size!r}")
        short = min(w, h)
        res = min(_RES_BY_SHORT_SIDE, key=lambda t: abs(t[0] - short))[1]
        ratio = min(_RATIOS, key=lambda k: abs(_RATIOS[k] - w / h))
        return {"width": w, "height": h, "resolution": size if short > 1080 or short < 400 else res, "aspect_ratio": ratio,
                "size": f"{w}x{h}"}  # fmt: skip
    return {"resolution": s}


_STATUS = {TaskStatus.PENDING.value: "queued", TaskStatus.PROCESSING.value: "generating",
           TaskStatus.STREAMING.value: "generating", TaskStatus.COMPLETED.value: "completed",
           TaskStatus.FAILED.value: "failed", TaskStatus.CANCELLED.value: "cancelled"}  # fmt: skip


def build_openai_routers(api) -> list[APIRouter]:
    images = APIRouter(prefix="/v1/images", tags=["images"])
    videos = APIRouter(prefix="/v1/videos", tags=["videos"])
    video_jobs: dict[str, dict] = {}

    def artifact_facts(task_id: str, path: str | None, media_type: str) -> dict | None:
        """Where a finished output lives, for callers that fetch it from the store rather than through the URL."""
        if not path or not Path(path).is_file():
            return None
        p = Path(path).resolve()
        try:
            rel = str(p.relative_to(Path(api.config.cache_dir).resolve()))
        except ValueError:
            rel = p.name
        return {"backend": "local", "relative_path": rel, "task_id": task_id, "media_type": media_type, "filename": p.name,
                "size_bytes": p.stat().st_size}  # fmt: skip

    async def run_image(task: str, req, request: Request, extra: dict) -> ImageResponse:
        from .api import b64_file

        out, peak, secs = [], None, None
        for i in range(req.n or 1):
            payload = {"task_id": f"img_{uuid.uuid4().hex[:16]}", "task": task, "prompt": req.prompt,
                       "negative_prompt": req.negative_prompt or "", "seed": (req.seed or 0) + i, "output_format": "png",
                       **parse_size(req.size), **extra}  # fmt: skip
            payload["output_path"] = f"{payload['task_id']}.png"
            resp = api.submit(payload)
            st = await api.wait_for_completion(resp.task_id)
            if st["status"] != TaskStatus.COMPLETED.value:
                raise HTTPException(500, st.get("error") or f"image task {st['status']}")
            path = st["output_path"]
            peak, secs = st.get("peak_memory_mb"), st.get("inference_time_s")
            d = ImageResponseData(file_path=path, artifact_id=resp.task_id, revised_prompt=req.prompt,
                                  artifact_metadata=artifact_facts(resp.task_id, path, "image"))  # fmt: skip
            if req.response_format == "b64_json":
                d.b64_json = b64_file(path)
            else:
                d.url = f"{api.base_url(request)}/v1/images/{resp.task_id}/content"
            out.append(d)
        return ImageResponse(data=out, peak_memory_mb=peak, inference_time_s=secs)

    @images.post("/generations", response_model=ImageResponse)
    async def generations(req: ImageGenerationsRequest, request: Request) -> ImageResponse:
        return await run_image("t2i", req, request, {})

    @images.post("/edits", response_model=ImageResponse)
    async def edits(req: ImageEditRequest, request: Request) -> ImageResponse:
        src = req.image or req.image_url
        if not src:
            raise HTTPException(400, "image or image_url is required")
        extra = {"first_image_path": src}
        if req.mask:
            extra["mask_path"] = req.mask
        meta = api.inference_service.metadata() if api.inference_service is not None else {}
        task = "edit" if "edit" in (meta.get("supported_tasks") or ()) else "i2i"
        return await run_image(task, req, request, extra)

    def content(task_id: str):
        t = api.task_manager.get_task(task_id)
        path = t.output_path if t is not None else None
        if path is None:
            rec = api.artifacts.get(task_id)
            path = rec.path if rec else None
        if not path or not Path(path).is_file():
            raise HTTPException(404, "content not found")
        return FileResponse(path, filename=Path(path).name)

    @images.get("/{image_id}/content")
    async def image_content(image_id: str):
        return content(image_id)

    def video_view(vid: str, request: Request | None = None) -> VideoResponse:
        job = video_jobs.get(vid)
        if job is None:
            raise HTTPException(404, "video not found")
        if job.get("deleted"):
            return VideoResponse(id=vid, status="deleted", created_at=job["created_at"], size=job["size"], seconds=job["seconds"])
        st = api.task_manager.get_status(vid) or {}
        status = _STATUS.get(st.get("status", "pending"), "queued")
        v = VideoResponse(id=vid, status=status, created_at=job["created_at"], size=job["size"], seconds=job["seconds"],
                          model=job["model"], progress=100 if status == "completed" else 50 if status == "generating" else 0,
                          peak_memory_mb=st.get("peak_memory_mb"), inference_time_s=st.get("inference_time_s"))  # fmt: skip
        if status == "completed":
            v.file_path, v.artifact_id = st.get("output_path"), vid
            v.artifact_metadata = artifact_facts(vid, v.file_path, "video")
            v.url = f"{api.base_url(request)}/v1/videos/{vid}/content"
            v.completed_at = int(time.time())
        elif status == "failed":
            v.error = {"message": st.get("error"), "type": "generation_error"}
        return v

    @videos.post("", response_model=VideoResponse)
    async def create_video(req: VideoGenerationsRequest, request: Request) -> VideoResponse:
        vid = f"video_{uuid.uuid4().hex[:16]}"
        ref = req.input_reference or req.reference_url
        payload = {"task_id": vid, "task": "i2v" if ref else "t2v", "prompt": req.prompt,
                   "negative_prompt": req.negative_prompt or "", "seed": req.seed if req.seed is not None else 1024,
                   "target_video_length": req.seconds or 4, "output_path": req.output_path or f"{vid}.mp4",
                   **parse_size(req.size)}  # fmt: skip
        if ref:
            payload["first_image_path"] = ref
        api.submit(payload)
        video_jobs[vid] = {"created_at": int(time.time()), "size": payload.get("size", req.size or ""),
                           "seconds": str(req.seconds or 4), "model": req.model or "telefuser"}  # fmt: skip
        return video_view(vid, request)

    @videos.get("", response_model=VideoListResponse)
    async def list_videos(request: Request, limit: int = 20, order: str = "desc") -> VideoListResponse:
        ids = sorted(video_jobs, key=lambda k: video_jobs[k]["created_at"], reverse=order != "asc")
        page = [video_view(i, request) for i in ids[:limit]]
        return VideoListResponse(data=page, has_more=len(ids) > limit, first_id=page[0].id if page else None,
                                 last_id=page[-1].id if page else None)  # fmt: skip

    @videos.get("/{video_id}", response_model=VideoResponse)
    async def get_video(video_id: str, request: Request) -> VideoResponse:
        return video_view(video_id, request)

    @videos.delete("/{video_id}", response_model=VideoResponse)
    async def delete_video(video_id: str) -> VideoResponse:
        if video_id not in video_jobs:
            raise HTTPException(404, "video not found")
        api.cancel(video_id)
        api.artifacts.delete(video_id)
        video_jobs[video_id]["deleted"] = True
        return video_view(video_id)

    @videos.get("/{video_id}/content")
    async def video_content(video_id: str):
        if video_jobs.get(video_id, {}).get("deleted"):
            raise HTTPException(404, "video was deleted")
        return content(video_id)

    return [images, videos]
