"""HTTP client of the task API plus helpers for fan-out over several servers.

Role parity: telefuser/client/tf_client.py:136-1000 (TFClient, create_*_task helpers,
wait_for_completion, download_result, send_and_monitor_task, find_idle_server, process_tasks_async).
"""

from __future__ import annotations

import base64
import os
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Any

import requests


class TeleFuserError(Exception):
    pass


class TaskCreationError(TeleFuserError):
    pass


class TaskFailedError(TeleFuserError):
    pass


class TaskTimeoutError(TeleFuserError):
    pass


_TERMINAL = ("completed", "failed", "cancelled")


class TFClient:
    def __init__(self, base_url: str = "http://localhost:8000", timeout: int = 300, session=None) -> None:
        self.base_url = base_url.rstrip("/")
        self.timeout = timeout
        self.session = session or requests.Session()

    def close(self) -> None:
        self.session.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    # ---- inputs ----
    @staticmethod
    def file_to_base64(file_path: str) -> str:
        with open(file_path, "rb") as f:
            return base64.b64encode(f.read()).decode()

    def _encode_file_input(self, path: str) -> str:
        """URLs and base64 go through as they are; an existing local file is sent as base64."""
        if not path or path.startswith(("http://", "https://", "data:")):
            return path
        return self.file_to_base64(path) if os.path.isfile(path) else path

    def _url(self, path: str) -> str:
        return f"{self.base_url}{path}"

    def _json(self, method: str, path: str, **kw) -> Any:
        r = self.session.request(method, self._url(path), timeout=kw.pop("timeout", self.timeout), **kw)
        if r.status_code >= 400:
            try:
                detail = r.json().get("detail")
            except ValueError:
                detail = r.text
            raise TeleFuserError(f"{method} {path} -> {r.status_code}: {detail}")
        return r.json()

    # ---- tasks ----
    def create_task(self, task_type: str, **params: Any) -> dict:
        body = {"task": task_type, **{k: v for k, v in params.items() if v is not None}}
        for key in ("first_image_path", "last_image_path", "ref_video_path", "audio_path", "mask_path"):
            if body.get(key):
                body[key] = self._encode_file_input(body[key])
        try:
            return self._json("POST", "/v1/tasks/create", json=body)
        except TeleFuserError as e:
            raise TaskCreationError(str(e)) from e

    def create_t2v_task(self, prompt: str, **kw) -> dict:
        return self.create_task("t2v", prompt=prompt, **kw)

    def create_i2v_task(self, prompt: str, image_path: str, **kw) -> dict:
        return self.create_task("i2v", prompt=prompt, first_image_path=image_path, **kw)

    def create_fl2v_task(self, prompt: str, first_image_path: str, last_image_path: str, **kw) -> dict:
        return self.create_task("fl2v", prompt=prompt, first_image_path=first_image_path, last_image_path=last_image_path, **kw)

    def create_vc_task(self, video_path: str, prompt: str = "", **kw) -> dict:
        return self.create_task("vc", prompt=prompt, ref_video_path=video_path, **kw)

    def create_s2v_task(self, image_path: str, audio_path: str, prompt: str = "", **kw) -> dict:
        return self.create_task("s2v", prompt=prompt, first_image_path=image_path, audio_path=audio_path, **kw)

    def create_vsr_task(self, video_path: str, **kw) -> dict:
        return self.create_task("vsr", ref_video_path=video_path, **kw)

    def create_t2i_task(self, prompt: str, **kw) -> dict:
        return self.create_task("t2i", prompt=prompt, **kw)

    def create_i2i_task(self, prompt: str, image_path: str, **kw) -> dict:
        return self.create_task("i2i", prompt=prompt, first_image_path=image_path, **kw)

    def create_edit_task(self, prompt: str, image_path: str, mask_path: str | None = None, **kw) -> dict:
        return self.create_task("edit", prompt=prompt, first_image_path=image_path, mask_path=mask_path, **kw)

    def get_task_status(self, task_id: str) -> dict:
        return self._json("GET", f"/v1/tasks/{task_id}/status")

    def wait_for_completion(self, task_id: str, poll_interval: float = 1.0, timeout: float | None = None,
                            raise_on_failure: bool = True) -> dict:  # fmt: skip
        deadline = time.monotonic() + (timeout if timeout is not None else self.timeout)
        while True:
            st = self.get_task_status(task_id)
            if st["status"] in _TERMINAL:
                if st["status"] != "completed" and raise_on_failure:
                    raise TaskFailedError(f"task {task_id} {st['status']}: {st.get('error')}")
                return st
            if time.monotonic() > deadline:
                raise TaskTimeoutError(f"task {task_id} still {st['status']} after the timeout")
            time.sleep(poll_interval)

    def cancel_task(self, task_id: str) -> dict:
        return self._json("DELETE", f"/v1/tasks/{task_id}")

    def download_result(self, task_id: str, output_path: str) -> bool:
        r = self.session.get(self._url(f"/v1/tasks/{task_id}/result"), timeout=self.timeout, stream=True)
        if r.status_code != 200:
            return False
        os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
        with open(output_path, "wb") as f:
            for chunk in r.iter_content(1 << 20):
                f.write(chunk)
        return True

    # ---- service ----
    def health_check(self) -> bool:
        try:
            return self.session.get(self._url("/v1/service/health"), timeout=5).status_code == 200
        except requests.RequestException:
            return False

    def get_service_status(self) -> dict:
        return self._json("GET", "/v1/service/status")

    def get_service_metadata(self) -> dict:
        return self._json("GET", "/v1/service/metadata")

    def get_queue_status(self) -> dict:
        return self._json("GET", "/v1/tasks/queue/status")


def send_and_monitor_task(url: str, task_type: str, params: dict, output_path: str | None = None,
                          poll_interval: float = 1.0, timeout: float = 3600.0) -> dict:  # fmt: skip
    with TFClient(url, timeout=int(timeout)) as c:
        resp = c.create_task(task_type, **params)
        st = c.wait_for_completion(resp["task_id"], poll_interval, timeout, raise_on_failure=False)
        if st["status"] == "completed" and output_path:
            c.download_result(resp["task_id"], output_path)
        return st


def get_available_urls(urls: list[str]) -> list[str]:
    return [u for u in urls if TFClient(u, timeout=5).health_check()]


def find_idle_server(available_urls: list[str], poll_interval: float = 0.5, timeout: float = 600.0) -> str:
    """The first server with no active task; if all are busy, the one with the shortest queue after the wait."""
    deadline = time.monotonic() + timeout
    best = available_urls[0]
    while time.monotonic() < deadline:
        loads = []
        for u in available_urls:
            try:
                loads.append((TFClient(u, timeout=5).get_queue_status().get("active_count", 0), u))
            except (TeleFuserError, requests.RequestException):
                continue
        if loads:
            n, best = min(loads)
            if n == 0:
                return best
        time.sleep(poll_interval)
    return best


def process_tasks_async(tasks: list[dict], urls: list[str], max_workers: int | None = None) -> list[dict]:
    """Runs `tasks` ({"task_type", "params", "output_path"?}) over the reachable servers, one in flight each."""
    live = get_available_urls(urls)
    if not live:
        raise TeleFuserError("no server is reachable")

    def run(i_task):
        i, t = i_task
        url = live[i % len(live)]
        try:
            return send_and_monitor_task(url, t["task_type"], t.get("params", {}), t.get("output_path"))
        except TeleFuserError as e:
            return {"status": "failed", "error": str(e)}

    with ThreadPoolExecutor(max_workers or len(live)) as ex:
        return list(ex.map(run, enumerate(tasks)))
