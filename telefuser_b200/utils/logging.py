"""Logging: one loguru logger configured from `TELEFUSER_LOG_*` environment variables.

Records carry rank and pid; a trace id / span id pair lives in context variables so that a
request can be followed across stages; worker ranks can log to per-rank files; decorators
`log_execution_time` and `log_exceptions` wrap sync and async callables.
Environment (same names as the reference, telefuser/utils/logging.py:219-268):
LEVEL, FORMAT (console|detailed|json), SINK (stderr|stdout|file), FILE, ROTATION, RETENTION,
COMPRESSION, ENQUEUE, BACKTRACE, DIAGNOSE, SERIALIZE, MULTIPROCESS, EXTRA_FIELDS, FILTER_MODULES.
"""

from __future__ import annotations

import contextvars
import functools
import inspect
import os
import sys
import time
import uuid
from dataclasses import dataclass, field

from loguru import logger as _logger

_trace_id: contextvars.ContextVar[str | None] = contextvars.ContextVar("tfb_trace_id", default=None)
_span_id: contextvars.ContextVar[str | None] = contextvars.ContextVar("tfb_span_id", default=None)


def _env(name: str, default: str) -> str:
    return os.environ.get(f"TELEFUSER_LOG_{name}", default)


def _env_bool(name: str, default: bool) -> bool:
    return _env(name, str(default)).lower() in ("1", "true", "yes", "on")


@dataclass
class LogConfig:
    level: str = "INFO"
    format: str = "console"
    sink: str = "stderr"
    file: str | None = None
    rotation: str | None = "100 MB"
    retention: str | None = "7 days"
    compression: str | None = None
    enqueue: bool = False
    backtrace: bool = False
    diagnose: bool = False
    serialize: bool = False
    multiprocess: bool = False
    extra_fields: dict = field(default_factory=dict)
    filter_modules: tuple = ()

    @classmethod
    def from_env(cls) -> "LogConfig":
        extra = {}
        for item in _env("EXTRA_FIELDS", "").split(","):
            if "=" in item:
                k, v = item.split("=", 1)
                extra[k.strip()] = v.strip()
        return cls(
            level=_env("LEVEL", "INFO").upper(), format=_env("FORMAT", "console"), sink=_env("SINK", "stderr"),
            file=os.environ.get("TELEFUSER_LOG_FILE"), rotation=_env("ROTATION", "100 MB") or None,
            retention=_env("RETENTION", "7 days") or None, compression=os.environ.get("TELEFUSER_LOG_COMPRESSION"),
            enqueue=_env_bool("ENQUEUE", False), backtrace=_env_bool("BACKTRACE", False),
            diagnose=_env_bool("DIAGNOSE", False), serialize=_env_bool("SERIALIZE", False),
            multiprocess=_env_bool("MULTIPROCESS", False), extra_fields=extra,
            filter_modules=tuple(m.strip() for m in _env("FILTER_MODULES", "").split(",") if m.strip()),
        )  # fmt: skip


FORMATS = {
    "console": "<green>{time:HH:mm:ss.SSS}</green> <level>{level: <7}</level> r{extra[rank]} {message}",
    "detailed": ("{time:YYYY-MM-DD HH:mm:ss.SSS} {level: <7} pid={extra[pid]} rank={extra[rank]} "
                 "trace={extra[trace_id]} span={extra[span_id]} {name}:{function}:{line} {message}"),  # fmt: skip
}


def _patch(record) -> None:
    extra = record["extra"]
    extra.setdefault("rank", int(os.environ.get("RANK", "0")))
    extra.setdefault("pid", os.getpid())
    extra["trace_id"] = _trace_id.get() or "-"
    extra["span_id"] = _span_id.get() or "-"


def setup_logging(config: LogConfig | None = None):
    cfg = config or LogConfig.from_env()
    _logger.remove()
    fmt = FORMATS.get(cfg.format, FORMATS["console"])
    flt = None
    if cfg.filter_modules:
        flt = lambda rec: not any(rec["name"].startswith(m) for m in cfg.filter_modules)  # noqa: E731
    common = dict(level=cfg.level, backtrace=cfg.backtrace, diagnose=cfg.diagnose, enqueue=cfg.enqueue, filter=flt,
                  serialize=cfg.serialize or cfg.format == "json")  # fmt: skip
    if cfg.sink == "file" and cfg.file:
        path = cfg.file
        if cfg.multiprocess:
            root, ext = os.path.splitext(path)
            path = f"{root}.rank{os.environ.get('RANK', '0')}{ext}"
        _logger.add(path, format=fmt, rotation=cfg.rotation, retention=cfg.retention, compression=cfg.compression,
                    **common)  # fmt: skip
    else:
        _logger.add(sys.stdout if cfg.sink == "stdout" else sys.stderr, format=fmt, **common)
    lg = _logger.patch(_patch)
    if cfg.extra_fields:
        lg = lg.bind(**cfg.extra_fields)
    return lg


logger = setup_logging()


def new_trace(trace_id: str | None = None) -> str:
    tid = trace_id or uuid.uuid4().hex[:16]
    _trace_id.set(tid)
    _span_id.set(None)
    return tid


def get_trace_id() -> str | None:
    return _trace_id.get()


class span:
    """`with span("vae"):` sets a span id for the records emitted inside and logs the duration at DEBUG."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self._token = _span_id.set(f"{self.name}-{uuid.uuid4().hex[:6]}")
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        logger.debug(f"span {self.name} took {(time.perf_counter() - self._t0) * 1e3:.1f} ms")
        _span_id.reset(self._token)
        return False


def log_execution_time(name: str | None = None, level: str = "INFO"):
    def deco(fn):
        label = name or fn.__qualname__
        if inspect.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def aw(*a, **k):
                t0 = time.perf_counter()
                try:
                    return await fn(*a, **k)
                finally:
                    logger.log(level, f"{label} took {(time.perf_counter() - t0) * 1e3:.1f} ms")

            return aw

        @functools.wraps(fn)
        def w(*a, **k):
            t0 = time.perf_counter()
            try:
                return fn(*a, **k)
            finally:
                logger.log(level, f"{label} took {(time.perf_counter() - t0) * 1e3:.1f} ms")

        return w

    return deco


def log_exceptions(reraise: bool = True):
    def deco(fn):
        if inspect.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def aw(*a, **k):
                try:
                    return await fn(*a, **k)
                except Exception:
                    logger.exception(f"{fn.__qualname__} failed")
                    if reraise:
                        raise

            return aw

        @functools.wraps(fn)
        def w(*a, **k):
            try:
                return fn(*a, **k)
            except Exception:
                logger.exception(f"{fn.__qualname__} failed")
                if reraise:
                    raise

        return w

    return deco
