"""Server assembly and entry functions.

`ServiceContainer` wires configuration -> pipeline service (one in-process pipeline) or pipeline pool
(data-parallel replicas) or stream service -> `ApiServer`; `run_server` / `run_stream_server` start
uvicorn and clean up on exit.
Role parity: telefuser/service/main.py:17-121, core/container.py.
"""

from __future__ import annotations

import asyncio
import sys
from pathlib import Path

from telefuser_b200.utils.logging import logger

from .api import ApiServer
from .pipeline_service import PipelinePool, PipelineService, ServerConfig
from .stream_service import StreamPipelineService


class ServiceContainer:
    def __init__(self, config: ServerConfig | None = None) -> None:
        self.config = config or ServerConfig()
        self.inference_service = None
        self.stream_service: StreamPipelineService | None = None
        self.api: ApiServer | None = None
        self.num_workers = 1

    def initialize_all(self, pipe_path: str, parallelism: int = 1, task: str | None = None,
                       skip_validation: bool = False) -> bool:  # fmt: skip
        cfg = self.config
        if cfg.num_replicas > 1:
            pool = PipelinePool(cfg)
            pool.start_all(pipe_path, task, parallelism, cfg.num_replicas, skip_validation=skip_validation)
            self.inference_service, self.num_workers = pool, len(pool.replicas)
        else:
            svc = PipelineService(cfg)
            svc.start_pipeline(pipe_path, task, parallelism, skip_validation)
            self.inference_service = svc
            self.num_workers = max(1, svc.contract.effective_max_concurrent_tasks if svc.contract else 1)
        return True

    def initialize_stream_service(self, pipe_path: str, gpu_num: int = 1, skip_validation: bool = False) -> bool:
        self.stream_service = StreamPipelineService(self.config)
        return self.stream_service.start_service(pipe_path, skip_validation, gpu_num)

    def get_api_app(self, enable_rate_limit: bool | None = None):
        if enable_rate_limit is not None:
            self.config.rate_limit_enabled = enable_rate_limit
        self.api = ApiServer(self.config, self.inference_service, self.stream_service, self.num_workers)
        if isinstance(self.inference_service, PipelinePool):
            self.inference_service.task_manager = self.api.task_manager
        return self.api.app

    async def cleanup(self) -> None:
        if self.inference_service is not None:
            await asyncio.to_thread(self.inference_service.stop)
        if self.stream_service is not None:
            await self.stream_service.aclose()


def _run(label: str, container: ServiceContainer, enable_rate_limit: bool) -> None:
    import uvicorn

    cfg = container.config
    try:
        app = container.get_api_app(enable_rate_limit)
        logger.info(f"starting {label} on {cfg.host}:{cfg.port}")
        uvicorn.run(app, host=cfg.host, port=cfg.port, log_level="warning")
    except KeyboardInterrupt:
        logger.info(f"{label} interrupted")
    except Exception as e:  # noqa: BLE001
        logger.error(f"{label} failed: {e}")
        sys.exit(1)
    finally:
        try:
            asyncio.run(container.cleanup())
        except Exception as e:  # noqa: BLE001
            logger.warning(f"cleanup error: {e}")


def run_server(pipe_path: str, task: str | None, port: int, host: str, cache_dir: str = "", parallelism: int = 1,
               enable_rate_limit: bool = True, num_replicas: int = 1, enable_latent_cache: bool | None = None,
               cache_mode: str | None = None, security_level: str | None = None, skip_validation: bool = False) -> None:  # fmt: skip
    cfg = ServerConfig()
    cfg.host, cfg.port, cfg.num_replicas = host, port, num_replicas
    if cache_dir:
        cfg.cache_dir = str(Path(cache_dir))
    from .contract import resolve_latent_cache_settings

    cache = resolve_latent_cache_settings(pipe_path, enable_latent_cache, cache_mode)  # CLI > the file's CACHE_CONFIG > off
    cfg.enable_latent_cache, cfg.latent_cache_mode = cache["enabled"], cache["mode"]
    if cache["directory"]:
        cfg.latent_cache_dir = str(cache["directory"])
    if cache["min_similarity"] is not None:
        cfg.latent_cache_min_similarity = float(cache["min_similarity"])
    if cfg.enable_latent_cache:
        logger.info(f"latent cache on ({cache['mode']}, decided by the {cache['source']})")
    if security_level:
        cfg.security_level = security_level.lower()
    container = ServiceContainer(cfg)
    container.initialize_all(pipe_path, parallelism, task, skip_validation)
    _run("server", container, enable_rate_limit)


def run_stream_server(pipe_path: str, port: int, host: str, enable_rate_limit: bool = True, skip_validation: bool = False,
                      security_level: str | None = None, gpu_num: int = 1) -> None:  # fmt: skip
    cfg = ServerConfig()
    cfg.host, cfg.port = host, port
    if security_level:
        cfg.security_level = security_level.lower()
    container = ServiceContainer(cfg)
    container.initialize_stream_service(pipe_path, gpu_num, skip_validation)
    _run("stream server", container, enable_rate_limit)
