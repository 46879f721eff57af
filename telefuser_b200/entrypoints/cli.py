"""Command line: `serve`, `stream-serve`, `validate`, `scan`.

Role parity: telefuser/entrypoints/cli/main.py (same commands and option names).
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import click

LEVELS = click.Choice(["none", "basic", "strict", "sandbox"], case_sensitive=False)


@click.group()
def main() -> None:
    """telefuser-b200: diffusion inference and serving on B200."""


def _print_validation(path: str, res: dict, as_json: bool) -> None:
    if as_json:
        click.echo(json.dumps({"file": path, **res}, indent=2))
        return
    click.echo(f"{path}: {'PASSED' if res['passed'] else 'FAILED'}")
    for v in res["violations"]:
        click.echo(f"  [{v['severity']}] {v['type']} line {v['line']}: {v['description']}  | {v['snippet']}")
    for w in res["warnings"]:
        click.echo(f"  [warning] {w['type']} line {w['line']}: {w['description']}")


def _validate(path: str, level: str) -> dict:
    from telefuser_b200.service.pipeline_service import PipelineService, ServerConfig

    return PipelineService(ServerConfig(security_level=level.lower())).validate_only(path)


@main.command()
@click.argument("pipe_path")
@click.option("--task", "-t", default="i2v", help="Task type (t2v, i2v, fl2v, vc, t2i, i2i, s2v, vsr)")
@click.option("--port", "-p", default=8000, type=int, help="Server port")
@click.option("--host", default="127.0.0.1", type=str, help="Server host")
@click.option("--cache-dir", default="work_dirs/server_cache", help="Cache directory for inputs and outputs")
@click.option("--parallelism", "--gpu-num", "-g", type=int, default=1, help="GPUs per pipeline replica")
@click.option("--num-replicas", default=1, type=int, help="Number of data-parallel pipeline replicas")
@click.option("--security-level", default="strict", type=LEVELS, help="Pipeline file validation level")
@click.option("--skip-validation", is_flag=True, default=False, help="Skip security validation")
@click.option("--validate-only", is_flag=True, default=False, help="Validate the pipeline file and exit")
@click.option("--enable-latent-cache/--disable-latent-cache", default=None, help="Latent cache on/off (default: the pipeline file's CACHE_CONFIG, else off)")
@click.option("--cache-mode", default=None, type=click.Choice(["read", "write", "readwrite", "read_only", "write_only", "read_write"]),
              help="Latent cache mode (default: the pipeline file's CACHE_CONFIG, else readwrite)")
@click.option("--rate-limit/--no-rate-limit", default=True, help="Sliding-window rate limit")
def serve(pipe_path, task, port, host, cache_dir, parallelism, num_replicas, security_level, skip_validation,
          validate_only, enable_latent_cache, cache_mode, rate_limit) -> None:  # fmt: skip
    """Serve a request/response pipeline file over HTTP."""
    if validate_only:
        res = _validate(pipe_path, security_level)
        _print_validation(pipe_path, res, False)
        sys.exit(0 if res["passed"] else 1)
    from telefuser_b200.service.main import run_server

    run_server(pipe_path, task, port, host, cache_dir, parallelism, rate_limit, num_replicas, enable_latent_cache,
               cache_mode, security_level, skip_validation)  # fmt: skip


@main.command(name="stream-serve")
@click.argument("pipe_path")
@click.option("--port", "-p", default=8088, type=int, help="Server port")
@click.option("--host", default="0.0.0.0", type=str, help="Server host")
@click.option("--gpu-num", "-g", default=1, type=int, help="GPUs for the streaming service")
@click.option("--security-level", default="strict", type=LEVELS, help="Pipeline file validation level")
@click.option("--skip-validation", is_flag=True, default=False, help="Skip security validation")
def stream_serve(pipe_path, port, host, gpu_num, security_level, skip_validation) -> None:
    """Serve a streaming pipeline file (`get_service`) over WebSocket / WebRTC."""
    from telefuser_b200.service.main import run_stream_server

    run_stream_server(pipe_path, port, host, True, skip_validation, security_level, gpu_num)


@main.command(name="validate")
@click.argument("pipeline_file", type=click.Path(exists=True))
@click.option("--level", default="strict", type=LEVELS, help="Validation level")
@click.option("--json", "as_json", is_flag=True, default=False, help="JSON output")
def validate(pipeline_file, level, as_json) -> None:
    """Run the security checks on one pipeline file."""
    res = _validate(pipeline_file, level)
    _print_validation(pipeline_file, res, as_json)
    sys.exit(0 if res["passed"] else 1)


@main.command(name="scan")
@click.argument("directory", type=click.Path(exists=True, file_okay=False))
@click.option("--level", default="strict", type=LEVELS, help="Validation level")
@click.option("--recursive/--no-recursive", default=True, help="Descend into sub-directories")
def scan(directory, level, recursive) -> None:
    """Run the security checks on every Python file of a directory."""
    files = sorted(Path(directory).rglob("*.py") if recursive else Path(directory).glob("*.py"))
    failed = 0
    for f in files:
        res = _validate(str(f), level)
        if not res["passed"]:
            failed += 1
            _print_validation(str(f), res, False)
    click.echo(f"scanned {len(files)} file(s): {len(files) - failed} passed, {failed} failed")
    sys.exit(0 if failed == 0 else 1)


if __name__ == "__main__":
    main()
