"""Small host utilities: free-port allocation for worker rendezvous, list splitting,
importing a callable from a file path (reference: telefuser/utils/system.py:10-228,
telefuser/utils/utils.py)."""

from __future__ import annotations

import importlib.util
import socket
import threading
from pathlib import Path


def find_free_port(host: str = "127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]


class PortAllocator:
    """Hands out distinct free ports (master ports of worker groups) within one process."""

    _lock = threading.Lock()
    _used: set[int] = set()

    @classmethod
    def allocate(cls, host: str = "127.0.0.1") -> int:
        with cls._lock:
            for _ in range(64):
                p = find_free_port(host)
                if p not in cls._used:
                    cls._used.add(p)
                    return p
        raise RuntimeError("no free port found")

    @classmethod
    def release(cls, port: int) -> None:
        with cls._lock:
            cls._used.discard(port)


def split_list(items: list, n: int) -> list[list]:
    """Splits `items` into `n` nearly equal contiguous parts."""
    k, r = divmod(len(items), n)
    out, i = [], 0
    for j in range(n):
        step = k + (1 if j < r else 0)
        out.append(items[i : i + step])
        i += step
    return out


def import_function_from_file(path: str | Path, name: str):
    path = Path(path)
    spec = importlib.util.spec_from_file_location(path.stem, path)
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot import {path}")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not hasattr(mod, name):
        raise AttributeError(f"{path} has no attribute {name}")
    return getattr(mod, name)
