"""Checkpoint I/O and identification.

* `load_state_dict(path)`: single safetensors / sharded `*.index.json` / `.bin` / `.pth` /
  a folder of shards / a list of files.
* `init_weights_on_device`: build a module without materialising weights (meta device).
* `hash_state_dict_keys`: MD5 over the sorted `key` and `key:shape` strings. The exact
  string format is part of the checkpoint-detection contract shared with the reference
  (telefuser/utils/model_weight.py:145-163), so hashes computed here equal the ones the
  published Wan checkpoints are registered under.
"""

from __future__ import annotations

import contextlib
import glob
import hashlib
import json
import os
import threading
from typing import Any

import torch


_CONSTRUCTION_LOCK = threading.RLock()
_INIT_FUNCTIONS = ("uniform_", "normal_", "trunc_normal_", "constant_", "ones_", "zeros_", "eye_", "dirac_", "xavier_uniform_",
                   "xavier_normal_", "kaiming_uniform_", "kaiming_normal_", "orthogonal_", "sparse_")  # fmt: skip


@contextlib.contextmanager
def init_weights_on_device(device: torch.device | str = "meta", include_buffers: bool = False):
    """Modules constructed inside get their PARAMETERS on `device` (the meta device: no storage, to be adopted from a
    checkpoint with `load_state_dict(assign=True)`), while everything else a constructor computes stays real: buffers
    (unless `include_buffers`), and plain tensor attributes such as normalisation constants or frequency tables, which
    no checkpoint restores. A blanket `torch.device("meta")` context would turn those into meta tensors as well.
    Weight initialisers are skipped while the context is open (their results would be thrown away), so the short-lived
    host allocation of a large layer is never written to and costs no time."""
    from torch import nn

    dev = torch.device(device)

    def parameter_on_device(module, name, param):
        register_parameter(module, name, param)
        if param is not None and param.device != dev:
            cls, extra = type(param), dict(param.__dict__)
            moved = cls(param.data.to(dev), requires_grad=param.requires_grad)
            moved.__dict__.update(extra)
            module._parameters[name] = moved

    def buffer_on_device(module, name, tensor, persistent=True):
        register_buffer(module, name, tensor, persistent=persistent)
        if tensor is not None and tensor.device != dev:
            module._buffers[name] = tensor.to(dev)

    # The hooks below are process-wide while the context is open, so loaders in different threads take turns; a module
    # that some other thread constructs in the meantime would get meta parameters too: construct models under this
    # context (or not at all) while one is open.
    with _CONSTRUCTION_LOCK:
        register_parameter, register_buffer = nn.Module.register_parameter, nn.Module.register_buffer
        saved = {n: getattr(nn.init, n) for n in _INIT_FUNCTIONS if hasattr(nn.init, n)}
        nn.Module.register_parameter = parameter_on_device
        if include_buffers:
            nn.Module.register_buffer = buffer_on_device
        for n in saved:
            setattr(nn.init, n, lambda tensor, *a, **k: tensor)
        try:
            yield
        finally:
            nn.Module.register_parameter, nn.Module.register_buffer = register_parameter, register_buffer
            for n, fn in saved.items():
                setattr(nn.init, n, fn)


def _load_one(path: str, device: str = "cpu") -> dict[str, torch.Tensor]:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        return load_file(path, device=device)
    sd = torch.load(path, map_location=device, weights_only=True)
    for key in ("state_dict", "module", "model"):
        if isinstance(sd, dict) and key in sd and isinstance(sd[key], dict):
            sd = sd[key]
    return sd


def expand_checkpoint_paths(path: str | list[str]) -> list[str]:
    """Resolves a path / wildcard / folder / index file / list into concrete weight files."""
    if isinstance(path, (list, tuple)):
        out: list[str] = []
        for p in path:
            out.extend(expand_checkpoint_paths(p))
        return out
    if any(ch in path for ch in "*?["):
        return sorted(glob.glob(path))
    if os.path.isdir(path):
        idx = sorted(glob.glob(os.path.join(path, "*.index.json")))
        if idx:
            return expand_checkpoint_paths(idx[0])
        files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
        return files or sorted(glob.glob(os.path.join(path, "*.bin")) + glob.glob(os.path.join(path, "*.pth")))
    if path.endswith(".index.json"):
        with open(path) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(os.path.dirname(path), s) for s in shards]
    return [path]


def load_state_dict(path: str | list[str], device: str = "cpu", torch_dtype: torch.dtype | None = None) -> dict:
    sd: dict[str, torch.Tensor] = {}
    files = expand_checkpoint_paths(path)
    if not files:
        raise FileNotFoundError(f"no weight files found for {path}")
    for f in files:
        sd.update(_load_one(f, device))
    if torch_dtype is not None:
        sd = {k: (v.to(torch_dtype) if isinstance(v, torch.Tensor) and v.is_floating_point() else v)
              for k, v in sd.items()}  # fmt: skip
    return sd


def state_dict_keys_string(state_dict: dict[str, Any], with_shape: bool = True) -> str:
    parts = []
    for key, value in state_dict.items():
        if isinstance(key, str):
            if isinstance(value, torch.Tensor) and with_shape:
                parts.append(f"{key}:{'_'.join(map(str, value.shape))}")
            parts.append(key)
        elif isinstance(value, dict):
            parts.append(f"{key}|{state_dict_keys_string(value, with_shape)}")
    parts.sort()
    return ",".join(parts)


def hash_state_dict_keys(state_dict: dict[str, Any], with_shape: bool = True) -> str:
    return hashlib.md5(state_dict_keys_string(state_dict, with_shape).encode("utf-8")).hexdigest()


def save_state_dict(state_dict: dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    from safetensors.torch import save_file

    # safetensors refuses aliased storage (fused projection views): store independent copies
    save_file({k: v.detach().clone().contiguous() for k, v in state_dict.items()}, path, metadata=metadata)
