"""Dataclass / enum / torch dtype -> JSON-friendly structures (reference: telefuser/core/config_serializer.py:15-54)."""

from __future__ import annotations

import dataclasses
from enum import Enum
from typing import Any

import torch


def to_jsonable(obj: Any) -> Any:
    if obj is None or isinstance(obj, (bool, int, float, str)):
        return obj
    if isinstance(obj, Enum):
        return obj.name
    if isinstance(obj, (torch.dtype, torch.device)):
        return str(obj)
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: to_jsonable(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if isinstance(obj, dict):
        return {str(k): to_jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set, frozenset)):
        return [to_jsonable(v) for v in obj]
    if isinstance(obj, torch.Tensor):
        return {"tensor": list(obj.shape), "dtype": str(obj.dtype)}
    return repr(obj)


def serialize_config(obj: Any) -> dict:
    return to_jsonable(obj)
