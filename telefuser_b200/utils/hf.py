"""Hugging Face helpers: id-vs-path test, snapshot resolution, task detection of a model folder. Component discovery
is in `hf_model_analyzer`. Role parity: telefuser/utils/hf_model_utils.py:21-209."""

from __future__ import annotations

import json
import os
import re


def is_hf_model_id(s: str) -> bool:
    return not os.path.exists(s) and re.fullmatch(r"[\w.\-]+/[\w.\-]+", s) is not None


def resolve_hf_path(model_id_or_path: str, cache_dir: str | None = None) -> str:
    """Local path as is; a hub id is resolved from the local cache (or downloaded when a network exists)."""
    if os.path.exists(model_id_or_path):
        return model_id_or_path
    zoo = os.environ.get("TF_MODEL_ZOO_PATH")
    if zoo and os.path.exists(os.path.join(zoo, model_id_or_path)):
        return os.path.join(zoo, model_id_or_path)
    if is_hf_model_id(model_id_or_path):
        from huggingface_hub import snapshot_download

        return snapshot_download(model_id_or_path, cache_dir=cache_dir)
    raise FileNotFoundError(model_id_or_path)


def get_component_path(root: str, component: str) -> str | None:
    p = os.path.join(root, component)
    return p if os.path.isdir(p) else None


def detect_model_task(root: str) -> str:
    """'i2v' when the folder's config names an image-conditioned model, else 't2v' ('t2i' for image models)."""
    for name in ("config.json", "model_index.json", os.path.join("transformer", "config.json")):
        f = os.path.join(root, name)
        if os.path.isfile(f):
            try:
                cfg = json.load(open(f))
            except (OSError, ValueError):
                continue
            blob = json.dumps(cfg).lower()
            if "i2v" in blob or cfg.get("model_type") == "i2v" or cfg.get("in_dim") == 36:
                return "i2v"
            if "image" in str(cfg.get("_class_name", "")).lower() and "video" not in blob:
                return "t2i"
    return "i2v" if "i2v" in os.path.basename(root).lower() else "t2v"


def __getattr__(name: str):
    # `HFModelAnalyzer` lives in `hf_model_analyzer` (which imports this module for the task detection).
    if name in ("HFModelAnalyzer", "ModelComponentInfo", "discover_model_components"):
        from . import hf_model_analyzer

        return getattr(hf_model_analyzer, name)
    raise AttributeError(name)
