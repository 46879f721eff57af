"""Registry mapping checkpoint fingerprints to model classes.

A fingerprint is the MD5 of a state dict's sorted key (+shape) strings
(`utils.model_weight.hash_state_dict_keys`). Model modules register entries at
import time; `ModelRegistry.autodiscover()` imports every module under
``telefuser_b200.models`` once so all registrations are present. Unlike a table of
literal hashes, entries here may be *derived*: `register_architecture` builds the
module on the meta device and fingerprints its own state dict, so a preset's hash
follows from its definition. Role parity: telefuser/core/model_registry.py:22-108.
"""

from __future__ import annotations

import importlib
import pkgutil
from dataclasses import dataclass
from typing import Callable

import torch
import torch.nn as nn

from telefuser_b200.utils.model_weight import hash_state_dict_keys


@dataclass
class RegistryEntry:
    keys_hash: str | None
    keys_hash_with_shape: str | None
    model_names: list[str]
    model_classes: list[type[nn.Module]]
    model_resource: str  # "official" | "diffusers" | "civitai"


class ModelRegistry:
    _instance: "ModelRegistry | None" = None

    def __init__(self) -> None:
        self._entries: list[RegistryEntry] = []
        self._discovered = False

    @classmethod
    def instance(cls) -> "ModelRegistry":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def register(self, keys_hash, keys_hash_with_shape, model_names, model_classes, model_resource) -> None:
        self._entries.append(RegistryEntry(keys_hash, keys_hash_with_shape, list(model_names), list(model_classes),
                                           model_resource))  # fmt: skip

    def autodiscover(self) -> None:
        if self._discovered:
            return
        self._discovered = True
        import telefuser_b200.models as models_pkg

        for info in pkgutil.iter_modules(models_pkg.__path__):
            if info.name.startswith("_"):
                continue
            try:
                importlib.import_module(f"telefuser_b200.models.{info.name}")
            except Exception as e:  # noqa: BLE001 - optional dependencies of a model family
                import warnings

                warnings.warn(f"model module {info.name} could not be imported: {e}", stacklevel=2)

    def get_configs(self) -> list[tuple]:
        self.autodiscover()
        return [(e.keys_hash, e.keys_hash_with_shape, e.model_names, e.model_classes, e.model_resource)
                for e in self._entries]  # fmt: skip

    def entries(self) -> list[RegistryEntry]:
        self.autodiscover()
        return list(self._entries)

    def match(self, state_dict: dict) -> RegistryEntry | None:
        self.autodiscover()
        with_shape = hash_state_dict_keys(state_dict, with_shape=True)
        for e in self._entries:
            if e.keys_hash_with_shape == with_shape:
                return e
        keys_only = hash_state_dict_keys(state_dict, with_shape=False)
        for e in self._entries:
            if e.keys_hash == keys_only:
                return e
        return None


def register_model_config(keys_hash, keys_hash_with_shape, model_names, model_classes, model_resource) -> None:
    ModelRegistry.instance().register(keys_hash, keys_hash_with_shape, model_names, model_classes, model_resource)


def register_architecture(name: str, model_class: type[nn.Module], build: Callable[[], nn.Module],
                          resource: str = "official", keys_only: bool = False) -> str:  # fmt: skip
    """Registers `model_class` under the fingerprint of the state dict that `build()` yields on the meta device."""
    with torch.device("meta"):
        sd = build().state_dict()
    h = hash_state_dict_keys(sd, with_shape=not keys_only)
    register_model_config(h if keys_only else None, None if keys_only else h, [name], [model_class], resource)
    return h
