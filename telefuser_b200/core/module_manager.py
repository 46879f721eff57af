"""ModuleManager: loads checkpoints, recognises which model they belong to, builds the
model without materialising weights twice, and hands modules to stages by name.

Flow (role parity with telefuser/core/module_manager.py:22-443): resolve the path(s)
to weight files -> read the state dict -> fingerprint it and look the fingerprint
up in the `ModelRegistry` (or take an explicit class) -> run the class's state-dict
converter (`from_official` / `from_diffusers`, which also returns constructor
kwargs) -> construct on the meta device -> `load_state_dict(assign=True)` -> dtype /
device -> optional quantisation. A model whose layout is not registered but whose
class has a shape-inferring converter can be loaded with `model_class=`.
"""

from __future__ import annotations

import os
from typing import Any

import torch
import torch.nn as nn

from telefuser_b200.core.config import QuantConfig
from telefuser_b200.core.model_registry import ModelRegistry
from telefuser_b200.utils.logging import logger
from telefuser_b200.utils.model_weight import expand_checkpoint_paths, init_weights_on_device, load_state_dict


def build_model_from_state_dict(state_dict, model_class, model_resource, torch_dtype, device,
                                low_cpu_mem_usage=False, converter_kwargs=None, quant_config=None):  # fmt: skip
    converter = model_class.state_dict_converter(**(converter_kwargs or {}))
    if converter is None:
        model_sd, ctor = state_dict, {}
    else:
        fn = {"official": "from_official", "diffusers": "from_diffusers", "civitai": "from_civitai"}.get(model_resource)
        if fn is None:
            raise ValueError(f"Unknown model_resource: {model_resource}")
        res = getattr(converter, fn)(state_dict)
        model_sd, ctor = res if isinstance(res, tuple) else (res, {})
    with init_weights_on_device("meta"):
        model = model_class(**ctor)
    model = model.eval().requires_grad_(False)
    if not low_cpu_mem_usage:
        model_sd = {k: v.to("cpu").clone() for k, v in model_sd.items()}
    model.load_state_dict(model_sd, assign=True)
    if torch_dtype != torch.float8_e4m3fn:
        model = model.to(dtype=torch_dtype)
    model = model.to(device)
    if quant_config is not None and quant_config.enabled:
        model.enable_quant(quant_config)
    elif torch_dtype == torch.float8_e4m3fn:
        model.enable_quant(torch_dtype)
    return model


class ModuleManager:
    def __init__(self, torch_dtype: torch.dtype = torch.bfloat16, device: str | None = None) -> None:
        self.torch_dtype = torch_dtype
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.modules: list[nn.Module] = []
        self.module_paths: list[Any] = []
        self.module_names: list[str] = []

    # ---- loading -----------------------------------------------------------
    def load_models(self, file_path_list, device=None, torch_dtype=None, low_cpu_mem_usage=False, quant_config=None):
        for p in file_path_list:
            self.load_model(p, device, torch_dtype, low_cpu_mem_usage, quant_config=quant_config)

    def load_model(self, file_path, device=None, torch_dtype=None, low_cpu_mem_usage=False, name=None,
                   model_class=None, model_resource="official", converter_kwargs=None,
                   quant_config: QuantConfig | None = None) -> bool:  # fmt: skip
        """Loads one checkpoint. Returns True when a model was recognised and added."""
        device = device or self.device
        torch_dtype = torch_dtype or self.torch_dtype
        if isinstance(file_path, str) and os.path.isdir(file_path):
            # a diffusers component folder
            for cand in ("diffusion_pytorch_model.safetensors.index.json", "diffusion_pytorch_model.safetensors"):
                if os.path.isfile(os.path.join(file_path, cand)):
                    file_path = os.path.join(file_path, cand)
                    break
        files = expand_checkpoint_paths(file_path)
        files = [f for f in files if os.path.isfile(f)]
        if not files:
            return False
        state_dict = load_state_dict(files)
        # a checkpoint quantised offline: recognise and build from its dense form, then put the stored payloads back
        from telefuser_b200.ops.quant import apply_quantized_state_, quantized_state_from_checkpoint

        state_dict, offline_quant = quantized_state_from_checkpoint(state_dict)
        if model_class is not None:
            names, classes, resource = [name or model_class.__name__], [model_class], model_resource
        else:
            entry = ModelRegistry.instance().match(state_dict)
            if entry is None:
                return False
            names, classes, resource = entry.model_names, entry.model_classes, entry.model_resource
            if name is not None:
                names = [name] * len(classes)
        for n, cls in zip(names, classes):
            model = build_model_from_state_dict(state_dict, cls, resource, torch_dtype, device, low_cpu_mem_usage,
                                                converter_kwargs, quant_config)  # fmt: skip
            if offline_quant:
                known = {name for name, _ in model.named_modules()}
                usable = {k: v for k, v in offline_quant.items() if k.rsplit(".", 1)[0] in known}
                done = apply_quantized_state_(model, usable, strict=False)
                total = sum(1 for k in offline_quant if k.endswith(".weight"))
                logger.info(f"{n}: {done} of {total} offline-quantised layers keep their stored form"
                            + ("" if done == total else " (the others were renamed by the key converter and stay dense)"))
            self.add_module(model, n, path=file_path)
        return True

    def load_from_huggingface(self, model_id_or_path: str, name: str, loader_class, torch_dtype=None, device=None,
                              **kwargs) -> nn.Module:  # fmt: skip
        """Loads a transformers / diffusers component with its own `from_pretrained` and registers it."""
        module = loader_class.from_pretrained(model_id_or_path, torch_dtype=torch_dtype or self.torch_dtype, **kwargs)
        module = module.to(device or self.device)
        self.add_module(module, name, path=model_id_or_path)
        return module

    # ---- registry of live modules ---------------------------------------------
    def add_module(self, module: nn.Module, name: str, path: Any = "manual") -> None:
        self.modules.append(module)
        self.module_paths.append(path)
        self.module_names.append(name)

    def remove_module(self, name: str) -> bool:
        removed = False
        for i in reversed(range(len(self.module_names))):
            if self.module_names[i] == name:
                del self.modules[i], self.module_paths[i], self.module_names[i]
                removed = True
        return removed

    def fetch_module(self, model_name: str, file_path: str | None = None, require_model_path: bool = False,
                     index: int | None = None):  # fmt: skip
        found = [(m, p) for m, p, n in zip(self.modules, self.module_paths, self.module_names)
                 if n == model_name and (file_path is None or file_path == p)]  # fmt: skip
        if not found:
            return (None, None) if require_model_path else None
        if len(found) == 1 or index is None:
            model, path = found[0]
        elif isinstance(index, int):
            model, path = [f[0] for f in found[:index]], [f[1] for f in found[:index]]
        else:
            model, path = [f[0] for f in found], [f[1] for f in found]
        return (model, path) if require_model_path else model

    def get_model_info(self) -> list[dict]:
        info = []
        for m, p, n in zip(self.modules, self.module_paths, self.module_names):
            params = sum(t.numel() for t in m.parameters()) if hasattr(m, "parameters") else 0
            first = next(iter(m.parameters()), None) if hasattr(m, "parameters") else None
            info.append({"name": n, "path": p, "class": type(m).__name__, "parameters": params,
                         "dtype": str(first.dtype) if first is not None else None,
                         "device": str(first.device) if first is not None else None})  # fmt: skip
        return info
