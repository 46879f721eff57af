"""Discovery of the components inside a model folder (Hugging Face / diffusers layout, or a flat folder of
official checkpoint files).

Three sources are consulted, in this order of trust:
1. `model_index.json` (diffusers): component name -> [library, class];
2. each sub-folder's own `config.json` (`_class_name`, `architectures`, `model_type`);
3. file and folder names (`*dit*`, `*t5*`, `*VAE*`, `*clip*`, ...), for official single-file releases.
Every component is classified into a role (transformer, transformer_2, vae, text_encoder, text_encoder_2,
image_encoder, tokenizer, tokenizer_2, scheduler, upsampler, lora) and reported with its weight files (sharded
checkpoints are returned as a sorted list), its class name when one is declared, and its size on disk.

Public surface follows telefuser/utils/hf_model_analyzer.py:19-382 (`ModelComponentInfo`, `HFModelAnalyzer`
with `analyze()` and the `get_*_path()` getters, `discover_model_components`).
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path

WEIGHT_SUFFIXES = (".safetensors", ".pth", ".pt", ".bin", ".ckpt")

# folder / file name fragments -> role (first match wins; checked on lower-cased names)
_NAME_RULES: tuple[tuple[str, str], ...] = (
    (r"transformer_2|low_noise", "transformer_2"),
    (r"transformer|high_noise|dit|unet|diffusion_pytorch_model|denoiser", "transformer"),
    (r"text_encoder_2|byt5|glyph", "text_encoder_2"),
    (r"text_encoder|umt5|t5|gemma|qwen2|llm|mt5", "text_encoder"),
    (r"image_encoder|clip|siglip|vision", "image_encoder"),
    (r"tokenizer_2", "tokenizer_2"),
    (r"tokenizer", "tokenizer"),
    (r"upsampl|upscal|latent_up", "upsampler"),
    (r"lora", "lora"),
    (r"vae|autoencoder|tae|decoder", "vae"),
    (r"scheduler", "scheduler"),
)
# declared class names -> role
_CLASS_RULES: tuple[tuple[str, str], ...] = (
    (r"tokenizer", "tokenizer"),
    (r"scheduler|solver", "scheduler"),
    (r"autoencoder|vae", "vae"),
    (r"clip.*vision|siglip|visionmodel|imageencoder", "image_encoder"),
    (r"t5|gemma|qwen2|llama|mistral|textencoder|causallm|encodermodel", "text_encoder"),
    (r"transformer|dit|unet", "transformer"),
)


@dataclass
class ModelComponentInfo:
    name: str  # folder or file stem as found on disk
    role: str
    path: str  # component folder (or the file for single-file components)
    files: list[str] = field(default_factory=list)  # weight files, sorted; empty for tokenizers / schedulers
    class_name: str | None = None
    library: str | None = None
    config: dict = field(default_factory=dict)
    size_bytes: int = 0

    @property
    def weights(self) -> str | list[str] | None:
        """One path, a list of shard paths, or None when the component has no weight file."""
        if not self.files:
            return None
        return self.files[0] if len(self.files) == 1 else list(self.files)


def _read_json(path: Path) -> dict:
    try:
        with open(path) as f:
            data = json.load(f)
        return data if isinstance(data, dict) else {}
    except (OSError, ValueError):
        return {}


def _role_from(text: str, rules) -> str | None:
    low = text.lower()
    for pattern, role in rules:
        if re.search(pattern, low):
            return role
    return None


def _weight_files(folder: Path, recursive: bool = False) -> list[str]:
    """Weight files of a component. A sharded checkpoint's index decides the list when present, so stray
    consolidated copies beside the shards are not loaded twice."""
    for index in sorted(folder.glob("*.safetensors.index.json")) + sorted(folder.glob("*.bin.index.json")):
        shards = sorted({v for v in _read_json(index).get("weight_map", {}).values()})
        files = [str(folder / s) for s in shards if (folder / s).is_file()]
        if files:
            return files
    it = folder.rglob("*") if recursive else folder.iterdir()
    found = sorted(str(p) for p in it if p.is_file() and p.suffix in WEIGHT_SUFFIXES)
    safes = [f for f in found if f.endswith(".safetensors")]
    return safes or found  # a folder that has both formats is loaded from safetensors


def _size(paths) -> int:
    total = 0
    for p in paths:
        try:
            total += Path(p).stat().st_size
        except OSError:
            pass
    return total


class HFModelAnalyzer:
    def __init__(self, model_root: str) -> None:
        self.root = Path(model_root)
        if not self.root.exists():
            raise FileNotFoundError(model_root)
        self.model_index = _read_json(self.root / "model_index.json")
        self.root_config = _read_json(self.root / "config.json")
        self._components: dict[str, ModelComponentInfo] | None = None

    # ---- analysis ---------------------------------------------------------------
    def analyze(self) -> dict[str, ModelComponentInfo]:
        """role -> component. When two components claim one role the first found keeps it and the second gets the
        `_2` role when that exists (two DiT experts, two text encoders), else it is listed under its own name."""
        if self._components is not None:
            return self._components
        out: dict[str, ModelComponentInfo] = {}

        def add(info: ModelComponentInfo) -> None:
            role = info.role
            if role in out:
                second = f"{role}_2"
                role = second if second not in out and role in ("transformer", "text_encoder", "tokenizer") else info.name
                info.role = role
            out[role] = info

        for info in self._from_model_index():
            add(info)
        seen = {c.path for c in out.values()}
        for info in self._from_subfolders():
            if info.path not in seen:
                add(info)
                seen.add(info.path)
        for info in self._from_loose_files():
            if info.path not in seen and not any(info.path in c.files for c in out.values()):
                add(info)
        self._components = out
        return out

    def _component(self, name: str, folder: Path, role: str | None, library=None, class_name=None) -> ModelComponentInfo | None:
        cfg = _read_json(folder / "config.json")
        declared = class_name or cfg.get("_class_name") or (cfg.get("architectures") or [None])[0]
        if not declared and (folder / "tokenizer_config.json").is_file():
            declared = _read_json(folder / "tokenizer_config.json").get("tokenizer_class")
            role = role or "tokenizer"
        if not declared and (folder / "scheduler_config.json").is_file():
            declared = _read_json(folder / "scheduler_config.json").get("_class_name")
            role = role or "scheduler"
        role = role or _role_from(name, _NAME_RULES) or (declared and _role_from(declared, _CLASS_RULES))
        if not role:
            return None
        files = [] if role.startswith(("tokenizer", "scheduler")) else _weight_files(folder)
        if not files and not role.startswith(("tokenizer", "scheduler")):
            return None
        return ModelComponentInfo(name, role, str(folder), files, declared, library, cfg,
                                  _size(files) if files else _size(p for p in folder.iterdir() if p.is_file()))  # fmt: skip

    def _from_model_index(self) -> list[ModelComponentInfo]:
        found = []
        for name, spec in self.model_index.items():
            if name.startswith("_") or not isinstance(spec, (list, tuple)) or len(spec) != 2 or spec[1] is None:
                continue
            folder = self.root / name
            if not folder.is_dir():
                continue
            library, class_name = spec
            role = _role_from(name, _NAME_RULES) or _role_from(str(class_name), _CLASS_RULES)
            info = self._component(name, folder, role, library, class_name)
            if info:
                found.append(info)
        return found

    def _from_subfolders(self) -> list[ModelComponentInfo]:
        found = []
        for folder in sorted(p for p in self.root.iterdir() if p.is_dir() and not p.name.startswith(".")):
            info = self._component(folder.name, folder, None)
            if info:
                found.append(info)
        return found

    def _from_loose_files(self) -> list[ModelComponentInfo]:
        """Official single-file releases: weight files directly in the root. Shards of one checkpoint (same stem up
        to the `-00001-of-0000N` counter) form one component."""
        groups: dict[str, list[str]] = {}
        loose = sorted(str(p) for p in self.root.iterdir() if p.is_file() and p.suffix in WEIGHT_SUFFIXES)
        for f in loose:
            stem = re.sub(r"-\d{5}-of-\d{5}$", "", Path(f).stem)
            groups.setdefault(stem, []).append(f)
        found = []
        for stem, files in sorted(groups.items()):
            role = _role_from(stem, _NAME_RULES)
            if role is None and len(groups) == 1:
                role = "transformer"  # a folder with a single checkpoint: the denoiser
            if role:
                cls = self.root_config.get("_class_name") if role == "transformer" else None
                found.append(ModelComponentInfo(stem, role, files[0] if len(files) == 1 else str(self.root), sorted(files),
                                                cls, None, self.root_config if role == "transformer" else {}, _size(files)))  # fmt: skip
        return found

    # ---- getters ------------------------------------------------------------------
    def _weights(self, *roles: str):
        comps = self.analyze()
        for role in roles:
            if role in comps and comps[role].weights is not None:
                return comps[role].weights
        return None

    def _folder(self, *roles: str) -> str | None:
        comps = self.analyze()
        for role in roles:
            if role in comps:
                return comps[role].path
        return None

    def get_transformer_path(self):
        return self._weights("transformer")

    def get_transformer_2_path(self):
        return self._weights("transformer_2")

    def get_vae_path(self):
        return self._weights("vae")

    def get_text_encoder_path(self):
        return self._weights("text_encoder")

    def get_text_encoder_2_path(self):
        return self._weights("text_encoder_2")

    def get_image_encoder_path(self):
        return self._weights("image_encoder")

    def get_tokenizer_path(self) -> str | None:
        return self._folder("tokenizer")

    def get_tokenizer_2_path(self) -> str | None:
        return self._folder("tokenizer_2")

    def get_scheduler_path(self) -> str | None:
        return self._folder("scheduler")

    def get_upsampler_path(self):
        return self._weights("upsampler")

    def get_distilled_lora_path(self):
        return self._weights("lora")

    def get_gemma_root_path(self) -> str | None:
        """Folder of a Gemma text encoder (LTX-2 keeps the language model as a whole transformers checkpoint)."""
        comps = self.analyze()
        for c in comps.values():
            if c.role.startswith("text_encoder") and "gemma" in f"{c.name} {c.class_name}".lower():
                return c.path
        return None

    def component_folder(self, role: str) -> str | None:
        return self._folder(role)

    def task(self) -> str:
        from .hf import detect_model_task

        return detect_model_task(str(self.root))

    def describe(self) -> str:
        lines = [f"{self.root} ({self.task()})"]
        for role, c in self.analyze().items():
            n = len(c.files)
            lines.append(f"  {role:<16} {c.class_name or '-':<40} {n} file{'s' if n != 1 else ''}  {c.size_bytes / 2**30:.2f} GiB  {c.name}")
        return "\n".join(lines)


def discover_model_components(model_root: str) -> dict[str, str | list[str]]:
    """role -> weight path(s) (folders for tokenizers and schedulers)."""
    out: dict[str, str | list[str]] = {}
    for role, c in HFModelAnalyzer(model_root).analyze().items():
        out[role] = c.weights if c.weights is not None else c.path
    return out
