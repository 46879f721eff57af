"""Checkpoint inspector: tree view of a (possibly sharded) safetensors / torch checkpoint.

`python -m telefuser_b200.tools.weight_viewer 'model-*.safetensors' [--max-depth N] [--no-merge] [--export out.json]`
prints the parameter count, dtype histogram, the registry fingerprint (which model class the loader would pick)
and a nested module tree in which siblings with identical structure (`blocks.0 ... blocks.39`) are folded into
one line. Only tensor metadata is read from safetensors files, so multi-GB checkpoints open instantly.
Role parity: tools/viewer/weight_viewer.py:19-512.
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import re
import struct
from typing import Any

_DTYPE_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1, "F8_E4M3": 1, "F8_E5M2": 1}


def expand_file_pattern(pattern: str) -> list:
    """Glob, then order shards numerically (`-00002-of-00007`, `_part3`) rather than lexically."""
    files = sorted(glob.glob(pattern)) if any(c in pattern for c in "*?[") else [pattern]

    def key(path: str):
        m = re.search(r"(\d+)-of-(\d+)", os.path.basename(path)) or re.search(r"part[_-]?(\d+)", os.path.basename(path))
        return (0, int(m.group(1))) if m else (1, os.path.basename(path))

    return sorted((f for f in files if os.path.isfile(f)), key=key)


def read_safetensors_header(path: str) -> dict:
    """name -> (dtype string, shape) without touching tensor data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return {k: (v["dtype"], tuple(v["shape"])) for k, v in header.items() if k != "__metadata__"}


def read_torch_checkpoint(path: str) -> dict:
    import torch

    obj = torch.load(path, map_location="cpu", weights_only=True)
    for wrapper in ("state_dict", "model", "module"):
        if isinstance(obj, dict) and isinstance(obj.get(wrapper), dict):
            obj = obj[wrapper]
    out = {}

    def walk(node, prefix=""):
        for k, v in node.items():
            name = f"{prefix}{k}"
            if isinstance(v, dict):
                walk(v, name + ".")
            elif hasattr(v, "shape"):
                out[name] = (str(v.dtype).replace("torch.", ""), tuple(v.shape))

    walk(obj)
    return out


class WeightViewer:
    def __init__(self) -> None:
        self.tensors: dict = {}
        self.files: list = []

    def load_weights(self, file_pattern: str) -> "WeightViewer":
        self.files = expand_file_pattern(file_pattern)
        if not self.files:
            raise FileNotFoundError(f"no checkpoint matches {file_pattern}")
        for f in self.files:
            self.tensors.update(read_safetensors_header(f) if f.endswith(".safetensors") else read_torch_checkpoint(f))
        return self

    @staticmethod
    def _numel(shape) -> int:
        n = 1
        for s in shape:
            n *= s
        return n

    def get_summary(self) -> dict:
        dtypes: dict = {}
        nbytes = 0
        for dt, shape in self.tensors.values():
            dtypes[dt] = dtypes.get(dt, 0) + self._numel(shape)
            nbytes += self._numel(shape) * _DTYPE_BYTES.get(dt.upper(), 4 if "32" in dt else 2 if "16" in dt else 1)
        top: dict = {}
        for name, (_, shape) in self.tensors.items():
            top[name.split(".")[0]] = top.get(name.split(".")[0], 0) + self._numel(shape)
        return {"files": len(self.files), "tensors": len(self.tensors), "parameters": sum(dtypes.values()), "bytes": nbytes, "dtypes": dtypes,
                "top_level": top, "fingerprint": self.fingerprint()}  # fmt: skip

    def fingerprint(self) -> dict:
        """The key / key+shape hashes the model registry matches on, and the registered model names if any."""
        try:
            import torch

            from telefuser_b200.core.model_registry import ModelRegistry, hash_state_dict_keys

            meta = {k: torch.empty(shape, device="meta") for k, (_, shape) in self.tensors.items()}
            entry = ModelRegistry.instance().match(meta)
            return {"keys": hash_state_dict_keys(meta, with_shape=False), "keys_and_shapes": hash_state_dict_keys(meta, with_shape=True),
                    "registered_as": list(entry.model_names) if entry is not None else None}  # fmt: skip
        except Exception as exc:  # noqa: BLE001 - the viewer still works when the registry cannot be imported
            return {"error": str(exc)}

    def build_tree(self) -> dict:
        root: dict = {}
        for name, leaf in self.tensors.items():
            node = root
            parts = name.split(".")
            for p in parts[:-1]:
                node = node.setdefault(p, {})
                if not isinstance(node, dict):  # a tensor and a module share a prefix: keep the tensor under "."
                    break
            else:
                node[parts[-1]] = leaf
        return root

    @classmethod
    def _signature(cls, node) -> Any:
        if not isinstance(node, dict):
            return node
        return tuple((k, cls._signature(v)) for k, v in sorted(node.items()))

    @classmethod
    def _count(cls, node) -> int:
        return cls._numel(node[1]) if not isinstance(node, dict) else sum(cls._count(v) for v in node.values())

    @staticmethod
    def format_number(n: int) -> str:
        for unit, div in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
            if n >= div:
                return f"{n / div:.2f}{unit}"
        return str(n)

    def render(self, max_depth: int = 5, merge_similar: bool = True) -> list:
        lines: list = []

        def walk(node: dict, depth: int, indent: str) -> None:
            keys = sorted(node, key=lambda k: (not k.isdigit(), int(k) if k.isdigit() else 0, k))
            i = 0
            while i < len(keys):
                k, v = keys[i], node[keys[i]]
                j = i + 1
                if merge_similar and isinstance(v, dict) and k.isdigit():
                    sig = self._signature(v)
                    while j < len(keys) and keys[j].isdigit() and isinstance(node[keys[j]], dict) and self._signature(node[keys[j]]) == sig:
                        j += 1
                label = k if j == i + 1 else f"{k}..{keys[j - 1]} (x{j - i}, identical)"
                if isinstance(v, dict):
                    lines.append(f"{indent}{label}/  [{self.format_number(self._count(v) * (j - i))}]")
                    if depth + 1 < max_depth:
                        walk(v, depth + 1, indent + "  ")
                else:
                    lines.append(f"{indent}{label}: {v[0]} {list(v[1])}")
                i = j

        walk(self.build_tree(), 0, "")
        return lines

    def export_to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"summary": self.get_summary(), "tensors": {k: {"dtype": d, "shape": list(s)} for k, (d, s) in self.tensors.items()}}, f, indent=1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Show the structure of a checkpoint")
    ap.add_argument("file_pattern", help="checkpoint path or glob (quote it)")
    ap.add_argument("--max-depth", type=int, default=5)
    ap.add_argument("--no-merge", action="store_true", help="do not fold structurally identical numbered siblings")
    ap.add_argument("--export", type=str, help="write summary and tensor list to this JSON file")
    ap.add_argument("--quiet", action="store_true", help="summary only")
    args = ap.parse_args(argv)
    viewer = WeightViewer().load_weights(args.file_pattern)
    s = viewer.get_summary()
    print(f"{s['files']} file(s), {s['tensors']} tensors, {viewer.format_number(s['parameters'])} parameters, {s['bytes'] / 2**30:.2f} GiB")
    print("dtypes:", ", ".join(f"{k}={viewer.format_number(v)}" for k, v in sorted(s["dtypes"].items())))
    print("fingerprint:", json.dumps(s["fingerprint"]))
    if not args.quiet:
        print("\n".join(viewer.render(args.max_depth, not args.no_merge)))
    if args.export:
        viewer.export_to_json(args.export)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
