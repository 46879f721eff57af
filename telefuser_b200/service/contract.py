"""Pipeline-file contract: what a served pipeline module declares and how requests are checked against it.

A pipeline file exposes `get_pipeline(parallelism=...)` + `run_with_file(...)` (request/response) or
`get_service(gpu_num=...)` (streaming) and may declare `PIPELINE_MANIFEST` / `PIPELINE_CONTRACT` /
`get_pipeline_contract()`: supported tasks, media type, required inputs and typed parameters with
defaults. Without a declaration a legacy contract is inferred from `run_with_file`'s signature.
Role parity: telefuser/service/core/pipeline_contract.py, contract_templates.py,
telefuser/service/api/task_contract_runtime.py:13-148.
"""

from __future__ import annotations

import inspect
import re
from dataclasses import dataclass, field
from types import ModuleType
from typing import Any

from .task_manager import IMAGE_TASKS, VIDEO_TASKS

TASK_NAME = re.compile(r"^[a-z][a-z0-9_]{1,31}$")
INPUT_FIELDS = ("prompt", "negative_prompt", "first_image_path", "last_image_path", "ref_video_path", "audio_path",
                "mask_path")  # fmt: skip


def infer_media_type_for_task(task: str) -> str:
    if task in IMAGE_TASKS:
        return "image"
    if task in VIDEO_TASKS:
        return "video"
    return "stream" if task == "bidirectional" else "video"


def validate_task_name_format(task: str) -> str:
    t = str(task).strip().lower()
    if not TASK_NAME.match(t):
        raise ValueError(f"invalid task name {task!r}")
    return t


def _strs(v) -> tuple:
    if v is None:
        return ()
    if isinstance(v, str):
        return (v,)
    return tuple(str(x) for x in v)


def _infer_type(default: Any) -> str:
    for t, name in ((bool, "boolean"), (int, "integer"), (float, "number"), (str, "string")):
        if isinstance(default, t):
            return name
    return "object" if isinstance(default, (dict, list, tuple)) else "string"


@dataclass(frozen=True)
class ParameterContract:
    type: str
    required: bool = False
    default: Any = None
    description: str = ""
    enum: tuple = ()
    exposed: bool = True

    @classmethod
    def from_mapping(cls, raw: dict) -> "ParameterContract":
        return cls(str(raw.get("type") or _infer_type(raw.get("default"))), bool(raw.get("required", False)),
                   raw.get("default"), str(raw.get("description") or ""), _strs(raw.get("enum")),
                   bool(raw.get("exposed", True)))  # fmt: skip

    def to_metadata(self) -> dict:
        return {"type": self.type, "required": self.required, "default": self.default, "description": self.description,
                "enum": list(self.enum), "exposed": self.exposed}  # fmt: skip

    def check(self, name: str, value: Any) -> None:
        ok = {"integer": lambda v: isinstance(v, int) and not isinstance(v, bool),
              "number": lambda v: isinstance(v, (int, float)) and not isinstance(v, bool),
              "boolean": lambda v: isinstance(v, bool), "string": lambda v: isinstance(v, str)}.get(self.type)  # fmt: skip
        if ok is not None and value is not None and not ok(value):
            raise ValueError(f"parameter {name} must be of type {self.type}")
        if self.enum and value is not None and str(value) not in self.enum:
            raise ValueError(f"parameter {name} must be one of {list(self.enum)}")


@dataclass(frozen=True)
class TaskContract:
    task: str
    media_type: str
    required_inputs: tuple = ()
    optional_inputs: tuple = ()
    parameters: dict = field(default_factory=dict)

    @classmethod
    def from_mapping(cls, task: str, raw: dict) -> "TaskContract":
        t = validate_task_name_format(task)
        params = {k: (v if isinstance(v, ParameterContract) else ParameterContract.from_mapping(v if isinstance(v, dict) else {"default": v}))
                  for k, v in (raw.get("parameters") or {}).items()}  # fmt: skip
        return cls(t, str(raw.get("media_type") or infer_media_type_for_task(t)), _strs(raw.get("required_inputs")),
                   _strs(raw.get("optional_inputs")), params)  # fmt: skip

    def to_metadata(self) -> dict:
        return {"media_type": self.media_type, "required_inputs": list(self.required_inputs),
                "optional_inputs": list(self.optional_inputs),
                "parameters": {n: c.to_metadata() for n, c in self.parameters.items() if c.exposed}}  # fmt: skip


@dataclass(frozen=True)
class PipelineContract:
    contract_version: str
    pipeline_name: str
    supported_tasks: tuple
    supported_media_types: tuple
    execution_mode: str
    effective_max_concurrent_tasks: int
    task_contracts: dict
    get_pipeline: str = "get_pipeline"
    run_with_file: str = "run_with_file"

    @classmethod
    def from_mapping(cls, raw: dict, fallback_name: str) -> "PipelineContract":
        name = str(raw.get("pipeline_name") or fallback_name).strip()
        if not name:
            raise ValueError("Pipeline contract requires a non-empty pipeline_name")
        tasks = tuple(validate_task_name_format(t) for t in _strs(raw.get("supported_tasks")))
        if not tasks:
            raise ValueError("Pipeline contract requires at least one supported task")
        tcs = {t: TaskContract.from_mapping(t, (raw.get("task_contracts") or raw.get("tasks") or {}).get(t, {})) for t in tasks}
        media = _strs(raw.get("supported_media_types")) or tuple(sorted({c.media_type for c in tcs.values()}))
        ep = raw.get("entrypoints") or {}
        return cls(str(raw.get("contract_version") or "1"), name, tasks, media, str(raw.get("execution_mode") or "sync"),
                   int(raw.get("effective_max_concurrent_tasks") or 1), tcs, ep.get("get_pipeline", "get_pipeline"),
                   ep.get("run_with_file", "run_with_file"))  # fmt: skip

    def to_metadata(self) -> dict:
        return {"contract_version": self.contract_version, "pipeline_name": self.pipeline_name,
                "supported_tasks": list(self.supported_tasks), "supported_media_types": list(self.supported_media_types),
                "execution_mode": self.execution_mode, "effective_max_concurrent_tasks": self.effective_max_concurrent_tasks,
                "entrypoints": {"get_pipeline": self.get_pipeline, "run_with_file": self.run_with_file},
                "task_contracts": {t: c.to_metadata() for t, c in self.task_contracts.items()},
                "tasks": {t: c.to_metadata() for t, c in self.task_contracts.items()}}  # fmt: skip  ("tasks": older clients)


TASK_TEMPLATES = {
    "t2v": {"required_inputs": ["prompt"], "optional_inputs": ["negative_prompt"]},
    "i2v": {"required_inputs": ["prompt", "first_image_path"], "optional_inputs": ["negative_prompt", "last_image_path"]},
    "fl2v": {"required_inputs": ["prompt", "first_image_path", "last_image_path"], "optional_inputs": ["negative_prompt"]},
    "vc": {"required_inputs": ["ref_video_path"], "optional_inputs": ["prompt"]},
    "s2v": {"required_inputs": ["first_image_path", "audio_path"], "optional_inputs": ["prompt"]},
    "vsr": {"required_inputs": ["ref_video_path"]},
    "t2i": {"required_inputs": ["prompt"], "optional_inputs": ["negative_prompt"]},
    "i2i": {"required_inputs": ["prompt", "first_image_path"]},
    "edit": {"required_inputs": ["prompt", "first_image_path"], "optional_inputs": ["mask_path"]},
}


def legacy_contract_from_module(module: ModuleType, task: str, name: str) -> PipelineContract:
    """Infers a contract from `run_with_file`'s signature: defaults become parameters."""
    fn = getattr(module, "run_with_file", None)
    params = {}
    if fn is not None:
        for pname, p in inspect.signature(fn).parameters.items():
            if pname in INPUT_FIELDS or pname in ("pipeline", "pipe", "output_path", "task", "kwargs"):
                continue
            if p.default is not inspect.Parameter.empty:
                params[pname] = {"default": p.default}
    tc = dict(TASK_TEMPLATES.get(task, {}))
    tc["parameters"] = params
    return PipelineContract.from_mapping({"pipeline_name": name, "supported_tasks": [task], "task_contracts": {task: tc}},
                                         fallback_name=name)  # fmt: skip


def declares_contract(module: ModuleType) -> bool:
    """Whether the pipeline file states its own contract (else one is derived from `run_with_file`'s signature)."""
    return any(isinstance(getattr(module, a, None), dict) for a in ("PIPELINE_MANIFEST", "PIPELINE_CONTRACT")) \
        or callable(getattr(module, "get_pipeline_contract", None))  # fmt: skip


def signature_parameters(module: ModuleType) -> dict:
    """`run_with_file`'s keyword defaults as parameter entries (inputs such as image paths and the plumbing arguments
    are not parameters)."""
    fn = getattr(module, "run_with_file", None)
    if fn is None:
        return {}
    return {n: {"default": p.default} for n, p in inspect.signature(fn).parameters.items()
            if n not in INPUT_FIELDS and n not in ("pipeline", "pipe", "output_path", "task", "kwargs", "stop_event", "latent_data")
            and p.default is not inspect.Parameter.empty}  # fmt: skip


def expand_short_manifest(raw: dict, module: ModuleType | None, name: str) -> dict:
    """The compact manifest form pipeline files may use,

        PIPELINE_MANIFEST = {"tasks": ["t2v", "i2v"], "media_type": "video", "required_inputs": {"t2v": ["prompt"], ...}}

    spelled out as a full contract mapping: one task contract per listed task with its required (and optional) inputs,
    the media type, and the keyword defaults of `run_with_file` as the task's parameters. A mapping that already has
    `supported_tasks` is returned unchanged."""
    if raw.get("supported_tasks") or not isinstance(raw.get("tasks"), (list, tuple)):
        return raw
    per_task = {key: raw.get(key) if isinstance(raw.get(key), dict) else {} for key in ("required_inputs", "optional_inputs", "parameters")}
    shared = signature_parameters(module) if module is not None else {}
    contracts = {}
    for t in raw["tasks"]:
        tc = dict(TASK_TEMPLATES.get(t, {}))
        if t in per_task["required_inputs"]:
            tc["required_inputs"] = list(per_task["required_inputs"][t])
        if t in per_task["optional_inputs"]:
            tc["optional_inputs"] = list(per_task["optional_inputs"][t])
        if isinstance(raw.get("media_type"), str) and len(raw["tasks"]) == 1:
            tc["media_type"] = raw["media_type"]  # with several tasks each keeps the media type its name implies (t2i next to t2v)
        inputs = set(tc.get("required_inputs", ())) | set(tc.get("optional_inputs", ()))
        tc["parameters"] = {**{n: v for n, v in shared.items() if n not in inputs}, **per_task["parameters"].get(t, {})}
        contracts[t] = tc
    rest = {k: v for k, v in raw.items() if k not in ("tasks", "media_type", "required_inputs", "optional_inputs", "parameters")}
    return {"pipeline_name": raw.get("pipeline_name") or (getattr(module, "PPL_CONFIG", None) or {}).get("name") or name,
            "supported_tasks": list(raw["tasks"]), "task_contracts": contracts, **rest}  # fmt: skip


def load_contract(module: ModuleType, task: str | None, name: str) -> PipelineContract:
    for attr in ("PIPELINE_MANIFEST", "PIPELINE_CONTRACT"):
        raw = getattr(module, attr, None)
        if isinstance(raw, dict):
            return PipelineContract.from_mapping(expand_short_manifest(raw, module, name), fallback_name=name)
    fn = getattr(module, "get_pipeline_contract", None)
    if callable(fn):
        raw = fn()
        return raw if isinstance(raw, PipelineContract) else PipelineContract.from_mapping(raw, fallback_name=name)
    return legacy_contract_from_module(module, task or "t2v", name)


def apply_task_contract_defaults(contract: PipelineContract, task: str, data: dict) -> dict:
    if task not in contract.task_contracts:
        raise ValueError(f"task {task!r} is not supported by pipeline {contract.pipeline_name} "
                         f"(supported: {list(contract.supported_tasks)})")  # fmt: skip
    out = dict(data)
    for name, pc in contract.task_contracts[task].parameters.items():
        if out.get(name) is None and pc.default is not None:
            out[name] = pc.default
    return out


def validate_required_task_parameters(contract: PipelineContract, task: str, data: dict) -> None:
    tc = contract.task_contracts[task]
    missing = [f for f in tc.required_inputs if not data.get(f)]
    missing += [n for n, pc in tc.parameters.items() if pc.required and data.get(n) is None]
    if missing:
        raise ValueError(f"missing required field(s) for task {task}: {missing}")
    for n, pc in tc.parameters.items():
        if n in data:
            pc.check(n, data[n])


# ---- CACHE_CONFIG: the pipeline file's own latent-cache settings --------------------------------------------------
CACHE_MODES = {"read": "read", "read_only": "read", "write": "write", "write_only": "write", "readwrite": "readwrite",
               "read_write": "readwrite"}  # fmt: skip


def _literal(node, env):
    """Value of an expression that is a literal, a container of such, or one of `os.getenv(name, default)`,
    `os.environ.get(name, default)`, `int / float / str / bool(<such>)`, `os.path.join(<such>, ...)`."""
    import ast
    import os

    if isinstance(node, ast.Constant):
        return node.value
    if isinstance(node, (ast.List, ast.Tuple)):
        return [_literal(e, env) for e in node.elts]
    if isinstance(node, ast.Dict):
        return {_literal(k, env): _literal(v, env) for k, v in zip(node.keys, node.values)}
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        return -_literal(node.operand, env)
    if isinstance(node, ast.Name) and node.id in env:
        return env[node.id]
    if isinstance(node, ast.Call):
        name = ast.unparse(node.func)
        args = [_literal(a, env) for a in node.args]
        if name in ("os.getenv", "os.environ.get"):
            return os.environ.get(args[0], args[1] if len(args) > 1 else None)
        if name in ("int", "float", "str", "bool") and len(args) == 1:
            return {"int": int, "float": float, "str": str, "bool": bool}[name](args[0])
        if name == "os.path.join":
            return os.path.join(*args)
        if name == "dict" and not args:
            return {kw.arg: _literal(kw.value, env) for kw in node.keywords}
    raise ValueError(f"not a plain value: {ast.unparse(node)}")


def load_cache_config(pipe_path: str) -> dict | None:
    """The `CACHE_CONFIG` mapping a pipeline file declares (or None), read WITHOUT importing the file: the server decides
    about the latent cache before any pipeline (or replica process) is started. Values may be literals, environment
    look-ups with defaults and simple casts of those; an entry written any other way is skipped."""
    import ast

    try:
        tree = ast.parse(open(pipe_path, encoding="utf-8").read())
    except (OSError, SyntaxError):
        return None
    env: dict = {}
    found = None
    for node in tree.body:
        if not (isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name)):
            continue
        target = node.targets[0].id
        if target != "CACHE_CONFIG":
            try:
                env[target] = _literal(node.value, env)  # module-level constants the mapping may refer to
            except (ValueError, TypeError, KeyError):
                pass
            continue
        entries: list = []
        if isinstance(node.value, ast.Dict):
            entries = [(k.value, v) for k, v in zip(node.value.keys, node.value.values) if isinstance(k, ast.Constant)]
        elif isinstance(node.value, ast.Call) and ast.unparse(node.value.func) == "dict":
            entries = [(kw.arg, kw.value) for kw in node.value.keywords if kw.arg]
        found = {}
        for key, value in entries:
            try:
                found[key] = _literal(value, env)
            except (ValueError, TypeError, KeyError):
                continue
    return found


def resolve_latent_cache_settings(pipe_path: str, enable: bool | None, mode: str | None) -> dict:
    """What the server should do about the latent cache: explicit arguments (the CLI) win, then the pipeline file's
    `CACHE_CONFIG`, then off / read-write. Returns {enabled, mode, directory, min_similarity, source}."""
    declared = load_cache_config(pipe_path) or {}
    out = {"enabled": bool(declared.get("enable_latent_cache", False)), "mode": "readwrite", "directory": declared.get("latent_cache_dir"),
           "min_similarity": declared.get("rerank_score_threshold"), "source": "pipeline file" if declared else "default"}  # fmt: skip
    declared_mode = declared.get("cache_mode")
    if declared_mode is not None:
        if str(declared_mode) not in CACHE_MODES:
            raise ValueError(f"{pipe_path}: CACHE_CONFIG cache_mode {declared_mode!r} is not one of {sorted(CACHE_MODES)}")
        out["mode"] = CACHE_MODES[str(declared_mode)]
    if enable is not None:
        out["enabled"], out["source"] = bool(enable), "command line"
    if mode:
        if mode not in CACHE_MODES:
            raise ValueError(f"cache mode {mode!r} is not one of {sorted(CACHE_MODES)}")
        out["mode"] = CACHE_MODES[mode]
    return out
