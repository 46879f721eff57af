"""Static checks of user-supplied pipeline files before they are imported into the server.

Levels: `none` (skip), `basic` (forbidden calls such as eval / exec / os.system / subprocess with
shell), `strict` (adds forbidden imports: sockets, ctypes, pickle, raw process control ...),
`sandbox` (strict + the module is executed with a restricted `__import__`). Code under
`if __name__ == "__main__":` is not analysed (it never runs in the server).
Role parity: telefuser/service/security/security_validator.py (ASTSecurityAnalyzer, SandboxedLoader,
PipelineSecurityValidator).
"""

from __future__ import annotations

import ast
import builtins
import re
import types
from dataclasses import dataclass, field
from enum import Enum


class SecurityLevel(str, Enum):
    NONE = "none"
    BASIC = "basic"
    STRICT = "strict"
    SANDBOX = "sandbox"


class SecurityError(Exception):
    pass


@dataclass
class SecurityViolation:
    type: str
    description: str
    line: int
    severity: str = "high"
    snippet: str = ""

    def to_dict(self) -> dict:
        return self.__dict__.copy()


@dataclass
class ValidationResult:
    passed: bool = True
    violations: list = field(default_factory=list)
    warnings: list = field(default_factory=list)

    def add_violation(self, v: SecurityViolation) -> None:
        self.violations.append(v)
        self.passed = False

    def add_warning(self, v: SecurityViolation) -> None:
        self.warnings.append(v)

    def has_critical(self) -> bool:
        return any(v.severity == "critical" for v in self.violations)


FORBIDDEN_CALLS = {"eval", "exec", "compile", "__import__", "execfile"}
FORBIDDEN_ATTR_CALLS = {("os", "system"), ("os", "popen"), ("os", "execv"), ("os", "execve"), ("os", "fork"),
                        ("os", "remove"), ("os", "rmdir"), ("os", "unlink"), ("shutil", "rmtree"), ("os", "kill"),
                        ("pty", "spawn")}  # fmt: skip
STRICT_FORBIDDEN_IMPORTS = {"socket", "ctypes", "pickle", "marshal", "pty", "telnetlib", "ftplib", "smtplib", "paramiko",
                            "multiprocessing.connection", "importlib.machinery"}  # fmt: skip
BASIC_FORBIDDEN_IMPORTS = {"pty", "telnetlib"}
SUSPICIOUS_PATTERNS = [(re.compile(r"base64\.b64decode\s*\(.*\)\s*\)?\s*\.decode"), "OBFUSCATION", "decoded payload"),
                       (re.compile(r"/etc/passwd|/etc/shadow|\.ssh/id_"), "SENSITIVE_PATH", "sensitive path literal")]


class ASTSecurityAnalyzer(ast.NodeVisitor):
    def __init__(self, source: str, filename: str = "<unknown>", level: SecurityLevel = SecurityLevel.STRICT) -> None:
        self.source, self.filename, self.level = source, filename, level
        self.lines = source.splitlines()
        self.result = ValidationResult()

    def analyze(self) -> ValidationResult:
        try:
            tree = ast.parse(self.source, filename=self.filename)
        except SyntaxError as e:
            self.result.add_violation(SecurityViolation("SYNTAX", f"cannot parse: {e}", e.lineno or 0, "critical"))
            return self.result
        self.visit(tree)
        return self.result

    def _snippet(self, node) -> str:
        ln = getattr(node, "lineno", 0)
        return self.lines[ln - 1].strip() if 0 < ln <= len(self.lines) else ""

    def _violation(self, node, vtype, desc, severity="high"):
        self.result.add_violation(SecurityViolation(vtype, desc, getattr(node, "lineno", 0), severity, self._snippet(node)))

    def _warning(self, node, vtype, desc):
        self.result.add_warning(SecurityViolation(vtype, desc, getattr(node, "lineno", 0), "low", self._snippet(node)))

    @staticmethod
    def _is_main_check(test) -> bool:
        return (isinstance(test, ast.Compare) and isinstance(test.left, ast.Name) and test.left.id == "__name__"
                and len(test.comparators) == 1 and isinstance(test.comparators[0], ast.Constant)
                and test.comparators[0].value == "__main__")  # fmt: skip

    def visit_If(self, node: ast.If) -> None:
        if self._is_main_check(node.test):
            for n in node.orelse:
                self.visit(n)
            return
        self.generic_visit(node)

    def _check_import(self, node, name: str) -> None:
        banned = STRICT_FORBIDDEN_IMPORTS if self.level in (SecurityLevel.STRICT, SecurityLevel.SANDBOX) else BASIC_FORBIDDEN_IMPORTS
        root = name.split(".")[0]
        if name in banned or root in banned:
            self._violation(node, "FORBIDDEN_IMPORT", f"import of '{name}' is not allowed")
        elif root == "subprocess":
            self._warning(node, "SUBPROCESS_IMPORT", "subprocess imported; shell=True calls are rejected")

    def visit_Import(self, node: ast.Import) -> None:
        for a in node.names:
            self._check_import(node, a.name)

    def visit_ImportFrom(self, node: ast.ImportFrom) -> None:
        if node.module:
            self._check_import(node, node.module)

    def visit_Call(self, node: ast.Call) -> None:
        f = node.func
        if isinstance(f, ast.Name) and f.id in FORBIDDEN_CALLS:
            self._violation(node, "FORBIDDEN_CALL", f"call to '{f.id}' is not allowed", "critical")
        elif isinstance(f, ast.Attribute):
            obj = f.value.id if isinstance(f.value, ast.Name) else ""
            if (obj, f.attr) in FORBIDDEN_ATTR_CALLS:
                self._violation(node, "FORBIDDEN_CALL", f"call to '{obj}.{f.attr}' is not allowed", "critical")
            if obj == "subprocess":
                for kw in node.keywords:
                    if kw.arg == "shell" and isinstance(kw.value, ast.Constant) and kw.value.value is True:
                        self._violation(node, "SHELL_EXEC", "subprocess with shell=True is not allowed", "critical")
        self.generic_visit(node)

    def visit_ClassDef(self, node: ast.ClassDef) -> None:
        if any(k.arg == "metaclass" for k in node.keywords):
            self._warning(node, "METACLASS", f"Metaclass definition detected: '{node.name}'")
        self.generic_visit(node)


class SandboxedLoader:
    """Executes module source with an import hook that only admits allow-listed top-level packages."""

    DEFAULT_ALLOWED = {"torch", "numpy", "PIL", "math", "os", "sys", "json", "typing", "dataclasses", "pathlib", "time",
                       "functools", "itertools", "collections", "random", "re", "einops", "telefuser_b200", "telefuser",
                       "__future__", "logging", "enum", "abc", "copy", "uuid", "threading", "asyncio", "io", "base64",
                       "tempfile", "warnings", "contextlib", "inspect", "types", "datetime", "cv2", "imageio", "tqdm",
                       "safetensors", "transformers", "argparse"}  # fmt: skip

    def __init__(self, allowed_modules: set | None = None) -> None:
        self.allowed = set(allowed_modules) if allowed_modules is not None else set(self.DEFAULT_ALLOWED)

    def import_hook(self, name, globals=None, locals=None, fromlist=(), level=0):  # noqa: A002
        if level == 0 and name.split(".")[0] not in self.allowed:
            raise SecurityError(f"import of '{name}' is blocked by the sandbox")
        return builtins.__import__(name, globals, locals, fromlist, level)

    def load_module(self, source: str, filename: str = "<sandbox>") -> types.ModuleType:
        mod = types.ModuleType("sandboxed_pipeline")
        mod.__file__ = filename
        safe = dict(vars(builtins))
        for banned in ("eval", "exec", "compile", "breakpoint"):
            safe.pop(banned, None)
        safe["__import__"] = self.import_hook
        mod.__dict__["__builtins__"] = safe
        exec(builtins.compile(source, filename, "exec"), mod.__dict__)  # noqa: S102 - source passed the static checks
        return mod


class PipelineSecurityValidator:
    def __init__(self, level: SecurityLevel | str = SecurityLevel.STRICT, allowed_modules: set | None = None) -> None:
        self.level = SecurityLevel(level) if not isinstance(level, SecurityLevel) else level
        self.loader = SandboxedLoader(allowed_modules)

    def validate_source(self, source: str, filename: str = "<unknown>") -> ValidationResult:
        if self.level == SecurityLevel.NONE:
            return ValidationResult()
        result = ASTSecurityAnalyzer(source, filename, self.level).analyze()
        for pat, vtype, desc in SUSPICIOUS_PATTERNS:
            m = pat.search(source)
            if m:
                line = source[: m.start()].count("\n") + 1
                v = SecurityViolation(vtype, desc, line, "medium")
                (result.add_violation if self.level != SecurityLevel.BASIC else result.add_warning)(v)
        return result

    def validate_file(self, path: str) -> ValidationResult:
        with open(path, encoding="utf-8") as f:
            return self.validate_source(f.read(), path)

    def check_file(self, path: str) -> None:
        res = self.validate_file(path)
        if not res.passed:
            lines = "; ".join(f"{v.type} line {v.line}: {v.description}" for v in res.violations)
            raise SecurityError(f"{path} failed security validation ({self.level.value}): {lines}")
