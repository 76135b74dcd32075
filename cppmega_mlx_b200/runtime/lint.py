"""AST lint for this code base's own anti-patterns (counterpart of the reference's ``tools/lint_mlx.py:91-755``, whose rules are
about MLX lazy evaluation; the rules here are about a stream-ordered PyTorch + CUDA-kernel design).

Rules
-----
``HS001``  host synchronisation inside a hot function: ``.item()``, ``.tolist()``, ``.cpu()``, ``.numpy()`` or
           ``torch.cuda.synchronize()`` in a ``forward`` / ``step`` / ``__call__`` body of a module under ``nn/``, ``models/``,
           ``ops/`` or ``training/``.  Each one stalls the launching thread until the stream drains.
``CL001``  a compatibility layer on the compute path: importing ``triton`` / ``tilelang`` / ``jax``, or calling
           ``torch.compile``.
``EX001``  a bare ``except:`` (it also swallows ``KeyboardInterrupt`` and the watchdog's exceptions).
``RZ001``  a distributed rendezvous address that is a host *name* (``localhost`` or similar) instead of ``127.0.0.1`` in a
           ``MASTER_ADDR`` assignment or ``init_method=`` string.
``PK001``  process control by pattern (``pkill``, ``killall``, ``pgrep``) in a subprocess command.

A line that ends with ``# lint: allow <RULE>`` (with a reason after it) is exempt from that rule.
"""
from __future__ import annotations

import ast
import os
import re
from dataclasses import dataclass

HOT_DIRS = ("nn", "models", "ops", "training")
HOT_FUNCTIONS = ("forward", "step", "__call__")
SYNC_METHODS = ("item", "tolist", "cpu", "numpy")
FORBIDDEN_IMPORTS = ("triton", "tilelang", "jax")
PATTERN_KILLERS = ("pkill", "killall", "pgrep")
ALLOW = re.compile(r"#\s*lint:\s*allow\s+([A-Z]{2}\d{3})")


@dataclass(frozen=True)
class Violation:
    path: str
    line: int
    rule: str
    message: str

    def __str__(self) -> str:
        return f"{self.path}:{self.line}: {self.rule} {self.message}"


def _is_hot_file(path: str) -> bool:
    parts = os.path.normpath(path).split(os.sep)
    return any(d in parts[:-1] for d in HOT_DIRS)


class _Visitor(ast.NodeVisitor):
    def __init__(self, path: str, lines: list[str]):
        self.path, self.lines = path, lines
        self.hot_file = _is_hot_file(path)
        self.stack: list[str] = []
        self.out: list[Violation] = []

    def _add(self, node: ast.AST, rule: str, message: str) -> None:
        line = getattr(node, "lineno", 1)
        end = getattr(node, "end_lineno", line) or line
        for ln in range(line, min(end, len(self.lines)) + 1):
            m = ALLOW.search(self.lines[ln - 1])
            if m and m.group(1) == rule:
                return
        self.out.append(Violation(self.path, line, rule, message))

    # ---- scopes
    def visit_FunctionDef(self, node):
        self.stack.append(node.name)
        self.generic_visit(node)
        self.stack.pop()

    visit_AsyncFunctionDef = visit_FunctionDef

    def _in_hot_function(self) -> bool:
        return self.hot_file and any(name in HOT_FUNCTIONS for name in self.stack)

    # ---- rules
    def visit_Import(self, node):
        for a in node.names:
            if a.name.split(".")[0] in FORBIDDEN_IMPORTS:
                self._add(node, "CL001", f"import of {a.name}")
        self.generic_visit(node)

    def visit_ImportFrom(self, node):
        if node.module and node.level == 0 and node.module.split(".")[0] in FORBIDDEN_IMPORTS:
            self._add(node, "CL001", f"import from {node.module}")
        self.generic_visit(node)

    def visit_ExceptHandler(self, node):
        if node.type is None:
            self._add(node, "EX001", "bare except")
        self.generic_visit(node)

    def visit_Call(self, node):
        f = node.func
        if isinstance(f, ast.Attribute):
            dotted = _dotted(f)
            if dotted == "torch.compile":
                self._add(node, "CL001", "torch.compile on the compute path")
            if self._in_hot_function():
                if f.attr in SYNC_METHODS and not node.args and not node.keywords:
                    self._add(node, "HS001", f".{f.attr}() synchronises the host inside {self.stack[-1]}()")
                elif dotted == "torch.cuda.synchronize":
                    self._add(node, "HS001", f"torch.cuda.synchronize() inside {self.stack[-1]}()")
        for kw in node.keywords:
            if kw.arg == "init_method" and isinstance(kw.value, ast.Constant) and isinstance(kw.value.value, str):
                self._check_addr(kw.value, kw.value.value.split("//")[-1].split(":")[0])
        for arg in node.args:
            self._check_command(arg)
        self.generic_visit(node)

    def visit_Assign(self, node):
        for t in node.targets:
            key = t.slice if isinstance(t, ast.Subscript) else None
            if isinstance(key, ast.Constant) and key.value == "MASTER_ADDR" and isinstance(node.value, ast.Constant) \
                    and isinstance(node.value.value, str):
                self._check_addr(node.value, node.value.value)
        self.generic_visit(node)

    def _check_addr(self, node, host: str) -> None:
        if host and not re.fullmatch(r"[0-9.]+|\[?[0-9a-fA-F:]+\]?", host):
            self._add(node, "RZ001", f"rendezvous host {host!r} is a name; use 127.0.0.1 or a literal address")

    def _check_command(self, node) -> None:
        words: list[str] = []
        if isinstance(node, ast.Constant) and isinstance(node.value, str):
            words = node.value.split()
        elif isinstance(node, (ast.List, ast.Tuple)):
            words = [e.value for e in node.elts if isinstance(e, ast.Constant) and isinstance(e.value, str)]
        if words and os.path.basename(words[0]) in PATTERN_KILLERS:
            self._add(node, "PK001", f"{words[0]} selects processes by pattern; signal the exact PID instead")


def _dotted(node: ast.AST) -> str:
    parts = []
    while isinstance(node, ast.Attribute):
        parts.append(node.attr)
        node = node.value
    if isinstance(node, ast.Name):
        parts.append(node.id)
    return ".".join(reversed(parts))


def lint_source(source: str, path: str = "<string>") -> list[Violation]:
    tree = ast.parse(source, filename=path)
    v = _Visitor(path, source.splitlines())
    v.visit(tree)
    return sorted(v.out, key=lambda x: (x.path, x.line, x.rule))


def lint_paths(paths) -> list[Violation]:
    out: list[Violation] = []
    for root in paths:
        files = [root] if os.path.isfile(root) else [os.path.join(d, f) for d, _, fs in os.walk(root) for f in fs if f.endswith(".py")]
        for f in sorted(files):
            with open(f, encoding="utf-8") as fh:
                out += lint_source(fh.read(), f)
    return out
