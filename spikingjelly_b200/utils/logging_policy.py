"""Lint for the package's logging conventions (the job of the reference's ``tools/check_logging_policy.py``):

* library code reports through the package logger (``spikingjelly_b200.logger.logger``): no ``print`` / ``pprint``, no writes to
  ``sys.stdout`` / ``sys.stderr``, no calls on the root ``logging`` module, no handler or ``basicConfig`` set-up, no private
  ``logging.getLogger(...)`` outside ``logger.py``;
* log calls pass arguments lazily (``logger.info("x=%s", x)``): a message built eagerly with ``%``, ``+``, ``str.format`` or an
  f-string costs its formatting even when the level is filtered out.

Examples, benchmarks, command-line entry points (``__main__`` blocks and functions named ``main``) and diagnostic helpers
listed in :data:`ALLOWED_PRINT_FUNCTIONS` may print.

    python -m spikingjelly_b200.utils.logging_policy [root]        # exit code 1 and one line per violation
"""
from __future__ import annotations

import ast
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterator, List, Optional, Sequence

__all__ = ["Violation", "check_source", "check_tree", "main", "ALLOWED_PRINT_FUNCTIONS"]

LOG_LEVELS = ("debug", "info", "warning", "warn", "error", "exception", "critical", "log")
SETUP_CALLS = ("basicConfig", "dictConfig", "fileConfig", "StreamHandler", "FileHandler")
#: directories whose files are scripts for people to read output from
SCRIPT_DIRS = ("examples", "example", "benchmark", "tests", "test", "docs")
#: functions whose purpose is to print a report for a person (surrogate gradient checks, model summaries)
ALLOWED_PRINT_FUNCTIONS = ("main", "check_manual_grad", "check_cuda_grad", "plot_surrogate_function", "print_summary")


@dataclass(frozen=True)
class Violation:
    path: str
    line: int
    rule: str
    detail: str

    def __str__(self) -> str:
        return f"{self.path}:{self.line}: [{self.rule}] {self.detail}"


def _dotted(node: ast.AST) -> Optional[str]:
    """``a.b.c`` for a chain of plain attribute accesses, else None."""
    parts = []
    while isinstance(node, ast.Attribute):
        parts.append(node.attr)
        node = node.value
    if isinstance(node, ast.Name):
        parts.append(node.id)
        return ".".join(reversed(parts))
    return None


def _eager(message: ast.AST) -> Optional[str]:
    if isinstance(message, ast.JoinedStr):
        return "f-string"
    if isinstance(message, ast.BinOp) and isinstance(message.op, (ast.Mod, ast.Add)):
        return "'%' formatting" if isinstance(message.op, ast.Mod) else "string concatenation"
    if isinstance(message, ast.Call) and isinstance(message.func, ast.Attribute) and message.func.attr == "format":
        return "str.format"
    return None


class _Rule:
    def __init__(self, name: str, test: Callable[[ast.Call, str, "_Context"], Optional[str]]):
        self.name, self.test = name, test


@dataclass
class _Context:
    is_logger_module: bool
    may_print: bool


def _rule_print(call, name, ctx):
    if name in ("print", "pprint", "builtins.print", "pprint.pprint") and not ctx.may_print:
        return f"direct {name}() in library code"


def _rule_stream(call, name, ctx):
    if name in ("sys.stdout.write", "sys.stderr.write") and not ctx.may_print:
        return f"direct {name}()"


def _rule_root_logging(call, name, ctx):
    if name.startswith("logging.") and name.split(".", 1)[1] in LOG_LEVELS:
        return f"{name}() logs through the root logger; use the package logger"


def _rule_setup(call, name, ctx):
    if name.startswith("logging.") and name.split(".", 1)[1] in SETUP_CALLS:
        return f"{name}() configures logging; that is the application's decision"
    if name == "logging.NullHandler" and not ctx.is_logger_module:
        return "logging.NullHandler() outside logger.py"


def _rule_private_logger(call, name, ctx):
    if name == "logging.getLogger" and not ctx.is_logger_module:
        return "logging.getLogger() outside logger.py; import `logger` from the package's logger module"


def _rule_lazy(call, name, ctx):
    head, _, level = name.rpartition(".")
    if head.split(".")[-1] in ("logger", "log", "_logger") and level in LOG_LEVELS and call.args:
        first = call.args[1] if level == "log" and len(call.args) > 1 else call.args[0]
        how = _eager(first)
        if how is not None:
            return f"log message built eagerly ({how}); pass the values as arguments instead"


RULES: Sequence[_Rule] = (_Rule("print", _rule_print), _Rule("stream-write", _rule_stream), _Rule("root-logger", _rule_root_logging),
                          _Rule("logging-setup", _rule_setup), _Rule("private-logger", _rule_private_logger),
                          _Rule("eager-format", _rule_lazy))


def _calls_with_scope(tree: ast.AST) -> Iterator[tuple]:
    """``(call node, names of the enclosing functions, inside an `if __name__ == "__main__"` block?)``."""
    def walk(node, funcs, in_main):
        for child in ast.iter_child_nodes(node):
            f, m = funcs, in_main
            if isinstance(child, (ast.FunctionDef, ast.AsyncFunctionDef)):
                f = funcs + (child.name,)
            elif isinstance(child, ast.If) and isinstance(child.test, ast.Compare) and _dotted(child.test.left) == "__name__":
                m = True
            if isinstance(child, ast.Call):
                yield child, f, m
            yield from walk(child, f, m)
    yield from walk(tree, (), False)


def check_source(source: str, path: str = "<string>", *, is_logger_module: bool = False, is_script: bool = False) -> List[Violation]:
    try:
        tree = ast.parse(source)
    except SyntaxError as problem:
        return [Violation(path, problem.lineno or 0, "syntax", str(problem))]
    found = []
    for call, funcs, in_main in _calls_with_scope(tree):
        name = _dotted(call.func)
        if name is None:
            continue
        ctx = _Context(is_logger_module, is_script or in_main or any(f in ALLOWED_PRINT_FUNCTIONS for f in funcs))
        for rule in RULES:
            detail = rule.test(call, name, ctx)
            if detail:
                found.append(Violation(path, call.lineno, rule.name, detail))
    return found


def check_tree(root) -> List[Violation]:
    """Lint every ``*.py`` below ``root`` (a package directory)."""
    root = Path(root)
    found: List[Violation] = []
    for path in sorted(root.rglob("*.py")):
        rel = path.relative_to(root)
        script = any(part in SCRIPT_DIRS for part in rel.parts[:-1]) or path.name.endswith("_example.py")
        found += check_source(path.read_text(encoding="utf-8"), str(path), is_logger_module=rel.as_posix() == "logger.py", is_script=script)
    return found


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    root = Path(args[0]) if args else Path(__file__).resolve().parents[1]
    found = check_tree(root)
    for v in found:
        print(v)
    print(f"{len(found)} violation(s) under {root}")
    return 1 if found else 0


if __name__ == "__main__":
    raise SystemExit(main())
