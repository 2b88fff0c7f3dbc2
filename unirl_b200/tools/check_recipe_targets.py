"""Static recipe check: every ``_target_:`` in every YAML under a directory must name a real symbol.

Resolution is by AST only — the module file is located on disk and parsed, nothing is imported, so
the check runs without torch or a GPU (the reference wires the same idea as a pre-commit hook,
``scripts/check_recipe_targets.py``).  ``python -m unirl_b200.tools.check_recipe_targets [dir]``.
"""

from __future__ import annotations

import ast
import os
import sys
from typing import Any, Iterator, List, Optional

import yaml

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_EXTERNAL_OK = ("builtins.", "collections.", "hydra.utils.get_class", "hydra.utils.get_method")


def _targets(node: Any) -> Iterator[str]:
    if isinstance(node, dict):
        for k, v in node.items():
            if k == "_target_" and isinstance(v, str):
                yield v
            else:
                yield from _targets(v)
    elif isinstance(node, list):
        for v in node:
            yield from _targets(v)


def _module_file(parts: List[str]) -> Optional[str]:
    base = os.path.join(_ROOT, *parts)
    if os.path.isfile(base + ".py"):
        return base + ".py"
    if os.path.isfile(os.path.join(base, "__init__.py")):
        return os.path.join(base, "__init__.py")
    return None


def _defines(path: str, names: List[str]) -> bool:
    with open(path) as f:
        tree = ast.parse(f.read())
    scope = tree.body
    inherited = False
    for depth, name in enumerate(names):
        found = None
        for n in scope:
            if isinstance(n, (ast.ClassDef, ast.FunctionDef, ast.AsyncFunctionDef)) and n.name == name:
                found = n
            elif isinstance(n, ast.Assign) and any(isinstance(t, ast.Name) and t.id == name for t in n.targets):
                found = n
            elif isinstance(n, (ast.Import, ast.ImportFrom)) and any((a.asname or a.name.split(".")[0]) == name for a in n.names):
                found = n
        if found is None:
            return inherited  # a name missing from a class body may come from a base class
        inherited = isinstance(found, ast.ClassDef) and bool(found.bases)
        if isinstance(found, ast.ClassDef):
            scope = found.body
        elif depth < len(names) - 1:
            return True  # attribute of an imported / assigned object: cannot look further statically
    return True


def _translate(target: str) -> str:
    """The name tables of ``config/aliases.py``, loaded from its file (pure data: no package import, so no torch)."""
    global _ALIAS_NS
    if _ALIAS_NS is None:
        import runpy

        _ALIAS_NS = runpy.run_path(os.path.join(_ROOT, "unirl_b200", "config", "aliases.py"))
    return _ALIAS_NS["translate"](target)


_ALIAS_NS: Any = None


def resolve(target: str) -> bool:
    if target.startswith(_EXTERNAL_OK):
        return True
    parts = _translate(target).split(".")
    for cut in range(len(parts) - 1, 0, -1):
        f = _module_file(parts[:cut])
        if f is not None:
            rest = parts[cut:]
            if _defines(f, rest):
                return True
            # a model family keeps its classes in fewer files than the reference: ``models.<family>.<file>.<Class>`` → the family's package
            return len(rest) >= 2 and parts[:cut][-2:-1] == ["models"] and _defines(f, rest[1:])
    return False


def check_tree(root: str) -> List[str]:
    problems: List[str] = []
    for dirpath, _d, files in os.walk(root):
        for fn in sorted(files):
            if not fn.endswith((".yaml", ".yml")):
                continue
            path = os.path.join(dirpath, fn)
            with open(path) as f:
                try:
                    doc = yaml.safe_load(f)
                except yaml.YAMLError as e:
                    problems.append(f"{path}: YAML error {e}")
                    continue
            for t in _targets(doc):
                if not resolve(t):
                    problems.append(f"{path}: unresolved _target_ '{t}'")
    return problems


def main(argv: Optional[List[str]] = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    bad = check_tree(argv[0] if argv else os.path.join(_ROOT, "examples"))
    for p in bad:
        print(p)
    print(f"{len(bad)} problem(s)")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
