"""``ConfigNode`` — attribute/dict access tree with lazy ``${...}`` interpolation.

A minimal stand-in for OmegaConf's ``DictConfig`` (neither Hydra nor OmegaConf is a dependency):
supports ``cfg.a.b``, ``cfg["a"]``, ``cfg.get(k, default)``, ``in``, iteration, and the resolvers
used by the reference recipes — ``${oc.env:VAR}``, ``${oc.env:VAR,default}`` (nestable), ``${oc.decode:…}``,
``${path.to.key}`` absolute and ``${.sibling}`` / ``${..parent.key}`` relative references (``config/README.md`` of the reference describes the
recipe grammar: flat single-file YAML, every object a ``_target_`` node).
"""

from __future__ import annotations

import os
from typing import Any, Dict, Iterator, List, Optional

_MISSING = object()


def _parse_scalar(text: str) -> Any:
    import yaml

    try:
        return yaml.safe_load(text)
    except Exception:
        return text


class ConfigNode:
    __slots__ = ("_data", "_root", "_path")

    def __init__(self, data: Dict[str, Any], root: Optional["ConfigNode"] = None, path: tuple = ()):
        object.__setattr__(self, "_data", data)
        object.__setattr__(self, "_root", root if root is not None else self)
        object.__setattr__(self, "_path", tuple(path))  # keys from the root to this mapping: the anchor of relative references

    # ---- interpolation ------------------------------------------------------------------------
    def _lookup_path(self, path: str) -> Any:
        cur: Any = self._root._data
        for part in path.split("."):
            if isinstance(cur, dict) and part in cur:
                cur = cur[part]
            elif isinstance(cur, list) and part.isdigit():
                cur = cur[int(part)]
            else:
                raise KeyError(f"interpolation key '{path}' not found")
        return self._resolve(cur)

    def _resolve_expr(self, expr: str) -> Any:
        expr = expr.strip()
        if expr.startswith("oc.env:"):
            body = expr[len("oc.env:"):]
            name, default = _split_top_comma(body)
            val = os.environ.get(name.strip())
            if val is not None:
                return val
            if default is _MISSING:
                raise KeyError(f"environment variable '{name.strip()}' is not set and has no default")
            d = self._resolve_str(default.strip())
            if isinstance(d, str) and d.lower() in ("null", "none", "~"):
                return None
            return d if d is None else str(d)
        if expr.startswith("oc.decode:"):  # a string (typically from the environment) read as a YAML scalar: "true" -> True, "3" -> 3, "null" -> None
            inner = self._resolve_str(expr[len("oc.decode:"):].strip())
            return _parse_scalar(inner) if isinstance(inner, str) else inner
        if expr.startswith("oc.select:"):
            name, default = _split_top_comma(expr[len("oc.select:"):])
            try:
                return self._lookup_path(name.strip())
            except KeyError:
                return None if default is _MISSING else _parse_scalar(default.strip())
        if expr.startswith("."):  # relative reference: ``${.key}`` a sibling in this mapping, ``${..key}`` one in the mapping above, ...
            ups = len(expr) - len(expr.lstrip("."))
            if ups - 1 > len(self._path):
                raise KeyError(f"relative interpolation '{expr}' climbs above the root from '{'.'.join(self._path)}'")
            base = self._path[: len(self._path) - (ups - 1)]
            return self._lookup_path(".".join([*base, expr[ups:]]))
        return self._lookup_path(expr)

    def _resolve_str(self, s: str) -> Any:
        if "${" not in s:
            return s
        out: List[Any] = []
        i = 0
        while i < len(s):
            j = s.find("${", i)
            if j < 0:
                out.append(s[i:])
                break
            if j > i:
                out.append(s[i:j])
            depth, k = 0, j
            while k < len(s):
                if s.startswith("${", k):
                    depth += 1
                    k += 2
                    continue
                if s[k] == "}":
                    depth -= 1
                    if depth == 0:
                        break
                k += 1
            if depth:
                raise ValueError(f"unbalanced interpolation in {s!r}")
            out.append(self._resolve_expr(s[j + 2 : k]))
            i = k + 1
        if len(out) == 1:
            return out[0]
        return "".join("" if o is None else str(o) for o in out)

    def _resolve(self, v: Any) -> Any:
        return self._resolve_str(v) if isinstance(v, str) else v

    def _wrap(self, v: Any, key: Optional[str] = None) -> Any:
        path = self._path if key is None else (*self._path, str(key))
        if isinstance(v, str) and v.startswith("${") and v.endswith("}") and v.count("${") == 1 and ":" not in v:
            # a whole-value reference (``params: ${sampling}``) stands for the node it names: relative references inside that node keep
            # resolving against the place the node lives at, not the place it is referenced from
            ref = v[2:-1].strip()
            if ref.startswith("."):
                ups = len(ref) - len(ref.lstrip("."))
                ref = ".".join([*self._path[: len(self._path) - (ups - 1)], ref[ups:]]) if ups - 1 <= len(self._path) else ref
            if not ref.startswith("."):
                path = tuple(ref.split("."))
        v = self._resolve(v)
        if isinstance(v, dict):
            return ConfigNode(v, self._root, path)
        if isinstance(v, list):
            holder = ConfigNode({}, self._root, path)  # entries of a list resolve relative references like the list's own mapping level
            return [holder._wrap(x, str(i)) if isinstance(x, dict) else self._wrap(x) for i, x in enumerate(v)]
        return v

    # ---- mapping API ----------------------------------------------------------------------------
    def __getattr__(self, key: str) -> Any:
        if key.startswith("__"):
            raise AttributeError(key)
        if key not in self._data:
            raise AttributeError(f"config has no key '{key}'")
        return self[key]

    def __setattr__(self, key: str, value: Any) -> None:
        self._data[key] = to_container(value)

    def __getitem__(self, key: str) -> Any:
        return self._wrap(self._data[key], key)

    def __setitem__(self, key: str, value: Any) -> None:
        self._data[key] = to_container(value)

    def __contains__(self, key: object) -> bool:
        return key in self._data

    def __iter__(self) -> Iterator[str]:
        return iter(self._data)

    def __len__(self) -> int:
        return len(self._data)

    def keys(self):
        return self._data.keys()

    def items(self):
        return [(k, self[k]) for k in self._data]

    def values(self):
        return [self[k] for k in self._data]

    def get(self, key: str, default: Any = None) -> Any:
        if key not in self._data:
            return default
        v = self[key]
        return default if v is None else v

    def __repr__(self) -> str:
        return f"ConfigNode({self._data!r})"

    def __reduce__(self):
        return (ConfigNode, (to_container(self, resolve=True),))


def _split_top_comma(body: str):
    depth = 0
    for i, ch in enumerate(body):
        if body.startswith("${", i):
            depth += 1
        elif ch == "}" and depth:
            depth -= 1
        elif ch == "," and depth == 0:
            return body[:i], body[i + 1 :]
    return body, _MISSING


def to_container(cfg: Any, resolve: bool = True) -> Any:
    """Plain ``dict``/``list`` copy of a config tree (interpolations resolved when asked)."""
    if isinstance(cfg, ConfigNode):
        if resolve:
            return {k: to_container(cfg[k], True) for k in cfg._data}
        return _deep_plain(cfg._data)
    if isinstance(cfg, dict):
        return {k: to_container(v, resolve) for k, v in cfg.items()}
    if isinstance(cfg, (list, tuple)):
        return [to_container(v, resolve) for v in cfg]
    return cfg


def _deep_plain(v: Any) -> Any:
    if isinstance(v, dict):
        return {k: _deep_plain(x) for k, x in v.items()}
    if isinstance(v, list):
        return [_deep_plain(x) for x in v]
    return v


def is_config(obj: Any) -> bool:
    return isinstance(obj, ConfigNode)


__all__ = ["ConfigNode", "to_container", "is_config"]
