"""``_target_`` resolution and instantiation.

``parse_cfg`` mirrors the reference's split of labour ("driver routes, worker materialises",
``unirl/utils/hydra.py:24-71``): it resolves only the top-level ``_target_`` to a class and leaves
nested ``_target_`` dicts as plain data for the worker to build inside its own CUDA context.
"""

from __future__ import annotations

import functools
import importlib
from typing import Any, Callable, Dict

from unirl_b200.config.node import ConfigNode, to_container

RESERVED = frozenset({"_target_", "_partial_", "_recursive_", "_convert_", "_args_"})

from unirl_b200.config.aliases import translate as _translate  # noqa: E402  (name tables for recipes written for the reference)


def get_method(path: str) -> Any:
    """Import ``pkg.mod.Attr[.attr…]`` and return the object (class, function or classmethod)."""
    path = _translate(path)
    parts = path.split(".")
    for cut in range(len(parts) - 1, 0, -1):
        try:
            obj: Any = importlib.import_module(".".join(parts[:cut]))
        except ModuleNotFoundError as e:
            if e.name and ".".join(parts[:cut]).startswith(e.name):
                continue
            raise
        rest = parts[cut:]
        # a model family keeps bundle / config / pipeline / diffusion classes in fewer files than the reference: a name asked for under
        # ``models.<family>.<file>.<Class>`` is looked up in the family's package when ``<file>`` is not a module of it
        if len(rest) >= 2 and parts[:cut][-2:-1] == ["models"] and not hasattr(obj, rest[0]) and hasattr(obj, rest[1]):
            rest = rest[1:]
        for attr in rest:
            obj = getattr(obj, attr)
        return obj
    raise ImportError(f"cannot resolve target '{path}'")


def get_class(path: str) -> type:
    obj = get_method(path)
    if not isinstance(obj, type):
        raise ValueError(f"'{path}' is not a class")
    return obj


def call_target(fn: Any, *pos: Any, **kw: Any) -> Any:
    """Call a recipe target.  A configuration dataclass that declares ``__extra_fields_ok__ = True`` (the model packages' pipeline
    configurations) also takes fields it does not declare: recipes written for the reference carry settings of its own loaders there
    (``use_lora``, ``lora_target_modules``, ``freeze_…``).  Such fields are kept as plain attributes of the object and named once in the log."""
    import dataclasses

    if isinstance(fn, type) and dataclasses.is_dataclass(fn) and getattr(fn, "__extra_fields_ok__", False):
        known = {f.name for f in dataclasses.fields(fn) if f.init}
        extra = {k: kw.pop(k) for k in list(kw) if k not in known}
        obj = fn(*pos, **kw)
        if extra:
            import logging

            for k, v in extra.items():
                setattr(obj, k, v)
            logging.getLogger(__name__).info("%s: fields without a declaration kept as attributes: %s", fn.__name__, sorted(extra))
        return obj
    return fn(*pos, **kw)


def instantiate(node: Any, *args: Any, _recursive_: bool = True, **overrides: Any) -> Any:
    """Build the object a ``{_target_: …}`` node describes (nested nodes first)."""
    if isinstance(node, ConfigNode):
        node = to_container(node, resolve=True)
    if isinstance(node, list):
        return [instantiate(x) if _recursive_ else x for x in node]
    if not isinstance(node, dict):
        return node
    if "_target_" not in node:
        return {k: instantiate(v) if _recursive_ else v for k, v in node.items()}
    recursive = bool(node.get("_recursive_", _recursive_))
    fn = get_method(node["_target_"])
    kw: Dict[str, Any] = {}
    for k, v in node.items():
        if k in RESERVED:
            continue
        kw[k] = instantiate(v) if recursive and isinstance(v, (dict, list)) else v
    kw.update(overrides)
    pos = list(node.get("_args_", [])) + list(args)
    if node.get("_partial_"):
        return functools.partial(fn, *pos, **kw)
    return call_target(fn, *pos, **kw)


def parse_cfg(cfg: Any) -> Dict[str, Any]:
    """``{"role_cls": <class or factory>, **plain fields}`` ready for ``remote(**…)``."""
    plain = to_container(cfg, resolve=True) if isinstance(cfg, ConfigNode) else dict(cfg)
    target = plain.get("_target_")
    if target is None:
        raise ValueError("config node has no _target_")
    if "role_cls" in plain:
        raise ValueError("config field 'role_cls' collides with remote()'s parameter")
    return {"role_cls": get_method(target), **{k: v for k, v in plain.items() if k not in RESERVED}}


parse_hydra_cfg = parse_cfg

__all__ = ["get_method", "get_class", "instantiate", "call_target", "parse_cfg", "parse_hydra_cfg", "RESERVED"]
