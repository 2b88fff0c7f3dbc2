"""Recipe loading + Hydra-style command line (``--config-dir``, ``--config-name``, ``k=v``, ``+k=v``, ``~k``)."""

from __future__ import annotations

import copy
import functools
import os
import sys
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import yaml

from unirl_b200.config.node import ConfigNode, _parse_scalar

_REPO_EXAMPLES = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "examples")


def _set_path(data: Dict[str, Any], dotted: str, value: Any, *, must_exist: bool) -> None:
    parts = dotted.split(".")
    cur = data
    for p in parts[:-1]:
        if p not in cur or not isinstance(cur[p], dict):
            if must_exist:
                raise KeyError(f"override '{dotted}': '{p}' not in config (prefix with '+' to add)")
            cur[p] = {}
        cur = cur[p]
    if must_exist and parts[-1] not in cur:
        raise KeyError(f"override '{dotted}': key not in config (prefix with '+' to add)")
    cur[parts[-1]] = value


def _del_path(data: Dict[str, Any], dotted: str) -> None:
    parts = dotted.split(".")
    cur = data
    for p in parts[:-1]:
        cur = cur[p]
    cur.pop(parts[-1], None)


def apply_overrides(data: Dict[str, Any], overrides: Sequence[str]) -> Dict[str, Any]:
    for ov in overrides:
        if ov.startswith("~"):
            _del_path(data, ov[1:].split("=")[0])
            continue
        if "=" not in ov:
            raise ValueError(f"malformed override '{ov}' (expected key=value)")
        key, raw = ov.split("=", 1)
        add = key.startswith("+")
        key = key.lstrip("+")
        _set_path(data, key, _parse_scalar(raw), must_exist=not add)
    return data


def load_recipe(path: str) -> Dict[str, Any]:
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    if not isinstance(data, dict):
        raise ValueError(f"recipe {path} must be a mapping at top level")
    return data


def compose(config_name: str, config_dir: Optional[str] = None, overrides: Sequence[str] = ()) -> ConfigNode:
    """Load ``<config_dir>/<config_name>.yaml`` and apply overrides."""
    base = config_dir or _REPO_EXAMPLES
    candidates = [config_name, os.path.join(base, config_name), os.path.join(base, config_name + ".yaml")]
    for c in candidates:
        if os.path.isfile(c):
            return ConfigNode(apply_overrides(load_recipe(c), overrides))
    raise FileNotFoundError(f"recipe '{config_name}' not found (looked in {base})")


def parse_cli(argv: Sequence[str]) -> Tuple[Optional[str], Optional[str], List[str], Dict[str, bool]]:
    name = cdir = None
    overrides: List[str] = []
    flags = {"cfg": False, "resolve": False}
    it = iter(argv)
    for a in it:
        if a in ("--config-name", "-cn"):
            name = next(it)
        elif a.startswith("--config-name="):
            name = a.split("=", 1)[1]
        elif a in ("--config-dir", "-cd", "--config-path", "-cp"):
            cdir = next(it)
        elif a.startswith("--config-dir=") or a.startswith("--config-path="):
            cdir = a.split("=", 1)[1]
        elif a in ("--cfg", "-c"):
            flags["cfg"] = True
            next(it, None)
        elif a == "--resolve":
            flags["resolve"] = True
        elif a == "--profile":  # bracket a window of steps for a profiler and emit NVTX ranges (utils/profiling.py)
            overrides.append("+profile.enabled=true")
        elif a.startswith("--profile="):  # --profile=START:COUNT
            st, _, cnt = a.split("=", 1)[1].partition(":")
            overrides += ["+profile.enabled=true", f"+profile.start_step={int(st or 3)}", f"+profile.num_steps={int(cnt or 1)}"]
        elif a.endswith((".yaml", ".yml")) and name is None and "=" not in a:
            name = a
        else:
            overrides.append(a)
    return name, cdir, overrides, flags


def main_entry(default_config: Optional[str] = None) -> Callable[[Callable[[ConfigNode], Any]], Callable[..., Any]]:
    """Decorator playing the part of ``@hydra.main(config_path=None)``."""

    def deco(fn: Callable[[ConfigNode], Any]) -> Callable[..., Any]:
        @functools.wraps(fn)
        def wrapper(argv: Optional[Sequence[str]] = None) -> Any:
            name, cdir, overrides, flags = parse_cli(sys.argv[1:] if argv is None else argv)
            name = name or default_config
            if name is None:
                raise SystemExit("no recipe given: pass --config-name=<domain>/<recipe> or a .yaml path")
            cfg = compose(name, cdir, overrides)
            if flags["cfg"]:
                from unirl_b200.config.node import to_container

                print(yaml.safe_dump(to_container(cfg, resolve=flags["resolve"]), sort_keys=False))
                return None
            if bool(cfg.get("validate", False)) or os.environ.get("UNIRL_B200_VALIDATE") == "1":
                from unirl_b200.config.validation import validate_recipe

                validate_recipe(cfg)
            return fn(cfg)

        return wrapper

    return deco


__all__ = ["compose", "load_recipe", "apply_overrides", "parse_cli", "main_entry"]
