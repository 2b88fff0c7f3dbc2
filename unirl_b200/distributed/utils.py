"""Small helpers shared by the dispatch and transport layers.

Parity: ``unirl/distributed/utils.py:25-95`` (``Broadcast``, ``collect_leaves``).
"""

from __future__ import annotations

import socket
from typing import Any, Callable, Dict, Iterator, List, Tuple


class Broadcast:
    """Marks a call argument as "replicate to every worker, never split along dim 0"."""

    __slots__ = ("value",)

    def __init__(self, value: Any):
        self.value = value

    def __repr__(self) -> str:
        return f"Broadcast({self.value!r})"


def free_port(host: str = "127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return int(s.getsockname()[1])


def iter_leaves(tree: Any, leaf_type: type, path: str = "") -> Iterator[Tuple[str, Any, Callable[[Any], None]]]:
    """Depth-first walk yielding ``(path, leaf, setter)`` for every ``leaf_type`` instance.

    Containers walked: ``Batch`` dataclasses (declared fields), dicts (sorted keys for
    deterministic order across processes), lists.  ``setter(new)`` writes a replacement into the
    parent container in place; a root-level leaf has a no-op setter (use :func:`map_leaves`).
    """
    from unirl_b200.distributed.tensor.batch import Batch
    import dataclasses

    if isinstance(tree, leaf_type):
        yield path, tree, lambda _new: None
        return

    def children(node: Any):
        if isinstance(node, Batch):
            for f in dataclasses.fields(node):
                yield f.name, getattr(node, f.name), (lambda v, o=node, a=f.name: setattr(o, a, v))
        elif isinstance(node, dict):
            for k in sorted(node, key=str):
                yield str(k), node[k], (lambda v, d=node, kk=k: d.__setitem__(kk, v))
        elif isinstance(node, list):
            for i, v in enumerate(node):
                yield str(i), v, (lambda nv, l=node, ii=i: l.__setitem__(ii, nv))
        elif isinstance(node, tuple):  # immutable: leaves are reported, setters are no-ops
            for i, v in enumerate(node):
                yield str(i), v, (lambda nv: None)

    for name, child, setter in children(tree):
        sub = f"{path}.{name}" if path else name
        if child is None:
            continue
        if isinstance(child, leaf_type):
            yield sub, child, setter
        else:
            yield from iter_leaves(child, leaf_type, sub)


def collect_leaves(tree: Any, leaf_type: type) -> Dict[str, Any]:
    return {p: leaf for p, leaf, _ in iter_leaves(tree, leaf_type)}


def map_leaves(tree: Any, leaf_type: type, fn: Callable[[Any], Any]) -> Any:
    """Functional leaf substitution: returns a tree where every ``leaf_type`` leaf is ``fn(leaf)``.

    Containers on a changed path are shallow-copied (the input tree is never mutated), untouched
    subtrees are shared.  ``Batch`` nodes keep their hidden ``cu_seqlens``.
    """
    from unirl_b200.distributed.tensor.batch import Batch
    import copy
    import dataclasses

    if isinstance(tree, leaf_type):
        return fn(tree)
    if isinstance(tree, Batch):
        out = None
        for f in dataclasses.fields(tree):
            v = getattr(tree, f.name)
            if v is None:
                continue
            nv = map_leaves(v, leaf_type, fn)
            if nv is not v:
                if out is None:
                    out = copy.copy(tree)
                setattr(out, f.name, nv)
        return tree if out is None else out
    if isinstance(tree, dict):
        new = {k: map_leaves(v, leaf_type, fn) for k, v in tree.items()}
        return new if any(new[k] is not tree[k] for k in tree) else tree
    if isinstance(tree, (list, tuple)):
        new_seq = [map_leaves(v, leaf_type, fn) for v in tree]
        if all(a is b for a, b in zip(new_seq, tree)):
            return tree
        return type(tree)(new_seq) if not hasattr(tree, "_fields") else type(tree)(*new_seq)
    return tree


__all__ = ["Broadcast", "free_port", "iter_leaves", "collect_leaves", "map_leaves"]
