"""RPC autograd: ``with enable_grad():`` records forward handle calls and replays them backwards.

On exit the context walks the recorded calls in reverse and issues ``_auto_backward`` RPCs,
feeding each call the ``.grad`` handles accumulated on its outputs and storing the returned input
gradients on the input handles (fan-out accumulates).  Parity:
``unirl/distributed/tensor/grad_context.py:50-110`` (context), ``:119-178`` (backward sweep).
"""

from __future__ import annotations

import contextlib
from typing import Any, Iterator, List, Tuple

from unirl_b200.distributed.tensor.transport import TensorMeta
from unirl_b200.distributed.utils import iter_leaves


class GradContext:
    def __init__(self) -> None:
        self.records: List[Tuple[Any, str, List[TensorMeta], List[TensorMeta]]] = []
        self.handles: List[Any] = []

    def attach(self, handle: Any) -> None:
        if handle not in self.handles:
            self.handles.append(handle)
        handle._grad_ctx = self

    def record(self, handle: Any, call_id: str, args: tuple, kwargs: dict, out: Any) -> None:
        ins = [m for _, m, _ in iter_leaves([list(args), kwargs], TensorMeta) if m.dtype is not None and m.dtype.is_floating_point]
        outs = [m for _, m, _ in iter_leaves([out], TensorMeta)]
        self.records.append((handle, call_id, ins, outs))

    def backward(self) -> None:
        for handle, call_id, ins, outs in reversed(self.records):
            if not any(o.grad is not None for o in outs):
                continue
            handle._grad_ctx = None
            try:
                new = handle._auto_backward(call_id, tuple(o.grad for o in outs), tuple(i.grad for i in ins))
            finally:
                handle._grad_ctx = self
            for m, g in zip(ins, new):
                if g is not None:
                    m.grad = g
        self.records.clear()

    def close(self) -> None:
        for h in self.handles:
            h._grad_ctx = None
            try:
                h._cleanup_all_grads()
            except Exception:  # noqa: BLE001
                pass
        self.handles.clear()
        self.records.clear()


@contextlib.contextmanager
def enable_grad(*handles: Any) -> Iterator[GradContext]:
    ctx = GradContext()
    for h in handles:
        ctx.attach(h)
    try:
        yield ctx
    finally:
        ctx.close()


__all__ = ["GradContext", "enable_grad"]
