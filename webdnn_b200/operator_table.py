"""Operator registry: ``opType -> [OperatorEntry]`` and backend/opset matching.

Restates ``core/operatorTable.ts:15-69`` including the special placement of shape-like ops (they
run where their data tensor lives, and the LAST backend of the order that holds it wins because
the loop does not break) and ``Shape`` always running on the cpu.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence


@dataclass
class OperatorEntry:
    """interface/core/operator.ts:20-30; opset_min inclusive, opset_max exclusive (None = open)."""
    op_type: str
    opset_min: int
    opset_max: Optional[int]
    backend: str
    factory: Callable[[], object]
    domain: Optional[str] = None


_registered: Dict[str, List[OperatorEntry]] = {}


def register_operators(entries: Sequence[OperatorEntry]) -> None:
    for e in entries:
        _registered.setdefault(e.op_type, []).append(e)


def registered_op_types(backend: str) -> List[str]:
    return sorted(t for t, es in _registered.items() if any(e.backend == backend for e in es))


def clear_registry() -> None:
    _registered.clear()


def instantiate_operator(op_type: str, opset: int, backend_order: Sequence[str],
                         current_tensors_backends: Sequence[Sequence[str]]):
    entries = _registered.get(op_type)
    if not entries:
        return None
    local_order = list(backend_order)
    if op_type in ("Flatten", "Pad", "Reshape", "Squeeze", "Transpose", "Unsqueeze"):
        for backend in backend_order:
            if current_tensors_backends and backend in current_tensors_backends[0]:
                local_order = [backend]
    elif op_type == "Shape":
        local_order = ["cpu"]
    def pick(order):
        for backend in order:
            for e in entries:
                if e.backend != backend:
                    continue
                if e.opset_min > opset:
                    continue
                if e.opset_max is not None and e.opset_max <= opset:
                    continue
                return e.factory()
        return None

    op = pick(local_order)
    if op is None and local_order != list(backend_order):
        # The reference gets here with null, throws, and reruns the node on its cpu backend
        # (runnerImpl.ts:511-520).  This backend has no cpu kernels to fall back to, so a shape-like
        # node whose data sits on the cpu (a graph input) is given to the regular backend order and
        # its input is moved to the device.
        op = pick(backend_order)
    return op
