"""Host-side ("cpu" backend) operators for shape tensors only.

WebDNN always keeps a cpu context next to the device backend (``index.ts:52-56,140-142``): ``Shape``
is pinned to it (``core/operatorTable.ts:48-51``), ``Constant`` produces cpu tensors, and the
reshape-like ops take their shape/axes operands from it.  This module registers exactly those
bookkeeping ops so that shape-computation sub-graphs of an exported model run where the reference
runs them.  No arithmetic operator of the hot path (Conv, Gemm, MatMul, pooling, Softmax,
reductions, unary/binary math on float tensors ...) is registered here: a graph node of such a type
that cannot run on ``cuda`` fails instead of falling back.
"""
from __future__ import annotations

from typing import List

import numpy as np

from ..backend import CPUTensor
from ..onnx_io import FLOAT, INT32, INT64, clip_long
from ..operator_table import OperatorEntry
from . import base
from .base import OperatorImpl, get_attr_int, get_attr_ints, get_attr_tensor

_MAX_HOST_ELEMENTS = 4096  # shape tensors are tiny; anything larger belongs on the device


def _small(t: CPUTensor, who: str) -> None:
    if t.length > _MAX_HOST_ELEMENTS:
        raise RuntimeError(f"{who}: tensor of {t.length} elements will not be processed on the host")


class HostShape(OperatorImpl):
    """operators/cpu/operators/standard/shape.ts:12-26: needs only the dims, from any backend."""

    def __init__(self):
        super().__init__("cpu")

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return [None]

    def run(self, context, inputs, n_outputs):
        dims = inputs[0].dims
        return [context.empty_tensor([len(dims)], "int32", np.asarray(dims, dtype=np.int32))]


class HostConstant(OperatorImpl):
    def __init__(self):
        super().__init__("cpu")

    def initialize(self, attribute):
        t = get_attr_tensor(attribute, "value")
        if t is None:
            raise ValueError("Constant: only the tensor-valued form is supported")
        if t.data_type == FLOAT:
            self.value = ("float32", t.dims, t.array.astype(np.float32))
        elif t.data_type == INT64:
            self.value = ("int32", t.dims, np.asarray([clip_long(int(v)) for v in t.array], dtype=np.int32))
        elif t.data_type == INT32:
            self.value = ("int32", t.dims, t.array.astype(np.int32))
        else:
            raise ValueError(f"Constant: dataType {t.data_type} is not supported")

    def run(self, context, inputs, n_outputs):
        dt, dims, arr = self.value
        return [context.empty_tensor(dims, dt, arr.copy())]


class HostConstantOfShape(OperatorImpl):
    def __init__(self):
        super().__init__("cpu")

    def initialize(self, attribute):
        t = get_attr_tensor(attribute, "value")
        if t is None:
            self.dt, self.v = "float32", 0.0
        elif t.data_type == FLOAT:
            self.dt, self.v = "float32", float(t.array[0])
        else:
            self.dt, self.v = "int32", clip_long(int(t.array[0]))

    def run(self, context, inputs, n_outputs):
        dims = [int(v) for v in inputs[0].data]
        n = int(np.prod(dims)) if dims else 1
        if n > _MAX_HOST_ELEMENTS:
            raise RuntimeError("ConstantOfShape: too large for the host")
        return [context.empty_tensor(dims, self.dt, np.full(n, self.v, dtype=np.float32 if self.dt == "float32" else np.int32))]


class HostReshapeLike(OperatorImpl):
    """cpu reshape5/flatten/squeeze/unsqueeze: new dims over the same array (reshape5.ts:20-27)."""

    def __init__(self, kind: str):
        super().__init__("cpu")
        self.kind = kind

    def initialize(self, attribute):
        if self.kind == "Flatten":
            self.helper = base.Flatten("cpu")
            self.helper.initialize(attribute)
        elif self.kind == "Reshape":
            self.helper = base.Reshape5("cpu")
            self.helper.initialize(attribute)
        else:
            self.axes = get_attr_ints(attribute, "axes", [])

    def run(self, context, inputs, n_outputs):
        x = inputs[0]
        if self.kind == "Flatten":
            dims = self.helper.calc_shape(x)
        elif self.kind == "Reshape":
            dims = self.helper.calc_shape(x, inputs[1])
        else:
            axes = [int(a) for a in inputs[1].data] if len(inputs) > 1 else self.axes
            dims = base.squeeze_shape(x.dims, axes) if self.kind == "Squeeze" else base.unsqueeze_shape(x.dims, axes)
        return [context.empty_tensor(dims, x.data_type, x.data)]


class HostGather(OperatorImpl):
    """gather.ts:20-33: scalar pick from a 1-D tensor only."""

    def __init__(self):
        super().__init__("cpu")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", 0)

    def run(self, context, inputs, n_outputs):
        data, indices = inputs
        if not (data.ndim == 1 and indices.ndim == 0 and self.axis == 0):
            raise ValueError("Gather: currently supports data.ndim === 1 && indices.ndim === 0 && axis === 0")
        return [context.empty_tensor([], data.data_type, data.data[[int(indices.data[0])]].copy())]


class HostConcat(OperatorImpl):
    def __init__(self):
        super().__init__("cpu")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", 0)

    def run(self, context, inputs, n_outputs):
        for t in inputs:
            _small(t, "Concat")
        axis = self.axis if self.axis >= 0 else inputs[0].ndim + self.axis
        out = np.concatenate([t.numpy() for t in inputs], axis=axis)
        return [context.empty_tensor(list(out.shape), inputs[0].data_type, np.ascontiguousarray(out).reshape(-1))]


class HostCast(OperatorImpl):
    def __init__(self):
        super().__init__("cpu")

    def initialize(self, attribute):
        self.to = get_attr_int(attribute, "to", 1)

    def run(self, context, inputs, n_outputs):
        x = inputs[0]
        _small(x, "Cast")
        if self.to == 1:
            return [context.empty_tensor(x.dims, "float32", x.data.astype(np.float32))]
        if self.to in (2, 6, 7):
            if x.data_type == "int32":
                return [context.empty_tensor(x.dims, "int32", x.data.copy())]
            d = x.data.astype(np.float64)
            t = np.where(np.isfinite(d), np.trunc(d), 0.0)
            m = np.mod(t, 4294967296.0)
            m = np.where(m >= 2147483648.0, m - 4294967296.0, m)
            return [context.empty_tensor(x.dims, "int32", m.astype(np.int32))]
        raise ValueError(f"Cast: converting to DataType {self.to} is not yet supported")


class HostIntBinary(OperatorImpl):
    """Add/Sub/Mul/Div on int32 shape tensors (binary7.ts semantics: double math, ToInt32 store)."""

    def __init__(self, op: str):
        super().__init__("cpu")
        self.op = op

    def run(self, context, inputs, n_outputs):
        a, b = inputs
        _small(a, self.op)
        _small(b, self.op)
        if a.data_type != "int32" or b.data_type != "int32":
            raise TypeError(f"{self.op}: the host backend only handles int32 shape tensors")
        x, y = np.broadcast_arrays(a.numpy().astype(np.float64), b.numpy().astype(np.float64))
        with np.errstate(all="ignore"):
            r = {"Add": x + y, "Sub": x - y, "Mul": x * y, "Div": x / y}[self.op]
        t = np.where(np.isfinite(r), np.trunc(r), 0.0)
        m = np.mod(t, 4294967296.0)
        m = np.where(m >= 2147483648.0, m - 4294967296.0, m)
        return [context.empty_tensor(list(r.shape), "int32", m.astype(np.int32).reshape(-1))]


def get_op_entries() -> List[OperatorEntry]:
    E = OperatorEntry
    entries = [
        E("Shape", 1, None, "cpu", HostShape),
        E("Constant", 1, None, "cpu", HostConstant),
        E("ConstantOfShape", 9, None, "cpu", HostConstantOfShape),
        E("Flatten", 1, None, "cpu", lambda: HostReshapeLike("Flatten")),
        E("Reshape", 5, None, "cpu", lambda: HostReshapeLike("Reshape")),
        E("Squeeze", 1, None, "cpu", lambda: HostReshapeLike("Squeeze")),
        E("Unsqueeze", 1, None, "cpu", lambda: HostReshapeLike("Unsqueeze")),
        E("Gather", 1, None, "cpu", HostGather),
        E("Concat", 1, None, "cpu", HostConcat),
        E("Cast", 6, None, "cpu", HostCast),
    ]
    for op in ("Add", "Sub", "Mul", "Div"):
        entries.append(E(op, 7, None, "cpu", lambda o=op: HostIntBinary(o)))
    return entries
