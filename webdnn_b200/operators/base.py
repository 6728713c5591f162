"""Backend-independent attribute parsing and shape math, one class per op family.

Restates ``src/descriptor_runner/operators/base/*.ts`` and ``operators/operatorUtil.ts`` /
``operatorImpl.ts`` so that the cuda operators subclass the same shape logic the reference's
backends share (the way ``operators/webgpu/operators/standard/gemm.ts:9-23`` subclasses
``base/gemm.ts``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

from ..onnx_io import Attribute, clip_long


# ---- operatorUtil.ts:19-133 --------------------------------------------------------------
# The reference's getAttrFloat / getAttrInt / getAttrString throw only when the field is null, and a message
# decoded by its protobuf binding never has null scalar fields: onnx/onnx.js:137-153 gives AttributeProto.f = 0,
# i = 0 and s = empty as prototype defaults.  So an attribute that is present but stored under another type reads
# as 0 / 0 / "" there (instancenormalization.ts:18 reads a float epsilon with getAttrInt and gets 0), and the same
# holds here.
def _get_attr(attribute: Sequence[Attribute], name: str) -> Optional[Attribute]:
    for a in attribute:
        if a.name == name:
            return a
    return None


def get_attr_float(attribute, name: str, default: float) -> float:
    a = _get_attr(attribute, name)
    if a is None:
        return default
    return a.f if a.f is not None else 0.0


def get_attr_int(attribute, name: str, default: int) -> int:
    a = _get_attr(attribute, name)
    if a is None:
        return default
    return clip_long(a.i) if a.i is not None else 0


def get_attr_ints(attribute, name: str, default: List[int]) -> List[int]:
    a = _get_attr(attribute, name)
    if a is None:
        return list(default)
    return [clip_long(v) for v in a.ints]


def get_attr_string(attribute, name: str, default: str) -> str:
    a = _get_attr(attribute, name)
    if a is None:
        return default
    return a.s.decode("utf-8") if a.s is not None else ""


def get_attr_tensor(attribute, name: str):
    a = _get_attr(attribute, name)
    return None if a is None else a.t


def array_prod(v: Sequence[int]) -> int:
    x = 1
    for i in v:
        x *= i
    return x


def calc_strides(dims: Sequence[int]) -> List[int]:
    strides: List[int] = []
    length = 1
    for d in reversed(dims):
        strides.insert(0, length)
        length *= d
    return strides


def broadcast_uni(dims_a: Sequence[int], dims_b: Sequence[int]) -> List[int]:
    """Strides of B broadcast to A's shape (operatorUtil.ts:178-209)."""
    if len(dims_a) < len(dims_b):
        raise ValueError(f"Unidirectional broadcast error: {dims_a}, {dims_b}")
    eb = [1] * (len(dims_a) - len(dims_b)) + list(dims_b)
    sb = calc_strides(eb)
    for i in range(len(dims_a)):
        if dims_a[i] != eb[i]:
            if eb[i] == 1:
                sb[i] = 0
            else:
                raise ValueError(f"Unidirectional broadcast error: {dims_a}, {dims_b}")
    return sb


def broadcast_multi(all_dims: Sequence[Sequence[int]]):
    """Output dims and per-input strides (operatorUtil.ts:211-245)."""
    nd = max(len(d) for d in all_dims)
    expanded = [[1] * (nd - len(d)) + list(d) for d in all_dims]
    dims = [max(e[i] for e in expanded) for i in range(nd)]
    all_strides = []
    for e in expanded:
        s = calc_strides(e)
        for i in range(nd):
            if e[i] != dims[i]:
                if e[i] == 1:
                    s[i] = 0
                else:
                    raise ValueError(f"Multidirectional broadcasting error: {all_dims}")
        all_strides.append(s)
    return dims, all_strides


# ---- operatorImpl.ts:7-29 ----------------------------------------------------------------
class OperatorImpl:
    def __init__(self, backend: str):
        self.backend = backend

    def initialize(self, attribute: Sequence[Attribute]) -> None:
        pass

    def get_tensor_backend_requirement(self, n_inputs: int, n_outputs: int):
        return [self.backend] * n_inputs

    def run(self, context, inputs, n_outputs: int):
        raise NotImplementedError


# ---- base/gemm.ts:7-62 -------------------------------------------------------------------
class Gemm(OperatorImpl):
    def initialize(self, attribute):
        super().initialize(attribute)
        self.alpha = get_attr_float(attribute, "alpha", 1.0)
        self.beta = get_attr_float(attribute, "beta", 1.0)
        self.trans_a = get_attr_int(attribute, "transA", 0)
        self.trans_b = get_attr_int(attribute, "transB", 0)

    def calc_shape(self, dims_a, dims_b):
        if len(dims_a) != 2 or len(dims_b) != 2:
            raise ValueError("Gemm: inputs must be 2-D")
        if self.trans_a:
            k, m = dims_a
            stride_a = [1, m]
        else:
            m, k = dims_a
            stride_a = [k, 1]
        if self.trans_b:
            n, kcheck = dims_b
            stride_b = [1, kcheck]
        else:
            kcheck, n = dims_b
            stride_b = [n, 1]
        if k != kcheck:
            raise ValueError("Gemm: inner dimensions differ")
        return m, n, k, stride_a, stride_b


# ---- base/matmul.ts:6-91 -----------------------------------------------------------------
class MatMul(OperatorImpl):
    def calc_shape(self, dims_a, dims_b):
        total = max(len(dims_a), len(dims_b), 2)
        ea = list(dims_a)
        if len(ea) == 0:
            raise ValueError("MatMul: scalar input")
        if len(ea) == 1:
            ea.insert(0, 1)
        ea = [1] * (total - len(ea)) + ea
        eb = list(dims_b)
        if len(eb) == 0:
            raise ValueError("MatMul: scalar input")
        if len(eb) == 1:
            eb.append(1)
        eb = [1] * (total - len(eb)) + eb
        result_dims = [ea[-2], eb[-1]]
        inner = ea[-1]
        if inner != eb[-2]:
            raise ValueError("MatMul: inner dimensions differ")
        sa, sb = calc_strides(ea), calc_strides(eb)
        for i in range(len(ea) - 3, -1, -1):
            rd = max(ea[i], eb[i])
            if ea[i] == 1:
                sa[i] = 0
            if eb[i] == 1:
                sb[i] = 0
            result_dims.insert(0, rd)
        result_strides = calc_strides(result_dims)
        squeezed = list(result_dims)
        if len(dims_a) == 1:
            del squeezed[len(squeezed) - 2]
        if len(dims_b) == 1:
            del squeezed[len(squeezed) - 1]
        return dict(result_dims=result_dims, result_strides=result_strides,
                    result_dims_after_squeeze=squeezed, strides_a=sa, strides_b=sb,
                    inner_product_length=inner)


# ---- base/conv.ts:7-79 -------------------------------------------------------------------
class Conv(OperatorImpl):
    def initialize(self, attribute):
        super().initialize(attribute)
        self.dilations = get_attr_ints(attribute, "dilations", [])
        self.group = get_attr_int(attribute, "group", 1)
        self.kernel_shape = get_attr_ints(attribute, "kernel_shape", [])
        self.pads = get_attr_ints(attribute, "pads", [])
        self.strides = get_attr_ints(attribute, "strides", [])

    def calc_shape(self, dims_x, dims_w):
        dil = self.dilations or [1, 1]
        ks = self.kernel_shape or [dims_w[2], dims_w[3]]
        pads = self.pads or [0, 0, 0, 0]
        st = self.strides or [1, 1]
        in_shape = [dims_x[2], dims_x[3]]
        out_shape = [
            math.floor((in_shape[0] + pads[0] + pads[2] - dil[0] * (ks[0] - 1) - 1) / st[0]) + 1,
            math.floor((in_shape[1] + pads[1] + pads[3] - dil[1] * (ks[1] - 1) - 1) / st[1]) + 1,
        ]
        ch_in = dims_x[1]
        ch_out = dims_w[0]
        return dict(batch=dims_x[0], dilations=dil, group=self.group, kernel_shape=ks, pads=pads,
                    strides=st, in_shape=in_shape, out_shape=out_shape, ch_in=ch_in,
                    ch_in_per_group=ch_in // self.group, ch_out=ch_out,
                    ch_out_per_group=ch_out // self.group)


# ---- base/maxpool.ts:6-138, base/averagepool.ts:7-105 -------------------------------------
class _Pool(OperatorImpl):
    has_dilations = False

    def initialize(self, attribute):
        super().initialize(attribute)
        self.auto_pad = get_attr_string(attribute, "auto_pad", "NOTSET")
        self.ceil_mode = get_attr_int(attribute, "ceil_mode", 0) != 0
        self.kernel_shape = get_attr_ints(attribute, "kernel_shape", [])
        self.pads = get_attr_ints(attribute, "pads", [])
        self.strides = get_attr_ints(attribute, "strides", [])
        self.dilations = get_attr_ints(attribute, "dilations", []) if self.has_dilations else []

    def calc_shape(self, dims_x):
        dil = self.dilations or [1, 1]
        ks = self.kernel_shape
        st = self.strides or [1, 1]
        in_shape = [dims_x[2], dims_x[3]]
        eff = [dil[i] * (ks[i] - 1) + 1 for i in range(2)]
        if self.auto_pad == "NOTSET":
            pads = self.pads or [0, 0, 0, 0]
            rnd = math.ceil if self.ceil_mode else math.floor
            out_shape = [rnd((in_shape[i] + pads[i] + pads[i + 2] - eff[i]) / st[i]) + 1 for i in range(2)]
        elif self.auto_pad in ("SAME_UPPER", "SAME_LOWER"):
            out_shape = [math.ceil(in_shape[i] / st[i]) for i in range(2)]
            sum_pad = [(out_shape[i] - 1) * st[i] + eff[i] - in_shape[i] for i in range(2)]
            lo = [math.floor(s / 2) for s in sum_pad]
            hi = [math.ceil(s / 2) for s in sum_pad]
            pads = lo + hi if self.auto_pad == "SAME_UPPER" else hi + lo
        elif self.auto_pad == "VALID":
            out_shape = [math.ceil((in_shape[i] - eff[i] + 1) / st[i]) for i in range(2)]
            pads = [0, 0, 0, 0]
        else:
            raise ValueError(f"Unknown auto_pad {self.auto_pad}")
        return dict(batch=dims_x[0], dilations=dil, kernel_shape=ks, pads=pads, strides=st,
                    in_shape=in_shape, out_shape=out_shape, ch=dims_x[1])


class MaxPool(_Pool):
    has_dilations = True

    def initialize(self, attribute):
        super().initialize(attribute)
        if get_attr_int(attribute, "storage_order", 0) != 0:
            raise ValueError("MaxPool: storage_order !== 0 is not supported.")


class AveragePool(_Pool):
    def initialize(self, attribute):
        super().initialize(attribute)
        self.count_include_pad = get_attr_int(attribute, "count_include_pad", 0) != 0


# ---- base/flatten.ts, reshape5.ts, squeeze.ts, unsqueeze.ts, transpose.ts ------------------
class Flatten(OperatorImpl):
    def initialize(self, attribute):
        super().initialize(attribute)
        if get_attr_int(attribute, "axis", 1) != 1:
            raise ValueError("Flatten: only axis === 1 is supported")

    def calc_shape(self, input):
        return [input.dims[0], array_prod(input.dims[1:])]


class Reshape5(OperatorImpl):
    def initialize(self, attribute):
        super().initialize(attribute)
        self.allowzero = get_attr_int(attribute, "allowzero", 0) != 0

    def calc_shape(self, input, shape_tensor) -> List[int]:
        shape_input = [int(v) for v in shape_tensor.data]
        explicit_prod, minus_dim = 1, -1
        for i, s in enumerate(shape_input):
            if s > 0:
                explicit_prod *= s
            elif s == 0 and not self.allowzero:
                explicit_prod *= input.dims[i]
            elif s == -1:
                if minus_dim >= 0:
                    raise ValueError("Reshape: multiple -1 dimensions")
                minus_dim = i
            elif s != 0:
                raise ValueError("Reshape: bad dimension")
        if minus_dim >= 0 and explicit_prod <= 0:
            raise ValueError("Reshape: cannot infer -1")
        minus_value = input.length // explicit_prod if explicit_prod > 0 else 0
        out = []
        for i, s in enumerate(shape_input):
            if s > 0 or (s == 0 and self.allowzero):
                out.append(s)
            elif s == 0:
                out.append(input.dims[i])
            else:
                out.append(minus_value)
        return out


def squeeze_shape(input_shape, axes) -> List[int]:
    if len(axes) == 0:
        return [s for s in input_shape if s != 1]
    nn = [a if a >= 0 else a + len(input_shape) for a in axes]
    return [s for i, s in enumerate(input_shape) if i not in nn]


def unsqueeze_shape(input_shape, axes) -> List[int]:
    nd = len(input_shape) + len(axes)
    nn = [a if a >= 0 else a + nd for a in axes]
    out, src = [], 0
    for d in range(nd):
        if d in nn:
            out.append(1)
        else:
            out.append(input_shape[src])
            src += 1
    return out


class Transpose(OperatorImpl):
    def initialize(self, attribute):
        super().initialize(attribute)
        self.perm = get_attr_ints(attribute, "perm", [])

    def calc_shape(self, input):
        perm = self.perm if self.perm else [input.ndim - 1 - i for i in range(input.ndim)]
        if len(perm) != input.ndim:
            raise ValueError("Transpose: perm length mismatch")
        out_shape = [input.dims[p] for p in perm]
        in_strides = [input.strides[p] for p in perm]
        return out_shape, in_strides


# ---- base/split.ts:7-100 -------------------------------------------------------------------
def split_params(input, n_outputs: int, axis: int, split_src: Sequence[int]):
    if axis < 0:
        axis += input.ndim
    if axis < 0 or axis >= input.ndim:
        raise ValueError(f"Split: axis {axis} out of range")
    axis_length = input.dims[axis]
    split = list(split_src) if len(split_src) > 0 else [axis_length // n_outputs] * n_outputs
    params, offset = [], 0
    for i in range(n_outputs):
        out_shape = list(input.dims)
        out_shape[axis] = split[i]
        params.append((split[i], offset, out_shape))
        offset += split[i]
    return axis, params
