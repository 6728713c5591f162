"""TEST INFRASTRUCTURE ONLY: runs an ONNX model with the CPU oracle, node by node.

Plays the role of ``WebDNN.load(dir, {backendOrder: ["cpu"]})`` + ``runner.run()``
(``core/runnerImpl.ts:315-596`` with only the cpu backend): initializers are narrowed the way
``extractInitializerTensor`` does (int64 saturates to int32), inputs are bound positionally to the
graph inputs that are not initializers, nodes execute in file order, outputs come back in
``graph.output`` order.  BatchNormalization and LSTM nodes, which the reference cannot execute,
use the ONNX-specification restatements of ``cpu_ops.c``.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from webdnn_b200 import onnx_io  # wire-format parser only; no compute

from . import ops
from .ops import _c


def _attrs(node) -> Dict[str, object]:
    out = {}
    for a in node.attribute:
        if a.t is not None:
            out[a.name] = a.t
        elif a.ints:
            out[a.name] = [onnx_io.clip_long(v) for v in a.ints]
        elif a.floats:
            out[a.name] = list(a.floats)
        elif a.i is not None:
            out[a.name] = onnx_io.clip_long(a.i)
        elif a.f is not None:
            out[a.name] = a.f
        elif a.s is not None:
            out[a.name] = a.s.decode("utf-8")
        elif a.type == onnx_io.A_INTS:
            out[a.name] = []
    return out


def _narrow(t) -> np.ndarray:
    if t.data_type == onnx_io.FLOAT:
        return _c(t.array, np.float32).reshape(t.dims)
    if t.data_type == onnx_io.INT64:
        return np.clip(t.array.astype(np.int64), -(2 ** 31), 2 ** 31 - 1).astype(np.int32).reshape(t.dims)
    if t.data_type == onnx_io.INT32:
        return _c(t.array, np.int32).reshape(t.dims)
    raise ValueError(f"Unsupported initializer dataType {t.data_type}")


_DYN_DEFAULTS = {"Elu": (("alpha", 1.0),), "HardSigmoid": (("alpha", 0.2), ("beta", 0.5)),
                 "LeakyRelu": (("alpha", 0.01),),
                 "Selu": (("alpha", 1.6732632423543772848170429916717), ("gamma", 1.0507009873554804934193349852946)),
                 "ThresholdedRelu": (("alpha", 1.0),)}


def run_node(node, ins: List[np.ndarray], opset: int) -> List[np.ndarray]:
    t, a = node.op_type, _attrs(node)
    if t in _DYN_DEFAULTS:
        ps = [float(np.float32(a.get(k, d))) if k in a else d for k, d in _DYN_DEFAULTS[t]] + [0.0]
        return [ops.unary(t, ins[0], ps[0], ps[1])]
    if t == "Clip":
        if opset >= 11:
            raise ValueError("Clip: opset >= 11 is not supported by the cpu backend")
        return [ops.unary("Clip", ins[0], a.get("min", -3.4028234663852886e38), a.get("max", 3.4028234663852886e38))]
    if t in ops.UNARY:
        return [ops.unary(t, ins[0])]
    if t in ("Add", "Sub", "Mul", "Div", "Pow"):
        return [ops.binary(t, ins[0], ins[1])]
    if t in ("Max", "Min", "Sum", "Mean"):
        acc = ins[0]
        for x in ins[1:]:
            acc = ops.binary({"Max": "Max", "Min": "Min", "Sum": "Add", "Mean": "Add"}[t], acc, x)
        if t == "Mean" and len(ins) > 1:
            acc = ops.binary("Div", acc, np.asarray(len(ins), np.float32))
        return [acc.copy() if acc is ins[0] else acc]
    if t == "Gemm":
        return [ops.gemm(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a.get("alpha", 1.0), a.get("beta", 1.0),
                         a.get("transA", 0), a.get("transB", 0))]
    if t == "MatMul":
        return [ops.matmul(ins[0], ins[1])]
    if t == "Conv":
        return [ops.conv2d(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a.get("strides") or (1, 1),
                           a.get("pads") or (0, 0, 0, 0), a.get("dilations") or (1, 1), a.get("group", 1))]
    if t == "BatchNormalization":
        return [ops.batchnorm(ins[0], ins[1], ins[2], ins[3], ins[4], a.get("epsilon", 1e-5))]
    if t == "MaxPool":
        return [ops.maxpool2d(ins[0], a["kernel_shape"], a.get("strides") or (1, 1), a.get("pads") or (0, 0, 0, 0),
                              a.get("dilations") or (1, 1), a.get("ceil_mode", 0) != 0, a.get("auto_pad", "NOTSET"))]
    if t == "AveragePool":
        return [ops.avgpool2d(ins[0], a["kernel_shape"], a.get("strides") or (1, 1), a.get("pads") or (0, 0, 0, 0),
                              a.get("ceil_mode", 0) != 0, a.get("count_include_pad", 0) != 0,
                              a.get("auto_pad", "NOTSET"))]
    if t == "GlobalAveragePool":
        return [ops.global_avgpool(ins[0])]
    if t == "Softmax":
        return [ops.softmax(ins[0], a.get("axis", -1))]
    if t in ops.REDUCE:
        if t == "ReduceSum" and opset >= 13:
            axes = [int(v) for v in ins[1].reshape(-1)] if len(ins) > 1 and ins[1].size else []
            if not axes and a.get("noop_with_empty_axes", 0):
                return [ins[0].copy()]
        else:
            axes = a.get("axes", [])
        return [ops.reduce(t, ins[0], axes, a.get("keepdims", 1) != 0)]
    if t == "Flatten":
        if a.get("axis", 1) != 1:
            raise ValueError("Flatten: only axis === 1 is supported")
        d = ins[0].shape   # flatten.ts:11-18: [dims[0], product of the rest], also when a dimension is 0
        return [ins[0].reshape(d[0], int(np.prod(d[1:], dtype=np.int64)))]
    if t == "Reshape":
        shape = [int(v) for v in ins[1].reshape(-1)]
        allowzero = a.get("allowzero", 0) != 0
        explicit, minus = 1, -1
        for i, s in enumerate(shape):
            if s > 0:
                explicit *= s
            elif s == 0 and not allowzero:
                explicit *= ins[0].shape[i]
            elif s == -1:
                if minus >= 0:
                    raise ValueError("Reshape: multiple -1 dimensions")
                minus = i
        out = []
        for i, s in enumerate(shape):
            if s > 0 or (s == 0 and allowzero):
                out.append(s)
            elif s == 0:
                out.append(ins[0].shape[i])
            else:
                out.append(ins[0].size // explicit)
        return [ins[0].reshape(out)]
    if t in ("Squeeze", "Unsqueeze"):
        axes = [int(v) for v in ins[1].reshape(-1)] if len(ins) > 1 else a.get("axes", [])
        shp = list(ins[0].shape)
        if t == "Squeeze":
            if not axes:
                new = [s for s in shp if s != 1]
            else:
                nn = [x if x >= 0 else x + len(shp) for x in axes]
                new = [s for i, s in enumerate(shp) if i not in nn]
        else:
            nd = len(shp) + len(axes)
            nn = [x if x >= 0 else x + nd for x in axes]
            new, src = [], 0
            for d in range(nd):
                if d in nn:
                    new.append(1)
                else:
                    new.append(shp[src])
                    src += 1
        return [ins[0].reshape(new)]
    if t == "Transpose":
        return [ops.transpose(ins[0], a.get("perm"))]
    if t == "Concat":
        axis = a.get("axis", 0)
        return [_c(np.concatenate(ins, axis=axis))]
    if t == "Split":
        axis = a.get("axis", 0)
        if axis < 0:
            axis += ins[0].ndim
        n_out = len(node.output)
        if opset >= 13:
            split = [int(v) for v in ins[1].reshape(-1)] if len(ins) > 1 else []
        else:
            split = a.get("split", [])
        if not split:
            split = [ins[0].shape[axis] // n_out] * n_out
        outs, off = [], 0
        for s in split:
            idx = [slice(None)] * ins[0].ndim
            idx[axis] = slice(off, off + s)
            outs.append(_c(ins[0][tuple(idx)]))
            off += s
        return outs
    if t == "Slice":
        return [ops.slice_(ins[0], ins[1].reshape(-1), ins[2].reshape(-1),
                           ins[3].reshape(-1).tolist() if len(ins) > 3 else None,
                           ins[4].reshape(-1).tolist() if len(ins) > 4 else None)]
    if t == "Gather":
        axis = a.get("axis", 0)
        idx = ins[1].astype(np.int64)
        idx = np.where(idx < 0, idx + ins[0].shape[axis], idx)
        return [_c(np.take(ins[0], idx, axis=axis))]
    if t == "Shape":
        return [np.asarray(ins[0].shape, np.int32)]
    if t == "Cast":
        return [ops.cast(ins[0], a.get("to", 1))]
    if t == "Constant":
        return [_narrow(a["value"])]
    if t == "Identity":
        return [ins[0].copy()]
    if t == "LSTM":
        if len(ins) == 5 or len(ins) > 7:
            raise ValueError("LSTM: sequence_lens unsupported")
        b = ins[3].reshape(-1) if len(ins) > 3 else None
        h0 = ins[5][0] if len(ins) > 5 else None
        c0 = ins[6][0] if len(ins) > 6 else None
        return list(ops.lstm(ins[0], ins[1][0], ins[2][0], b, h0, c0))[:len(node.output)]
    if t == "ArgMax":
        return [ops.argmax(ins[0], a.get("axis", 0), a.get("keepdims", 1) != 0, a.get("select_last_index", 0) != 0)]
    if t == "LayerNormalization":
        return [ops.layernorm_chain(ins[0], ins[1] if len(ins) > 1 else None, ins[2] if len(ins) > 2 else None,
                                    float(np.float32(a.get("epsilon", 1e-5))))]
    if t == "ConvTranspose":
        if a.get("auto_pad", "NOTSET") != "NOTSET":
            raise ValueError("ConvTranspose: auto_pad !== NOTSET is not yet supported.")
        if a.get("output_shape"):
            raise ValueError("ConvTranspose: explicit output_shape is not yet supported.")
        return [ops.conv_transpose2d(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a.get("strides") or (1, 1),
                                     a.get("pads") or (0, 0, 0, 0), a.get("dilations") or (1, 1), a.get("group", 1),
                                     a.get("output_padding") or (0, 0))]
    if t == "InstanceNormalization":
        # instancenormalization.ts:18 reads epsilon with getAttrInt: a float attribute has integer field 0
        eps = 1e-5 if "epsilon" not in a else (float(a["epsilon"]) if isinstance(a["epsilon"], int) else 0.0)
        return [ops.instance_norm(ins[0], ins[1], ins[2], eps)]
    if t == "Pad":
        if opset < 11:
            raise NotImplementedError(f"Operator implementation for {t}, opset={opset} does not exist.")
        value = ins[2].reshape(-1)[0] if len(ins) > 2 else 0
        return [ops.pad(ins[0], [int(v) for v in ins[1].reshape(-1)], a.get("mode", "constant"), value)]
    if t == "Tile":
        return [ops.tile(ins[0], [int(v) for v in ins[1].reshape(-1)])]
    raise NotImplementedError(f"Operator implementation for {t}, opset={opset} does not exist.")


def run_model(model: onnx_io.Model, inputs: Sequence[np.ndarray], return_all: bool = False):
    g = model.graph
    values: Dict[str, np.ndarray] = {t.name: _narrow(t) for t in g.initializer}
    init_names = set(values)
    free_inputs = [vi for vi in g.input if vi.name not in init_names]
    if len(free_inputs) != len(inputs):
        raise ValueError("length of inputs mismatch")
    for vi, arr in zip(free_inputs, inputs):
        values[vi.name] = _c(arr)
    opset = int(model.opset_import[0][1])
    # like the reference's runner (runnerImpl.ts:523-532) an intermediate value is dropped after its last consumer,
    # unless every value was asked for; without this a batch-32 ResNet-50 keeps several GB of activations alive
    last_use: Dict[str, int] = {}
    for i, node in enumerate(g.node):
        for n in node.input:
            last_use[n] = i
    keep = init_names | {vi.name for vi in g.output} | {vi.name for vi in free_inputs}
    for i, node in enumerate(g.node):
        outs = run_node(node, [values[n] for n in node.input], opset)
        for name, arr in zip(node.output, outs):
            values[name] = arr
        if not return_all:
            for n in node.input:
                if last_use.get(n) == i and n not in keep:
                    values.pop(n, None)
    if return_all:
        return values
    return [values[vi.name] for vi in g.output]
