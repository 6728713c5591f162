"""Operators of the ``cuda`` backend and their registry entries.

Each class follows the reference's operator contract (``interface/core/operator.ts:6-30``):
``initialize(attribute)`` parses attributes, ``get_tensor_backend_requirement`` says where each
input must live, ``run(context, inputs, n_outputs)`` computes shapes on the host with the shared
base class, allocates outputs with ``context.empty_tensor`` and enqueues kernels without waiting
for the device — the shape of ``operators/webgpu/operators/standard/{gemm,conv,unary,binary7}.ts``.
``get_op_entries()`` returns ``OperatorEntry`` records like every ``getOpEntries()`` the generated
``opEntriesStandard.ts`` aggregates (``scripts/make_operator_entries.py:5-33``).

Ops that exist in no reference backend (BatchNormalization, LayerNormalization, ArgMax, LSTM and
the fused types the load-time graph rewrite emits) follow the ONNX operator specification.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_void_p
from typing import List

import numpy as np

from ..backend import NP_DTYPE, CPUTensor, CudaTensor, WebDNNCudaContext
from ..lib import BINARY_OPS, REDUCE_KINDS, UNARY_OPS, AttentionDesc, ConvDesc, ConvTransposeDesc, GemmDesc, PoolDesc
from ..operator_table import OperatorEntry
from . import base
from .base import (OperatorImpl, array_prod, broadcast_multi, broadcast_uni, get_attr_float, get_attr_int,
                   get_attr_ints, get_attr_string, squeeze_shape, unsqueeze_shape)


def _p(t):
    return c_void_p(t.ptr) if t is not None else None


# ------------------------------------------------------------------------------ pointwise
class CudaUnary(OperatorImpl):
    """unary.ts:10-32 on the device; keeps the input's storage layout."""

    def __init__(self, op_type: str, allow=("float32",)):
        super().__init__("cuda")
        self.op_type = op_type
        self.allow = allow
        self.p0 = self.p1 = 0.0

    def initialize(self, attribute):
        a = attribute
        t = self.op_type
        if t == "Elu":
            self.p0 = get_attr_float(a, "alpha", 1.0)
        elif t == "HardSigmoid":
            self.p0, self.p1 = get_attr_float(a, "alpha", 0.2), get_attr_float(a, "beta", 0.5)
        elif t == "LeakyRelu":
            self.p0 = get_attr_float(a, "alpha", 0.01)
        elif t == "Selu":
            self.p0 = get_attr_float(a, "alpha", 1.6732632423543772848170429916717)
            self.p1 = get_attr_float(a, "gamma", 1.0507009873554804934193349852946)
        elif t == "ThresholdedRelu":
            self.p0 = get_attr_float(a, "alpha", 1.0)
        elif t == "Clip":  # opset < 11: limits are attributes (clip.ts:39-49)
            self.p0 = get_attr_float(a, "min", -3.4028234663852886e38)
            self.p1 = get_attr_float(a, "max", 3.4028234663852886e38)

    def run(self, context: WebDNNCudaContext, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = inputs[0]
        if x.data_type not in self.allow:
            raise TypeError(f"{self.op_type}: DataType {x.data_type} not supported")
        y = context.empty_tensor(x.dims, x.data_type, layout=x.layout)
        context.unary(UNARY_OPS[self.op_type], x, y, self.p0, self.p1)
        return [y]


class CudaBinary7(OperatorImpl):
    """binary7.ts:16-68 on the device (float32 and int32, multidirectional broadcast <= 6-D)."""

    def __init__(self, op_type: str):
        super().__init__("cuda")
        self.op_type = op_type

    def run(self, context: WebDNNCudaContext, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        a, b = inputs
        if a.data_type != b.data_type:
            raise TypeError(f"Binary: input dataTypes mismatch: {a.data_type} !== {b.data_type}")
        tmp = []
        if a.layout == b.layout == "nhwc" and a.dims == b.dims:
            layout = "nhwc"  # same physical order on both sides: plain elementwise
        else:
            layout = "nchw"
            ca, cb = context.canonical(a), context.canonical(b)
            tmp = [t for t, o in ((ca, a), (cb, b)) if t is not o]
            a, b = ca, cb
        out_shape, (sa, sb) = broadcast_multi([a.dims, b.dims])
        if len(out_shape) > 6:
            raise ValueError(f"Binary: input ndim {len(out_shape)} > 6 is not supported")
        y = context.empty_tensor(out_shape, a.data_type, layout=layout)
        context.binary(BINARY_OPS[self.op_type], a, b, y, out_shape, sa, sb)
        for t in tmp:
            t.dispose()
        return [y]


class CudaEachElementwise(OperatorImpl):
    """Max / Min / Sum / Mean over N inputs (eachelementwise.ts), folded pairwise on the device."""

    def __init__(self, op_type: str):
        super().__init__("cuda")
        self.op_type = op_type

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        code = {"Max": "Max", "Min": "Min", "Sum": "Add", "Mean": "Add"}[self.op_type]
        acc = context.canonical(inputs[0])
        acc_owned = acc is not inputs[0]
        for t in inputs[1:]:
            ct = context.canonical(t)
            out_shape, (sa, sb) = broadcast_multi([acc.dims, ct.dims])
            y = context.empty_tensor(out_shape, acc.data_type)
            context.binary(BINARY_OPS[code], acc, ct, y, out_shape, sa, sb)
            if ct is not t:
                ct.dispose()
            if acc_owned:
                acc.dispose()
            acc, acc_owned = y, True
        if self.op_type == "Mean" and len(inputs) > 1:
            n = context.move_tensor(
                context.cpu_context.empty_tensor([], "float32", np.array([len(inputs)], np.float32)))
            y = context.empty_tensor(acc.dims, acc.data_type)
            context.binary(BINARY_OPS["Div"], acc, n, y, acc.dims, acc.strides, [0] * acc.ndim)
            n.dispose()
            acc.dispose()
            acc = y
        if not acc_owned:  # single input: the output must be its own tensor
            y = context.empty_tensor(acc.dims, acc.data_type)
            context.unary(UNARY_OPS["Identity"], acc, y)
            acc = y
        return [acc]


class CudaCast(OperatorImpl):
    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.to = get_attr_int(attribute, "to", 1)

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        if self.to == 1:
            dt = "float32"
        elif self.to in (2, 6, 7):
            dt = "int32"
        else:
            raise ValueError(f"Cast: converting to DataType {self.to} is not yet supported")
        y = context.empty_tensor(x.dims, dt)
        code = {"float32": 0, "int32": 1}
        context._call("wdc_cast", code[x.data_type], code[dt], _p(x), _p(y), x.length)
        if x is not inputs[0]:
            x.dispose()
        return [y]


# --------------------------------------------------------------------------- contractions
class CudaGemm(base.Gemm):
    """gemm.ts:21-61; C is broadcast unidirectionally to [m, n]."""

    def __init__(self, relu: bool = False):
        super().__init__("cuda")
        self.relu = relu

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        owned = []
        ins = []
        for t in inputs:
            c = context.canonical(t)
            if c is not t:
                owned.append(c)
            ins.append(c)
        a, b = ins[0], ins[1]
        c = ins[2] if len(ins) > 2 else None
        m, n, k, sa, sb = self.calc_shape(a.dims, b.dims)
        d = GemmDesc(batch=1, m=m, n=n, k=k, sab=0, sa0=sa[0], sa1=sa[1], sbb=0, sb0=sb[0], sb1=sb[1],
                     sc0=0, sc1=0, alpha=self.alpha, beta=self.beta, relu=int(self.relu))
        if c is not None:
            sc = broadcast_uni([m, n], c.dims)
            d.sc0, d.sc1 = sc
        y = context.empty_tensor([m, n], "float32")
        context.gemm(d, a, b, c, y)
        for t in owned:
            t.dispose()
        return [y]


class CudaMatMul(base.MatMul):
    """matmul.ts:11-111, result rank <= 3 like the cpu backend (plus any rank whose leading
    dims collapse to one batch axis)."""

    def __init__(self):
        super().__init__("cuda")

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        a, b = (context.canonical(t) for t in inputs)
        owned = [t for t, o in ((a, inputs[0]), (b, inputs[1])) if t is not o]
        if a.data_type != "float32" or b.data_type != "float32":
            raise TypeError("only float32 is supported")
        s = self.calc_shape(a.dims, b.dims)
        rd, sa, sb = s["result_dims"], s["strides_a"], s["strides_b"]
        if len(rd) > 3:
            raise ValueError("MatMul: result rank > 3 is not supported")
        batch = rd[0] if len(rd) == 3 else 1
        d = GemmDesc(batch=batch, m=rd[-2], n=rd[-1], k=s["inner_product_length"],
                     sab=sa[0] if len(rd) == 3 else 0, sa0=sa[-2], sa1=sa[-1],
                     sbb=sb[0] if len(rd) == 3 else 0, sb0=sb[-2], sb1=sb[-1],
                     sc0=0, sc1=0, alpha=1.0, beta=0.0, relu=0)
        y = context.empty_tensor(s["result_dims_after_squeeze"], "float32")
        context.gemm(d, a, b, None, y)
        for t in owned:
            t.dispose()
        return [y]


class CudaMatMulBias(OperatorImpl):
    """``MatMul(A, W) + b`` [+ Relu] [+ residual] in one launch: A [..., k] (leading dims stacked into rows), W a
    constant [k, n], b a constant vector of n, residual an activation of the result's shape (load-time rewrite of
    MatMul + Add [+ Relu | + Add], matmul.ts:11-111 and binary7.ts broadcasting for the reference semantics).

    With a residual the launch goes through ``wdc_conv2d`` as a 1x1 convolution over the rows (its epilogue takes a
    per-column addend and a residual tensor together); W is transposed to [n, k] once and kept with the weight."""

    def __init__(self):
        super().__init__("cuda")
        self.relu = False
        self.has_residual = False

    def initialize(self, attribute):
        self.relu = get_attr_int(attribute, "relu", 0) != 0
        self.has_residual = get_attr_int(attribute, "has_residual", 0) != 0

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        a = context.canonical(inputs[0])
        w, b = inputs[1], inputs[2]
        k, n = w.dims
        if a.ndim < 1 or a.dims[-1] != k:
            raise ValueError("CudaMatMulBias: inner dimensions do not match")
        m = a.length // k
        out_dims = list(a.dims[:-1]) + [n]
        res = context.canonical(inputs[3]) if self.has_residual else None
        owned = [t for t, o in ((a, inputs[0]), (res, inputs[3] if self.has_residual else None)) if t is not o]
        y = context.empty_tensor(out_dims, "float32")
        fused_res = res is not None and list(res.dims) == out_dims and res.data_type == "float32" and m < 2 ** 31
        if y.length and fused_res:
            wt = w.aux.get("nk")
            if wt is None:
                wt = context.empty_tensor([n, k], "float32")
                context.strided_copy(w, wt, [n, k], [1, n], 0, [k, 1], 0)
                w.aux["nk"] = wt
            d = ConvDesc(batch=1, ch_in=k, in_h=1, in_w=m, ch_out=n, k_h=1, k_w=1, out_h=1, out_w=m, stride_h=1,
                         stride_w=1, pad_t=0, pad_l=0, dil_h=1, dil_w=1, group=1, relu=int(self.relu), x_nchw=0)
            context.conv2d(d, a, wt, None, b, res, y)
        elif y.length:
            d = GemmDesc(batch=1, m=m, n=n, k=k, sab=0, sa0=k, sa1=1, sbb=0, sb0=n, sb1=1, sc0=0, sc1=1,
                         alpha=1.0, beta=1.0, relu=int(self.relu))
            context.gemm(d, a, w, b, y)
        for t in owned:
            t.dispose()
        if res is not None and not fused_res:
            # shapes differ (the Add broadcasts): keep the reference's two steps
            add = CudaBinary7("Add")
            out = add.run(context, [y, inputs[3]], 1)
            y.dispose()
            return out
        return [y]


class CudaAttention(OperatorImpl):
    """softmax(scale * Q K^T) V as one launch (load-time rewrite of MatMul -> Mul -> Softmax -> MatMul;
    matmul.ts:11-111, binary7.ts:16-68, softmax.ts:15-59 give the reference semantics).

    Inputs are either rank-3 [batch*heads, tokens, c] tensors (``heads`` attribute 0), or the tensors
    in front of the head split, [batch, tokens, heads*c] in memory, read through strides.  With
    ``merge_heads`` the result is written as [batch, tq, heads*c], else as [batch*heads, tq, c]."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.scale = get_attr_float(attribute, "scale", 1.0)
        self.batch = get_attr_int(attribute, "batch", 0)
        self.heads = get_attr_int(attribute, "heads", 0)
        self.head_size = get_attr_int(attribute, "head_size", 0)
        self.merge = get_attr_int(attribute, "merge_heads", 0) != 0

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        q, k, v = (context.canonical(t) for t in inputs)
        owned = [t for t, o in zip((q, k, v), inputs) if t is not o]
        if any(t.data_type != "float32" for t in (q, k, v)):
            raise TypeError("only float32 is supported")
        if self.heads:
            b, h = self.batch, self.heads
            if k.length != v.length:
                raise ValueError("CudaAttention: operand sizes do not match the head split")
            c = self.head_size
            if c <= 0 or q.length % (b * h * c) or k.length % (b * h * c):
                raise ValueError("CudaAttention: operand sizes do not match the head split")
            tq, tk = q.length // (b * h * c), k.length // (b * h * c)
            sq = (tq * h * c, c, h * c)
            sk = (tk * h * c, c, h * c)
        else:
            if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
                raise ValueError("CudaAttention: operands must have rank 3")
            b, h = q.dims[0], 1
            tq, c = q.dims[1], q.dims[2]
            tk = k.dims[1]
            if k.dims != [b, tk, c] or v.dims != [b, tk, c]:
                raise ValueError("CudaAttention: operand shapes do not match")
            sq = (tq * c, 0, c)
            sk = (tk * c, 0, c)
        if self.merge:
            y = context.empty_tensor([b, tq, h * c], "float32")
            sy = (tq * h * c, c, h * c)
        else:
            y = context.empty_tensor([b * h, tq, c], "float32")
            sy = (h * tq * c, tq * c, c)
        if y.length:
            if c in (32, 64):
                d = AttentionDesc(batch=b, heads=h, tq=tq, tk=tk, dh=c,
                                  q_sb=sq[0], q_sh=sq[1], q_st=sq[2], k_sb=sk[0], k_sh=sk[1], k_st=sk[2],
                                  v_sb=sk[0], v_sh=sk[1], v_st=sk[2], y_sb=sy[0], y_sh=sy[1], y_st=sy[2],
                                  scale=self.scale)
                context._call("wdc_attention", byref(d), _p(q), _p(k), _p(v), _p(y))
            elif self.heads:
                raise ValueError("CudaAttention: a head split is only absorbed for head sizes 32 and 64")
            else:
                # other head sizes: the same chain as three launches (the scale rides on the first contraction)
                sc = context.empty_tensor([b, tq, tk], "float32")
                context.gemm(GemmDesc(batch=b, m=tq, n=tk, k=c, sab=tq * c, sa0=c, sa1=1, sbb=tk * c, sb0=1, sb1=c,
                                      sc0=0, sc1=0, alpha=self.scale, beta=0.0, relu=0), q, k, None, sc)
                pr = context.empty_tensor([b, tq, tk], "float32")
                context._call("wdc_softmax", _p(sc), _p(pr), b * tq, tk)
                sc.dispose()
                context.gemm(GemmDesc(batch=b, m=tq, n=c, k=tk, sab=tq * tk, sa0=tk, sa1=1, sbb=tk * c, sb0=c, sb1=1,
                                      sc0=0, sc1=0, alpha=1.0, beta=0.0, relu=0), pr, v, None, y)
                pr.dispose()
        for t in owned:
            t.dispose()
        return [y]


def _packed_weight(context: WebDNNCudaContext, w: CudaTensor) -> CudaTensor:
    """[Cout, Cin/g, kh, kw] -> [Cout, kh, kw, Cin/g], cached on the (persistent) weight tensor."""
    pk = w.aux.get("krsc")
    if pk is None:
        co, cig, kh, kw = w.dims
        pk = context.empty_tensor([co, kh, kw, cig], "float32")
        context._call("wdc_pack_conv_weight", _p(w), _p(pk), co, cig, kh, kw)
        w.aux["krsc"] = pk
    return pk


class CudaConv(base.Conv):
    """conv.ts:134-221 as one implicit-GEMM launch; activations are kept channels-last.

    ``fused`` instances take the inputs the load-time rewrite produced:
    [X, W, (scale), (shift), (residual)] selected by the ``has_*`` attributes.
    """

    def __init__(self, fused: bool = False):
        super().__init__("cuda")
        self.fused = fused
        self.relu = False
        self.has_scale = self.has_shift = self.has_residual = False

    def initialize(self, attribute):
        super().initialize(attribute)
        if self.fused:
            self.relu = get_attr_int(attribute, "relu", 0) != 0
            self.has_scale = get_attr_int(attribute, "has_scale", 0) != 0
            self.has_shift = get_attr_int(attribute, "has_shift", 0) != 0
            self.has_residual = get_attr_int(attribute, "has_residual", 0) != 0

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x, w = inputs[0], inputs[1]
        if x.ndim != 4:
            raise ValueError("Conv other than 2D is not yet supported")
        rest = list(inputs[2:])
        scale = shift = residual = None
        if self.fused:
            if self.has_scale:
                scale = rest.pop(0)
            if self.has_shift:
                shift = rest.pop(0)
            if self.has_residual:
                residual = rest.pop(0)
        elif rest:
            shift = rest.pop(0)  # plain Conv bias
        s = self.calc_shape(x.dims, w.dims)
        # the first layer of an image network: its few-channel NCHW input is re-laid out inside the
        # library anyway, so the separate NCHW -> NHWC conversion is skipped
        direct = (x.layout == "nchw" and s["group"] == 1 and s["ch_in"] <= 4 and s["kernel_shape"][1] <= 8
                  and s["ch_out"] % 4 == 0 and s["in_shape"][0] * s["in_shape"][1] > 1)
        oh, ow = s["out_shape"]
        # The epilogue reads residual[pixel, channel] for every output element, so the addend rides in it only
        # when it is a float32 tensor of exactly the output's shape.  An Add that broadcasts ([1,C,H,W],
        # [N,C,1,1], ... : binary7.ts broadcasts multidirectionally) keeps the reference's separate steps below.
        unfused_res = None
        if residual is not None and (list(residual.dims) != [s["batch"], s["ch_out"], oh, ow]
                                     or residual.data_type != "float32"):
            unfused_res, residual = residual, None
        relu_here = self.relu and unfused_res is None
        xcl = x if direct else context.channels_last(x)
        rcl = context.channels_last(residual) if residual is not None else None
        wp = _packed_weight(context, w)
        y = context.empty_tensor([s["batch"], s["ch_out"], oh, ow], "float32", layout="nhwc")
        d = ConvDesc(batch=s["batch"], ch_in=s["ch_in"], in_h=s["in_shape"][0], in_w=s["in_shape"][1],
                     ch_out=s["ch_out"], k_h=s["kernel_shape"][0], k_w=s["kernel_shape"][1], out_h=oh,
                     out_w=ow, stride_h=s["strides"][0], stride_w=s["strides"][1], pad_t=s["pads"][0],
                     pad_l=s["pads"][1], dil_h=s["dilations"][0], dil_w=s["dilations"][1],
                     group=s["group"], relu=int(relu_here), x_nchw=int(direct))
        context.conv2d(d, xcl, wp, scale, shift, rcl, y)
        if xcl is not x:
            xcl.dispose()
        if rcl is not None and rcl is not residual:
            rcl.dispose()
        if unfused_res is not None:
            (t,) = CudaBinary7("Add").run(context, [y, unfused_res], 1)
            y.dispose()
            y = t
            if self.relu:
                (t,) = CudaUnary("Relu").run(context, [y], 1)
                y.dispose()
                y = t
        return [y]


class CudaBatchNormalization(OperatorImpl):
    """Inference-form BatchNormalization (ONNX spec): y = (x - mean) / sqrt(var + eps) * scale + B.
    The per-channel scale/shift pair is derived once in float64 on the host from the four parameter
    vectors (which the requirement list keeps on the cpu) and cached on the scale tensor."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.epsilon = get_attr_float(attribute, "epsilon", 1e-5)

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return ["cuda"] + ["cpu"] * (n_inputs - 1)

    def run(self, context, inputs, n_outputs):
        x, gamma, beta, mean, var = inputs
        cache = gamma.__dict__.setdefault("_cuda_bn", {})
        key = (id(context), self.epsilon)
        if key not in cache:
            g, b, m, v = (t.data.astype(np.float64) for t in (gamma, beta, mean, var))
            sc = g / np.sqrt(v + float(np.float32(self.epsilon)))
            sh = b - m * sc
            cache[key] = tuple(
                context.move_tensor(context.cpu_context.empty_tensor([len(a)], "float32", a.astype(np.float32)))
                for a in (sc, sh))
        dsc, dsh = cache[key]
        y = context.empty_tensor(x.dims, "float32", layout=x.layout)
        ch = x.dims[1]
        if x.layout == "nhwc":
            outer, inner = x.length // ch, 1
        else:
            outer, inner = x.dims[0], array_prod(x.dims[2:])
        context._call("wdc_channel_affine", _p(x), _p(dsc), _p(dsh), _p(y), outer, ch, inner, 0)
        return [y]


# -------------------------------------------------------------------------------- pooling
def _pool_desc(s, x: CudaTensor, y: CudaTensor, count_include_pad: bool) -> PoolDesc:
    xs, ys = x.nchw_strides(), y.nchw_strides()
    return PoolDesc(batch=s["batch"], ch=s["ch"], in_h=s["in_shape"][0], in_w=s["in_shape"][1],
                    out_h=s["out_shape"][0], out_w=s["out_shape"][1], k_h=s["kernel_shape"][0],
                    k_w=s["kernel_shape"][1], stride_h=s["strides"][0], stride_w=s["strides"][1],
                    pad_t=s["pads"][0], pad_l=s["pads"][1], dil_h=s["dilations"][0], dil_w=s["dilations"][1],
                    xs_n=xs[0], xs_c=xs[1], xs_h=xs[2], xs_w=xs[3], ys_n=ys[0], ys_c=ys[1], ys_h=ys[2],
                    ys_w=ys[3], count_include_pad=int(count_include_pad))


class CudaMaxPool(base.MaxPool):
    def __init__(self):
        super().__init__("cuda")

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = inputs[0]
        if n_outputs != 1:
            raise ValueError("MaxPool: output indices is not yet supported")
        if x.ndim != 4:
            raise ValueError("MaxPool other than 2D is not yet supported")
        s = self.calc_shape(x.dims)
        y = context.empty_tensor([s["batch"], s["ch"], *s["out_shape"]], "float32", layout=x.layout)
        context.pool("max", _pool_desc(s, x, y, False), x, y)
        return [y]


class CudaAveragePool(base.AveragePool):
    def __init__(self):
        super().__init__("cuda")

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = inputs[0]
        if x.ndim != 4:
            raise ValueError("AveragePool other than 2D is not yet supported")
        s = self.calc_shape(x.dims)
        y = context.empty_tensor([s["batch"], s["ch"], *s["out_shape"]], "float32", layout=x.layout)
        context.pool("avg", _pool_desc(s, x, y, self.count_include_pad), x, y)
        return [y]


class CudaGlobalAveragePool(OperatorImpl):
    def __init__(self):
        super().__init__("cuda")

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = inputs[0]
        if x.ndim != 4:
            raise ValueError("GlobalAveragePool other than 2D is not yet supported")
        n, c, h, w = x.dims
        y = context.empty_tensor([n, c, 1, 1], "float32")
        xs = x.nchw_strides()
        context._call("wdc_global_avgpool", _p(x), _p(y), n, c, h * w, xs[0], xs[1], xs[3])
        return [y]


# -------------------------------------------------------------------------------- row ops
class CudaSoftmax(OperatorImpl):
    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", -1)

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = context.canonical(inputs[0])
        axis = self.axis + x.ndim if self.axis < 0 else self.axis
        if axis != x.ndim - 1:
            raise ValueError("Softmax: currently only reducing final axis is supported")
        ln = x.dims[axis]
        y = context.empty_tensor(x.dims, x.data_type)
        context._call("wdc_softmax", _p(x), _p(y), x.length // ln if ln else 0, ln)
        if x is not inputs[0]:
            x.dispose()
        return [y]


class CudaReduce(OperatorImpl):
    """reduce.ts:41-103: one device pass per reduced axis, axes sorted ascending."""

    def __init__(self, op_type: str, axes_from_input: bool):
        super().__init__("cuda")
        self.op_type = op_type
        self.axes_from_input = axes_from_input

    def initialize(self, attribute):
        self.axes = get_attr_ints(attribute, "axes", [])
        self.keepdims = get_attr_int(attribute, "keepdims", 1) != 0
        self.noop_with_empty_axes = get_attr_int(attribute, "noop_with_empty_axes", 0) != 0

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return ["cuda"] + ["cpu"] * (n_inputs - 1)

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        if self.axes_from_input:
            axes = [int(a) for a in inputs[1].data] if len(inputs) > 1 and inputs[1].length > 0 else []
            if not axes and not self.noop_with_empty_axes:
                axes = list(range(x.ndim))
        else:
            axes = self.axes or list(range(x.ndim))
        sorted_axes = sorted(a if a >= 0 else a + x.ndim for a in axes)
        kind = REDUCE_KINDS[self.op_type]
        cur, shape, total = x, list(x.dims), 1
        for i, axis in enumerate(sorted_axes):
            red = shape[axis]
            total *= red
            outer, inner = array_prod(shape[:axis]), array_prod(shape[axis + 1:])
            new_shape = list(shape)
            new_shape[axis] = 1
            nxt = context.empty_tensor(new_shape, "float32")
            context._call("wdc_reduce_axis", kind, int(i == len(sorted_axes) - 1), _p(cur), _p(nxt), outer,
                          red, inner, total)
            if cur is not inputs[0]:
                cur.dispose()
            cur, shape = nxt, new_shape
        final = shape if self.keepdims else [s for i, s in enumerate(shape) if i not in sorted_axes]
        if cur is inputs[0] or cur is x:
            y = context.empty_tensor(final, "float32")
            context.unary(UNARY_OPS["Identity"], cur, y)
            if x is not inputs[0]:
                x.dispose()
            return [y]
        out = cur.alias(final)
        cur.dispose()
        return [out]


class CudaLayerNormalization(OperatorImpl):
    """ONNX LayerNormalization (opset 17) over the last axis; not in the reference."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", -1)
        self.epsilon = get_attr_float(attribute, "epsilon", 1e-5)

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = context.canonical(inputs[0])
        axis = self.axis + x.ndim if self.axis < 0 else self.axis
        if axis != x.ndim - 1:
            raise ValueError("LayerNormalization: only the last axis is supported")
        gamma = inputs[1] if len(inputs) > 1 else None
        beta = inputs[2] if len(inputs) > 2 else None
        ln = x.dims[-1]
        y = context.empty_tensor(x.dims, "float32")
        context._call("wdc_layernorm", _p(x), _p(gamma), _p(beta), _p(y), x.length // ln, ln, self.epsilon)
        if x is not inputs[0]:
            x.dispose()
        return [y]


class CudaArgMax(OperatorImpl):
    """ONNX ArgMax; output is int32 (the runtime has no int64, constants.ts:9-15)."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", 0)
        self.keepdims = get_attr_int(attribute, "keepdims", 1) != 0
        self.select_last = get_attr_int(attribute, "select_last_index", 0) != 0

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        axis = self.axis + x.ndim if self.axis < 0 else self.axis
        owned = [x] if x is not inputs[0] else []
        if axis != x.ndim - 1:  # move the axis last
            perm = [i for i in range(x.ndim) if i != axis] + [axis]
            t = context.empty_tensor([x.dims[p] for p in perm], "float32")
            context.strided_copy(x, t, t.dims, [x.strides[p] for p in perm], 0, t.strides, 0)
            owned.append(t)
            src = t
        else:
            src = x
        ln = src.dims[-1]
        out_dims = list(x.dims)
        if self.keepdims:
            out_dims[axis] = 1
        else:
            del out_dims[axis]
        y = context.empty_tensor(out_dims, "int32")
        context._call("wdc_argmax", _p(src), _p(y), src.length // ln, ln, int(self.select_last))
        for t in owned:
            t.dispose()
        return [y]


# -------------------------------------------------------------------------- data movement
class CudaReshapeLike(OperatorImpl):
    """Flatten / Reshape / Squeeze / Unsqueeze: new dims over the same device memory, like
    operators/webgl/operators/standard/reshape5.ts:30 (no copy).  Shape/axes inputs stay on cpu."""

    def __init__(self, kind: str):
        super().__init__("cuda")
        self.kind = kind
        self.helper = None

    def initialize(self, attribute):
        if self.kind == "Flatten":
            self.helper = base.Flatten("cuda")
            self.helper.initialize(attribute)
        elif self.kind == "Reshape":
            self.helper = base.Reshape5("cuda")
            self.helper.initialize(attribute)
        else:
            self.axes = get_attr_ints(attribute, "axes", [])

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return ["cuda"] + ["cpu"] * (n_inputs - 1)

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        if self.kind == "Flatten":
            dims = self.helper.calc_shape(x)
        elif self.kind == "Reshape":
            dims = self.helper.calc_shape(x, inputs[1])
        else:
            axes = [int(a) for a in inputs[1].data] if len(inputs) > 1 else self.axes
            dims = squeeze_shape(x.dims, axes) if self.kind == "Squeeze" else unsqueeze_shape(x.dims, axes)
        y = x.alias(dims)
        if x is not inputs[0]:
            x.dispose()
        return [y]


class CudaTranspose(base.Transpose):
    def __init__(self):
        super().__init__("cuda")

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = inputs[0]
        if x.ndim > 6:
            raise ValueError(f"Transpose: ndim {x.ndim} > 6 is not supported")
        if x.layout == "nhwc":
            # logical strides of the physical storage: no canonical copy needed
            src_strides = x.nchw_strides()
            perm = self.perm if self.perm else [3, 2, 1, 0]
            out_shape = [x.dims[p] for p in perm]
            in_strides = [src_strides[p] for p in perm]
        else:
            out_shape, in_strides = self.calc_shape(x)
        y = context.empty_tensor(out_shape, x.data_type)
        context.strided_copy(x, y, out_shape, in_strides, 0, y.strides, 0)
        return [y]


class CudaConcat(OperatorImpl):
    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", 0)

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        ins = [context.canonical(t) for t in inputs]
        axis = self.axis if self.axis >= 0 else ins[0].ndim + self.axis
        if axis < 0 or axis >= ins[0].ndim:
            raise ValueError(f"Concat: axis {axis} out of range")
        out_shape = list(ins[0].dims)
        out_shape[axis] = sum(t.dims[axis] for t in ins)
        y = context.empty_tensor(out_shape, ins[0].data_type)
        off = 0
        for t in ins:
            if t.length:
                context.strided_copy(t, y, t.dims, t.strides, 0, y.strides, off * y.strides[axis])
            off += t.dims[axis]
        for t, o in zip(ins, inputs):
            if t is not o:
                t.dispose()
        return [y]


class CudaSplit(OperatorImpl):
    def __init__(self, split_from_input: bool):
        super().__init__("cuda")
        self.split_from_input = split_from_input

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", 0)
        self.split = get_attr_ints(attribute, "split", [])

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return ["cuda"] + ["cpu"] * (n_inputs - 1)

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        split = self.split
        if self.split_from_input and len(inputs) > 1:
            split = [int(v) for v in inputs[1].data]
        axis, params = base.split_params(x, n_outputs, self.axis, split)
        outs = []
        for dim, offset, out_shape in params:
            y = context.empty_tensor(out_shape, x.data_type)
            if y.length:
                context.strided_copy(x, y, out_shape, x.strides, offset * x.strides[axis], y.strides, 0)
            outs.append(y)
        if x is not inputs[0]:
            x.dispose()
        return outs


class CudaSlice(OperatorImpl):
    """slice.ts:12-90 (opset >= 10: starts/ends/axes/steps are cpu tensors)."""

    def __init__(self):
        super().__init__("cuda")

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return ["cuda"] + ["cpu"] * (n_inputs - 1)

    def run(self, context, inputs, n_outputs):
        import math
        x = context.canonical(inputs[0])
        starts, ends = inputs[1], inputs[2]
        axes = [int(a) for a in inputs[3].data] if len(inputs) > 3 else list(range(x.ndim))
        axes = [a + x.ndim if a < 0 else a for a in axes]
        steps = [int(s) for s in inputs[4].data] if len(inputs) > 4 else [1] * len(axes)
        ranges = [[0, d, 1, d] for d in x.dims]
        for i, ax in enumerate(axes):
            ranges[ax] = [int(starts.data[i]), int(ends.data[i]), steps[i], x.dims[ax]]
        out_dims, sstr, soff = [], [], 0
        for ax, (start, stop, step, size) in enumerate(ranges):
            if start < 0:
                start += size
            start = max(min(start, size - 1), 0)
            if stop < 0:
                stop += size
            stop = max(min(stop, size), -1)
            n = max(math.ceil((stop - start) / step), 0)
            out_dims.append(n)
            sstr.append(x.strides[ax] * step)
            soff += start * x.strides[ax]
        y = context.empty_tensor(out_dims, x.data_type)
        if y.length:
            # a negative step is a negative source stride from the (clamped) start element
            context.strided_copy(x, y, out_dims, sstr, soff, y.strides, 0)
        if x is not inputs[0]:
            x.dispose()
        return [y]


class CudaGather(OperatorImpl):
    """Gather along one axis with int32 indices (the cpu backend only picks a scalar from a 1-D
    tensor, gather.ts:20-33; that case gives the same result here)."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.axis = get_attr_int(attribute, "axis", 0)

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        data = context.canonical(inputs[0])
        idx = inputs[1]
        if idx.data_type != "int32":
            raise TypeError("Gather: indices must be int32")
        axis = self.axis + data.ndim if self.axis < 0 else self.axis
        outer, inner = array_prod(data.dims[:axis]), array_prod(data.dims[axis + 1:])
        out_dims = data.dims[:axis] + idx.dims + data.dims[axis + 1:]
        y = context.empty_tensor(out_dims, data.data_type)
        context._call("wdc_gather", _p(data), _p(idx), _p(y), outer, data.dims[axis], inner, idx.length)
        if data is not inputs[0]:
            data.dispose()
        return [y]


class CudaConvTranspose(OperatorImpl):
    """convtranspose.ts:30-263 with the shape rule of base/convtranspose.ts:34-104 (2-D only,
    auto_pad NOTSET, no explicit output_shape, like the reference)."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.auto_pad = get_attr_string(attribute, "auto_pad", "NOTSET")
        self.dilations = get_attr_ints(attribute, "dilations", [])
        self.group = get_attr_int(attribute, "group", 1)
        self.kernel_shape = get_attr_ints(attribute, "kernel_shape", [])
        self.output_padding = get_attr_ints(attribute, "output_padding", [])
        self.output_shape = get_attr_ints(attribute, "output_shape", [])
        self.pads = get_attr_ints(attribute, "pads", [])
        self.strides = get_attr_ints(attribute, "strides", [])

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        if inputs[0].ndim != 4:
            raise ValueError("ConvTranspose other than 2D is not yet supported")
        if self.auto_pad != "NOTSET":
            raise ValueError("ConvTranspose: auto_pad !== NOTSET is not yet supported.")
        if self.output_shape:
            raise ValueError("ConvTranspose: explicit output_shape is not yet supported.")
        x = context.canonical(inputs[0])
        w = context.canonical(inputs[1])
        bias = inputs[2] if len(inputs) > 2 else None
        dil = self.dilations or [1, 1]
        ks = self.kernel_shape or [w.dims[2], w.dims[3]]
        pads = self.pads or [0, 0, 0, 0]
        st = self.strides or [1, 1]
        op = self.output_padding or [0, 0]
        batch, ch_in, in_h, in_w = x.dims
        out_h = st[0] * (in_h - 1) + op[0] + (ks[0] - 1) * dil[0] + 1 - pads[0] - pads[2]
        out_w = st[1] * (in_w - 1) + op[1] + (ks[1] - 1) * dil[1] + 1 - pads[1] - pads[3]
        cog = w.dims[1]
        # Shapes the library runs as one tensor-core GEMM over the input pixels + col2im take the weight re-laid out
        # as [ch_in, k_h, k_w, ch_out] (made once, kept with the persistent weight tensor like a Conv's packed
        # weight), so that its hi/lo split stays cached and the run can be recorded as a graph.
        wk = w
        w_layout = 0
        n_cols = cog * ks[0] * ks[1]
        if (self.group == 1 and ch_in % 4 == 0 and ch_in >= 32 and n_cols % 4 == 0 and batch * in_h * in_w >= 128
                and w is inputs[1]):
            wk = inputs[1].aux.get("ckkc")
            if wk is None:
                taps = ks[0] * ks[1]
                wk = context.empty_tensor([ch_in, ks[0], ks[1], cog], "float32")
                context.strided_copy(w, wk, [ch_in, taps, cog], [cog * taps, 1, taps], 0, [taps * cog, cog, 1], 0)
                inputs[1].aux["ckkc"] = wk
            w_layout = 1
        d = ConvTransposeDesc(batch=batch, ch_in=ch_in, in_h=in_h, in_w=in_w, ch_out_per_group=cog, group=self.group,
                              k_h=ks[0], k_w=ks[1], out_h=out_h, out_w=out_w, stride_h=st[0], stride_w=st[1],
                              pad_t=pads[0], pad_l=pads[1], dil_h=dil[0], dil_w=dil[1], w_layout=w_layout)
        y = context.empty_tensor([batch, cog * self.group, out_h, out_w], "float32")
        context._call("wdc_conv_transpose2d", byref(d), _p(x), _p(wk), _p(bias) if bias is not None else None, _p(y))
        for t, o in ((x, inputs[0]), (w, inputs[1])):
            if t is not o:
                t.dispose()
        return [y]


class CudaInstanceNormalization(OperatorImpl):
    """instancenormalization.ts:9-53.  The reference reads ``epsilon`` with getAttrInt (:18): absent it
    is 1e-5, but an attribute stored as a float (the ONNX way) has an integer field of 0, so a given
    epsilon acts as 0.  That is kept: the same graph gives the reference's numbers."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.epsilon = float(get_attr_int(attribute, "epsilon", 1e-5))

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        x = context.canonical(inputs[0])
        scale, bias = inputs[1], inputs[2]
        y = context.empty_tensor(x.dims, "float32")
        area = array_prod(x.dims[2:])
        if x.length:
            context._call("wdc_instance_norm", _p(x), _p(scale), _p(bias), _p(y), x.dims[0], x.dims[1], area,
                          ctypes.c_double(self.epsilon))
        if x is not inputs[0]:
            x.dispose()
        return [y]


def _gather_axis(context, t, axis: int, index: np.ndarray):
    """t with axis `axis` re-indexed by `index` (int32 positions along that axis)."""
    idx = context.move_tensor(CPUTensor.from_array(np.ascontiguousarray(index, dtype=np.int32)))
    out_dims = list(t.dims)
    out_dims[axis] = int(index.size)
    y = context.empty_tensor(out_dims, t.data_type)
    context._call("wdc_gather", _p(t), _p(idx), _p(y), array_prod(t.dims[:axis]), t.dims[axis],
                  array_prod(t.dims[axis + 1:]), int(index.size))
    idx.dispose()
    return y


class CudaPad11(OperatorImpl):
    """pad11.ts (cpu) / base/pad11.ts:14-50: constant, reflect and edge padding of up to 6-D tensors;
    pads (and the optional constant) are cpu tensors.  Every mode maps an output index to an input
    index axis by axis, so reflect/edge are one gather per padded axis and constant is a fill plus
    one strided copy of the part of the input that stays visible (negative pads crop)."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.mode = get_attr_string(attribute, "mode", "constant")

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return [self.backend, "cpu"] if n_inputs == 2 else [self.backend, "cpu", "cpu"]

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        if x.ndim > 6:
            raise ValueError(f"Pad: input.ndim = {x.ndim} > 6 is not yet supported")
        pads = [int(v) for v in inputs[1].get_data()]
        nd = x.ndim
        out_dims = [x.dims[i] + pads[i] + pads[i + nd] for i in range(nd)]
        if self.mode == "constant":
            value = inputs[2].get_data()[0] if len(inputs) > 2 else 0
            y = context.empty_tensor(out_dims, x.data_type)
            bits = int(np.asarray(value, dtype=NP_DTYPE[x.data_type]).view(np.uint32))
            if y.length:
                context._call("wdc_fill_u32", _p(y), bits, y.length)
            lo = [max(0, -pads[i]) for i in range(nd)]                           # first visible input index
            hi = [min(x.dims[i], out_dims[i] - pads[i]) for i in range(nd)]     # one past the last
            region = [h - l for l, h in zip(lo, hi)]
            if nd == 0:
                context.unary(UNARY_OPS["Identity"], x, y)
            elif all(r > 0 for r in region):
                soff = sum(l * s for l, s in zip(lo, x.strides))
                doff = sum((l + pads[i]) * s for i, (l, s) in enumerate(zip(lo, y.strides)))
                context.strided_copy(x, y, region, list(x.strides), soff, list(y.strides), doff)
        elif self.mode in ("reflect", "edge"):
            cur = x
            for i in range(nd):
                if pads[i] == 0 and pads[i + nd] == 0:
                    continue
                n = cur.dims[i]
                src = np.arange(out_dims[i], dtype=np.int64) - pads[i]
                if self.mode == "edge":
                    src = np.clip(src, 0, n - 1)
                else:
                    period = n * 2 - 2
                    neg = src < 0
                    m = np.where(neg, (-src) % period if period else 0, src % period if period else 0)
                    m = np.where((neg | (src >= n)), m, src)
                    src = np.where(m >= n, n * 2 - m - 2, m)
                nxt = _gather_axis(context, cur, i, src)
                if cur is not x:
                    cur.dispose()
                cur = nxt
            y = cur if cur is not x else context.empty_tensor(out_dims, x.data_type)
            if cur is x:
                context.unary(UNARY_OPS["Identity"], x, y)
        else:
            raise ValueError(f"Pad: unknown mode {self.mode}")
        if x is not inputs[0]:
            x.dispose()
        return [y]


class CudaTile6(OperatorImpl):
    """tile.ts:11-70: out[d] = in[d mod dims], up to 4-D like the reference; repeats is a cpu tensor.
    One gather per repeated axis."""

    def __init__(self):
        super().__init__("cuda")

    def get_tensor_backend_requirement(self, n_inputs, n_outputs):
        return [self.backend, "cpu"]

    def run(self, context, inputs, n_outputs):
        x = context.canonical(inputs[0])
        if x.ndim > 4:
            raise ValueError(f"Tile: input.ndim = {x.ndim} > 4 is not yet supported")
        repeats = [int(v) for v in inputs[1].get_data()]
        cur = x
        for i in range(x.ndim):
            if repeats[i] == 1:
                continue
            n = x.dims[i]
            nxt = _gather_axis(context, cur, i, np.arange(n * repeats[i], dtype=np.int64) % max(n, 1))
            if cur is not x:
                cur.dispose()
            cur = nxt
        if cur is x:
            y = context.empty_tensor(x.dims, x.data_type)
            context.unary(UNARY_OPS["Identity"], x, y)
            cur = y
        if x is not inputs[0]:
            x.dispose()
        return [cur]


class CudaLSTM(OperatorImpl):
    """ONNX LSTM, forward direction, inputs [X, W, R, (B), (sequence_lens), (initial_h),
    (initial_c)] given without empty-name placeholders: the runner cannot bind ""
    (runnerImpl.ts:392-409), so trailing optional inputs are simply absent."""

    def __init__(self):
        super().__init__("cuda")

    def initialize(self, attribute):
        self.hidden_size = get_attr_int(attribute, "hidden_size", 0)
        self.direction = base.get_attr_string(attribute, "direction", "forward")
        if self.direction != "forward":
            raise ValueError("LSTM: only direction=forward is supported")
        if get_attr_int(attribute, "input_forget", 0) != 0:
            raise ValueError("LSTM: input_forget is not supported")
        # The kernels implement the operator's defaults only; anything else must fail here rather than
        # return the default's numbers.
        for a in attribute:
            if a.name == "activations":
                acts = [v.decode("utf-8") if isinstance(v, bytes) else str(v) for v in a.strings]
                if [v.lower() for v in acts] != ["sigmoid", "tanh", "tanh"]:
                    raise ValueError(f"LSTM: activations {acts} are not supported (only Sigmoid, Tanh, Tanh)")
            elif a.name in ("activation_alpha", "activation_beta") and len(a.floats) > 0:
                raise ValueError(f"LSTM: {a.name} is not supported")
        if get_attr_float(attribute, "clip", 0.0) != 0.0 or any(a.name == "clip" for a in attribute):
            raise ValueError("LSTM: clip is not supported")
        if get_attr_int(attribute, "layout", 0) != 0:
            raise ValueError("LSTM: layout=1 (batch-major) is not supported")

    def run(self, context, inputs, n_outputs):
        context.asserts_cuda_tensor_array(inputs)
        if len(inputs) == 5 or len(inputs) > 7:
            raise ValueError("LSTM: sequence_lens is not supported")
        for j, t in enumerate(inputs):
            if j != 4 and t.data_type != "float32":     # input 4 is sequence_lens (int32)
                raise TypeError(f"LSTM: DataType {t.data_type} not supported")
        x, w, r = inputs[0], inputs[1], inputs[2]
        b = inputs[3] if len(inputs) > 3 else None
        h0 = inputs[5] if len(inputs) > 5 else None
        c0 = inputs[6] if len(inputs) > 6 else None
        T, Bt, I = x.dims
        H = self.hidden_size or r.dims[2]
        if w.dims != [1, 4 * H, I] or r.dims != [1, 4 * H, H]:
            raise ValueError("LSTM: weight shapes do not match hidden_size")
        y = context.empty_tensor([T, 1, Bt, H], "float32")
        yh = context.empty_tensor([1, Bt, H], "float32")
        yc = context.empty_tensor([1, Bt, H], "float32")
        context._call("wdc_lstm", _p(x), _p(w), _p(r), _p(b), _p(h0), _p(c0), _p(y), _p(yh), _p(yc), T, Bt, I, H)
        outs = [y, yh, yc][:n_outputs]
        for t in [y, yh, yc][n_outputs:]:
            t.dispose()
        return outs


# ------------------------------------------------------------------------------- registry
def get_op_entries() -> List[OperatorEntry]:
    E = OperatorEntry
    entries: List[OperatorEntry] = []
    int_ok = {"Abs", "Neg", "Relu", "Sign"}
    for name in ["Abs", "Acos", "Acosh", "Asin", "Asinh", "Atan", "Atanh", "Ceil", "Cos", "Cosh", "Exp",
                 "Floor", "HardSwish", "Log", "Neg", "Reciprocal", "Relu", "Round", "Sigmoid", "Sign",
                 "Sin", "Softplus", "Softsign", "Sqrt", "Tan", "Tanh", "Elu", "HardSigmoid", "LeakyRelu",
                 "Selu", "ThresholdedRelu", "Identity"]:
        allow = ("float32", "int32") if name in int_ok or name == "Identity" else ("float32",)
        entries.append(E(name, 1, None, "cuda", lambda n=name, a=allow: CudaUnary(n, a)))
    entries.append(E("Clip", 1, 11, "cuda", lambda: CudaUnary("Clip")))
    for name in ["Add", "Sub", "Mul", "Div", "Pow"]:
        entries.append(E(name, 7, None, "cuda", lambda n=name: CudaBinary7(n)))
    for name in ["Max", "Min", "Sum", "Mean"]:
        entries.append(E(name, 1, None, "cuda", lambda n=name: CudaEachElementwise(n)))
    entries += [
        E("Cast", 6, None, "cuda", CudaCast),
        E("Gemm", 1, None, "cuda", CudaGemm),
        E("CudaGemmRelu", 1, None, "cuda", lambda: CudaGemm(relu=True)),
        E("CudaMatMulBias", 1, None, "cuda", CudaMatMulBias),
        E("CudaAttention", 1, None, "cuda", CudaAttention),
        E("MatMul", 1, None, "cuda", CudaMatMul),
        E("Conv", 1, None, "cuda", CudaConv),
        E("CudaConvFused", 1, None, "cuda", lambda: CudaConv(fused=True)),
        E("BatchNormalization", 9, None, "cuda", CudaBatchNormalization),
        E("MaxPool", 1, None, "cuda", CudaMaxPool),
        E("AveragePool", 1, None, "cuda", CudaAveragePool),
        E("GlobalAveragePool", 1, None, "cuda", CudaGlobalAveragePool),
        E("Softmax", 1, None, "cuda", CudaSoftmax),
        E("LayerNormalization", 17, None, "cuda", CudaLayerNormalization),
        E("CudaLayerNorm", 1, None, "cuda", CudaLayerNormalization),
        E("ArgMax", 1, None, "cuda", CudaArgMax),
        E("Flatten", 1, None, "cuda", lambda: CudaReshapeLike("Flatten")),
        E("Reshape", 5, None, "cuda", lambda: CudaReshapeLike("Reshape")),
        E("Squeeze", 1, None, "cuda", lambda: CudaReshapeLike("Squeeze")),
        E("Unsqueeze", 1, None, "cuda", lambda: CudaReshapeLike("Unsqueeze")),
        E("Transpose", 1, None, "cuda", CudaTranspose),
        E("Concat", 1, None, "cuda", CudaConcat),
        E("Split", 1, 13, "cuda", lambda: CudaSplit(False)),
        E("Split", 13, None, "cuda", lambda: CudaSplit(True)),
        E("Slice", 10, None, "cuda", CudaSlice),
        E("Gather", 1, None, "cuda", CudaGather),
        E("ConvTranspose", 1, None, "cuda", CudaConvTranspose),
        E("InstanceNormalization", 1, None, "cuda", CudaInstanceNormalization),
        E("Pad", 11, None, "cuda", CudaPad11),
        E("Tile", 6, None, "cuda", CudaTile6),
        E("LSTM", 7, None, "cuda", CudaLSTM),
    ]
    for name in REDUCE_KINDS:
        if name == "ReduceSum":
            entries.append(E(name, 1, 13, "cuda", lambda n=name: CudaReduce(n, False)))
            entries.append(E(name, 13, None, "cuda", lambda n=name: CudaReduce(n, True)))
        else:
            entries.append(E(name, 1, None, "cuda", lambda n=name: CudaReduce(n, False)))
    return entries
