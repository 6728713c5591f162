"""Synthetic ONNX graphs for the benchmark and parity configurations.

The reference builds its benchmark models by exporting pretrained PyTorch networks
(``example/benchmark/make_models.py:130-164``); there is no network access and no ONNX exporter
here, so the same topologies are written out node by node with seeded random parameters.  The
graphs use only operator forms the reference's cpu backend accepts (last-axis Softmax, rank <= 3
MatMul, 2-D NCHW Conv/Pool, Flatten axis 1) plus BatchNormalization and LSTM, which the task's
configurations name although no reference backend implements them.

Weight init: seed 0 -- conv/linear weights N(0, 2/fan_in), biases U(-0.1, 0.1), BatchNormalization
gamma U(0.5, 1.5), beta N(0, 0.1), mean N(0, 0.1), var U(0.5, 1.5).  Inputs come from
``make_input`` with seed 1.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

from .onnx_io import FLOAT, Graph, Model, ValueInfo, make_node, make_tensor


class _Builder:
    def __init__(self, seed: int = 0):
        self.rng = np.random.default_rng(seed)
        self.nodes = []
        self.inits = []
        self.counter = 0

    def name(self, prefix: str) -> str:
        self.counter += 1
        return f"{prefix}_{self.counter}"

    def init(self, name: str, arr: np.ndarray) -> str:
        self.inits.append(make_tensor(name, arr))
        return name

    def he(self, shape, fan_in) -> np.ndarray:
        return (self.rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)

    def bias(self, n) -> np.ndarray:
        return self.rng.uniform(-0.1, 0.1, n).astype(np.float32)

    def node(self, op, inputs, n_out=1, **attrs) -> List[str]:
        outs = [self.name(op.lower()) for _ in range(n_out)]
        self.nodes.append(make_node(op, inputs, outs, name=self.name(op), **attrs))
        return outs

    def conv(self, x, cin, cout, k, stride=1, pad=0, bias=False, group=1, dilation=1) -> str:
        w = self.init(self.name("w"), self.he((cout, cin // group, k, k), (cin // group) * k * k))
        ins = [x, w]
        if bias:
            ins.append(self.init(self.name("b"), self.bias(cout)))
        return self.node("Conv", ins, kernel_shape=[k, k], strides=[stride, stride],
                         pads=[pad, pad, pad, pad], dilations=[dilation, dilation], group=group)[0]

    def bn(self, x, c) -> str:
        r = self.rng
        g = self.init(self.name("bn_gamma"), r.uniform(0.5, 1.5, c).astype(np.float32))
        b = self.init(self.name("bn_beta"), (r.standard_normal(c) * 0.1).astype(np.float32))
        m = self.init(self.name("bn_mean"), (r.standard_normal(c) * 0.1).astype(np.float32))
        v = self.init(self.name("bn_var"), r.uniform(0.5, 1.5, c).astype(np.float32))
        return self.node("BatchNormalization", [x, g, b, m, v], epsilon=1e-5)[0]

    def linear(self, x, cin, cout, trans_b=True) -> str:
        w = self.he((cout, cin), cin)
        if not trans_b:
            w = np.ascontiguousarray(w.T)
        wn = self.init(self.name("fc_w"), w)
        bn = self.init(self.name("fc_b"), self.bias(cout))
        return self.node("Gemm", [x, wn, bn], transB=int(trans_b))[0]

    def model(self, inputs: List[Tuple[str, List[int]]], outputs: List[Tuple[str, List[int]]], opset=13,
              name="graph") -> Model:
        g = Graph(name, self.nodes, self.inits,
                  [ValueInfo(n, FLOAT, s) for n, s in inputs], [ValueInfo(n, FLOAT, s) for n, s in outputs])
        return Model(g, ir_version=7, opset_import=[("", opset)], producer_name="webdnn_b200.zoo")


def mlp(batch: int = 64, trans_b: bool = True) -> Model:
    """784 -> 512 -> 512 -> 10 with Relu and a final Softmax."""
    b = _Builder(0)
    h = b.node("Relu", [b.linear("input", 784, 512, trans_b)])[0]
    h = b.node("Relu", [b.linear(h, 512, 512, trans_b)])[0]
    h = b.linear(h, 512, 10, trans_b)
    out = b.node("Softmax", [h], axis=-1)[0]
    return b.model([("input", [batch, 784])], [(out, [batch, 10])], name="mlp")


def conv_bn_relu(batch: int = 32, ch: int = 64, size: int = 56) -> Model:
    """One 3x3 stride-1 pad-1 Conv with bias, BatchNormalization and Relu."""
    b = _Builder(0)
    h = b.conv("input", ch, ch, 3, 1, 1, bias=True)
    h = b.bn(h, ch)
    out = b.node("Relu", [h])[0]
    return b.model([("input", [batch, ch, size, size])], [(out, [batch, ch, size, size])], name="conv_bn_relu")


def _bottleneck(b: _Builder, x: str, cin: int, planes: int, stride: int, downsample: bool) -> str:
    out = b.node("Relu", [b.bn(b.conv(x, cin, planes, 1), planes)])[0]
    out = b.node("Relu", [b.bn(b.conv(out, planes, planes, 3, stride, 1), planes)])[0]  # v1.5: stride on 3x3
    out = b.bn(b.conv(out, planes, planes * 4, 1), planes * 4)
    identity = x
    if downsample:
        identity = b.bn(b.conv(x, cin, planes * 4, 1, stride), planes * 4)
    out = b.node("Add", [out, identity])[0]
    return b.node("Relu", [out])[0]


def resnet_trunk(b: _Builder, x: str, width: int = 64, blocks=(3, 4, 6, 3)) -> Tuple[str, int]:
    h = b.node("Relu", [b.bn(b.conv(x, 3, width, 7, 2, 3), width)])[0]
    h = b.node("MaxPool", [h], kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])[0]
    cin = width
    for stage, n in enumerate(blocks):
        planes = width * (2 ** stage)
        for i in range(n):
            stride = 2 if (i == 0 and stage > 0) else 1
            h = _bottleneck(b, h, cin, planes, stride, downsample=(i == 0))
            cin = planes * 4
    return h, cin


def resnet50(batch: int = 1, size: int = 224, width: int = 64, blocks=(3, 4, 6, 3), classes: int = 1000,
             softmax: bool = True) -> Model:
    """ResNet-50 v1.5 (torchvision topology), NCHW input [batch, 3, size, size]."""
    b = _Builder(0)
    h, c = resnet_trunk(b, "input", width, blocks)
    h = b.node("GlobalAveragePool", [h])[0]
    h = b.node("Flatten", [h], axis=1)[0]
    h = b.linear(h, c, classes)
    if softmax:
        h = b.node("Softmax", [h], axis=-1)[0]
    return b.model([("input", [batch, 3, size, size])], [(h, [batch, classes])], name="resnet50")


class _Transformer:
    """Node-by-node pieces of a post-norm encoder/decoder (DETR style), written only with operator
    forms the reference's cpu backend runs: MatMul of rank <= 3, last-axis Softmax, LayerNorm as the
    ReduceMean / Sub / Mul / Add / Sqrt / Div chain (opset 13)."""

    def __init__(self, b: _Builder, batch: int, d: int, heads: int, ffn: int):
        self.b, self.batch, self.d, self.heads, self.ffn = b, batch, d, heads, ffn
        self.dh = d // heads
        self.scale = b.init(b.name("attn_scale"), np.array(1.0 / np.sqrt(self.dh), np.float32))
        self.eps = b.init(b.name("ln_eps"), np.array(1e-5, np.float32))

    def shape(self, dims) -> str:
        return self.b.init(self.b.name("shape"), np.array(dims, np.int64))

    def linear(self, x: str, cin: int, cout: int) -> str:
        b = self.b
        w = b.init(b.name("w"), b.he((cin, cout), cin))
        bias = b.init(b.name("b"), b.bias(cout))
        return b.node("Add", [b.node("MatMul", [x, w])[0], bias])[0]

    def layer_norm(self, x: str) -> str:
        b = self.b
        g = b.init(b.name("ln_g"), b.rng.uniform(0.5, 1.5, self.d).astype(np.float32))
        be = b.init(b.name("ln_b"), (b.rng.standard_normal(self.d) * 0.1).astype(np.float32))
        mean = b.node("ReduceMean", [x], axes=[-1], keepdims=1)[0]
        xc = b.node("Sub", [x, mean])[0]
        var = b.node("ReduceMean", [b.node("Mul", [xc, xc])[0]], axes=[-1], keepdims=1)[0]
        std = b.node("Sqrt", [b.node("Add", [var, self.eps])[0]])[0]
        y = b.node("Div", [xc, std])[0]
        return b.node("Add", [b.node("Mul", [y, g])[0], be])[0]

    def split_heads(self, x: str, tokens: int) -> str:
        b = self.b
        h = b.node("Reshape", [x, self.shape([self.batch, tokens, self.heads, self.dh])])[0]
        h = b.node("Transpose", [h], perm=[0, 2, 1, 3])[0]
        return b.node("Reshape", [h, self.shape([self.batch * self.heads, tokens, self.dh])])[0]

    def attention(self, q_in: str, k_in: str, v_in: str, tq: int, tk: int) -> str:
        b = self.b
        q = self.split_heads(self.linear(q_in, self.d, self.d), tq)
        k = self.split_heads(self.linear(k_in, self.d, self.d), tk)
        v = self.split_heads(self.linear(v_in, self.d, self.d), tk)
        kt = b.node("Transpose", [k], perm=[0, 2, 1])[0]
        scores = b.node("Mul", [b.node("MatMul", [q, kt])[0], self.scale])[0]
        p = b.node("Softmax", [scores], axis=-1)[0]
        ctx = b.node("MatMul", [p, v])[0]
        ctx = b.node("Reshape", [ctx, self.shape([self.batch, self.heads, tq, self.dh])])[0]
        ctx = b.node("Transpose", [ctx], perm=[0, 2, 1, 3])[0]
        ctx = b.node("Reshape", [ctx, self.shape([self.batch, tq, self.d])])[0]
        return self.linear(ctx, self.d, self.d)

    def feed_forward(self, x: str) -> str:
        h = self.b.node("Relu", [self.linear(x, self.d, self.ffn)])[0]
        return self.linear(h, self.ffn, self.d)

    def add_norm(self, x: str, y: str) -> str:
        return self.layer_norm(self.b.node("Add", [x, y])[0])


def detr(batch: int = 1, size: int = 800, d: int = 256, heads: int = 8, enc_layers: int = 6, dec_layers: int = 6,
         ffn: int = 2048, queries: int = 100, classes: int = 92, width: int = 64, blocks=(3, 4, 6, 3)) -> Model:
    """DETR-style detector: ResNet trunk, 1x1 projection to d channels, learned position embeddings,
    post-norm transformer encoder / decoder with `queries` object queries, class head and 3-layer box
    head.  Input [batch, 3, size, size]; outputs logits [batch, queries, classes] and boxes
    [batch, queries, 4].  Tokens are kept batch-first so that every MatMul has rank <= 3."""
    b = _Builder(0)
    h, c = resnet_trunk(b, "input", width, blocks)
    side = size
    for _ in range(5):
        side = (side + 1) // 2
    tokens = side * side
    h = b.conv(h, c, d, 1, bias=True)
    t = _Transformer(b, batch, d, heads, ffn)
    h = b.node("Reshape", [h, t.shape([batch, d, tokens])])[0]
    src = b.node("Transpose", [h], perm=[0, 2, 1])[0]                       # [batch, tokens, d]
    pos = b.init("pos_embed", b.rng.standard_normal((1, tokens, d)).astype(np.float32))
    for _ in range(enc_layers):
        qk = b.node("Add", [src, pos])[0]
        src = t.add_norm(src, t.attention(qk, qk, src, tokens, tokens))
        src = t.add_norm(src, t.feed_forward(src))
    memory = src
    mem_k = b.node("Add", [memory, pos])[0]
    qpos = b.init("query_embed", b.rng.standard_normal((1, queries, d)).astype(np.float32))
    tgt = b.init("tgt0", np.zeros((batch, queries, d), np.float32))
    for _ in range(dec_layers):
        q = b.node("Add", [tgt, qpos])[0]
        tgt = t.add_norm(tgt, t.attention(q, q, tgt, queries, queries))
        q = b.node("Add", [tgt, qpos])[0]
        tgt = t.add_norm(tgt, t.attention(q, mem_k, memory, queries, tokens))
        tgt = t.add_norm(tgt, t.feed_forward(tgt))
    logits = t.linear(tgt, d, classes)
    box = b.node("Relu", [t.linear(tgt, d, d)])[0]
    box = b.node("Relu", [t.linear(box, d, d)])[0]
    box = b.node("Sigmoid", [t.linear(box, d, 4)])[0]
    return b.model([("input", [batch, 3, size, size])],
                   [(logits, [batch, queries, classes]), (box, [batch, queries, 4])], name="detr")


def lstm(seq: int = 128, batch: int = 64, input_size: int = 256, hidden: int = 512) -> Model:
    """Single forward LSTM node; inputs [X, W, R, B] only (zero initial state by omission)."""
    b = _Builder(0)
    lim = 1.0 / np.sqrt(hidden)
    r = b.rng
    w = b.init("W", r.uniform(-lim, lim, (1, 4 * hidden, input_size)).astype(np.float32))
    rr = b.init("R", r.uniform(-lim, lim, (1, 4 * hidden, hidden)).astype(np.float32))
    bb = b.init("B", r.uniform(-lim, lim, (1, 8 * hidden)).astype(np.float32))
    y, yh, yc = b.node("LSTM", ["X", w, rr, bb], n_out=3, hidden_size=hidden, direction="forward")
    return b.model([("X", [seq, batch, input_size])],
                   [(y, [seq, 1, batch, hidden]), (yh, [1, batch, hidden]), (yc, [1, batch, hidden])],
                   name="lstm")


def make_input(shape, kind: str = "normal", seed: int = 1) -> np.ndarray:
    rng = np.random.default_rng(seed)
    if kind == "uniform":
        return rng.uniform(0.0, 1.0, shape).astype(np.float32)
    return rng.standard_normal(shape).astype(np.float32)


def contraction_flops(model: Model, input_shapes: Dict[str, List[int]]) -> int:
    """Algorithmic FLOPs of the Conv / Gemm nodes of a zoo graph: 2 * MACs, by shape propagation
    over the few op types these graphs contain."""
    import math
    shapes: Dict[str, List[int]] = dict(input_shapes)
    for t in model.graph.initializer:
        shapes[t.name] = list(t.dims)
    flops = 0
    for n in model.graph.node:
        a = {x.name: x for x in n.attribute}
        if n.op_type == "Conv":
            x, w = shapes[n.input[0]], shapes[n.input[1]]
            k, s, p = a["kernel_shape"].ints, a["strides"].ints, a["pads"].ints
            d = a["dilations"].ints
            oh = math.floor((x[2] + p[0] + p[2] - d[0] * (k[0] - 1) - 1) / s[0]) + 1
            ow = math.floor((x[3] + p[1] + p[3] - d[1] * (k[1] - 1) - 1) / s[1]) + 1
            shapes[n.output[0]] = [x[0], w[0], oh, ow]
            flops += 2 * x[0] * w[0] * oh * ow * w[1] * k[0] * k[1]
        elif n.op_type == "Gemm":
            x, w = shapes[n.input[0]], shapes[n.input[1]]
            tb = a["transB"].i if "transB" in a else 0
            nn = w[0] if tb else w[1]
            shapes[n.output[0]] = [x[0], nn]
            flops += 2 * x[0] * nn * x[1]
        elif n.op_type == "MaxPool":
            x = shapes[n.input[0]]
            k, s, p = a["kernel_shape"].ints, a["strides"].ints, a["pads"].ints
            oh = math.floor((x[2] + p[0] + p[2] - k[0]) / s[0]) + 1
            ow = math.floor((x[3] + p[1] + p[3] - k[1]) / s[1]) + 1
            shapes[n.output[0]] = [x[0], x[1], oh, ow]
        elif n.op_type == "GlobalAveragePool":
            x = shapes[n.input[0]]
            shapes[n.output[0]] = [x[0], x[1], 1, 1]
        elif n.op_type == "Flatten":
            x = shapes[n.input[0]]
            shapes[n.output[0]] = [x[0], int(np.prod(x[1:]))]
        else:
            shapes[n.output[0]] = list(shapes[n.input[0]])
    return flops
