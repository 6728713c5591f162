"""Generates tests/golden/torch_cases.npz: inputs and float64-PyTorch expectations for single ops.

The reference commits no golden tensors: its legacy op zoo (test/model_test/make_models.py:575-732)
and its e2e fixtures (test/fixtures/generate_fixtures.py) compute expectations at test time with
PyTorch / onnxruntime.  This script restates that approach with the same case shapes (trimmed where
a case is large) and PyTorch in float64 on the CPU, then rounds to float32.  It needs only torch and
numpy; it is run by hand when cases change:  python tests/golden/make_golden.py

Each case stores: op type, attributes (JSON), input arrays, expected output arrays.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch
import torch.nn.functional as F

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_cases.npz")
rng = np.random.default_rng(0)
cases = {}


def f32(*shape, scale=1.0, positive=False):
    a = rng.random(shape) if positive else rng.standard_normal(shape)
    return (a * scale).astype(np.float32)


def t64(a):
    return torch.tensor(a, dtype=torch.float64)


def add(name, op, attrs, inputs, outputs):
    cases[name] = dict(op=op, attrs=attrs, n_in=len(inputs), n_out=len(outputs))
    for i, a in enumerate(inputs):
        cases[name][f"in{i}"] = np.asarray(a)
    for i, a in enumerate(outputs):
        cases[name][f"out{i}"] = np.asarray(a)


def conv_case(name, cin, cout, k, stride, pad, dil, groups, bias, shape):
    x = f32(*shape)
    w = f32(cout, cin // groups, k, k, scale=(2.0 / ((cin // groups) * k * k)) ** 0.5)
    b = f32(cout) if bias else None
    y = F.conv2d(t64(x), t64(w), t64(b) if bias else None, stride, pad, dil, groups)
    attrs = dict(kernel_shape=[k, k], strides=[stride, stride], pads=[pad] * 4, dilations=[dil, dil], group=groups)
    add(name, "Conv", attrs, [x, w] + ([b] if bias else []), [y.numpy().astype(np.float32)])


# shapes of test/model_test/make_models.py:617-636 (conv8/10/11 trimmed: same code paths, fewer channels)
conv_case("conv1", 2, 4, 3, 1, 0, 1, 1, False, (1, 2, 8, 8))
conv_case("conv2", 3, 4, 7, 2, 3, 1, 1, False, (2, 3, 8, 16))
conv_case("conv3", 4, 8, 7, 2, 3, 1, 2, False, (3, 4, 8, 16))
conv_case("conv4", 4, 8, 3, 2, 3, 2, 2, False, (3, 4, 8, 16))
conv_case("conv5", 4, 8, 3, 2, 3, 2, 2, True, (3, 4, 8, 16))
conv_case("conv6", 16, 32, 3, 1, 1, 1, 1, False, (2, 16, 28, 28))
conv_case("conv7", 16, 33, 3, 1, 1, 1, 1, False, (2, 16, 28, 28))
conv_case("conv8", 256, 64, 3, 1, 1, 1, 64, False, (1, 256, 7, 7))
conv_case("conv9", 64, 64, 3, 1, 1, 1, 64, False, (1, 64, 7, 7))
conv_case("conv_c64_56", 64, 64, 3, 1, 1, 1, 1, True, (1, 64, 20, 20))
conv_case("conv_1x1_s2", 64, 128, 1, 2, 0, 1, 1, False, (2, 64, 14, 14))
conv_case("conv_fixture", 1, 1, 2, 1, 0, 1, 1, False, (1, 1, 3, 3))

# gemm / matmul (make_models.py:613-615, generate_fixtures.py:66-85)
a, b, c = f32(2, 3), f32(3, 4), f32(4)
add("gemm_fixture", "Gemm", dict(alpha=1.0, beta=1.0), [a, b, c], [(t64(a) @ t64(b) + t64(c)).numpy().astype(np.float32)])
a, b, c = f32(3, 128), f32(64, 128), f32(64)
add("gemm_transb", "Gemm", dict(transB=1, alpha=0.5, beta=2.0), [a, b, c],
    [(0.5 * (t64(a) @ t64(b).T) + 2.0 * t64(c)).numpy().astype(np.float32)])
a, b, c = f32(70, 5), f32(70, 9), f32(5, 1)
add("gemm_transa", "Gemm", dict(transA=1), [a, b, c], [(t64(a).T @ t64(b) + t64(c)).numpy().astype(np.float32)])
a, b = f32(3, 128), f32(128, 8)
add("matmul", "MatMul", {}, [a, b], [(t64(a) @ t64(b)).numpy().astype(np.float32)])
a, b = f32(1, 3, 128), f32(4, 128, 1)
add("matmul2", "MatMul", {}, [a, b], [(t64(a) @ t64(b)).numpy().astype(np.float32)])
a, b = f32(8, 50, 32), f32(8, 32, 50)
add("matmul_attn", "MatMul", {}, [a, b], [(t64(a) @ t64(b)).numpy().astype(np.float32)])
a, b = f32(128), f32(128)
add("matmul_1d", "MatMul", {}, [a, b], [np.asarray((t64(a) @ t64(b)).numpy(), np.float32)])

# pools (make_models.py:643-653)
x = f32(2, 3, 10, 12)
add("maxpool1", "MaxPool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[0, 0, 0, 0]), [x],
    [F.max_pool2d(t64(x), 3, 2, 0).numpy().astype(np.float32)])
add("maxpool2", "MaxPool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[0, 0, 0, 0], ceil_mode=1), [x],
    [F.max_pool2d(t64(x), 3, 2, 0, ceil_mode=True).numpy().astype(np.float32)])
add("maxpool_resnet", "MaxPool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1]), [x],
    [F.max_pool2d(t64(x), 3, 2, 1).numpy().astype(np.float32)])
add("avgpool3", "AveragePool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[0, 0, 0, 0], ceil_mode=1,
                                    count_include_pad=0), [x],
    [F.avg_pool2d(t64(x), 3, 2, 0, ceil_mode=True, count_include_pad=False).numpy().astype(np.float32)])
add("avgpool_pad", "AveragePool", dict(kernel_shape=[3, 3], strides=[1, 1], pads=[1, 1, 1, 1], count_include_pad=1),
    [x], [F.avg_pool2d(t64(x), 3, 1, 1, count_include_pad=True).numpy().astype(np.float32)])
add("globalavgpool", "GlobalAveragePool", {}, [x], [t64(x).mean((2, 3), keepdim=True).numpy().astype(np.float32)])

# softmax / reductions (make_models.py:718-727)
x = f32(3, 4, 5, 6)
add("softmax", "Softmax", dict(axis=-1), [x], [torch.softmax(t64(x), -1).numpy().astype(np.float32)])
x2 = f32(4, 1500, scale=3.0)
add("softmax_long", "Softmax", dict(axis=-1), [x2], [torch.softmax(t64(x2), -1).numpy().astype(np.float32)])
add("reducemax", "ReduceMax", dict(axes=[1], keepdims=0), [x], [t64(x).amax(1).numpy().astype(np.float32)])
add("reducemin", "ReduceMin", dict(axes=[1], keepdims=0), [x], [t64(x).amin(1).numpy().astype(np.float32)])
add("reducemean", "ReduceMean", dict(axes=[1], keepdims=0), [x], [t64(x).mean(1).numpy().astype(np.float32)])
add("reduceprod", "ReduceProd", dict(axes=[1], keepdims=0), [x], [t64(x).prod(1).numpy().astype(np.float32)])
add("reducesum_multi", "ReduceSum", dict(axes=[1, 3], keepdims=1, _opset=11), [x],
    [t64(x).sum((1, 3), keepdim=True).numpy().astype(np.float32)])
add("reducemean_last", "ReduceMean", dict(axes=[-1], keepdims=1), [x],
    [t64(x).mean(-1, keepdim=True).numpy().astype(np.float32)])
add("reducel2", "ReduceL2", dict(axes=[2], keepdims=0), [x], [t64(x).pow(2).sum(2).sqrt().numpy().astype(np.float32)])

# unary / binary (make_models.py:585-612, 668-688)
x = f32(3, 4)
for op, fn in [("Sigmoid", torch.sigmoid), ("Tanh", torch.tanh), ("Exp", torch.exp), ("Softplus", F.softplus),
               ("Softsign", F.softsign), ("Sin", torch.sin), ("Cos", torch.cos), ("Tan", torch.tan),
               ("Atan", torch.atan), ("Abs", torch.abs), ("Neg", torch.neg), ("Ceil", torch.ceil),
               ("Floor", torch.floor), ("Relu", torch.relu)]:
    add(f"unary_{op.lower()}", op, {}, [x], [fn(t64(x)).numpy().astype(np.float32)])
xp = f32(3, 4, positive=True)
add("unary_sqrt", "Sqrt", {}, [xp], [torch.sqrt(t64(xp)).numpy().astype(np.float32)])
add("unary_log", "Log", {}, [xp + 1], [torch.log(t64(xp + 1)).numpy().astype(np.float32)])
add("unary_acos", "Acos", {}, [xp], [torch.acos(t64(xp)).numpy().astype(np.float32)])
add("unary_asin", "Asin", {}, [xp], [torch.asin(t64(xp)).numpy().astype(np.float32)])
x4 = f32(3, 4, 5, 6)
add("elu", "Elu", dict(alpha=2.0), [x4], [F.elu(t64(x4), 2.0).numpy().astype(np.float32)])
add("leakyrelu", "LeakyRelu", dict(alpha=0.5), [x4], [F.leaky_relu(t64(x4), 0.5).numpy().astype(np.float32)])
add("selu", "Selu", {}, [x4], [F.selu(t64(x4)).numpy().astype(np.float32)])
big, bc, sc = f32(2, 3, 10, 12), f32(1, 3, 1, 12), f32()
for op, fn in [("Add", torch.add), ("Sub", torch.sub), ("Mul", torch.mul), ("Div", torch.div)]:
    add(f"{op.lower()}1", op, {}, [big, big[::-1].copy()], [fn(t64(big), t64(big[::-1].copy())).numpy().astype(np.float32)])
    add(f"{op.lower()}2", op, {}, [big, sc], [fn(t64(big), t64(sc)).numpy().astype(np.float32)])
    add(f"{op.lower()}3", op, {}, [big, bc], [fn(t64(big), t64(bc)).numpy().astype(np.float32)])
    sc2 = f32()
    add(f"{op.lower()}4", op, {}, [sc, sc2], [np.asarray(fn(t64(sc), t64(sc2)).numpy(), np.float32)])
pb, pe = f32(2, 3, 10, 12, positive=True), f32(1, 3, 1, 12, positive=True)
add("pow3", "Pow", {}, [pb, pe], [torch.pow(t64(pb), t64(pe)).numpy().astype(np.float32)])

# ops the reference does not implement (ONNX spec; cross-check only)
x = f32(2, 6, 5, 7)
g, bt, mu, var = f32(6, positive=True) + 0.5, f32(6, scale=0.1), f32(6, scale=0.1), f32(6, positive=True) + 0.5
add("batchnorm", "BatchNormalization", dict(epsilon=1e-5), [x, g, bt, mu, var],
    [F.batch_norm(t64(x), t64(mu), t64(var), t64(g), t64(bt), False, 0.0, 1e-5).numpy().astype(np.float32)])
x = f32(7, 5, 48)
g, bt = f32(48), f32(48)
add("layernorm", "LayerNormalization", dict(axis=-1, epsilon=1e-5, _opset=17), [x, g, bt],
    [F.layer_norm(t64(x), (48,), t64(g), t64(bt), 1e-5).numpy().astype(np.float32)])
T, B, I, H = 6, 3, 10, 16
X = f32(T, B, I)
lim = 1.0 / np.sqrt(H)
W = rng.uniform(-lim, lim, (1, 4 * H, I)).astype(np.float32)
R = rng.uniform(-lim, lim, (1, 4 * H, H)).astype(np.float32)
Bv = rng.uniform(-lim, lim, (1, 8 * H)).astype(np.float32)


def iofc_to_ifgo(m):
    i, o, f, c = np.split(m, 4, axis=0)
    return np.concatenate([i, f, c, o], 0)


lstm = torch.nn.LSTM(I, H).double()
with torch.no_grad():
    lstm.weight_ih_l0.copy_(t64(iofc_to_ifgo(W[0])))
    lstm.weight_hh_l0.copy_(t64(iofc_to_ifgo(R[0])))
    lstm.bias_ih_l0.copy_(t64(iofc_to_ifgo(Bv[0, :4 * H])))
    lstm.bias_hh_l0.copy_(t64(iofc_to_ifgo(Bv[0, 4 * H:])))
    y, (hn, cn) = lstm(t64(X))
add("lstm", "LSTM", dict(hidden_size=H, direction="forward"), [X, W, R, Bv],
    [y.numpy().astype(np.float32).reshape(T, 1, B, H), hn.numpy().astype(np.float32), cn.numpy().astype(np.float32)])
x = f32(4, 9, 11)
add("argmax", "ArgMax", dict(axis=1, keepdims=0), [x], [t64(x).argmax(1).numpy().astype(np.int32)])


# ---- operators of the cpu backend outside the benchmark configurations (make_models.py:583, 645-676, 731)
def convt_case(name, cin, cout, k, stride, pad, outpad, groups, dil, bias, shape):
    x = f32(*shape)
    w = f32(cin, cout // groups, k, k, scale=(2.0 / (cin * k * k)) ** 0.5)
    b = f32(cout) if bias else None
    y = F.conv_transpose2d(t64(x), t64(w), t64(b) if bias else None, stride, pad, outpad, groups, dil)
    attrs = dict(kernel_shape=[k, k], strides=[stride, stride], pads=[pad] * 4, dilations=[dil, dil], group=groups,
                 output_padding=[outpad, outpad])
    add(name, "ConvTranspose", attrs, [x, w] + ([b] if bias else []), [y.numpy().astype(np.float32)])


convt_case("convtranspose1", 16, 32, 3, 1, 0, 0, 1, 1, False, (1, 16, 7, 7))
convt_case("convtranspose2", 16, 32, 3, 2, 0, 0, 1, 1, True, (2, 16, 7, 9))
convt_case("convtranspose3", 16, 32, 3, 2, 0, 0, 2, 1, False, (2, 16, 7, 9))
convt_case("convtranspose4", 16, 32, 3, 2, 1, 1, 1, 1, False, (2, 16, 7, 9))
convt_case("convtranspose5", 16, 32, 3, 2, 1, 1, 1, 2, False, (2, 16, 7, 9))


def pad_case(name, torch_pads, shape, mode="constant", constant=0.0):
    """torch_pads is F.pad's order (last axis first); ONNX wants all begins then all ends."""
    x = f32(*shape)
    nd = len(shape)
    begins, ends = [0] * nd, [0] * nd
    for j in range(len(torch_pads) // 2):
        begins[nd - 1 - j], ends[nd - 1 - j] = torch_pads[2 * j], torch_pads[2 * j + 1]
    tmode = {"constant": "constant", "reflect": "reflect", "edge": "replicate"}[mode]
    xt = torch.tensor(x)
    if mode == "constant":
        y = F.pad(xt, torch_pads, value=constant)
    else:
        y = F.pad(xt, torch_pads, mode=tmode)
    ins = [x, np.array(begins + ends, np.int64)]
    if mode == "constant" and constant != 0.0:
        ins.append(np.array(constant, np.float32))
    add(name, "Pad", dict(mode=mode, _opset=11), ins, [y.numpy()])


pad_case("pad1", (1, 2), (2,))
pad_case("pad2", (1, 2, 3, 4), (2, 3))
pad_case("pad3", (1, 2, 3, 4, 5, 6), (2, 3, 4))
pad_case("pad4", (1, 2, 3, 4, 5, 6, 7, 8), (2, 3, 4, 5))
pad_case("pad5", (1, 2, 1, 0, 2, 1, 0, 1, 1, 1), (2, 3, 4, 5, 6))
pad_case("pad6", (1, 0, 0, 1, 1, 1, 2, 0, 0, 2, 1, 1), (2, 3, 4, 5, 6, 7))
pad_case("padc2", (1, 2, 3, 4), (2, 3), constant=-1.0)
pad_case("padc4", (1, 2, 3, 4, 5, 6, 7, 8), (2, 3, 4, 5), constant=-1.0)
pad_case("padr3", (2, 1), (2, 3, 4), mode="reflect")
pad_case("padr4", (4, 3, 2, 1), (2, 3, 4, 5), mode="reflect")
pad_case("padr5", (6, 5, 4, 3, 2, 1), (3, 4, 5, 6, 7), mode="reflect")
pad_case("pade3", (2, 1), (2, 3, 4), mode="edge")
pad_case("pade4", (4, 3, 2, 1), (2, 3, 4, 5), mode="edge")
pad_case("pade5", (6, 5, 4, 3, 2, 1), (3, 4, 5, 6, 7), mode="edge")
xt_ = f32(3, 4, 5, 6, positive=True)
add("tile", "Tile", dict(_opset=6), [xt_, np.array([2, 3, 1, 2], np.int64)], [np.tile(xt_, (2, 3, 1, 2))])
xi = f32(3, 4, 5, 6, positive=True)
gi, bi = f32(4, positive=True), f32(4, positive=True)
# epsilon left at its default: the reference reads a given epsilon as 0 (instancenormalization.ts:18)
add("instancenorm1", "InstanceNormalization", {}, [xi, gi, bi],
    [F.instance_norm(t64(xi), weight=t64(gi), bias=t64(bi), eps=1e-5).numpy().astype(np.float32)])

flat = {}
meta = {}
for name, c in cases.items():
    meta[name] = dict(op=c["op"], attrs=c["attrs"], n_in=c["n_in"], n_out=c["n_out"])
    for k, v in c.items():
        if isinstance(v, np.ndarray):
            flat[f"{name}/{k}"] = v
flat["__meta__"] = np.frombuffer(json.dumps(meta).encode("utf-8"), dtype=np.uint8)
np.savez_compressed(OUT, **flat)
print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(cases), "cases")
