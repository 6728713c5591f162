"""TEST INFRASTRUCTURE ONLY: Python face of the CPU oracle.

ctypes wrappers over ``cpu_ops.c`` (arithmetic restated from ``operators/cpu/**`` of the reference)
plus numpy restatements of the indexing ops, and an ONNX graph walker that executes a model with
these ops the way ``RunnerImpl.run()`` does with ``backendOrder = ["cpu"]``.  Shape math is written
here independently of the shipped backend (from ``operators/base/*.ts``) so that a mistake in one
copy shows up as a parity failure instead of cancelling out.

Tensors are numpy arrays: float32 / int32, C-contiguous.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import POINTER, c_double, c_int, c_int64, c_void_p
from typing import Dict, List, Sequence

import numpy as np

from .build import build

_lib = None

UNARY = {"Abs": 0, "Acos": 1, "Acosh": 2, "Asin": 3, "Asinh": 4, "Atan": 5, "Atanh": 6, "Ceil": 7, "Cos": 8,
         "Cosh": 9, "Exp": 10, "Floor": 11, "HardSwish": 12, "Log": 13, "Neg": 14, "Reciprocal": 15,
         "Relu": 16, "Round": 17, "Sigmoid": 18, "Sign": 19, "Sin": 20, "Softplus": 21, "Softsign": 22,
         "Sqrt": 23, "Tan": 24, "Tanh": 25, "Elu": 32, "HardSigmoid": 33, "LeakyRelu": 34, "Selu": 35,
         "ThresholdedRelu": 36, "Clip": 40, "Identity": 41}
BINARY = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3, "Pow": 4, "Max": 5, "Min": 6}
REDUCE = {"ReduceSum": 0, "ReduceMean": 1, "ReduceMax": 2, "ReduceMin": 3, "ReduceProd": 4, "ReduceL1": 5,
          "ReduceL2": 6, "ReduceLogSum": 7, "ReduceLogSumExp": 8, "ReduceSumSquare": 9}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_num_threads.restype = c_int
    return _lib


def set_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


def num_threads() -> int:
    return lib().orc_num_threads()


def _p(a: np.ndarray):
    return a.ctypes.data_as(c_void_p) if a is not None else None


def _i64(v: Sequence[int]):
    return (c_int64 * max(len(v), 1))(*[int(x) for x in v])


def _c(a, dtype=None) -> np.ndarray:
    """C-contiguous array that keeps 0-d arrays 0-d (np.ascontiguousarray promotes them to 1-d)."""
    a = np.asarray(a, dtype=dtype)
    return a if a.flags.c_contiguous else a.copy(order="C")


def _f32(a) -> np.ndarray:
    return _c(a, dtype=np.float32)


def strides_of(dims: Sequence[int]) -> List[int]:
    s, n = [], 1
    for d in reversed(dims):
        s.insert(0, n)
        n *= d
    return s


# --------------------------------------------------------------------------- arithmetic
def unary(op: str, x: np.ndarray, p0: float = 0.0, p1: float = 0.0) -> np.ndarray:
    x = _c(x)
    y = np.empty_like(x)
    dt = 0 if x.dtype == np.float32 else 1
    st = lib().orc_unary(UNARY[op], dt, _p(x), _p(y), c_int64(x.size), c_double(p0), c_double(p1))
    if st:
        raise ValueError(f"Unary: DataType {x.dtype} not supported for {op}")
    return y


def broadcast_multi(all_dims):
    nd = max(len(d) for d in all_dims)
    ex = [[1] * (nd - len(d)) + list(d) for d in all_dims]
    dims = [max(e[i] for e in ex) for i in range(nd)]
    strides = []
    for e in ex:
        s = strides_of(e)
        for i in range(nd):
            if e[i] != dims[i]:
                if e[i] != 1:
                    raise ValueError("Multidirectional broadcasting error")
                s[i] = 0
        strides.append(s)
    return dims, strides


def binary(op: str, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _c(a), _c(b)
    if a.dtype != b.dtype:
        raise TypeError("Binary: input dataTypes mismatch")
    dims, (sa, sb) = broadcast_multi([a.shape, b.shape])
    if len(dims) > 6:
        raise ValueError("Binary: rank > 6")
    out = np.empty(dims, dtype=a.dtype)
    dt = 0 if a.dtype == np.float32 else 1
    lib().orc_binary(BINARY[op], dt, _p(a), _p(b), _p(out), len(dims), _i64(dims), _i64(sa), _i64(sb))
    return out


def gemm(a, b, c=None, alpha=1.0, beta=1.0, trans_a=0, trans_b=0) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    if a.ndim != 2 or b.ndim != 2:
        raise ValueError("Gemm: 2-D inputs only")
    if trans_a:
        k, m = a.shape
        sa = (1, m)
    else:
        m, k = a.shape
        sa = (k, 1)
    if trans_b:
        n, k2 = b.shape
        sb = (1, k2)
    else:
        k2, n = b.shape
        sb = (n, 1)
    if k != k2:
        raise ValueError("Gemm: inner dims differ")
    y = np.empty((m, n), np.float32)
    sc = (0, 0)
    if c is not None:
        c = _f32(c)
        ec = [1] * (2 - c.ndim) + list(c.shape)
        sc = strides_of(ec)
        for i, (want, have) in enumerate(zip((m, n), ec)):
            if want != have:
                if have != 1:
                    raise ValueError("Unidirectional broadcast error")
                sc[i] = 0
    lib().orc_gemm(_p(a), _p(b), _p(c), _p(y), *map(c_int64, (m, n, k, sa[0], sa[1], sb[0], sb[1])),
                   c_int(c is not None), c_int64(sc[0]), c_int64(sc[1]), c_double(alpha), c_double(beta))
    return y


def matmul(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    da, db = list(a.shape), list(b.shape)
    total = max(len(da), len(db), 2)
    ea = ([1] + da) if len(da) == 1 else da
    ea = [1] * (total - len(ea)) + ea
    eb = (db + [1]) if len(db) == 1 else db
    eb = [1] * (total - len(eb)) + eb
    if ea[-1] != eb[-2]:
        raise ValueError("MatMul: inner dims differ")
    rd = [max(x, y) for x, y in zip(ea[:-2], eb[:-2])] + [ea[-2], eb[-1]]
    if len(rd) > 3:
        raise ValueError("MatMul: result rank > 3 unsupported by the cpu backend")
    sa, sb = strides_of(ea), strides_of(eb)
    for i in range(len(ea) - 2):
        if ea[i] == 1:
            sa[i] = 0
        if eb[i] == 1:
            sb[i] = 0
    batch = rd[0] if len(rd) == 3 else 1
    y = np.empty(rd, np.float32)
    lib().orc_matmul(_p(a), _p(b), _p(y), *map(c_int64, (
        batch, rd[-2], rd[-1], ea[-1], sa[0] if len(rd) == 3 else 0, sa[-2], sa[-1],
        sb[0] if len(rd) == 3 else 0, sb[-2], sb[-1])))
    sq = list(rd)
    if len(da) == 1:
        del sq[-2]
    if len(db) == 1:
        del sq[-1]
    return y.reshape(sq)


def conv_out_shape(in_hw, k, pads, strides, dil):
    return [math.floor((in_hw[i] + pads[i] + pads[i + 2] - dil[i] * (k[i] - 1) - 1) / strides[i]) + 1
            for i in range(2)]


def conv2d(x, w, bias=None, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    if x.ndim != 4:
        raise ValueError("Conv other than 2D is not yet supported")
    n, cin, ih, iw = x.shape
    cout, _, kh, kw = w.shape
    oh, ow = conv_out_shape((ih, iw), (kh, kw), pads, strides, dilations)
    y = np.empty((n, cout, oh, ow), np.float32)
    b = _f32(bias) if bias is not None else None
    lib().orc_conv2d(_p(x), _p(w), _p(b), _p(y), *map(c_int64, (
        n, cin, ih, iw, cout, kh, kw, oh, ow, strides[0], strides[1], pads[0], pads[1], dilations[0],
        dilations[1], group)))
    return y


def pool_out_shape(in_hw, k, pads, strides, dil, ceil_mode, auto_pad):
    eff = [dil[i] * (k[i] - 1) + 1 for i in range(2)]
    if auto_pad == "NOTSET":
        rnd = math.ceil if ceil_mode else math.floor
        return [rnd((in_hw[i] + pads[i] + pads[i + 2] - eff[i]) / strides[i]) + 1 for i in range(2)], list(pads)
    if auto_pad in ("SAME_UPPER", "SAME_LOWER"):
        out = [math.ceil(in_hw[i] / strides[i]) for i in range(2)]
        sp = [(out[i] - 1) * strides[i] + eff[i] - in_hw[i] for i in range(2)]
        lo, hi = [math.floor(s / 2) for s in sp], [math.ceil(s / 2) for s in sp]
        return out, (lo + hi if auto_pad == "SAME_UPPER" else hi + lo)
    if auto_pad == "VALID":
        return [math.ceil((in_hw[i] - eff[i] + 1) / strides[i]) for i in range(2)], [0, 0, 0, 0]
    raise ValueError(f"Unknown auto_pad {auto_pad}")


def maxpool2d(x, kernel, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), ceil_mode=False,
              auto_pad="NOTSET") -> np.ndarray:
    x = _f32(x)
    n, c, ih, iw = x.shape
    (oh, ow), pads = pool_out_shape((ih, iw), kernel, pads, strides, dilations, ceil_mode, auto_pad)
    y = np.empty((n, c, oh, ow), np.float32)
    lib().orc_maxpool(_p(x), _p(y), *map(c_int64, (n, c, ih, iw, kernel[0], kernel[1], oh, ow, strides[0],
                                                   strides[1], pads[0], pads[1], dilations[0], dilations[1])))
    return y


def avgpool2d(x, kernel, strides=(1, 1), pads=(0, 0, 0, 0), ceil_mode=False, count_include_pad=False,
              auto_pad="NOTSET") -> np.ndarray:
    x = _f32(x)
    n, c, ih, iw = x.shape
    (oh, ow), pads = pool_out_shape((ih, iw), kernel, pads, strides, (1, 1), ceil_mode, auto_pad)
    y = np.empty((n, c, oh, ow), np.float32)
    lib().orc_avgpool(_p(x), _p(y), c_int(bool(count_include_pad)), *map(c_int64, (
        n, c, ih, iw, kernel[0], kernel[1], oh, ow, strides[0], strides[1], pads[0], pads[1])))
    return y


def global_avgpool(x) -> np.ndarray:
    x = _f32(x)
    n, c, ih, iw = x.shape
    y = np.empty((n, c, 1, 1), np.float32)
    lib().orc_avgpool(_p(x), _p(y), c_int(1), *map(c_int64, (n, c, ih, iw, ih, iw, 1, 1, 1, 1, 0, 0)))
    return y


def softmax(x, axis=-1) -> np.ndarray:
    x = _f32(x)
    if axis < 0:
        axis += x.ndim
    if axis != x.ndim - 1:
        raise ValueError("Softmax: currently only reducing final axis is supported")
    y = np.empty_like(x)
    ln = x.shape[-1]
    lib().orc_softmax(_p(x), _p(y), c_int64(x.size // ln if ln else 0), c_int64(ln))
    return y


def reduce(op: str, x, axes=None, keepdims=True) -> np.ndarray:
    x = _f32(x)
    axes = sorted(a if a >= 0 else a + x.ndim for a in (axes if axes else range(x.ndim)))
    cur, shape, total = x, list(x.shape), 1
    for i, ax in enumerate(axes):
        red = shape[ax]
        total *= red
        outer, inner = int(np.prod(shape[:ax], dtype=np.int64)), int(np.prod(shape[ax + 1:], dtype=np.int64))
        new_shape = list(shape)
        new_shape[ax] = 1
        nxt = np.empty(new_shape, np.float32)
        lib().orc_reduce_axis(REDUCE[op], c_int(i == len(axes) - 1), _p(cur), _p(nxt), *map(c_int64, (
            outer, red, inner, total)))
        cur, shape = nxt, new_shape
    if not keepdims:
        cur = cur.reshape([s for i, s in enumerate(shape) if i not in axes])
    return cur


def batchnorm(x, scale, bias, mean, var, eps=1e-5) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    n, c = x.shape[0], x.shape[1]
    area = x.size // (n * c) if n * c else 0
    lib().orc_batchnorm(_p(x), _p(_f32(scale)), _p(_f32(bias)), _p(_f32(mean)), _p(_f32(var)), _p(y),
                        c_int64(n), c_int64(c), c_int64(area), c_double(float(np.float32(eps))))
    return y


def lstm(x, w, r, b=None, h0=None, c0=None):
    x, w, r = _f32(x), _f32(w), _f32(r)
    T, Bt, I = x.shape
    H = r.shape[-1]
    y = np.empty((T, 1, Bt, H), np.float32)
    yh = np.empty((1, Bt, H), np.float32)
    yc = np.empty((1, Bt, H), np.float32)
    bb = _f32(b) if b is not None else None
    hh = _f32(h0) if h0 is not None else None
    cc = _f32(c0) if c0 is not None else None
    lib().orc_lstm(_p(x), _p(w), _p(r), _p(bb), _p(hh), _p(cc), _p(y), _p(yh), _p(yc),
                   *map(c_int64, (T, Bt, I, H)))
    return y, yh, yc


def layernorm_chain(x, gamma=None, beta=None, eps=1e-5) -> np.ndarray:
    """The decomposed LayerNorm the reference would execute, node by node."""
    mean = reduce("ReduceMean", x, [-1])
    d = binary("Sub", x, mean)
    var = reduce("ReduceMean", binary("Mul", d, d), [-1])
    den = unary("Sqrt", binary("Add", var, np.asarray(eps, np.float32)))
    y = binary("Div", d, den)
    if gamma is not None:
        y = binary("Mul", y, _f32(gamma))
    if beta is not None:
        y = binary("Add", y, _f32(beta))
    return y


def argmax(x, axis=0, keepdims=True, select_last=False) -> np.ndarray:
    x = _f32(x)
    if axis < 0:
        axis += x.ndim
    xm = _c(np.moveaxis(x, axis, -1))
    ln = xm.shape[-1]
    out = np.empty(xm.shape[:-1], np.int32)
    lib().orc_argmax(_p(xm), _p(out), c_int64(xm.size // ln), c_int64(ln), c_int(bool(select_last)))
    return np.expand_dims(out, axis) if keepdims else out


# ------------------------------------------------------------------------------ indexing
def strided_copy(src: np.ndarray, dims, sstr, soff=0) -> np.ndarray:
    src = _c(src)
    out = np.empty(dims, dtype=src.dtype)
    lib().orc_strided_copy(_p(src), _p(out), len(dims), _i64(dims), _i64(sstr), c_int64(soff))
    return out


def transpose(x, perm=None) -> np.ndarray:
    x = _c(x)
    perm = list(perm) if perm else list(range(x.ndim))[::-1]
    st = strides_of(x.shape)
    return strided_copy(x, [x.shape[p] for p in perm], [st[p] for p in perm])


def cast(x, to: int) -> np.ndarray:
    x = _c(x)
    if to == 1:
        return x.astype(np.float32)
    if to in (2, 6, 7):
        if x.dtype == np.int32:
            return x.copy()
        out = np.empty(x.shape, np.int32)
        lib().orc_cast_f32_i32(_p(_f32(x)), _p(out), c_int64(x.size))
        return out
    raise ValueError(f"Cast: converting to DataType {to} is not yet supported")


def slice_(x, starts, ends, axes=None, steps=None) -> np.ndarray:
    x = _c(x)
    axes = [a + x.ndim if a < 0 else a for a in (axes if axes is not None else range(x.ndim))]
    steps = list(steps) if steps is not None else [1] * len(axes)
    ranges = [[0, d, 1, d] for d in x.shape]
    for i, ax in enumerate(axes):
        ranges[ax] = [int(starts[i]), int(ends[i]), int(steps[i]), x.shape[ax]]
    st = strides_of(x.shape)
    dims, sstr, soff = [], [], 0
    for ax, (start, stop, step, size) in enumerate(ranges):
        if start < 0:
            start += size
        start = max(min(start, size - 1), 0)
        if stop < 0:
            stop += size
        stop = max(min(stop, size), -1)
        dims.append(max(math.ceil((stop - start) / step), 0))
        sstr.append(st[ax] * step)
        soff += start * st[ax]
    if any(d == 0 for d in dims):
        return np.empty(dims, x.dtype)
    return strided_copy(x, dims, sstr, soff)


def conv_transpose2d(x, w, bias=None, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1,
                     output_padding=(0, 0)) -> np.ndarray:
    """convtranspose.ts:30-263 with its rounding points: the channel contraction of every (input
    pixel, output channel, tap) in double, stored as float32 (matmul :218-240); the taps that land on
    an output pixel summed in double in (k0, k1) order, stored as float32 (col2im :139-196); bias
    added in float32 (:242-262).  Shape rule: base/convtranspose.ts:53-72."""
    x, w = _f32(x), _f32(w)
    batch, ch_in, in_h, in_w = x.shape
    cig, cog, kh, kw = ch_in // group, w.shape[1], w.shape[2], w.shape[3]
    out_h = strides[0] * (in_h - 1) + output_padding[0] + (kh - 1) * dilations[0] + 1 - pads[0] - pads[2]
    out_w = strides[1] * (in_w - 1) + output_padding[1] + (kw - 1) * dilations[1] + 1 - pads[1] - pads[3]
    y = np.zeros((batch, group * cog, out_h, out_w), np.float64)
    for g in range(group):
        xg = x[:, g * cig:(g + 1) * cig].astype(np.float64)
        wg = w[g * cig:(g + 1) * cig].astype(np.float64)
        # NB: einsum's double sum over ci may associate differently from the JS loop; the result is
        # rounded to float32 right after, so a difference needs a near-tie in the double sum
        part = np.einsum("bchw,cokl->bohwkl", xg, wg).astype(np.float32).astype(np.float64)
        for k0 in range(kh):
            for k1 in range(kw):
                for i0 in range(in_h):
                    o0 = i0 * strides[0] - pads[0] + k0 * dilations[0]
                    if o0 < 0 or o0 >= out_h:
                        continue
                    for i1 in range(in_w):
                        o1 = i1 * strides[1] - pads[1] + k1 * dilations[1]
                        if o1 < 0 or o1 >= out_w:
                            continue
                        y[:, g * cog:(g + 1) * cog, o0, o1] += part[:, :, i0, i1, k0, k1]
    out = y.astype(np.float32)
    if bias is not None:
        out = (out + _f32(bias)[None, :, None, None]).astype(np.float32)
    return out


def instance_norm(x, scale, bias, eps) -> np.ndarray:
    """instancenormalization.ts:24-53: left-to-right double sums per (batch, channel) row."""
    x = _f32(x)
    n, c = x.shape[:2]
    rows = x.reshape(n, c, -1).astype(np.float64)
    length = rows.shape[2]
    total = np.cumsum(rows, axis=2)[:, :, -1]
    sq = np.cumsum(rows * rows, axis=2)[:, :, -1]
    mean = total / length
    variance = sq / length - mean * mean
    invstd = 1.0 / np.sqrt(variance + eps)
    chscale = _f32(scale).astype(np.float64)[None, :] * invstd
    chbias = -mean * chscale + _f32(bias).astype(np.float64)[None, :]
    return (rows * chscale[:, :, None] + chbias[:, :, None]).astype(np.float32).reshape(x.shape)


def pad(x, pads, mode="constant", value=0) -> np.ndarray:
    """pad11.ts: every mode maps an output index d to an input index per axis: constant i = d - pad
    (outside -> value, :139-149), edge clamps (:900-907), reflect folds with period 2n-2 (:408-420)."""
    x = np.asarray(x)
    nd = x.ndim
    if nd > 6:
        raise ValueError(f"Pad: input.ndim = {nd} > 6 is not yet supported")
    pads = [int(p) for p in pads]
    out_shape = [x.shape[i] + pads[i] + pads[i + nd] for i in range(nd)]
    maps, valid = [], []
    for i in range(nd):
        n = x.shape[i]
        src = np.arange(out_shape[i], dtype=np.int64) - pads[i]
        ok = (src >= 0) & (src < n)
        if mode == "edge":
            src = np.clip(src, 0, n - 1)
        elif mode == "reflect":
            period = n * 2 - 2
            with np.errstate(divide="ignore", invalid="ignore"):
                folded = np.where(src < 0, np.fmod(-src, period) if period else 0, np.fmod(src, period) if period else 0)
            folded = np.where(folded >= n, n * 2 - folded - 2, folded)
            src = np.where(ok, src, folded)
        elif mode != "constant":
            raise ValueError(f"Pad: unknown mode {mode}")
        maps.append(src)
        valid.append(ok)
    if mode == "constant":
        out = np.full(out_shape, value, dtype=x.dtype)
        if all(v.any() for v in valid) or nd == 0:
            dst = tuple(np.nonzero(v)[0] for v in valid)
            out[np.ix_(*dst)] = x[np.ix_(*[m[v] for m, v in zip(maps, valid)])] if nd else x
        return out
    return x[np.ix_(*maps)] if nd else x.copy()


def tile(x, repeats) -> np.ndarray:
    """tile.ts:19-70: out[d] = in[d mod dims] (at most 4-D in the reference)."""
    x = np.asarray(x)
    if x.ndim > 4:
        raise ValueError(f"Tile: input.ndim = {x.ndim} > 4 is not yet supported")
    idx = [np.arange(x.shape[i] * int(repeats[i])) % max(x.shape[i], 1) for i in range(x.ndim)]
    return x[np.ix_(*idx)] if x.ndim else x.copy()
