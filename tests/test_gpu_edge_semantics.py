"""GPU parity on the awkward values: JavaScript number semantics of the reference's cpu backend (doubles stored
into typed arrays) that a native kernel gets wrong by default: int32 wrap-around and division by zero, casts of
NaN / infinities / out-of-range values, infinities and NaNs flowing through contractions, pools and softmax, slices
with negative steps and clamped bounds.  Every case runs through the shipped runner on the cuda backend and is
compared with the CPU oracle: integers bit for bit, floats with equal NaN / infinity patterns and 1e-4 * L_inf.
"""
import numpy as np
import pytest

from oracle import ref_runner

from util import max_err_rel_linf, run_cuda, single_op_model

pytestmark = pytest.mark.gpu
I32 = np.int32
F32 = np.float32
BIG = 2 ** 31 - 1


def _check(model, inputs, ctx):
    want = ref_runner.run_model(model, inputs)
    got = run_cuda(model, inputs, ctx)
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert list(g.shape) == list(w.shape), (g.shape, w.shape)
        if w.dtype == np.int32:
            assert g.dtype == np.int32 and np.array_equal(g, w), (g, w)
        else:
            assert max_err_rel_linf(g, w) <= 1e-4, (g, w)


def _check_contraction(model, inputs, ctx, exact_infinities):
    """Contractions with non-finite operands.  NaN in the reference <-> NaN here; finite values agree to 1e-4 * L_inf
    of the finite part.  An infinity of the reference is reproduced exactly by the CUDA-core kernel; the tensor-core
    kernel computes a * w as three products of split operands, and inf * (a low part of either sign, or zero) makes
    NaN of what the reference calls +-inf: there the result only has to be non-finite."""
    want = ref_runner.run_model(model, inputs)
    got = run_cuda(model, inputs, ctx)
    for g, w in zip(got, want):
        assert list(g.shape) == list(w.shape)
        assert np.isnan(g[np.isnan(w)]).all()
        fin = np.isfinite(w)
        assert np.isfinite(g[fin]).all(), "a finite result of the reference came out non-finite"
        if fin.any():
            assert np.abs(g[fin] - w[fin]).max() <= 1e-4 * np.abs(w[fin]).max()
        inf = np.isinf(w)
        if exact_infinities:
            assert np.array_equal(g[inf], w[inf])
        else:
            assert (~np.isfinite(g[inf])).all()


INT_BINARY = [
    ("Add", [BIG, -BIG - 1, 5, 0], [1, -1, -7, 0]),
    ("Sub", [-BIG - 1, BIG, 5, 0], [1, -1, -7, 0]),
    ("Mul", [65536, -65536, 46341, BIG, 3], [65536, 65536, 46341, BIG, -5]),
    ("Div", [7, -7, 7, -7, 5, -5, 0, -BIG - 1], [2, 2, -2, -2, 0, 0, 0, -1]),
    ("Pow", [2, -3, 2, 0, 7], [10, 3, 31, 0, -1]),
]


@pytest.mark.parametrize("op,a,b", INT_BINARY, ids=[c[0] for c in INT_BINARY])
def test_int32_binary_follows_js_numbers(cuda_context, op, a, b):
    a, b = np.asarray(a, I32), np.asarray(b, I32)
    _check(single_op_model(op, {}, [a, b]), [a, b], cuda_context)


@pytest.mark.parametrize("op", ["Abs", "Neg", "Sign", "Relu"])
def test_int32_unary_extremes(cuda_context, op):
    x = np.asarray([-BIG - 1, -BIG, -1, 0, 1, BIG], I32)
    _check(single_op_model(op, {}, [x]), [x], cuda_context)


def test_cast_float_to_int32_wraps_and_zeroes_nan(cuda_context):
    x = np.asarray([np.nan, np.inf, -np.inf, 3e9, -3e9, 4294967296.0 + 5, -0.9, 0.9, -1.5, 2147483648.0, 1e20], F32)
    _check(single_op_model("Cast", {"to": 6}, [x]), [x], cuda_context)


def test_cast_int32_to_float_rounds(cuda_context):
    x = np.asarray([BIG, -BIG - 1, 16777217, -16777217, 0], I32)
    _check(single_op_model("Cast", {"to": 1}, [x]), [x], cuda_context)


def test_gemm_beta_zero_still_multiplies_c(cuda_context):
    """gemm.ts adds C * beta unconditionally: a NaN or infinity in C survives beta = 0 as NaN."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((5, 8)).astype(F32)
    b = rng.standard_normal((8, 6)).astype(F32)
    c = rng.standard_normal((5, 6)).astype(F32)
    c[1, 2], c[3, 0] = np.nan, np.inf
    _check(single_op_model("Gemm", {"alpha": 0.5, "beta": 0.0}, [a, b, c], n_graph_inputs=1), [a], cuda_context)
    _check(single_op_model("Gemm", {"alpha": 0.5, "beta": 0.0}, [a, b, c]), [a, b, c], cuda_context)


@pytest.mark.parametrize("m,k,n", [(6, 8, 5), (64, 64, 64), (130, 96, 72)])
def test_matmul_with_infinities_and_nans(cuda_context, m, k, n):
    """inf * finite stays inf (not NaN), inf * 0 and inf - inf are NaN, NaN spreads along its row / column only."""
    rng = np.random.default_rng(m)
    a = rng.standard_normal((m, k)).astype(F32)
    b = rng.standard_normal((k, n)).astype(F32)
    a[0, 1] = np.inf
    a[1, 2] = -np.inf
    a[2, 0] = np.nan
    a[3, 3], a[3, 4] = np.inf, np.inf
    b[3, 0], b[4, 0] = 1.0, -1.0          # row 3 x column 0: inf - inf
    b[1, 1] = 0.0                         # row 0 x column 1: inf * 0
    b[5, 3] = np.inf
    small = m < 32                        # below the tensor-core kernel's sizes: CUDA-core kernel, plain fp32 products
    _check_contraction(single_op_model("MatMul", {}, [a, b], n_graph_inputs=1), [a], cuda_context, small)
    _check_contraction(single_op_model("MatMul", {}, [a, b]), [a, b], cuda_context, small)


def test_conv_with_infinities_and_nans(cuda_context):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 32, 9, 9)).astype(F32)
    w = (rng.standard_normal((32, 32, 3, 3)) * 0.1).astype(F32)
    x[0, 0, 4, 4] = np.inf
    x[0, 5, 0, 0] = -np.inf
    x[1, 3, 8, 8] = np.nan
    w[7, 0, 1, 1] = 0.0                   # inf * 0 at the centre tap of output channel 7
    w[9, 2, 0, 0] = np.inf
    attrs = dict(kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[1, 1])
    _check_contraction(single_op_model("Conv", attrs, [x, w], n_graph_inputs=1), [x], cuda_context, False)


def test_softmax_rows_with_infinities(cuda_context):
    x = np.asarray([[1, 2, 3, 4], [np.inf, 1, 2, 3], [-np.inf, -np.inf, 0, 1], [-np.inf] * 4, [np.nan, 0, 0, 0],
                    [np.inf, np.inf, 0, 0], [88.0, 89.0, -104.0, 0.0]], F32)
    _check(single_op_model("Softmax", {"axis": -1}, [x], opset=13), [x], cuda_context)


@pytest.mark.parametrize("op,attrs", [
    ("MaxPool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])),
    ("MaxPool", dict(kernel_shape=[2, 2], strides=[2, 2], ceil_mode=1)),
    ("AveragePool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1], count_include_pad=1)),
    ("AveragePool", dict(kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])),
    ("GlobalAveragePool", {}),
])
def test_pools_with_infinities_and_nans(cuda_context, op, attrs):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((1, 4, 7, 7)).astype(F32)
    x[0, 0, 0, 0] = -np.inf
    x[0, 1, 3, 3] = np.nan
    x[0, 2, 6, 6] = np.inf
    x[0, 3, :, :] = -np.inf
    _check(single_op_model(op, attrs, [x]), [x], cuda_context)


@pytest.mark.parametrize("starts,ends,axes,steps", [
    ([5], [0], [1], [-1]), ([-1], [-100], [1], [-2]), ([0], [BIG], [0], [1]), ([100], [200], [1], [1]),
    ([-3, 1], [BIG, -1], [0, 1], [2, 3]), ([6], [-8], [1], [-3]),
])
def test_slice_clamping_and_negative_steps(cuda_context, starts, ends, axes, steps):
    x = np.arange(5 * 7, dtype=F32).reshape(5, 7)
    ins = [x] + [np.asarray(v, np.int64) for v in (starts, ends, axes, steps)]
    _check(single_op_model("Slice", {}, ins, n_graph_inputs=1, opset=11), [x], cuda_context)


def test_unary_special_values(cuda_context):
    x = np.asarray([np.nan, np.inf, -np.inf, -0.0, 0.0, 0.5, -0.5, 1.5, 2.5, -1.5, -2.5, 1e-45, -1e-45, 3.4e38], F32)
    for op in ("Round", "Ceil", "Floor", "Sign", "Abs", "Neg", "Sqrt", "Exp", "Log", "Tanh", "Sigmoid", "Reciprocal",
               "Relu", "Atan", "Cosh"):
        _check(single_op_model(op, {}, [x]), [x], cuda_context)


def test_binary_special_values(cuda_context):
    a = np.asarray([np.inf, np.inf, 0.0, -0.0, 1.0, np.nan, -np.inf, 2.0, -8.0, 0.0], F32)
    b = np.asarray([np.inf, -np.inf, 0.0, 0.0, 0.0, 1.0, np.inf, 0.5, 1.0 / 3.0, -1.0], F32)
    for op in ("Add", "Sub", "Mul", "Div", "Pow"):
        _check(single_op_model(op, {}, [a, b]), [a, b], cuda_context)
