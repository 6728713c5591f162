"""GPU parity sweep of the data-movement, shape and broadcasting operators: many small variants of each (negative
axes, default attributes, broadcasting forms, uneven splits, higher ranks, int32 data) through the shipped runner on
the cuda backend against the CPU oracle.  Copies and integer results bit for bit; Gemm / MatMul to 1e-4 * L_inf.
"""
import numpy as np
import pytest

from oracle import ref_runner

from util import max_err_rel_linf, run_cuda, single_op_model

pytestmark = pytest.mark.gpu
F32, I32, I64 = np.float32, np.int32, np.int64


def _rand(shape, seed=0, dtype=F32):
    rng = np.random.default_rng(seed)
    if dtype == I32:
        return rng.integers(-50, 50, shape).astype(I32)
    return rng.standard_normal(shape).astype(F32)


def _check(op, attrs, ins, n_run=None, n_out=1, opset=13, exact=True):
    def run(ctx):
        k = len(ins) if n_run is None else n_run
        model = single_op_model(op, attrs, ins, n_out=n_out, n_graph_inputs=k, opset=opset)
        want = ref_runner.run_model(model, ins[:k])
        got = run_cuda(model, ins[:k], ctx)
        assert len(got) == len(want)
        for g, w in zip(got, want):
            assert list(g.shape) == list(w.shape), (op, attrs, g.shape, w.shape)
            assert g.dtype == w.dtype, (op, g.dtype, w.dtype)
            if exact or w.dtype == I32:
                assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), (op, attrs)
            else:
                assert max_err_rel_linf(g, w) <= 1e-4, (op, attrs)
    return run


CASES = {
    # Transpose: default perm reverses; unit dims; 6-D
    "transpose_default_2d": _check("Transpose", {}, [_rand((3, 5))]),
    "transpose_default_4d": _check("Transpose", {}, [_rand((2, 3, 4, 5))]),
    "transpose_unit_dims": _check("Transpose", {"perm": [2, 0, 3, 1]}, [_rand((1, 7, 1, 3))]),
    "transpose_6d": _check("Transpose", {"perm": [5, 3, 1, 0, 2, 4]}, [_rand((2, 3, 2, 3, 2, 3))]),
    "transpose_int32": _check("Transpose", {"perm": [1, 0, 2]}, [_rand((4, 3, 5), dtype=I32)]),
    "transpose_inner_kept": _check("Transpose", {"perm": [1, 0, 2]}, [_rand((33, 65, 8))]),
    "transpose_batched_2d": _check("Transpose", {"perm": [0, 2, 1]}, [_rand((3, 40, 70))]),
    "transpose_narrow": _check("Transpose", {"perm": [0, 2, 3, 1]}, [_rand((2, 3, 9, 11))]),
    # Concat
    "concat_neg_axis": _check("Concat", {"axis": -1}, [_rand((2, 3, 4)), _rand((2, 3, 1), 1), _rand((2, 3, 6), 2)]),
    "concat_axis0_int": _check("Concat", {"axis": 0}, [_rand((1, 5), dtype=I32), _rand((3, 5), 1, I32)]),
    "concat_middle": _check("Concat", {"axis": 1}, [_rand((2, 1, 3, 2)), _rand((2, 4, 3, 2), 1)]),
    "concat_single": _check("Concat", {"axis": 1}, [_rand((2, 3))]),
    # Split
    "split_equal": _check("Split", {"axis": 1}, [_rand((2, 6, 3))], n_out=3, opset=11),
    "split_uneven_attr": _check("Split", {"axis": -1, "split": [1, 4, 2]}, [_rand((3, 7))], n_out=3, opset=11),
    "split_uneven_input": _check("Split", {"axis": 0}, [_rand((5, 4)), np.asarray([2, 3], I64)], n_run=1, n_out=2),
    # Gather
    "gather_axis0": _check("Gather", {"axis": 0}, [_rand((5, 4)), np.asarray([4, 0, 2], I64)], n_run=1),
    "gather_axis1_neg_index": _check("Gather", {"axis": 1}, [_rand((3, 6, 2)), np.asarray([-1, 0, -6], I64)], n_run=1),
    "gather_neg_axis_2d_index": _check("Gather", {"axis": -1}, [_rand((2, 7)), np.asarray([[0, 6], [3, 3]], I64)], n_run=1),
    "gather_scalar_index": _check("Gather", {"axis": 0}, [_rand((5,), dtype=I32), np.asarray(3, I64)], n_run=1),
    # Reshape / Squeeze / Unsqueeze / Flatten
    "reshape_zero_copies_dim": _check("Reshape", {}, [_rand((2, 3, 4)), np.asarray([0, -1], I64)], n_run=1),
    "reshape_minus_one_middle": _check("Reshape", {}, [_rand((2, 3, 4)), np.asarray([4, -1, 2], I64)], n_run=1),
    "squeeze_all": _check("Squeeze", {}, [_rand((1, 3, 1, 2))], opset=11),
    "squeeze_neg_axes_attr": _check("Squeeze", {"axes": [-2]}, [_rand((3, 1, 2))], opset=11),
    "squeeze_axes_input": _check("Squeeze", {}, [_rand((1, 3, 1)), np.asarray([0, -1], I64)], n_run=1),
    "unsqueeze_attr": _check("Unsqueeze", {"axes": [0, 3]}, [_rand((3, 2))], opset=11),
    "unsqueeze_input_neg": _check("Unsqueeze", {}, [_rand((3, 2)), np.asarray([-1], I64)], n_run=1),
    "flatten_4d": _check("Flatten", {}, [_rand((2, 3, 4, 5))]),
    # Gemm: every documented form of C
    "gemm_c_scalar": _check("Gemm", {}, [_rand((4, 6)), _rand((6, 5), 1), _rand((1,), 2)], exact=False),
    "gemm_c_row": _check("Gemm", {}, [_rand((4, 6)), _rand((6, 5), 1), _rand((1, 5), 2)], exact=False),
    "gemm_c_col": _check("Gemm", {}, [_rand((4, 6)), _rand((6, 5), 1), _rand((4, 1), 2)], exact=False),
    "gemm_c_full_alpha_beta": _check("Gemm", {"alpha": -1.5, "beta": 0.25},
                                     [_rand((4, 6)), _rand((6, 5), 1), _rand((4, 5), 2)], exact=False),
    "gemm_ta_tb": _check("Gemm", {"transA": 1, "transB": 1}, [_rand((6, 4)), _rand((5, 6), 1), _rand((5,), 2)],
                         exact=False),
    "gemm_no_c": _check("Gemm", {"transA": 1}, [_rand((6, 4)), _rand((6, 5), 1)], exact=False, opset=11),
    # MatMul broadcasting
    "matmul_3d_2d": _check("MatMul", {}, [_rand((2, 3, 4)), _rand((4, 5), 1)], exact=False),
    "matmul_2d_3d": _check("MatMul", {}, [_rand((3, 4)), _rand((2, 4, 5), 1)], exact=False),
    "matmul_1d_2d": _check("MatMul", {}, [_rand((4,)), _rand((4, 5), 1)], exact=False),
    "matmul_2d_1d": _check("MatMul", {}, [_rand((3, 4)), _rand((4,), 1)], exact=False),
    "matmul_1d_1d": _check("MatMul", {}, [_rand((4,)), _rand((4,), 1)], exact=False),
    "matmul_batch_broadcast": _check("MatMul", {}, [_rand((1, 3, 4)), _rand((5, 4, 2), 1)], exact=False),
    # n-ary elementwise
    "max3": _check("Max", {}, [_rand((2, 3)), _rand((3,), 1), _rand((2, 1), 2)]),
    "min3": _check("Min", {}, [_rand((2, 3)), _rand((3,), 1), _rand((2, 1), 2)]),
    "sum3": _check("Sum", {}, [_rand((2, 3)), _rand((3,), 1), _rand((2, 1), 2)], exact=False),
    "mean3": _check("Mean", {}, [_rand((2, 3)), _rand((3,), 1), _rand((2, 1), 2)], exact=False),
    "max1": _check("Max", {}, [_rand((2, 3))]),
    # Shape / Cast / Identity
    "shape": _check("Shape", {}, [_rand((2, 3, 5))]),
    "cast_f2i": _check("Cast", {"to": 6}, [_rand((3, 4)) * 10]),
    "cast_i2f": _check("Cast", {"to": 1}, [_rand((3, 4), dtype=I32)]),
    "identity": _check("Identity", {}, [_rand((2, 2))]),
    # ArgMax
    "argmax_ties_first": _check("ArgMax", {"axis": 1, "keepdims": 0},
                                [np.asarray([[1, 3, 3, 0], [2, 2, 2, 2], [0, -1, 0, -1]], F32)]),
    "argmax_ties_last": _check("ArgMax", {"axis": 1, "keepdims": 1, "select_last_index": 1},
                               [np.asarray([[1, 3, 3, 0], [2, 2, 2, 2], [0, -1, 0, -1]], F32)]),
    "argmax_axis0": _check("ArgMax", {"axis": 0}, [_rand((5, 3, 2))]),
    # pooling attribute forms
    "maxpool_same_upper": _check("MaxPool", {"kernel_shape": [3, 3], "strides": [2, 2], "auto_pad": "SAME_UPPER"},
                                 [_rand((1, 2, 8, 9))]),
    "maxpool_same_lower": _check("MaxPool", {"kernel_shape": [2, 2], "strides": [2, 2], "auto_pad": "SAME_LOWER"},
                                 [_rand((1, 2, 7, 7))]),
    "maxpool_dilated": _check("MaxPool", {"kernel_shape": [2, 2], "dilations": [2, 2]}, [_rand((1, 2, 7, 7))]),
    "avgpool_ceil": _check("AveragePool", {"kernel_shape": [3, 3], "strides": [2, 2], "ceil_mode": 1},
                           [_rand((1, 2, 8, 8))], exact=False),
    "avgpool_ceil_pad_incl": _check("AveragePool", {"kernel_shape": [3, 3], "strides": [2, 2], "ceil_mode": 1,
                                                    "pads": [1, 1, 1, 1], "count_include_pad": 1},
                                    [_rand((1, 2, 8, 8))], exact=False),
    # Conv attribute forms on the CUDA-core path
    "conv_group": _check("Conv", {"kernel_shape": [3, 3], "group": 2, "pads": [1, 1, 1, 1]},
                         [_rand((2, 4, 6, 6)), _rand((6, 2, 3, 3), 1), _rand((6,), 2)], n_run=1, exact=False),
    "conv_depthwise_dilated": _check("Conv", {"kernel_shape": [3, 3], "group": 4, "dilations": [2, 2],
                                              "pads": [2, 2, 2, 2]},
                                     [_rand((1, 4, 9, 9)), _rand((4, 1, 3, 3), 1)], n_run=1, exact=False),
    "conv_asym_pads_stride": _check("Conv", {"kernel_shape": [2, 3], "strides": [2, 1], "pads": [0, 1, 1, 2]},
                                    [_rand((1, 3, 7, 8)), _rand((5, 3, 2, 3), 1)], n_run=1, exact=False),
}

# row operators over many lengths (warp kernels up to 1024 elements, block kernels beyond) and every reduction kind
for _len in (1, 2, 31, 33, 256, 1024, 1025, 4097):
    CASES[f"softmax_len{_len}"] = _check("Softmax", {"axis": -1}, [_rand((3, _len), _len) * 3], exact=False)
    CASES[f"layernorm_len{_len}"] = _check("LayerNormalization", {"axis": -1, "epsilon": 1e-5},
                                           [_rand((5, _len), _len), _rand((_len,), 1), _rand((_len,), 2)],
                                           n_run=1, opset=17, exact=False)
for _kind in ("ReduceSum", "ReduceMean", "ReduceMax", "ReduceMin", "ReduceProd", "ReduceL1", "ReduceL2",
              "ReduceLogSum", "ReduceLogSumExp", "ReduceSumSquare"):
    _x = np.abs(_rand((3, 4, 5, 6), 7)) + 0.5 if "Log" in _kind else _rand((3, 4, 5, 6), 7)
    CASES[f"{_kind.lower()}_axes13_keep"] = _check(_kind, {"axes": [1, 3], "keepdims": 1}, [_x], opset=11, exact=False)
    CASES[f"{_kind.lower()}_axis_last_drop"] = _check(_kind, {"axes": [-1], "keepdims": 0}, [_x], opset=11, exact=False)
    CASES[f"{_kind.lower()}_all"] = _check(_kind, {"keepdims": 0}, [_x], opset=11, exact=False)
CASES["reducesum_long_rows"] = _check("ReduceSum", {"axes": [1], "keepdims": 0}, [_rand((7, 5000), 3)], opset=11,
                                      exact=False)
CASES["reducemax_long_cols"] = _check("ReduceMax", {"axes": [0], "keepdims": 0}, [_rand((3000, 9), 3)], opset=11)

# the operators added last: ConvTranspose and InstanceNormalization over attribute forms
for _i, (_cin, _cout, _k, _s, _p, _d, _g, _op) in enumerate([
        (4, 6, 3, 2, 1, 1, 1, 1), (6, 4, 2, 2, 0, 1, 2, 0), (3, 5, 3, 1, 1, 2, 1, 0), (8, 8, 4, 3, 2, 1, 4, 2),
        (2, 3, 1, 1, 0, 1, 1, 0), (5, 2, 5, 2, 2, 1, 1, 1)]):
    _attrs = {"kernel_shape": [_k, _k], "strides": [_s, _s], "pads": [_p] * 4, "dilations": [_d, _d], "group": _g}
    if _op:
        _attrs["output_padding"] = [min(_op, _s - 1)] * 2
    CASES[f"convtranspose_v{_i}"] = _check(
        "ConvTranspose", _attrs, [_rand((2, _cin, 5, 6), _i), _rand((_cin, _cout // _g, _k, _k), _i + 1) * 0.3,
                                  _rand((_cout,), _i + 2)], n_run=1, exact=False)
for _i, (_shape, _eps) in enumerate([((2, 3, 4, 5), 1e-5), ((1, 7, 1, 1), 1e-3), ((3, 2, 33, 31), 1e-5),
                                     ((2, 5, 64, 64), 0.1)]):
    CASES[f"instancenorm_v{_i}"] = _check("InstanceNormalization", {"epsilon": _eps},
                                          [_rand(_shape, _i) * 2 + 1, _rand((_shape[1],), 9), _rand((_shape[1],), 8)],
                                          n_run=1, exact=False)


@pytest.mark.parametrize("name", sorted(CASES))
def test_variant(cuda_context, name):
    CASES[name](cuda_context)
