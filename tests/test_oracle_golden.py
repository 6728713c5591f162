"""CPU: the oracle against the reference's known answers and the float64-PyTorch golden cases."""
import base64

import numpy as np
import pytest

from oracle import ops, ref_runner
from webdnn_b200 import onnx_io

from util import known_answers, max_err_rel_linf, single_op_model, torch_cases

KA = known_answers()


def test_relu_known_answer_from_reference_unit_test():
    ka = KA["relu_vector"]
    y = ops.unary("Relu", np.asarray(ka["input"], np.float32))
    assert y.tolist() == ka["expected"]
    assert list(y.shape) == ka["dims"]


def test_relu_readme_example():
    ka = KA["relu_readme"]
    y = ops.unary("Relu", np.asarray(ka["input"], np.float32).reshape(ka["dims"]))
    assert y.reshape(-1).tolist() == np.asarray(ka["expected"], np.float32).tolist()


def test_relu_js_edge_semantics():
    x = np.asarray([np.nan, -0.0, 0.0, -1.0, np.inf, -np.inf], np.float32)
    y = ops.unary("Relu", x)
    assert np.isnan(y[0])
    assert y[1] == 0 and not np.signbit(y[1])  # Math.max(-0, 0) is +0
    assert y[3] == 0 and y[4] == np.inf and y[5] == 0


def test_minimum_model_fixture_runs_relu():
    ka = KA["minimum_model"]
    model = onnx_io.decode_model(base64.b64decode(ka["base64"]))
    x = np.asarray([[1, -2, 3], [-4, 5, -6]], np.float32)
    (y,) = ref_runner.run_model(model, [x])
    assert y.tolist() == [[1, 0, 3], [0, 5, 0]]


def test_int32_typed_array_semantics():
    a = np.asarray([2147483647, -2147483648, 7, -7, 123456789], np.int32)
    b = np.asarray([1, -1, 2, 2, 987654321], np.int32)
    assert ops.binary("Add", a, b).tolist() == [-2147483648, 2147483647, 9, -5, 1111111110]
    assert ops.binary("Div", a, b).tolist() == [2147483647, -2147483648, 3, -3, 0]
    # product computed in double then ToInt32: 123456789*987654321 = 121932631112635269
    exact = 123456789 * 987654321
    as_double = int(float(exact))
    expect = ((as_double + 2 ** 31) % 2 ** 32) - 2 ** 31
    assert ops.binary("Mul", a, b)[4] == expect
    assert ops.binary("Div", np.asarray([5], np.int32), np.asarray([0], np.int32)).tolist() == [0]
    assert ops.unary("Abs", np.asarray([-2147483648], np.int32)).tolist() == [-2147483648]
    assert ops.cast(np.asarray([3.9, -3.9, np.nan, 4294967808.0, -1e30], np.float32), 6).tolist()[:4] == [3, -3, 0, 512]


@pytest.mark.parametrize("name", sorted(torch_cases()))
def test_oracle_matches_float64_pytorch(name):
    case = torch_cases()[name]
    n_in = next((i for i, a in enumerate(case["inputs"]) if a.dtype == np.int64), len(case["inputs"]))   # from the first int64 operand on: graph constants
    model = single_op_model(case["op"], case["attrs"], case["inputs"], n_out=len(case["outputs"]), n_graph_inputs=n_in)
    outs = ref_runner.run_model(model, case["inputs"][:n_in])
    for got, want in zip(outs, case["outputs"]):
        assert list(got.shape) == list(want.shape)
        if want.dtype == np.int32:
            assert np.array_equal(got, want)
        else:
            # double accumulation rounded once to float: at most an ulp or two from float64 torch
            assert max_err_rel_linf(got, want) <= 2e-6, name


def test_reduce_quirks_of_the_reference_are_kept():
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4) / 7
    # ReduceL2 over two axes squares on every pass (reduce.ts:250-282): sqrt(sum_j (sum_i x^2)^2)
    got = ops.reduce("ReduceL2", x, [0, 2], keepdims=False)
    first = (x.astype(np.float64) ** 2).sum(0).astype(np.float32).astype(np.float64)
    want = np.sqrt((first ** 2).sum(1)).astype(np.float32)
    assert np.allclose(got, want, rtol=1e-6)


def test_softmax_rounding_points():
    x = np.asarray([[0.1, 2.5, -3.0, 7.25]], np.float32)
    e = np.exp(x.astype(np.float64) - 7.25)
    want = (e.astype(np.float32).astype(np.float64) / e.sum()).astype(np.float32)
    assert np.array_equal(ops.softmax(x), want)


def test_pad_examples_written_in_the_reference_source():
    """The edge / reflect examples in the comment block of the reference's Pad implementation."""
    ka = known_answers()["pad_examples"]
    x = np.asarray(ka["input"], np.float32)
    for c in ka["cases"]:
        assert ops.pad(x, c["pads"], c["mode"]).tolist() == c["expected"], c


def test_instance_norm_epsilon_is_read_like_the_reference():
    """instancenormalization.ts:18 reads epsilon with getAttrInt: absent -> 1e-5; given as a float
    attribute -> its integer field, 0.  The oracle keeps that."""
    rng = np.random.default_rng(0)
    x, s, b = rng.random((2, 3, 4, 5)).astype(np.float32), rng.random(3).astype(np.float32), rng.random(3).astype(np.float32)
    (default,) = ref_runner.run_model(single_op_model("InstanceNormalization", {}, [x, s, b]), [x, s, b])
    (given,) = ref_runner.run_model(single_op_model("InstanceNormalization", {"epsilon": 0.5}, [x, s, b]), [x, s, b])
    assert np.array_equal(default, ops.instance_norm(x, s, b, 1e-5))
    assert np.array_equal(given, ops.instance_norm(x, s, b, 0.0))
