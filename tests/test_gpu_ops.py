"""GPU parity: every single-op case runs through the shipped runner on the cuda backend (which calls
the C ABI) and is compared with the CPU oracle on the same inputs, and with the golden tensors.

Tolerances: integer / indexing ops bit-exact; floating point max|a-e| <= 1e-4 * ||e||_inf.
"""
import numpy as np
import pytest

from oracle import ops, ref_runner

from util import known_answers, max_err_rel_linf, run_cuda, single_op_model, torch_cases

pytestmark = pytest.mark.gpu
TOL = 1e-4
EXACT_UNARY = {"Relu", "Abs", "Neg", "Ceil", "Floor", "Sign", "Round", "Identity"}


def _check_all_on_cuda(runner):
    assert runner.node_backends and all(b == "cuda" for _, _, b in runner.node_backends), runner.node_backends


def test_relu_known_answer(cuda_context):
    ka = known_answers()["relu_vector"]
    x = np.asarray(ka["input"], np.float32)
    (y,), r = run_cuda(single_op_model("Relu", {}, [x]), [x], cuda_context, return_runner=True)
    _check_all_on_cuda(r)
    assert y.tolist() == ka["expected"] and list(y.shape) == ka["dims"]
    r.dispose()


def test_relu_js_edge_semantics(cuda_context):
    x = np.asarray([np.nan, -0.0, 0.0, -1.0, np.inf, -np.inf, 1e-45], np.float32)
    (y,) = run_cuda(single_op_model("Relu", {}, [x]), [x], cuda_context)
    e = ops.unary("Relu", x)
    assert np.array_equal(y.view(np.uint32)[1:], e.view(np.uint32)[1:]) and np.isnan(y[0])


@pytest.mark.parametrize("name", sorted(torch_cases()))
def test_case_matches_oracle_and_golden(cuda_context, name):
    case = torch_cases()[name]
    # from the first int64 operand (pads, repeats) on, operands are constants of the graph, like an exporter writes them
    n_run = next((i for i, a in enumerate(case["inputs"]) if a.dtype == np.int64), len(case["inputs"]))
    model = single_op_model(case["op"], case["attrs"], case["inputs"], n_out=len(case["outputs"]), n_graph_inputs=n_run)
    want = ref_runner.run_model(model, case["inputs"][:n_run])
    got, r = run_cuda(model, case["inputs"][:n_run], cuda_context, return_runner=True)
    _check_all_on_cuda(r)
    r.dispose()
    for g, w, gold in zip(got, want, case["outputs"]):
        assert list(g.shape) == list(w.shape), (g.shape, w.shape)
        if w.dtype == np.int32:
            assert np.array_equal(g, w, equal_nan=True), (op, g, w)
            continue
        if case["op"] in EXACT_UNARY or case["op"] in ("MaxPool", "ReduceMax", "ReduceMin", "Pad", "Tile"):
            assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), name
        assert max_err_rel_linf(g, w) <= TOL, name
        assert max_err_rel_linf(g, gold) <= TOL, name


UNARY_DOMAINS = {"Acos": (-1, 1), "Asin": (-1, 1), "Acosh": (1, 5), "Atanh": (-0.95, 0.95), "Log": (0.01, 10),
                 "Sqrt": (0, 10), "Reciprocal": (0.1, 5), "Exp": (-10, 10), "Cosh": (-5, 5), "Tan": (-1.3, 1.3)}


@pytest.mark.parametrize("op", ["Abs", "Acos", "Acosh", "Asin", "Asinh", "Atan", "Atanh", "Ceil", "Cos", "Cosh",
                                "Exp", "Floor", "HardSwish", "Log", "Neg", "Reciprocal", "Relu", "Round",
                                "Sigmoid", "Sign", "Sin", "Softplus", "Softsign", "Sqrt", "Tan", "Tanh", "Elu",
                                "HardSigmoid", "LeakyRelu", "Selu", "ThresholdedRelu"])
def test_unary_ops(cuda_context, op):
    rng = np.random.default_rng(3)
    lo, hi = UNARY_DOMAINS.get(op, (-6, 6))
    x = rng.uniform(lo, hi, (7, 129)).astype(np.float32)  # odd length: vector body + scalar tail
    x[0, :8] = [0.0, -0.0, 0.5, -0.5, 1.5, 2.5, -2.5, 3.0][:8] if op in ("Round", "Sign", "Relu", "HardSwish", "Ceil", "Floor") else x[0, :8]
    model = single_op_model(op, {}, [x])
    (want,) = ref_runner.run_model(model, [x])
    (got,) = run_cuda(model, [x], cuda_context)
    if op in EXACT_UNARY:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert max_err_rel_linf(got, want) <= TOL


def test_clip_opset6(cuda_context):
    x = np.linspace(-3, 3, 50, dtype=np.float32)
    model = single_op_model("Clip", {"min": -1.0, "max": 1.5, "_opset": 6}, [x])
    (want,) = ref_runner.run_model(model, [x])
    (got,) = run_cuda(model, [x], cuda_context)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("op", ["Add", "Sub", "Mul", "Div", "Pow"])
def test_int32_binary_bit_exact(cuda_context, op):
    rng = np.random.default_rng(5)
    a = rng.integers(-2 ** 31, 2 ** 31, (4, 1, 33), dtype=np.int64).astype(np.int32)
    b = rng.integers(-2 ** 31, 2 ** 31, (1, 5, 33), dtype=np.int64).astype(np.int32)
    if op == "Pow":
        a = rng.integers(-9, 10, (4, 1, 33)).astype(np.int32)
        b = rng.integers(0, 9, (1, 5, 33)).astype(np.int32)
    a[0, 0, :4] = [2147483647, -2147483648, 123456789, 5]
    # Pow stays below 2^53 where the double result is exact in every libm; beyond that the low bits
    # depend on the pow() implementation (V8's is not specified), so no parity claim is possible
    b[0, 0, :4] = [1, -1, 987654321, 0] if op != "Pow" else [1, 1, 1, 0]
    model = single_op_model(op, {}, [a, b])
    (want,) = ref_runner.run_model(model, [a, b])
    (got,) = run_cuda(model, [a, b], cuda_context)
    assert got.dtype == np.int32 and np.array_equal(got, want)


@pytest.mark.parametrize("op", ["Abs", "Neg", "Relu", "Sign"])
def test_int32_unary_bit_exact(cuda_context, op):
    x = np.asarray([-2147483648, 2147483647, 0, -5, 7], np.int32)
    model = single_op_model(op, {}, [x])
    (want,) = ref_runner.run_model(model, [x])
    (got,) = run_cuda(model, [x], cuda_context)
    assert np.array_equal(got, want)


def test_broadcast_ranks_up_to_6(cuda_context):
    rng = np.random.default_rng(6)
    for sa, sb in [((2, 1, 3, 1, 4, 5), (1, 3, 1, 2, 1, 5)), ((3, 4, 5), (5,)), ((3, 4, 5), (4, 1)), ((), (2, 3)),
                   ((6, 1), (1, 7)), ((0, 3), (0, 3))]:
        a, b = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
        model = single_op_model("Sub", {}, [a, b])
        (want,) = ref_runner.run_model(model, [a, b])
        (got,) = run_cuda(model, [a, b], cuda_context)
        assert got.shape == want.shape and np.array_equal(got, want)  # IEEE sub is exact either way


def test_indexing_ops_bit_exact(cuda_context):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((3, 4, 5, 6)).astype(np.float32)
    cases = [
        ("Transpose", {"perm": [2, 0, 3, 1]}, [x], 1),
        ("Transpose", {}, [x[0]], 1),
        ("Transpose", {"perm": [0, 2, 3, 1]}, [rng.standard_normal((2, 40, 9, 9)).astype(np.float32)], 1),
        ("Concat", {"axis": 1}, [x, x[:, :2], x[:, 1:]], 1),
        ("Concat", {"axis": -1}, [x, x], 1),
        ("Split", {"axis": -1, "split": [2, 3, 1], "_opset": 11}, [x], 3),
        ("Split", {"axis": 0}, [rng.standard_normal((30, 4)).astype(np.float32)], 3),
        ("Flatten", {"axis": 1}, [x], 1),
        ("Squeeze", {"axes": [2, 4], "_opset": 11}, [rng.standard_normal((3, 4, 1, 5, 1, 6)).astype(np.float32)], 1),
        ("Unsqueeze", {"axes": [0, 3], "_opset": 11}, [x], 1),
        ("Cast", {"to": 6}, [(x * 100).astype(np.float32)], 1),
        ("Identity", {}, [x], 1),
    ]
    for op, attrs, ins, n_out in cases:
        model = single_op_model(op, attrs, ins, n_out=n_out)
        want = ref_runner.run_model(model, ins)
        got = run_cuda(model, ins, cuda_context)
        for g, w in zip(got, want):
            assert g.shape == w.shape and g.dtype == w.dtype, (op, g.shape, w.shape)
            assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), op


def test_reshape_slice_gather_with_cpu_operands(cuda_context):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((100, 200)).astype(np.float32)
    for op, attrs, ins, n_graph in [
        ("Reshape", {}, [x, np.asarray([0, 10, -1], np.int64)], 1),
        ("Slice", {}, [x, np.asarray([10, 20], np.int64), np.asarray([50, -20], np.int64)], 1),
        ("Slice", {}, [x, np.asarray([5], np.int64), np.asarray([90], np.int64), np.asarray([1], np.int64),
                       np.asarray([3], np.int64)], 1),
        ("Gather", {"axis": 1}, [x, np.asarray([3, -1, 7, 7], np.int32)], 2),
    ]:
        model = single_op_model(op, attrs, ins, n_graph_inputs=n_graph)
        want = ref_runner.run_model(model, ins[:n_graph])
        got = run_cuda(model, ins[:n_graph], cuda_context)
        assert got[0].shape == want[0].shape and np.array_equal(got[0], want[0]), op


def test_softmax_edge_rows(cuda_context):
    x = np.zeros((5, 10), np.float32)
    x[1] = 1e4
    x[2, 3] = -np.inf
    x[3] = np.linspace(-80, 80, 10)
    x[4] = -1e30
    for arr in (x, np.zeros((0, 7), np.float32), np.random.default_rng(0).standard_normal((3, 1, 1)).astype(np.float32)):
        model = single_op_model("Softmax", {"axis": -1}, [arr])
        (want,) = ref_runner.run_model(model, [arr])
        (got,) = run_cuda(model, [arr], cuda_context)
        assert got.shape == want.shape
        if arr.size:
            assert max_err_rel_linf(got, want) <= TOL


def test_gemm_larger_and_odd_shapes(cuda_context):
    rng = np.random.default_rng(9)
    for m, n, k, ta, tb in [(64, 512, 784, 0, 1), (64, 10, 512, 0, 1), (129, 67, 33, 1, 0), (1, 1, 1, 0, 0),
                            (256, 1000, 2048, 0, 1)]:
        a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
        b = (rng.standard_normal((n, k) if tb else (k, n)) * np.sqrt(2.0 / k)).astype(np.float32)
        c = rng.uniform(-0.1, 0.1, n).astype(np.float32)
        model = single_op_model("Gemm", {"transA": ta, "transB": tb}, [a, b, c])
        (want,) = ref_runner.run_model(model, [a, b, c])
        (got,) = run_cuda(model, [a, b, c], cuda_context)
        assert max_err_rel_linf(got, want) <= TOL, (m, n, k)


def test_eightbit_decode_on_device_is_bit_exact(cuda_context):
    """wdc_decode_eightbit against the host decoder (itself pinned to the reference's table and
    encoder by tests/test_tensor_loader.py) for every code value, odd lengths and several scales."""
    from webdnn_b200 import tensor_loader
    rng = np.random.default_rng(9)
    for n, scale in [(256, 1.0), (1, 0.37), (15, 1e-20), (16, 3.25), (100003, 0.0123), (1 << 20, 7.5)]:
        codes = rng.integers(0, 256, n, dtype=np.uint8) if n != 256 else np.arange(256, dtype=np.uint8)
        want = tensor_loader.scaled_table(scale)[codes]
        t = cuda_context.decode_eightbit(codes, scale, [n])
        got = t.get_data()
        t.dispose()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_pad_examples_written_in_the_reference_source(cuda_context):
    ka = known_answers()["pad_examples"]
    x = np.asarray(ka["input"], np.float32)
    for c in ka["cases"]:
        pads = np.asarray(c["pads"], np.int64)
        model = single_op_model("Pad", {"mode": c["mode"], "_opset": 11}, [x, pads], n_graph_inputs=1)
        (y,) = run_cuda(model, [x], cuda_context)
        assert y.tolist() == c["expected"], c


def test_pad_negative_pads_crop_and_int32(cuda_context):
    x = np.arange(2 * 3 * 4, dtype=np.int32).reshape(2, 3, 4)
    pads = np.asarray([0, -1, 2, 1, 0, -1], np.int64)
    model = single_op_model("Pad", {"_opset": 11}, [x, pads, np.asarray(-7, np.int32)], n_graph_inputs=1)
    model.graph.input[0].elem_type = 6
    (y,) = run_cuda(model, [x], cuda_context)
    assert np.array_equal(y, ops.pad(x, pads.tolist(), "constant", -7))


EMPTY_CASES = {
    "Relu": ({}, [np.zeros((0, 4), np.float32)], 13),
    "Transpose": ({"perm": [1, 0]}, [np.zeros((0, 4), np.float32)], 13),
    "Concat": ({"axis": 0}, [np.zeros((0, 4), np.float32), np.ones((2, 4), np.float32)], 13),
    "MatMul": ({}, [np.zeros((0, 4), np.float32), np.ones((4, 3), np.float32)], 13),
    "Gemm": ({}, [np.zeros((0, 4), np.float32), np.ones((4, 3), np.float32), np.ones((3,), np.float32)], 13),
    "ReduceSum": ({"axes": [0], "keepdims": 0}, [np.zeros((0, 4), np.float32)], 11),
    "ReduceMax": ({"axes": [0], "keepdims": 1}, [np.zeros((0, 4), np.float32)], 11),
    "ReduceMean": ({"axes": [0], "keepdims": 0}, [np.zeros((0, 4), np.float32)], 11),
    "ReduceProd": ({"axes": [1], "keepdims": 0}, [np.zeros((3, 0, 2), np.float32)], 11),
    "Softmax": ({"axis": -1}, [np.zeros((0, 4), np.float32)], 11),
    "Flatten": ({}, [np.zeros((0, 4, 2), np.float32)], 13),
    "GlobalAveragePool": ({}, [np.zeros((0, 3, 2, 2), np.float32)], 13),
    "Conv": ({"kernel_shape": [1, 1]}, [np.zeros((0, 4, 3, 3), np.float32), np.ones((2, 4, 1, 1), np.float32)], 13),
    "MaxPool": ({"kernel_shape": [2, 2]}, [np.zeros((0, 4, 4, 4), np.float32)], 13),
}


@pytest.mark.parametrize("op", sorted(EMPTY_CASES))
def test_empty_batch(cuda_context, op):
    """Tensors with a zero dimension: same shapes and, for reductions over an empty axis, the same values as the
    oracle (sum 0, product 1, mean 0/0 = NaN, max of nothing = NaN like the reference's typed-array store)."""
    attrs, ins, opset = EMPTY_CASES[op]
    n_run = 1 if op in ("MatMul", "Gemm", "Conv") else len(ins)
    model = single_op_model(op, attrs, ins, opset=opset, n_graph_inputs=n_run)
    want = ref_runner.run_model(model, ins[:n_run])
    got = run_cuda(model, ins[:n_run], cuda_context)
    for g, w in zip(got, want):
        assert list(g.shape) == list(w.shape), (op, g.shape, w.shape)
        assert np.array_equal(g, w, equal_nan=True), (op, g, w)


@pytest.mark.parametrize("addend_shape", [(1, 32, 9, 9), (3, 32, 1, 1), (3, 1, 9, 9), (3, 32, 9, 9), (32, 1, 1)])
@pytest.mark.parametrize("relu", [False, True])
def test_conv_bn_add_with_a_broadcasting_addend(cuda_context, addend_shape, relu):
    """Conv + BatchNormalization + Add [+ Relu] is rewritten to one CudaConvFused node whatever the second operand of
    the Add is; only an addend of exactly the output's shape may ride in the epilogue.  A broadcasting Add
    (binary7.ts:16-68 broadcasts multidirectionally) must give the reference's numbers and shape."""
    from webdnn_b200 import zoo
    b = zoo._Builder(5)
    h = b.bn(b.conv("input", 16, 32, 3, 1, 1, bias=True), 32)
    h = b.node("Add", [h, "addend"])[0]
    if relu:
        h = b.node("Relu", [h])[0]
    model = b.model([("input", [3, 16, 9, 9]), ("addend", list(addend_shape))], [(h, [3, 32, 9, 9])])
    rng = np.random.default_rng(8)
    x = rng.standard_normal((3, 16, 9, 9)).astype(np.float32)
    a = rng.standard_normal(addend_shape).astype(np.float32)
    (want,) = ref_runner.run_model(model, [x, a])
    (got,), r = run_cuda(model, [x, a], cuda_context, return_runner=True)
    _check_all_on_cuda(r)
    assert [t for _, t, _ in r.node_backends] == ["CudaConvFused"]
    r.dispose()
    assert got.shape == want.shape == (3, 32, 9, 9)
    assert max_err_rel_linf(got, want) <= TOL


@pytest.mark.parametrize("length", [1, 31, 33, 625, 1024, 1025, 2047, 2048, 4096, 4100, 8192, 8193, 9000])
def test_softmax_and_layernorm_row_lengths(cuda_context, length):
    """Every row kernel: one warp per row (up to 1024), one CTA with the row in registers (up to 8192), and the
    re-reading CTA kernel beyond; ragged lengths on both sides of each boundary."""
    rng = np.random.default_rng(length)
    x = (rng.standard_normal((5, length)) * 3).astype(np.float32)
    x[1] += 50.0                       # a row with a large common offset
    model = single_op_model("Softmax", {"axis": -1}, [x])
    (want,) = ref_runner.run_model(model, [x])
    (got,) = run_cuda(model, [x], cuda_context)
    assert max_err_rel_linf(got, want) <= TOL
    assert np.allclose(got.sum(axis=-1), 1.0, atol=1e-4)
    if length > 1:
        gamma = rng.uniform(0.5, 1.5, length).astype(np.float32)
        beta = (rng.standard_normal(length) * 0.1).astype(np.float32)
        want_ln = ops.layernorm_chain(x, gamma, beta, 1e-5)
        ln = single_op_model("LayerNormalization", {"axis": -1, "epsilon": 1e-5}, [x, gamma, beta], opset=17)
        (got_ln,) = run_cuda(ln, [x, gamma, beta], cuda_context)
        assert max_err_rel_linf(got_ln, want_ln) <= TOL


@pytest.mark.parametrize("shape", [(3, 5, 7, 7), (2, 130, 1, 1), (4, 9, 5, 6), (2, 3, 8, 9), (1, 2, 11, 12), (2, 2, 40, 40)])
def test_global_average_pool_on_nchw_maps_of_every_size(cuda_context, shape):
    """NCHW input (a graph input, not a convolution's channels-last output): the grouped-lanes kernel for maps of at
    most 128 pixels (4, 8 or 16 lanes per map) and the warp-per-map kernel above that."""
    x = np.random.default_rng(sum(shape)).standard_normal(shape).astype(np.float32)
    model = single_op_model("GlobalAveragePool", {}, [x])
    (want,) = ref_runner.run_model(model, [x])
    (got,) = run_cuda(model, [x], cuda_context)
    assert got.shape == want.shape == shape[:2] + (1, 1)
    assert max_err_rel_linf(got, want) <= 1e-6


@pytest.mark.parametrize("shape", [(3, 64, 96), (2, 100, 36), (1, 132, 260), (2, 33, 64), (1, 1024, 68)])
def test_batched_transpose_tiles_are_bit_exact(cuda_context, shape):
    """[b, r, c] -> [b, c, r] through the 64x64 tile kernel with 16-byte accesses (both sizes multiples of 4 and at
    least 32) and through the 32x32 kernel (33 rows): ragged tile edges on both axes."""
    x = np.random.default_rng(sum(shape)).standard_normal(shape).astype(np.float32)
    model = single_op_model("Transpose", {"perm": [0, 2, 1]}, [x])
    (want,) = ref_runner.run_model(model, [x])
    (got,) = run_cuda(model, [x], cuda_context)
    assert got.shape == want.shape and np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("cin,cout,k,stride,pad,dil,outpad,bias,size", [
    (32, 16, 3, 2, 0, 1, 0, False, (12, 12)),     # the reference benchmark's form (3x3, stride 2, no padding), small
    (64, 40, 3, 2, 1, 1, 1, True, (9, 15)),       # padding, output_padding, bias, channel tile edge (40 of 64)
    (32, 8, 4, 2, 1, 1, 0, True, (8, 16)),        # even kernel
    (48, 33, 2, 1, 0, 1, 0, False, (12, 11)),     # stride 1; 33 output channels (N = 132, a multiple of 4)
    (32, 12, 3, 3, 2, 2, 0, True, (10, 13)),      # stride 3 with dilation 2
])
def test_conv_transpose_through_matmul_and_col2im(cuda_context, cin, cout, k, stride, pad, dil, outpad, bias, size):
    """ConvTranspose shapes large enough for the tensor-core route (convtranspose.ts:139-240 as one GEMM over the
    input pixels and a col2im pass) against the oracle; two images, so the batch offset of col2im is covered."""
    rng = np.random.default_rng(cin + cout + k)
    x = rng.standard_normal((2, cin) + size).astype(np.float32)
    w = (rng.standard_normal((cin, cout, k, k)) * 0.1).astype(np.float32)
    ins = [x, w] + ([rng.uniform(-0.5, 0.5, cout).astype(np.float32)] if bias else [])
    attrs = dict(kernel_shape=[k, k], strides=[stride, stride], pads=[pad] * 4, dilations=[dil, dil],
                 output_padding=[outpad, outpad])
    model = single_op_model("ConvTranspose", attrs, ins, n_graph_inputs=1)
    (want,) = ref_runner.run_model(model, [x])
    before = cuda_context.stats()["tensor_core_launches"]
    (got,) = run_cuda(model, [x], cuda_context)
    assert cuda_context.stats()["tensor_core_launches"] == before + 1
    assert got.shape == want.shape
    assert max_err_rel_linf(got, want) <= TOL


def test_conv_add_that_broadcasts_the_conv_output_up(cuda_context):
    """The Add's other operand is larger than the convolution's output ([1,C,H,W] + [3,C,H,W]): the fused node must
    return the broadcast shape, like binary7.ts does, not the convolution's."""
    from webdnn_b200 import zoo
    b = zoo._Builder(6)
    h = b.conv("input", 16, 32, 3, 1, 1, bias=True)
    h = b.node("Relu", [b.node("Add", ["addend", h])[0]])[0]
    model = b.model([("input", [1, 16, 9, 9]), ("addend", [3, 32, 9, 9])], [(h, [3, 32, 9, 9])])
    rng = np.random.default_rng(9)
    x = rng.standard_normal((1, 16, 9, 9)).astype(np.float32)
    a = rng.standard_normal((3, 32, 9, 9)).astype(np.float32)
    (want,) = ref_runner.run_model(model, [x, a])
    (got,), r = run_cuda(model, [x, a], cuda_context, return_runner=True)
    assert [t for _, t, _ in r.node_backends] == ["CudaConvFused"]
    r.dispose()
    assert got.shape == want.shape == (3, 32, 9, 9)
    assert max_err_rel_linf(got, want) <= TOL
