"""GPU parity of the tcgen05 (3xTF32) implicit-GEMM kernel against the CPU oracle, through the
runner and the C ABI.  Each case also checks that the tensor-core kernel really launched."""
import numpy as np
import pytest

from oracle import ops, ref_runner

from util import max_err_rel_linf, run_cuda, single_op_model

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _conv_case(ctx, n, cin, cout, size, k, stride, pad, dil=1, bias=True, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, cin, size[0], size[1])).astype(np.float32)
    w = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    ins = [x, w] + ([rng.uniform(-0.1, 0.1, cout).astype(np.float32)] if bias else [])
    attrs = dict(kernel_shape=[k, k], strides=[stride, stride], pads=[pad] * 4, dilations=[dil, dil])
    model = single_op_model("Conv", attrs, ins, n_graph_inputs=1)
    (want,) = ref_runner.run_model(model, [x])
    before = ctx.stats()["tensor_core_launches"]
    (got,) = run_cuda(model, [x], ctx)
    assert ctx.stats()["tensor_core_launches"] > before, "tensor-core kernel did not launch"
    assert got.shape == want.shape
    return max_err_rel_linf(got, want)


@pytest.mark.parametrize("n,cin,cout,size,k,stride,pad,dil", [
    (2, 64, 64, (56, 56), 3, 1, 1, 1),      # layer1 3x3
    (3, 64, 256, (17, 19), 1, 1, 0, 1),     # 1x1, M = 969 (tail rows), N = 2 tiles
    (2, 128, 128, (28, 28), 3, 2, 1, 1),    # stride-2 3x3
    (2, 256, 512, (14, 14), 1, 2, 0, 1),    # stride-2 1x1 downsample
    (1, 512, 512, (7, 7), 3, 1, 1, 1),      # K = 4608, single partly filled M tile
    (1, 32, 32, (9, 11), 3, 1, 2, 2),       # dilation 2, tile_n 32
    (2, 96, 72, (12, 12), 3, 1, 1, 1),      # Cout not a multiple of 32 (masked columns)
    (1, 64, 64, (160, 128), 1, 1, 0, 1),    # 160 M tiles: more tiles than SMs, several per CTA
])
def test_conv_shapes(cuda_context, n, cin, cout, size, k, stride, pad, dil):
    assert _conv_case(cuda_context, n, cin, cout, size, k, stride, pad, dil) <= TOL


def test_fused_epilogue_through_c_abi(cuda_context):
    """scale/shift/residual/Relu epilogue against conv -> affine -> add -> relu on the oracle."""
    from ctypes import byref
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.lib import ConvDesc
    ctx = cuda_context
    rng = np.random.default_rng(1)
    n, c, h, w_, co = 2, 64, 20, 20, 128
    x = rng.standard_normal((n, c, h, w_)).astype(np.float32)
    wt = (rng.standard_normal((co, c, 3, 3)) * 0.06).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, co).astype(np.float32)
    shift = rng.standard_normal(co).astype(np.float32)
    res = rng.standard_normal((n, co, h, w_)).astype(np.float32)
    conv = ops.conv2d(x, wt, None, (1, 1), (1, 1, 1, 1))
    want = conv.astype(np.float64) * scale[None, :, None, None] + shift[None, :, None, None] + res
    want = np.maximum(want, 0).astype(np.float32)
    dx = ctx.channels_last(ctx.move_tensor(CPUTensor.from_array(x)))
    dres = ctx.channels_last(ctx.move_tensor(CPUTensor.from_array(res)))
    dw = ctx.move_tensor(CPUTensor.from_array(wt))
    dwp = ctx.empty_tensor([co, 3, 3, c])
    ctx._call("wdc_pack_conv_weight", dw.ptr, dwp.ptr, co, c, 3, 3)
    dsc, dsh = ctx.move_tensor(CPUTensor.from_array(scale)), ctx.move_tensor(CPUTensor.from_array(shift))
    y = ctx.empty_tensor([n, co, h, w_], layout="nhwc")
    d = ConvDesc(batch=n, ch_in=c, in_h=h, in_w=w_, ch_out=co, k_h=3, k_w=3, out_h=h, out_w=w_, stride_h=1,
                 stride_w=1, pad_t=1, pad_l=1, dil_h=1, dil_w=1, group=1, relu=1)
    before = ctx.stats()["tensor_core_launches"]
    ctx.conv2d(d, dx, dwp, dsc, dsh, dres, y)
    got = y.get_data().reshape(n, co, h, w_)
    assert ctx.stats()["tensor_core_launches"] == before + 1
    assert max_err_rel_linf(got, want) <= TOL
    for t in (dx, dres, dw, dwp, dsc, dsh, y):
        t.dispose()


@pytest.mark.parametrize("m,n,k", [(64, 512, 784), (64, 10, 512), (256, 1000, 2048), (8192, 2048, 256), (33, 40, 36)])
def test_gemm_transb_on_tensor_cores(cuda_context, m, n, k):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((n, k)) * np.sqrt(2.0 / k)).astype(np.float32)
    c = rng.uniform(-0.1, 0.1, n).astype(np.float32)
    model = single_op_model("Gemm", {"transB": 1, "alpha": 0.75, "beta": 1.5}, [a, b, c])
    (want,) = ref_runner.run_model(model, [a, b, c])
    before = cuda_context.stats()["tensor_core_launches"]
    (got,) = run_cuda(model, [a, b, c], cuda_context)
    assert cuda_context.stats()["tensor_core_launches"] > before
    assert max_err_rel_linf(got, want) <= TOL


def test_split_precision_is_fp32_class(cuda_context):
    """Values chosen so that a single-pass TF32 product (10-bit mantissa) would be off by ~5e-4.
    All terms are positive and the sum is 512x a term: the worst case for the tensor core's fp32
    accumulator, which truncates when it aligns addends (a small negative bias per accumulation,
    ~3e-6 relative here).  The 3xTF32 result must still be two orders below single-pass TF32."""
    rng = np.random.default_rng(3)
    m, n, k = 128, 64, 512
    a = (1.0 + rng.uniform(0, 1, (m, k)) * 2.0 ** -9).astype(np.float32)   # low-order mantissa bits matter
    b = (1.0 + rng.uniform(0, 1, (n, k)) * 2.0 ** -9).astype(np.float32)
    model = single_op_model("Gemm", {"transB": 1}, [a, b])
    (want,) = ref_runner.run_model(model, [a, b])
    (got,) = run_cuda(model, [a, b], cuda_context)
    assert max_err_rel_linf(got, want) <= 1e-5


def test_precision_option_selects_single_pass_tf32(cuda_context):
    """backendOptions.cuda.precision = "tf32x1": one MMA per multiply-add on operands cut to 10 mantissa bits.  On
    the values of the test above it must be visibly worse than the default (else the option did nothing) and still
    TF32-class (< 2e-3); switching back restores fp32-class results.  Unknown values are refused."""
    from webdnn_b200.lib import CudaBackendError
    ctx = cuda_context
    rng = np.random.default_rng(3)
    m, n, k = 128, 64, 512
    a = (1.0 + rng.uniform(0, 1, (m, k)) * 2.0 ** -9).astype(np.float32)
    b = (1.0 + rng.uniform(0, 1, (n, k)) * 2.0 ** -9).astype(np.float32)
    model = single_op_model("Gemm", {"transB": 1}, [a, b])
    (want,) = ref_runner.run_model(model, [a, b])
    try:
        ctx.set_precision("tf32x1")
        before = ctx.stats()["tensor_core_launches"]
        (one,) = run_cuda(model, [a, b], ctx)
        assert ctx.stats()["tensor_core_launches"] > before
    finally:
        ctx.set_precision("tf32x3")
    (three,) = run_cuda(model, [a, b], ctx)
    e1, e3 = max_err_rel_linf(one, want), max_err_rel_linf(three, want)
    assert e3 <= 1e-5 and 1e-4 < e1 < 2e-3, (e1, e3)
    with pytest.raises(ValueError):
        ctx.set_precision("fp16")
    with pytest.raises(CudaBackendError, match="precision is 0"):
        ctx.set_option("precision", 7)
    with pytest.raises(CudaBackendError, match="unknown option"):
        ctx.set_option("no_such_option", 1)


def test_weight_split_cache_follows_buffer_lifetime(cuda_context):
    """The cached hi/lo split of a weight buffer must not outlive the buffer: a new tensor that lands
    on the same address with other values has to give the new result."""
    rng = np.random.default_rng(4)
    a = rng.standard_normal((64, 64)).astype(np.float32)
    for seed in (10, 11, 12):
        b = np.random.default_rng(seed).standard_normal((32, 64)).astype(np.float32)
        model = single_op_model("Gemm", {"transB": 1}, [a, b])
        (want,) = ref_runner.run_model(model, [a, b])
        (got,) = run_cuda(model, [a, b], cuda_context)
        assert max_err_rel_linf(got, want) <= TOL


def test_weight_split_cache_sees_in_place_writes(cuda_context):
    """A weight buffer rewritten on the device (here: negated in place by wdc_unary, and then one
    half of it overwritten through wdc_strided_copy at an offset) must not be served from the cached
    split of its old contents."""
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.lib import GemmDesc
    from webdnn_b200.lib import UNARY_OPS
    ctx = cuda_context
    rng = np.random.default_rng(5)
    m, n, k = 64, 64, 128
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((n, k)).astype(np.float32)
    da, db = ctx.move_tensor(CPUTensor.from_array(a)), ctx.move_tensor(CPUTensor.from_array(b))
    dy = ctx.empty_tensor([m, n])
    d = GemmDesc(batch=1, m=m, n=n, k=k, sab=0, sa0=k, sa1=1, sbb=0, sb0=1, sb1=k, sc0=0, sc1=0, alpha=1.0, beta=0.0,
                 relu=0)
    ctx.gemm(d, da, db, None, dy)
    assert max_err_rel_linf(dy.get_data().reshape(m, n), a @ b.T) <= TOL
    ctx.unary(UNARY_OPS["Neg"], db, db)                      # in place
    ctx.gemm(d, da, db, None, dy)
    assert max_err_rel_linf(dy.get_data().reshape(m, n), -(a @ b.T)) <= TOL
    half = ctx.move_tensor(CPUTensor.from_array(np.zeros((n // 2, k), np.float32)))
    ctx.strided_copy(half, db, [n // 2, k], [k, 1], 0, [k, 1], (n // 2) * k)   # second half of b := 0
    ctx.gemm(d, da, db, None, dy)
    want = -(a @ b.T)
    want[:, n // 2:] = 0
    assert max_err_rel_linf(dy.get_data().reshape(m, n), want) <= TOL
    for t in (da, db, dy, half):
        t.dispose()


def test_weight_split_cache_sees_a_write_that_starts_before_the_operand(cuda_context):
    """B sits at an offset inside a larger allocation.  Rewriting the whole allocation from its base starts before
    the cached operand and covers it: the next contraction must see the new values, and so must one after a
    wdc_gemm whose C aliases Y (the in-place accumulate of the CUDA-core kernel)."""
    from ctypes import byref, c_void_p
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.lib import GemmDesc
    ctx = cuda_context
    rng = np.random.default_rng(15)
    m, n, k, lead = 64, 64, 128, 4096   # B starts `lead` floats into its allocation
    a = rng.standard_normal((m, k)).astype(np.float32)
    big = rng.standard_normal(lead + n * k).astype(np.float32)
    da, dbig = ctx.move_tensor(CPUTensor.from_array(a)), ctx.move_tensor(CPUTensor.from_array(big))
    dy = ctx.empty_tensor([m, n])
    d = GemmDesc(batch=1, m=m, n=n, k=k, sab=0, sa0=k, sa1=1, sbb=0, sb0=1, sb1=k, sc0=0, sc1=0, alpha=1.0, beta=0.0,
                 relu=0)

    def gemm_at_offset():
        ctx._call("wdc_gemm", byref(d), c_void_p(da.ptr), c_void_p(dbig.ptr + 4 * lead), None, c_void_p(dy.ptr))
        return dy.get_data().reshape(m, n).copy()

    b = big[lead:].reshape(n, k)
    assert max_err_rel_linf(gemm_at_offset(), a @ b.T) <= TOL
    big2 = rng.standard_normal(lead + n * k).astype(np.float32)
    dbig.set_data(big2)                                  # upload from the base of the allocation
    assert max_err_rel_linf(gemm_at_offset(), a @ big2[lead:].reshape(n, k).T) <= TOL
    ctx.unary(16, dbig, dbig)                            # Relu in place over the whole allocation, from its base
    b3 = np.maximum(big2[lead:], 0).reshape(n, k)
    y3 = gemm_at_offset()
    assert max_err_rel_linf(y3, a @ b3.T) <= TOL
    # Y = A B^T + Y through the public entry point: C == Y
    d2 = GemmDesc(batch=1, m=m, n=n, k=k, sab=0, sa0=k, sa1=1, sbb=0, sb0=1, sb1=k, sc0=n, sc1=1, alpha=1.0, beta=1.0,
                  relu=0)
    ctx._call("wdc_gemm", byref(d2), c_void_p(da.ptr), c_void_p(dbig.ptr + 4 * lead), c_void_p(dy.ptr), c_void_p(dy.ptr))
    assert max_err_rel_linf(dy.get_data().reshape(m, n), 2.0 * (a.astype(np.float64) @ b3.T)) <= TOL
    for t in (da, dbig, dy):
        t.dispose()


def test_captured_graph_goes_stale_when_its_weight_is_rewritten(cuda_context):
    """A captured run holds the addresses of the cached weight splits.  Rewriting the weight drops the split, so a
    replay would read freed memory: wdc_graph_launch must refuse instead, and a fresh capture works again."""
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.lib import CudaBackendError, GemmDesc
    ctx = cuda_context
    rng = np.random.default_rng(16)
    m, n, k = 128, 64, 64
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((n, k)).astype(np.float32)
    da, db = ctx.move_tensor(CPUTensor.from_array(a)), ctx.move_tensor(CPUTensor.from_array(b))
    dy = ctx.empty_tensor([m, n])
    d = GemmDesc(batch=1, m=m, n=n, k=k, sab=0, sa0=k, sa1=1, sbb=0, sb0=1, sb1=k, sc0=0, sc1=0, alpha=1.0, beta=0.0,
                 relu=0)
    ctx.gemm(d, da, db, None, dy)          # one-time split happens here
    ctx.capture_begin()
    ctx.gemm(d, da, db, None, dy)
    g = ctx.capture_end()
    ctx.graph_launch(g)
    assert max_err_rel_linf(dy.get_data().reshape(m, n), a @ b.T) <= TOL
    b2 = rng.standard_normal((n, k)).astype(np.float32)
    db.set_data(b2)
    with pytest.raises(CudaBackendError, match="capture the run again"):
        ctx.graph_launch(g)
    ctx.graph_destroy(g)
    ctx.gemm(d, da, db, None, dy)
    ctx.capture_begin()
    ctx.gemm(d, da, db, None, dy)
    g = ctx.capture_end()
    ctx.graph_launch(g)
    assert max_err_rel_linf(dy.get_data().reshape(m, n), a @ b2.T) <= TOL
    ctx.graph_destroy(g)
    for t in (da, db, dy):
        t.dispose()


@pytest.mark.parametrize("shape_a,shape_b", [
    ((64, 256), (256, 512)),          # 2-D, B stored [k, n]
    ((8, 625, 256), (256, 256)),      # rank-3 A times a shared 2-D B: one tall matrix
    ((3, 40, 2048), (2048, 256)),     # K = 2048, M = 120 (partly filled tile)
])
def test_matmul_row_major_b_on_tensor_cores(cuda_context, shape_a, shape_b):
    rng = np.random.default_rng(6)
    a = rng.standard_normal(shape_a).astype(np.float32)
    b = (rng.standard_normal(shape_b) * np.sqrt(2.0 / shape_b[0])).astype(np.float32)
    model = single_op_model("MatMul", {}, [a, b])
    (want,) = ref_runner.run_model(model, [a, b])
    before = cuda_context.stats()["tensor_core_launches"]
    (got,) = run_cuda(model, [a, b], cuda_context)
    assert cuda_context.stats()["tensor_core_launches"] > before
    assert got.shape == want.shape
    assert max_err_rel_linf(got, want) <= TOL


def test_gemm_trans_b_0_on_tensor_cores(cuda_context):
    rng = np.random.default_rng(7)
    a = rng.standard_normal((96, 128)).astype(np.float32)
    b = (rng.standard_normal((128, 72)) * 0.1).astype(np.float32)
    c = rng.uniform(-0.1, 0.1, 72).astype(np.float32)
    model = single_op_model("Gemm", {"alpha": 1.25, "beta": 0.5}, [a, b, c])
    (want,) = ref_runner.run_model(model, [a, b, c])
    before = cuda_context.stats()["tensor_core_launches"]
    (got,) = run_cuda(model, [a, b, c], cuda_context)
    assert cuda_context.stats()["tensor_core_launches"] > before
    assert max_err_rel_linf(got, want) <= TOL


@pytest.mark.parametrize("seed", range(10))
def test_conv_random_geometry(cuda_context, seed):
    """Random kernel sizes (k_h != k_w), strides, dilations and asymmetric pads: the im2col tensor map's
    corner offsets, traversal strides and tap offsets against the oracle's direct loops."""
    rng = np.random.default_rng(100 + seed)
    cin, cout = int(rng.choice([32, 64, 96])), int(rng.choice([8, 36, 64, 132]))
    kh, kw = int(rng.integers(1, 6)), int(rng.integers(1, 6))
    sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
    dh, dw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
    pads = [int(v) for v in rng.integers(0, 4, 4)]                      # [top, left, bottom, right]
    h = int(rng.integers((kh - 1) * dh + 1, (kh - 1) * dh + 14))
    w_ = int(rng.integers((kw - 1) * dw + 1, (kw - 1) * dw + 14))
    n = int(rng.integers(1, 4))
    x = rng.standard_normal((n, cin, h, w_)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, kh, kw)) * np.sqrt(2.0 / (cin * kh * kw))).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    attrs = dict(kernel_shape=[kh, kw], strides=[sh, sw], pads=pads, dilations=[dh, dw])
    model = single_op_model("Conv", attrs, [x, wt, b], n_graph_inputs=1)
    (want,) = ref_runner.run_model(model, [x])
    before = cuda_context.stats()["tensor_core_launches"]
    (got,) = run_cuda(model, [x], cuda_context)
    assert cuda_context.stats()["tensor_core_launches"] > before
    assert got.shape == want.shape, (attrs, x.shape)
    assert max_err_rel_linf(got, want) <= TOL, (attrs, x.shape)


@pytest.mark.parametrize("n,cin,cout,size,k,stride,pad,res", [
    (1, 512, 512, (7, 7), 3, 1, 1, False),      # 49 rows, K = 4608: many ranges
    (1, 2048, 512, (7, 7), 1, 1, 0, False),     # 1x1, K = 2048
    (2, 256, 256, (14, 14), 3, 1, 1, True),     # with residual + Relu in the second pass
    (1, 1024, 36, (5, 5), 1, 1, 0, False),      # narrow output (N = 36), ragged last range (K blocks 32 = 4 x 8)
    (1, 320, 64, (9, 9), 3, 2, 1, False),       # K blocks = 90: ranges of unequal length
])
def test_split_reduction(cuda_context, n, cin, cout, size, k, stride, pad, res):
    """Small outputs with long reductions run as (tile, K range) work units plus a reduction pass: the
    result must not depend on that (parity with the oracle, and with the unsplit kernel)."""
    import os
    from ctypes import byref
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.lib import ConvDesc
    ctx = cuda_context
    rng = np.random.default_rng(8)
    x = rng.standard_normal((n, cin, size[0], size[1])).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    shift = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    oh = (size[0] + 2 * pad - k) // stride + 1
    ow = (size[1] + 2 * pad - k) // stride + 1
    r = rng.standard_normal((n, cout, oh, ow)).astype(np.float32) if res else None
    want = ops.conv2d(x, wt, shift, (stride, stride), (pad,) * 4).astype(np.float64)
    if res:
        want = np.maximum(want + r, 0)
    want = want.astype(np.float32)
    dx = ctx.channels_last(ctx.move_tensor(CPUTensor.from_array(x)))
    dw = ctx.move_tensor(CPUTensor.from_array(np.ascontiguousarray(wt.transpose(0, 2, 3, 1))))
    dsh = ctx.move_tensor(CPUTensor.from_array(shift))
    dr = ctx.channels_last(ctx.move_tensor(CPUTensor.from_array(r))) if res else None
    d = ConvDesc(batch=n, ch_in=cin, in_h=size[0], in_w=size[1], ch_out=cout, k_h=k, k_w=k, out_h=oh, out_w=ow,
                 stride_h=stride, stride_w=stride, pad_t=pad, pad_l=pad, dil_h=1, dil_w=1, group=1, relu=int(res))
    warm = ctx.empty_tensor([n, cout, oh, ow], layout="nhwc")
    ctx.conv2d(d, dx, dw, None, dsh, dr, warm)     # first use of the weights: their one-time split
    warm.dispose()
    outs = []
    for no_split in (False, True):
        ctx.set_option("split_k", 0 if no_split else 1)
        try:
            dy = ctx.empty_tensor([n, cout, oh, ow], layout="nhwc")
            before = ctx.stats()["launches"]
            ctx.conv2d(d, dx, dw, None, dsh, dr, dy)
            launches = ctx.stats()["launches"] - before
            outs.append((ctx.canonical(dy).get_data().reshape(n, cout, oh, ow), launches))
            dy.dispose()
        finally:
            ctx.set_option("split_k", 1)
    (split, l_split), (single, l_single) = outs
    assert l_split == l_single + 1, (l_split, l_single)    # the reduction pass really ran
    assert max_err_rel_linf(split, want) <= TOL
    assert max_err_rel_linf(single, want) <= TOL
    assert max_err_rel_linf(split, single) <= 1e-5


@pytest.mark.parametrize("n,cin,cout,size,k,stride,pad,dil", [
    (2, 48, 64, (13, 15), 3, 1, 1, 1),     # 48 channels: one full and one half K block per tap
    (1, 100, 32, (9, 9), 3, 2, 1, 1),      # 100 channels: the last block of a tap has 4 of 32
    (2, 24, 40, (11, 7), 5, 1, 2, 1),      # fewer than 32 channels: every block is short
    (1, 72, 128, (8, 8), 1, 1, 0, 1),      # 1x1
    (1, 40, 64, (12, 12), 3, 1, 2, 2),     # dilation
])
def test_conv_channels_not_multiple_of_32(cuda_context, n, cin, cout, size, k, stride, pad, dil):
    assert _conv_case(cuda_context, n, cin, cout, size, k, stride, pad, dil) <= TOL


@pytest.mark.parametrize("n,cin,cout,size,k,stride,pad", [
    (2, 3, 16, (20, 22), 5, 1, 2),     # stride 1: one 16-byte plane per tap
    (2, 3, 64, (33, 31), 7, 2, 3),     # stride 2, odd sizes: pixel-pair planes
    (1, 1, 8, (12, 12), 3, 1, 1),      # a single input channel
    (3, 4, 32, (9, 14), 3, 2, 0),      # four channels, no padding
])
def test_first_layer_reads_nchw_input_directly(cuda_context, n, cin, cout, size, k, stride, pad):
    """Few-channel first layers take the network's NCHW input as it is (no separate layout conversion
    launch): one padding pass, one contraction."""
    before = cuda_context.stats()["launches"]
    assert _conv_case(cuda_context, n, cin, cout, size, k, stride, pad) <= TOL
    # weight packing + weight split + padding pass + contraction (+ the output's conversion for the host)
    assert cuda_context.stats()["launches"] - before <= 5


@pytest.mark.parametrize("seed", range(32))
def test_fused_block_random_sweep(cuda_context, seed):
    """Conv (+bias) -> BatchNormalization -> Add(residual) -> Relu as one fused launch, over random channel counts
    (multiples of 4, also far from multiples of 32; 1 and 3 for first-layer shapes), square kernels of 1..7, strides
    1..3, pads 0..3, dilation 1..2, image sizes from a handful of pixels to several tiles, with and without each
    epilogue part; the unfused oracle chain is the expectation."""
    from webdnn_b200.zoo import _Builder
    rng = np.random.default_rng(500 + seed)
    first_layer = seed % 8 == 7
    cin = int(rng.choice([1, 3])) if first_layer else int(rng.choice([4, 8, 12, 20, 36, 64, 100, 160, 256]))
    cout = int(rng.choice([4, 12, 32, 60, 64, 128, 200, 260]))
    k = int(rng.integers(1, 8)) if first_layer else int(rng.choice([1, 1, 2, 3, 3, 5]))
    stride = int(rng.integers(1, 4))
    pad = int(rng.integers(0, min(k, 4)))
    dil = 1 if first_layer else int(rng.integers(1, 3))
    size = int(rng.integers((k - 1) * dil + 1, (k - 1) * dil + 40))
    n = int(rng.integers(1, 5))
    use_bias, use_bn, use_res, use_relu = (bool(v) for v in rng.integers(0, 2, 4))
    b = _Builder(seed)
    h = b.conv("x", cin, cout, k, stride=stride, pad=pad, bias=use_bias, dilation=dil)
    if use_bn:
        h = b.bn(h, cout)
    out = (size + 2 * pad - dil * (k - 1) - 1) // stride + 1
    ins = [("x", [n, cin, size, size])]
    feeds = [rng.standard_normal((n, cin, size, size)).astype(np.float32)]
    if use_res:
        h = b.node("Add", [h, "r"])[0]
        ins.append(("r", [n, cout, out, out]))
        feeds.append(rng.standard_normal((n, cout, out, out)).astype(np.float32))
    if use_relu:
        h = b.node("Relu", [h])[0]
    model = b.model(ins, [(h, [n, cout, out, out])])
    (want,) = ref_runner.run_model(model, feeds)
    before = cuda_context.stats()["tensor_core_launches"]
    (got,), r = run_cuda(model, feeds, cuda_context, return_runner=True)
    kinds = [kd for _, kd, _ in r.node_backends]
    r.dispose()
    assert len(kinds) == 1 or not (use_bias or use_bn or use_res or use_relu) or kinds == ["CudaConvFused"], kinds
    desc = dict(cin=cin, cout=cout, k=k, stride=stride, pad=pad, dil=dil, size=size, n=n, bias=use_bias, bn=use_bn,
                res=use_res, relu=use_relu)
    assert got.shape == want.shape, desc
    assert max_err_rel_linf(got, want) <= TOL, desc
    if cin % 4 == 0 and cout % 4 == 0:
        assert cuda_context.stats()["tensor_core_launches"] > before, desc


@pytest.mark.parametrize("seed", range(24))
def test_gemm_matmul_random_sweep(cuda_context, seed):
    """Gemm with every C form (none, scalar, row, column, full), alpha / beta, transA / transB, and MatMul with a
    constant or a run-time right operand and stacked left operands, over random sizes on both sides of the
    tensor-core kernel's limits (k % 4, k >= 32, m >= 32)."""
    rng = np.random.default_rng(900 + seed)
    m = int(rng.choice([1, 5, 31, 32, 33, 100, 129, 300]))
    n = int(rng.choice([1, 4, 10, 36, 64, 100, 130, 257]))
    k = int(rng.choice([3, 8, 32, 36, 50, 64, 100, 260]))
    a = rng.standard_normal((m, k)).astype(np.float32)
    bm = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    if seed % 2 == 0:
        ta, tb = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        c_form = ["none", "scalar", "row", "col", "full"][int(rng.integers(0, 5))]
        c = {"none": None, "scalar": rng.standard_normal((1,)), "row": rng.standard_normal((n,)),
             "col": rng.standard_normal((m, 1)), "full": rng.standard_normal((m, n))}[c_form]
        ins = [np.ascontiguousarray(a.T) if ta else a, np.ascontiguousarray(bm.T) if tb else bm]
        if c is not None:
            ins.append(c.astype(np.float32))
        attrs = dict(alpha=float(rng.choice([1.0, 0.5, -2.0])), beta=float(rng.choice([1.0, 0.0, 0.25])), transA=ta,
                     transB=tb)
        const_w = bool(rng.integers(0, 2))
        model = single_op_model("Gemm", attrs, ins, n_graph_inputs=1 if const_w else len(ins), opset=11)
        feeds = ins[:1] if const_w else ins
        desc = dict(op="Gemm", m=m, n=n, k=k, c=c_form, const_w=const_w, **attrs)
    else:
        lead = [(), (3,), (5,)][int(rng.integers(0, 3))]      # result rank <= 3, like the reference
        a = rng.standard_normal(lead + (m, k)).astype(np.float32)
        const_w = bool(rng.integers(0, 2))
        model = single_op_model("MatMul", {}, [a, bm], n_graph_inputs=1 if const_w else 2)
        feeds = [a] if const_w else [a, bm]
        desc = dict(op="MatMul", lead=lead, m=m, n=n, k=k, const_w=const_w)
    (want,) = ref_runner.run_model(model, feeds)
    (got,) = run_cuda(model, feeds, cuda_context)
    assert got.shape == want.shape, desc
    assert max_err_rel_linf(got, want) <= TOL, desc
