"""GPU parity of the fused attention kernel (wdc_attention) against the chain of reference operators it
replaces: MatMul -> Mul -> Softmax -> MatMul on the CPU oracle (matmul.ts, binary7.ts, softmax.ts).

Tolerance: max|a-e| <= 1e-4 * ||e||_inf.
"""
from ctypes import byref, c_void_p

import numpy as np
import pytest

from oracle import ops, ref_runner

from util import max_err_rel_linf, run_cuda
from webdnn_b200.backend import CPUTensor
from webdnn_b200.lib import AttentionDesc
from webdnn_b200.zoo import _Builder, _Transformer

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _oracle_chain(q, k, v, scale):
    """[bh, t, c] operands through the reference operators."""
    s = ops.binary("Mul", ops.matmul(q, ops.transpose(k, [0, 2, 1])), np.asarray(scale, np.float32))
    return ops.matmul(ops.softmax(s, -1), v)


def _device(ctx, a):
    return ctx.move_tensor(CPUTensor.from_array(np.ascontiguousarray(a, np.float32)))


@pytest.mark.parametrize("bh,tq,tk,dh", [(3, 70, 130, 32), (2, 64, 64, 32), (5, 1, 7, 32), (2, 100, 625, 32),
                                         (3, 65, 129, 64), (1, 128, 200, 64), (2, 129, 1, 32), (1, 300, 63, 64),
                                         (4, 257, 65, 32), (1, 5, 1000, 64)])
def test_contiguous_heads_match_the_operator_chain(cuda_context, bh, tq, tk, dh):
    rng = np.random.default_rng(bh * 1000 + tq + tk + dh)
    q, k, v = (rng.standard_normal((bh, t, dh)).astype(np.float32) for t in (tq, tk, tk))
    scale = float(np.float32(dh ** -0.5))
    want = _oracle_chain(q, k, v, scale)
    ctx = cuda_context
    dq, dk, dv = (_device(ctx, a) for a in (q, k, v))
    y = ctx.empty_tensor([bh, tq, dh], "float32")
    d = AttentionDesc(batch=bh, heads=1, tq=tq, tk=tk, dh=dh, q_sb=tq * dh, q_sh=0, q_st=dh, k_sb=tk * dh, k_sh=0,
                      k_st=dh, v_sb=tk * dh, v_sh=0, v_st=dh, y_sb=tq * dh, y_sh=0, y_st=dh, scale=scale)
    before = ctx.stats()["tensor_core_launches"]
    ctx._call("wdc_attention", byref(d), *(c_void_p(t.ptr) for t in (dq, dk, dv, y)))
    assert ctx.stats()["tensor_core_launches"] == before + 1      # the tcgen05 kernel ran, not the CUDA-core one
    got = y.get_data().reshape(bh, tq, dh)
    assert max_err_rel_linf(got, want) <= TOL
    for t in (dq, dk, dv, y):
        t.dispose()


def test_full_size_encoder_block_through_head_strides(cuda_context):
    """The encoder self-attention of the DETR-style configuration at its full size (batch 8, 8 heads of 32 channels,
    625 tokens), operands laid out [batch, tokens, heads * 32] and read through strides, result written merged."""
    b, h, t, c = 8, 8, 625, 32
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((b, t, h * c)).astype(np.float32) for _ in range(3))
    scale = float(np.float32(c ** -0.5))
    heads = lambda a: np.ascontiguousarray(a.reshape(b, t, h, c).transpose(0, 2, 1, 3).reshape(b * h, t, c))
    want = _oracle_chain(heads(q), heads(k), heads(v), scale).reshape(b, h, t, c).transpose(0, 2, 1, 3).reshape(b, t, h * c)
    ctx = cuda_context
    dq, dk, dv = (_device(ctx, a) for a in (q, k, v))
    y = ctx.empty_tensor([b, t, h * c], "float32")
    st = dict(sb=t * h * c, sh=c, st=h * c)
    d = AttentionDesc(batch=b, heads=h, tq=t, tk=t, dh=c, scale=scale,
                      **{f"{n}_{key}": val for n in "qkvy" for key, val in st.items()})
    ctx._call("wdc_attention", byref(d), *(c_void_p(x.ptr) for x in (dq, dk, dv, y)))
    assert max_err_rel_linf(y.get_data().reshape(b, t, h * c), want) <= TOL
    for x in (dq, dk, dv, y):
        x.dispose()


def test_sharp_softmax_rows_and_large_scores(cuda_context):
    """Scores spread over hundreds of units: the running maximum has to move between key chunks."""
    rng = np.random.default_rng(7)
    bh, tq, tk, dh = 2, 40, 300, 32
    q = (rng.standard_normal((bh, tq, dh)) * 6).astype(np.float32)
    k = (rng.standard_normal((bh, tk, dh)) * 6).astype(np.float32)
    k = np.sort(k, axis=1)                              # larger keys later, so later chunks raise the maximum
    v = rng.standard_normal((bh, tk, dh)).astype(np.float32)
    want = _oracle_chain(q, k, v, 1.0)
    ctx = cuda_context
    dq, dk, dv = (_device(ctx, a) for a in (q, k, v))
    y = ctx.empty_tensor([bh, tq, dh], "float32")
    d = AttentionDesc(batch=bh, heads=1, tq=tq, tk=tk, dh=dh, q_sb=tq * dh, q_sh=0, q_st=dh, k_sb=tk * dh, k_sh=0,
                      k_st=dh, v_sb=tk * dh, v_sh=0, v_st=dh, y_sb=tq * dh, y_sh=0, y_st=dh, scale=1.0)
    ctx._call("wdc_attention", byref(d), *(c_void_p(t.ptr) for t in (dq, dk, dv, y)))
    assert max_err_rel_linf(y.get_data().reshape(bh, tq, dh), want) <= TOL
    for t in (dq, dk, dv, y):
        t.dispose()


def test_unsupported_head_size_is_an_error_not_a_fallback(cuda_context):
    ctx = cuda_context
    x = _device(ctx, np.zeros((1, 4, 16), np.float32))
    y = ctx.empty_tensor([1, 4, 16], "float32")
    d = AttentionDesc(batch=1, heads=1, tq=4, tk=4, dh=16, q_sb=64, q_sh=0, q_st=16, k_sb=64, k_sh=0, k_st=16,
                      v_sb=64, v_sh=0, v_st=16, y_sb=64, y_sh=0, y_st=16, scale=1.0)
    with pytest.raises(RuntimeError, match="head size"):
        ctx._call("wdc_attention", byref(d), *(c_void_p(t.ptr) for t in (x, x, x, y)))
    x.dispose()
    y.dispose()


@pytest.mark.parametrize("d_model,heads,tq,tk", [(64, 2, 37, 90), (128, 2, 70, 70), (64, 4, 20, 33)])
def test_attention_block_graph_runs_as_one_node(cuda_context, d_model, heads, tq, tk):
    """A whole multi-head attention block (projections, head split, scores, softmax, context, head merge, output
    projection) as the graph exporters write it; head sizes 32 / 64 read the projections through strides, head
    size 16 takes the rank-3 form and the three-launch path."""
    batch = 2
    b = _Builder(3)
    t = _Transformer(b, batch, d_model, heads, 2 * d_model)
    y = t.attention("xq", "xk", "xv", tq, tk)
    model = b.model([("xq", [batch, tq, d_model]), ("xk", [batch, tk, d_model]), ("xv", [batch, tk, d_model])],
                    [(y, [batch, tq, d_model])])
    rng = np.random.default_rng(11)
    xs = [rng.standard_normal(s).astype(np.float32) for s in ((batch, tq, d_model), (batch, tk, d_model),
                                                              (batch, tk, d_model))]
    want = ref_runner.run_model(model, xs)
    got, r = run_cuda(model, xs, cuda_context, return_runner=True)
    kinds = [k for _, k, _ in r.node_backends]
    assert kinds.count("CudaAttention") == 1 and "Softmax" not in kinds and "MatMul" not in kinds, kinds
    assert all(bk == "cuda" for _, _, bk in r.node_backends)
    if d_model // heads in (32, 64):
        assert "Transpose" not in kinds and "Reshape" not in kinds, kinds
    r.dispose()
    assert list(got[0].shape) == list(want[0].shape)
    assert max_err_rel_linf(got[0], want[0]) <= TOL
