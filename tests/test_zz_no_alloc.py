"""GPU: the allocation-free LSTM entry point against the CPU oracle and the regular entry point, through the C ABI.

wdc_lstm_static exists for hosts that may not allocate device memory while running (their own memory pool owns the
GPU, a real-time loop, a sandbox): its scratch is a fixed array inside the library.  This file is named so that
pytest collects it last; the check must hold both in a fresh process and after every other test has used the
device, and on two calls in a row (the second call sees the scratch the first one left behind).
"""
from ctypes import c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LSTM_TOL = 1e-3   # the LSTM tolerance of the suite, relative to the output's largest magnitude


def _upload(ctx, arrays):
    from webdnn_b200.backend import CPUTensor
    return [ctx.move_tensor(CPUTensor.from_array(a)) for a in arrays]


def _call(ctx, entry, dev_in, shape):
    """One call of `entry` on resident operands; returns the three output tensors (still on the device)."""
    T, Bt, I, H = shape
    dx, dw, dr, db = dev_in
    y, yh, yc = ctx.empty_tensor([T, 1, Bt, H]), ctx.empty_tensor([1, Bt, H]), ctx.empty_tensor([1, Bt, H])
    p = lambda t: c_void_p(t.ptr)
    ctx._call(entry, p(dx), p(dw), p(dr), p(db), None, None, p(y), p(yh), p(yc), T, Bt, I, H)
    return [y, yh, yc]


def test_static_scratch_lstm_matches_oracle_twice(cuda_context):
    from oracle import ops as oracle_ops
    ctx = cuda_context
    rng = np.random.default_rng(21)
    T, Bt, I, H = 12, 16, 64, 96
    lim = 1.0 / np.sqrt(H)
    w = rng.uniform(-lim, lim, (1, 4 * H, I)).astype(np.float32)
    r = rng.uniform(-lim, lim, (1, 4 * H, H)).astype(np.float32)
    b = rng.uniform(-lim, lim, (1, 8 * H)).astype(np.float32)
    for call in range(2):  # second call: different input, scratch still holds the first call's last step
        x = rng.standard_normal((T, Bt, I)).astype(np.float32)
        oracle = oracle_ops.lstm(x, w[0], r[0], b[0])
        dev_in = _upload(ctx, (x, w, r, b))
        arena_outs = _call(ctx, "wdc_lstm", dev_in, (T, Bt, I, H))
        arena = [t.get_data().copy() for t in arena_outs]
        for t in arena_outs:
            t.dispose()
        ctx.sync()
        before = ctx.stats(device_memory=True)
        outs = _call(ctx, "wdc_lstm_static", dev_in, (T, Bt, I, H))
        ctx.sync()
        after = ctx.stats(device_memory=True)
        # the three output tensors of this test are the only arena allocations, the arena did not grow, and
        # (second call, when every module is certainly loaded) the GPU's free memory did not move at all
        assert after["allocs"] - before["allocs"] == 3
        assert after["reserved_bytes"] == before["reserved_bytes"]
        if call == 1:
            assert after["device_free_bytes"] == before["device_free_bytes"]
        got = [t.get_data().copy() for t in outs]
        for t in dev_in + outs:
            t.dispose()
        for g, e, a in zip(got, oracle, arena):
            scale = np.abs(e).max()
            assert np.abs(g.astype(np.float64) - e.reshape(g.shape)).max() <= LSTM_TOL * scale, ("oracle", call)
            assert np.abs(g.astype(np.float64) - a).max() <= LSTM_TOL * scale, ("wdc_lstm", call)


def test_static_scratch_limit_is_enforced(cuda_context):
    from webdnn_b200.lib import CudaBackendError
    ctx = cuda_context
    t = ctx.empty_tensor([4])
    p = c_void_p(t.ptr)
    with pytest.raises(CudaBackendError, match="exceeds the static scratch"):
        ctx._call("wdc_lstm_static", p, p, p, None, None, None, p, p, p, 1, 1024, 8, 512)  # 1024*4*512 > 2^20
    t.dispose()
