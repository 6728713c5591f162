"""GPU: the allocation-free LSTM entry point against the regular one, through the C ABI.

wdc_lstm_static exists for hosts that may not allocate device memory while running (their own memory pool owns the
GPU, a real-time loop, a sandbox): its scratch is a fixed array inside the library.  This file is named so that
pytest collects it last; the check must hold both in a fresh process and after every other test has used the
device, and on two calls in a row (the second call sees the scratch the first one left behind).
"""
from ctypes import c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(ctx, entry, x, w, r, b):
    from webdnn_b200.backend import CPUTensor
    T, Bt, I = x.shape
    H = r.shape[-1]
    dx, dw, dr, db = (ctx.move_tensor(CPUTensor.from_array(a)) for a in (x, w, r, b))
    y, yh, yc = ctx.empty_tensor([T, 1, Bt, H]), ctx.empty_tensor([1, Bt, H]), ctx.empty_tensor([1, Bt, H])
    p = lambda t: c_void_p(t.ptr)
    ctx._call(entry, p(dx), p(dw), p(dr), p(db), None, None, p(y), p(yh), p(yc), T, Bt, I, H)
    out = [t.get_data().copy() for t in (y, yh, yc)]
    for t in (dx, dw, dr, db, y, yh, yc):
        t.dispose()
    return out


def test_static_scratch_lstm_matches_arena_lstm_twice(cuda_context):
    ctx = cuda_context
    rng = np.random.default_rng(21)
    T, Bt, I, H = 12, 16, 64, 96
    lim = 1.0 / np.sqrt(H)
    w = rng.uniform(-lim, lim, (1, 4 * H, I)).astype(np.float32)
    r = rng.uniform(-lim, lim, (1, 4 * H, H)).astype(np.float32)
    b = rng.uniform(-lim, lim, (1, 8 * H)).astype(np.float32)
    for call in range(2):  # second call: different input, scratch still holds the first call's last step
        x = rng.standard_normal((T, Bt, I)).astype(np.float32)
        want = _run(ctx, "wdc_lstm", x, w, r, b)
        allocs_before = ctx.stats()["allocs"]
        reserved_before = ctx.stats()["reserved_bytes"]
        dx_tensors = 7  # the test's own input/output tensors are the only arena allocations
        got = _run(ctx, "wdc_lstm_static", x, w, r, b)
        assert ctx.stats()["allocs"] - allocs_before == dx_tensors
        assert ctx.stats()["reserved_bytes"] == reserved_before
        for g, e in zip(got, want):
            scale = np.abs(e).max()
            assert np.abs(g.astype(np.float64) - e).max() <= 1e-3 * scale, call  # the LSTM tolerance of the suite


def test_static_scratch_limit_is_enforced(cuda_context):
    from webdnn_b200.lib import CudaBackendError
    ctx = cuda_context
    t = ctx.empty_tensor([4])
    p = c_void_p(t.ptr)
    with pytest.raises(CudaBackendError, match="exceeds the static scratch"):
        ctx._call("wdc_lstm_static", p, p, p, None, None, None, p, p, p, 1, 1024, 8, 512)  # 1024*4*512 > 2^20
    t.dispose()
