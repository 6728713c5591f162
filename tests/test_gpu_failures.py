"""GPU: failure handling of the cuda backend, none of which faults, traps or hangs the device.

What the reference does at these points: a backend that cannot initialise is skipped by WebDNN.load
(index.ts:68-79) and a throwing operator surfaces as a JS exception (core/runnerImpl.ts:511-520) with the runner
object still usable.  Here every C-ABI call returns a status, the arena has an optional byte budget, tensors refuse
use after dispose, and a device-side wait that runs out is reported at the next waiting call.
"""
from ctypes import byref, c_int64, c_void_p

import numpy as np
import pytest

from oracle import ref_runner
from webdnn_b200 import zoo

from util import max_err_rel_linf, run_cuda

pytestmark = pytest.mark.gpu


def _new_context(arena_bytes=0):
    from webdnn_b200.backend import WebDNNCudaContext
    ctx = WebDNNCudaContext(arena_bytes=arena_bytes)
    ctx.initialize()
    return ctx


def test_arena_budget_gives_oom_and_the_context_stays_usable():
    from webdnn_b200.lib import CudaBackendError
    ctx = _new_context(arena_bytes=8 << 20)
    try:
        small = ctx.empty_tensor([1024, 1024])           # 4 MiB: fits
        with pytest.raises(CudaBackendError) as e:
            ctx.empty_tensor([2048, 1024])               # 8 MiB more: over the budget
        assert e.value.status == 3 and "arena budget" in str(e.value)   # WDC_ERR_OOM
        # a whole model whose activations cannot fit fails the same way, from inside runner.run() ...
        with pytest.raises(CudaBackendError) as e:
            run_cuda(zoo.conv_bn_relu(8, 64, 56), [zoo.make_input((8, 64, 56, 56))], ctx)
        assert e.value.status == 3
        # ... and the context still computes: nothing leaked past the budget, small work goes through
        small.dispose()
        model = zoo.conv_bn_relu(1, 16, 8)
        x = zoo.make_input((1, 16, 8, 8))
        (want,) = ref_runner.run_model(model, [x])
        (got,) = run_cuda(model, [x], ctx)
        assert max_err_rel_linf(got, want) <= 1e-4
    finally:
        ctx.close()


def test_use_after_dispose_and_foreign_tensors_raise(cuda_context):
    from webdnn_b200.backend import CPUTensor
    ctx = cuda_context
    t = ctx.move_tensor(CPUTensor.from_array(np.arange(6, dtype=np.float32).reshape(2, 3)))
    assert t.get_data().tolist() == [0, 1, 2, 3, 4, 5]
    t.dispose()
    with pytest.raises(RuntimeError):
        t.get_data()
    with pytest.raises(RuntimeError):
        t.set_data(np.zeros(6, np.float32))
    with pytest.raises(RuntimeError):
        _ = t.ptr
    # a cpu tensor handed to a cuda operator is refused by the operator's own check (assertsCudaTensorArray)
    from webdnn_b200.operators.cuda import CudaUnary
    with pytest.raises(TypeError):
        CudaUnary("Relu").run(ctx, [CPUTensor.from_array(np.zeros(3, np.float32))], 1)
    # a tensor of another context is refused as well
    other = _new_context()
    try:
        foreign = other.empty_tensor([3])
        with pytest.raises(TypeError):
            CudaUnary("Relu").run(ctx, [foreign], 1)
        foreign.dispose()
    finally:
        other.close()


def test_null_and_invalid_arguments_return_a_status(cuda_context):
    from webdnn_b200.lib import CudaBackendError, Library
    L = Library().lib
    ctx = cuda_context
    # null context: every entry point answers WDC_ERR_INVALID (1) instead of dereferencing it
    assert L.wdc_sync(None) == 1
    assert L.wdc_alloc(None, 16, byref(c_void_p())) == 1
    assert L.wdc_softmax(None, None, None, 1, 1) == 1
    assert L.wdc_lstm(None, *([None] * 9), 1, 1, 1, 1) == 1
    assert L.wdc_set_option(None, b"precision", 0) == 1
    assert L.wdc_graph_launch(None, None) == 1
    # an out-of-range device and a null output pointer at creation
    h = c_void_p()
    assert L.wdc_create(4096, 0, byref(h)) == 1 and not h.value
    assert b"out of range" in L.wdc_last_error(None)
    # freeing an address that is not a live allocation of this context
    with pytest.raises(CudaBackendError, match="not a live allocation"):
        ctx._call("wdc_free", c_void_p(0x1000))
    t = ctx.empty_tensor([8])
    with pytest.raises(CudaBackendError, match="not a live allocation"):
        ctx._call("wdc_free", c_void_p(t.ptr + 16))     # inside a block, not its start
    t.dispose()
    # shapes the library must refuse before any launch
    with pytest.raises(CudaBackendError):
        ctx._call("wdc_softmax", None, None, -1, 4)
    with pytest.raises(CudaBackendError):
        ctx._call("wdc_alloc", -5, byref(c_void_p()))
    with pytest.raises(CudaBackendError, match="outside"):
        ctx._call("wdc_selftest_device_wait", c_int64(5))
    ctx.sync()     # none of the refused calls left anything behind


def test_a_device_wait_that_runs_out_is_reported_and_the_context_survives():
    """The persistent LSTM kernel is told to wait for one CTA more than its grid has, with a 1 ms limit: the wait
    runs out, the kernel returns by itself, the next sync reports WDC_ERR_DEVICE_WAIT exactly once, and the same
    context then runs the real LSTM correctly."""
    import time
    from webdnn_b200.lib import CudaBackendError
    ctx = _new_context()
    try:
        ctx.sync()
        t0 = time.perf_counter()
        ctx._call("wdc_selftest_device_wait", c_int64(1_000_000))
        with pytest.raises(CudaBackendError) as e:
            ctx.sync()
        assert e.value.status == 5 and "kernel status 61" in str(e.value)     # WDC_ERR_DEVICE_WAIT, the step counter
        assert time.perf_counter() - t0 < 5.0
        ctx.sync()                                                             # reported once, then clean
        model = zoo.lstm(6, 8, 16, 128)
        x = zoo.make_input((6, 8, 16))
        want = ref_runner.run_model(model, [x])
        got = run_cuda(model, [x], ctx)
        for g, w in zip(got, want):
            assert max_err_rel_linf(g, w) <= 1e-4
    finally:
        ctx.close()


def test_a_backend_that_cannot_initialise_is_skipped_by_load():
    """index.ts:68-79: load() tries the next name of backendOrder.  A cuda device that does not exist falls through
    to the host backend, which has no arithmetic operators, so running a Conv there raises instead of silently
    computing on the CPU."""
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.runner import load
    r = load(zoo.conv_bn_relu(1, 8, 6), backend_order=["cuda", "cpu"], backend_options={"cuda": {"device": 4096}})
    assert r.backend_order == ["cpu"]
    with pytest.raises(RuntimeError, match="does not exist"):
        r.run([CPUTensor.from_array(zoo.make_input((1, 8, 6, 6)))])
