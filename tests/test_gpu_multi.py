"""In-process replicas on two GPUs: batch slices run on their own devices and the outputs are gathered
either through the host or by peer copies into the first device.  Skipped on a single-GPU box."""
import numpy as np
import pytest

from oracle import ref_runner
from webdnn_b200 import zoo

from util import max_err_rel_linf

pytestmark = pytest.mark.gpu


def _device_count():
    from webdnn_b200.lib import Library
    return Library().device_count()


@pytest.mark.parametrize("gather", ["host", "peer"])
def test_two_replicas_match_one_oracle_run(gather):
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    from webdnn_b200.replicas import ReplicaGroup
    model = zoo.conv_bn_relu(6, 32, 14)
    x = zoo.make_input((6, 32, 14, 14))
    (want,) = ref_runner.run_model(model, [x])
    group = ReplicaGroup(model, devices=[0, 1])
    try:
        (got,) = group.run([x], gather=gather)
        assert got.shape == want.shape
        assert max_err_rel_linf(got, want) <= 1e-4
        # later runs are served by each replica's recorded graph (from the third run of a shape on): new inputs
        # every time, the same answers as the oracle
        for seed in (11, 12, 13):
            x2 = zoo.make_input((6, 32, 14, 14), seed=seed)
            (want2,) = ref_runner.run_model(model, [x2])
            (got2,) = group.run([x2], gather=gather, deadline_s=60)
            assert max_err_rel_linf(got2, want2) <= 1e-4, seed
        assert all(r._captured for r in group.replicas)
    finally:
        group.close()


def test_two_outputs_over_two_gpus():
    """Four images over two GPUs through a network with two outputs (the DETR-style heads, whose reshapes fix the
    per-replica batch at 2): slice offsets of the peer gather for both outputs."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    from webdnn_b200.replicas import ReplicaGroup
    model = zoo.detr(batch=2, size=128, d=64, heads=4, enc_layers=1, dec_layers=1, ffn=128, queries=6, classes=9,
                     width=16, blocks=(1, 1, 1, 1))
    x = zoo.make_input((4, 3, 128, 128))
    halves = [ref_runner.run_model(model, [np.ascontiguousarray(x[i:i + 2])]) for i in (0, 2)]
    want = [np.concatenate([h[j] for h in halves], axis=0) for j in range(2)]
    group = ReplicaGroup(model, devices=[0, 1], graph_replay=False)
    try:
        for gather in ("peer", "host"):
            got = group.run([x], gather=gather)
            for g, w in zip(got, want):
                assert g.shape == w.shape
                assert max_err_rel_linf(g, w) <= 1e-4, gather
    finally:
        group.close()


@pytest.mark.parametrize("devices", [[0], [0, 1]])
def test_pipelined_group_runs_equal_synchronous_runs(devices):
    """ReplicaGroup.run_async: two steps in flight (the second started before the first result is taken), node by
    node at first and as replayed graphs from the third step of the shape on; every result equals the synchronous
    call's bit for bit.  The one-device group runs on any box."""
    if _device_count() < len(devices):
        pytest.skip("needs two GPUs")
    from webdnn_b200.replicas import ReplicaGroup
    model = zoo.conv_bn_relu(8, 32, 14)
    xs = [zoo.make_input((8, 32, 14, 14), seed=s) for s in range(21, 27)]
    group = ReplicaGroup(model, devices=devices)
    try:
        want = [group.run([x])[0] for x in xs]
        pend = group.run_async([xs[0]])
        got = []
        for x in xs[1:]:
            nxt = group.run_async([x])
            got.append(pend.result(deadline_s=60)[0])
            pend = nxt
        got.append(pend.result()[0])
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
        (oracle0,) = ref_runner.run_model(model, [xs[0]])
        assert max_err_rel_linf(got[0], oracle0) <= 1e-4
    finally:
        group.close()
