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
    finally:
        group.close()
    assert got.shape == want.shape
    assert max_err_rel_linf(got, want) <= 1e-4
