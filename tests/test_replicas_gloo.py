"""CPU, world_size 2 over gloo: the batch-sharded replica path (slice -> run -> gather) gives the same result as
one full-batch run.  The per-rank compute here is the CPU oracle; on GPUs each rank would run its cuda runner."""
import os
import socket

import numpy as np
import pytest

from webdnn_b200.replicas import shard_for_rank, slice_bounds


def test_slice_bounds_cover_the_batch_exactly():
    for n in (0, 1, 7, 64, 255, 256):
        for parts in (1, 2, 3, 4, 8):
            edges = [slice_bounds(n, parts, i) for i in range(parts)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            assert all(edges[i][1] == edges[i + 1][0] for i in range(parts - 1))
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        slice_bounds(4, 2, 2)


def test_shard_axis_one_for_lstm_inputs():
    x = np.arange(3 * 8 * 2, dtype=np.float32).reshape(3, 8, 2)
    a, b = (shard_for_rank([x], r, 2, axis=1)[0] for r in range(2))
    assert a.shape == (3, 4, 2) and np.array_equal(np.concatenate([a, b], axis=1), x)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from oracle import ops, ref_runner
    from webdnn_b200 import zoo
    from webdnn_b200.replicas import gather_outputs
    ops.set_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = zoo.mlp(batch)  # shapes in the graph are not checked by the runner: any batch works
        x = zoo.make_input((batch, 784), "uniform")
        mine = shard_for_rank([x], rank, world)
        local = ref_runner.run_model(model, mine)
        gathered = gather_outputs(local)
        full = ref_runner.run_model(model, [x])
        ok = all(np.array_equal(g, f) for g, f in zip(gathered, full))
        queue.put((rank, ok, gathered[0].shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [8, 7])  # even and uneven slices
def test_two_gloo_ranks_reproduce_the_full_batch(batch):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(ok for _, ok, _ in results), results
    assert all(shape == (batch, 10) for _, _, shape in results)


# ---- one process, several replicas: stand-ins that compute with the CPU oracle, fail, or stall (no GPU involved) ----
class _OracleReplica:
    """Behaves like CudaReplica towards ReplicaGroup: start(shard) takes the slice, finish() returns host arrays."""

    def __init__(self, model, fail=None, stall_s=0.0):
        self.model, self.fail, self.stall_s = model, fail, stall_s
        self.shard = None
        self.closed = False

    def start(self, shard):
        if self.fail == "start":
            from webdnn_b200.lib import CudaBackendError
            raise CudaBackendError(3, "wdc_alloc: 1024 bytes would exceed the arena budget")   # what a full arena reports
        self.shard = [np.asarray(a) for a in shard]

    def finish(self):
        import time
        from oracle import ref_runner
        if self.stall_s:
            time.sleep(self.stall_s)
        if self.fail == "finish":
            from webdnn_b200.lib import CudaBackendError
            raise CudaBackendError(5, "a bounded device-side wait expired (kernel status 61)")
        return ref_runner.run_model(self.model, self.shard)

    def close(self):
        self.closed = True


def test_replica_group_slices_and_gathers_like_one_run():
    from oracle import ref_runner
    from webdnn_b200 import zoo
    from webdnn_b200.replicas import ReplicaGroup
    model = zoo.mlp(7)
    x = zoo.make_input((7, 784), "uniform")
    (full,) = ref_runner.run_model(model, [x])
    for n in (1, 2, 3):
        group = ReplicaGroup(replicas=[_OracleReplica(model) for _ in range(n)])
        (got,) = group.run([x], gather="host", deadline_s=60)
        assert got.shape == full.shape and np.array_equal(got, full)      # uneven slices, offsets and order
        group.close()
        assert all(r.closed for r in group.replicas)
    with pytest.raises(ValueError):
        ReplicaGroup(replicas=[])


class _QueueingReplica(_OracleReplica):
    """Like CudaReplica's queue: start_async may be called again before the first step is finished."""

    def __init__(self, model):
        super().__init__(model)
        self.queue = []

    def start_async(self, shard):
        self.queue.append([np.asarray(a) for a in shard])

    def finish(self):
        if self.queue:
            self.shard = self.queue.pop(0)
        return super().finish()


def test_replica_group_pipelined_steps_come_back_in_order():
    from oracle import ref_runner
    from webdnn_b200 import zoo
    from webdnn_b200.replicas import ReplicaGroup
    model = zoo.mlp(6)
    xs = [zoo.make_input((6, 784), "uniform", seed=s) for s in (1, 2, 3)]
    want = [ref_runner.run_model(model, [x])[0] for x in xs]
    group = ReplicaGroup(replicas=[_QueueingReplica(model) for _ in range(2)])
    first = group.run_async([xs[0]])
    second = group.run_async([xs[1]])
    with pytest.raises(RuntimeError, match="order"):
        second.result()                      # the older step's result has not been taken yet
    with pytest.raises(RuntimeError, match="in flight"):
        group.run([xs[2]])                   # the synchronous call does not jump the queue
    assert np.array_equal(first.result(deadline_s=60)[0], want[0])
    third = group.run_async([xs[2]])
    assert np.array_equal(second.result()[0], want[1])
    assert np.array_equal(third.result()[0], want[2])
    assert np.array_equal(group.run([xs[0]])[0], want[0])     # nothing in flight any more
    group.close()


def test_replica_group_pipelined_step_that_fails_names_the_replica():
    from webdnn_b200 import zoo
    from webdnn_b200.lib import CudaBackendError
    from webdnn_b200.replicas import ReplicaError, ReplicaGroup
    model = zoo.mlp(6)
    x = zoo.make_input((6, 784), "uniform")

    class _FailsLater(_QueueingReplica):
        def finish(self):
            raise CudaBackendError(5, "a bounded device-side wait expired (kernel status 61)")

    group = ReplicaGroup(replicas=[_QueueingReplica(model), _FailsLater(model)])
    pend = group.run_async([x])
    with pytest.raises(ReplicaError) as e:
        pend.result(deadline_s=60)
    assert list(e.value.failures) == [1] and e.value.failures[1].status == 5
    group.close()      # what a caller does after a failed step
    assert all(r.closed for r in group.replicas)


def test_replica_group_names_the_replica_that_failed_or_stalled():
    from webdnn_b200 import zoo
    from webdnn_b200.lib import CudaBackendError
    from webdnn_b200.replicas import ReplicaError, ReplicaGroup
    model = zoo.mlp(6)
    x = zoo.make_input((6, 784), "uniform")
    # an error status while enqueueing (arena budget) on replica 1
    group = ReplicaGroup(replicas=[_OracleReplica(model), _OracleReplica(model, fail="start"), _OracleReplica(model)])
    with pytest.raises(ReplicaError) as e:
        group.run([x])
    assert list(e.value.failures) == [1] and isinstance(e.value.failures[1], CudaBackendError)
    assert e.value.failures[1].status == 3
    # an error status reported at the waiting call (a device wait that ran out) on replica 2
    group = ReplicaGroup(replicas=[_OracleReplica(model), _OracleReplica(model), _OracleReplica(model, fail="finish")])
    with pytest.raises(ReplicaError) as e:
        group.run([x])
    assert list(e.value.failures) == [2] and e.value.failures[2].status == 5
    # a replica that does not answer before the host-side deadline
    group = ReplicaGroup(replicas=[_OracleReplica(model, stall_s=5.0), _OracleReplica(model)])
    with pytest.raises(ReplicaError) as e:
        group.run([x], deadline_s=0.5)
    assert list(e.value.failures) == [0] and isinstance(e.value.failures[0], TimeoutError)


# ---- one process per replica over gloo: a rank whose step failed, and a rank that never arrives ----
def _failing_worker(rank, world, port, mode, queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    import torch.distributed as dist
    from webdnn_b200.replicas import ReplicaError, check_all_ranks_ok
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        dist.barrier()
        if mode == "error":
            # rank 1's step returned an error status; every rank must learn of it before the gather
            err = RuntimeError("WDC_ERR_OOM: arena budget") if rank == 1 else None
            try:
                check_all_ranks_ok(err)
                queue.put((rank, "no error seen"))
            except ReplicaError as e:
                queue.put((rank, sorted(e.failures)))
        else:
            # rank 1 leaves between steps and never joins the next collective: the others' collective ends with
            # the process group's short timeout instead of waiting for ever
            if rank == 1:
                queue.put((rank, "left"))
                return
            try:
                check_all_ranks_ok(None)
                queue.put((rank, "no timeout"))
            except ReplicaError:
                queue.put((rank, "replica error"))
            except Exception as e:       # gloo's timeout / connection-closed error
                queue.put((rank, "collective failed"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("mode", ["error", "absent"])
def test_gloo_ranks_learn_of_a_failed_or_absent_rank(mode):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    if mode == "error":
        assert results == {0: [1], 1: [1]}
    else:
        assert results[1] == "left" and results[0] == "collective failed"
