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
