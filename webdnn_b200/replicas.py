"""Batch-sharded replicas: the multi-GPU form of the operator-execution path.

Every operator on the path is independent across the batch axis (rows of Gemm/Conv, per-row Softmax, per-(n,c)
pooling; for LSTM the batch is axis 1), so N GPUs run N independent replicas of the same runner on contiguous
slices of the batch.  There is no exchange step inside the graph and therefore no collective on the data path.

Two deployment shapes:
* one process per GPU (``torch.distributed.run``): ``shard_for_rank`` picks this rank's slice, the rank runs its own
  ``load(...)``-ed runner, ``gather_outputs`` concatenates the per-rank results on every rank (host-side
  all-gather; gloo on CPU tensors, so it also runs without GPUs);
* one process, several contexts: ``ReplicaGroup`` owns one context + runner per device, enqueues all replicas
  before it waits for any of them, and concatenates the outputs.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np


def slice_bounds(n: int, parts: int, index: int):
    """Contiguous split of n items into `parts` nearly equal slices (the first n % parts get one more)."""
    if parts <= 0 or not 0 <= index < parts:
        raise ValueError("bad replica index")
    base, extra = divmod(n, parts)
    start = index * base + min(index, extra)
    return start, start + base + (1 if index < extra else 0)


def shard_for_rank(inputs: Sequence[np.ndarray], rank: int, world: int, axis: int = 0) -> List[np.ndarray]:
    out = []
    for a in inputs:
        lo, hi = slice_bounds(a.shape[axis], world, rank)
        idx = [slice(None)] * a.ndim
        idx[axis] = slice(lo, hi)
        out.append(np.ascontiguousarray(a[tuple(idx)]))
    return out


def gather_outputs(local: Sequence[np.ndarray], axis: int = 0, group=None) -> List[np.ndarray]:
    """All-gather per-rank output slices (possibly of different lengths) and concatenate along `axis`."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    results = []
    for a in local:
        t = torch.from_numpy(np.ascontiguousarray(a))
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([a.shape[axis]], dtype=torch.int64), group=group)
        parts = []
        for r in range(world):
            shape = list(a.shape)
            shape[axis] = int(sizes[r].item())
            parts.append(torch.empty(shape, dtype=t.dtype))
        dist.all_gather(parts, t, group=group) if len({tuple(p.shape) for p in parts}) == 1 else _gather_uneven(parts, t, group)
        results.append(np.concatenate([p.numpy() for p in parts], axis=axis))
    return results


def _gather_uneven(parts, mine, group) -> None:
    import torch.distributed as dist
    rank = dist.get_rank(group)
    for r, p in enumerate(parts):
        if r == rank:
            p.copy_(mine)
        dist.broadcast(p, src=dist.get_global_rank(group, r) if group is not None else r, group=group)


class ReplicaGroup:
    """N runners on N devices inside one process; batch slices run concurrently on their own streams."""

    def __init__(self, source, devices: Sequence[int], batch_axis: int = 0, output_axes: Optional[Sequence[int]] = None):
        from .backend import WebDNNCudaContext
        from .runner import load
        self.batch_axis = batch_axis
        self.output_axes = output_axes
        self.contexts = []
        self.runners = []
        for d in devices:
            ctx = WebDNNCudaContext(device=d)
            ctx.initialize()
            self.contexts.append(ctx)
            self.runners.append(load(source, backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": ctx}}))

    def run(self, inputs: Sequence[np.ndarray], gather: str = "host") -> List[np.ndarray]:
        """``gather="host"``: every replica copies its output slice to the host.  ``gather="peer"``: the
        slices are first collected on the first device by peer copies over NVLink (batch axis 0 only:
        a replica's slice is then one contiguous range) and leave in one device-to-host transfer."""
        from .backend import CPUTensor
        if gather not in ("host", "peer"):
            raise ValueError("gather must be 'host' or 'peer'")
        n = len(self.runners)
        pending = []
        for i, runner in enumerate(self.runners):  # enqueue everything first: nothing here waits for a GPU
            shard = shard_for_rank(inputs, i, n, self.batch_axis)
            dev_in = [runner.backend_contexts["cuda"].move_tensor(CPUTensor.from_array(a)) for a in shard]
            outs = runner.run(dev_in, outputs_on_device=True)
            pending.append((dev_in, outs))
        axes = self.output_axes or [self.batch_axis] * len(pending[0][1])
        if gather == "peer":
            if any(a != 0 for a in axes):
                raise ValueError("gather='peer' needs outputs sharded along axis 0")
            ctx0 = self.contexts[0]
            results = []
            for j in range(len(pending[0][1])):
                parts = [ctx.canonical(outs[j]) for ctx, (_, outs) in zip(self.contexts, pending)]
                dims = [sum(p.dims[0] for p in parts)] + list(parts[0].dims[1:])
                whole = ctx0.empty_tensor(dims, parts[0].data_type)
                off = 0
                for ctx, p in zip(self.contexts, parts):
                    ctx0.peer_copy_from(whole, off, ctx, p, p.length)
                    off += p.length
                results.append(whole.get_data().reshape(dims))
                whole.dispose()
                for p, (_, outs) in zip(parts, pending):
                    if p is not outs[j]:
                        p.dispose()
            for dev_in, outs in pending:
                for t in list(outs) + list(dev_in):
                    t.dispose()
            return results
        per_output: List[List[np.ndarray]] = []
        for dev_in, outs in pending:               # now drain, replica by replica
            arrays = []
            for o in outs:
                arrays.append(o.get_data().reshape(o.dims))
                o.dispose()
            for t in dev_in:
                t.dispose()
            per_output.append(arrays)
        return [np.concatenate([rep[j] for rep in per_output], axis=axes[j]) for j in range(len(per_output[0]))]

    def close(self) -> None:
        for r in self.runners:
            r.dispose()
        for c in self.contexts:
            c.close()
