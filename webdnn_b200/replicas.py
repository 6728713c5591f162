"""Batch-sharded replicas: the multi-GPU form of the operator-execution path.

Every operator on the path is independent across the batch axis (rows of Gemm/Conv, per-row Softmax, per-(n,c)
pooling; for LSTM the batch is axis 1), so N GPUs run N independent replicas of the same runner on contiguous
slices of the batch.  There is no exchange step inside the graph and therefore no collective on the data path.

Two deployment shapes:
* one process per GPU (``torch.distributed.run``): ``shard_for_rank`` picks this rank's slice, the rank runs its own
  ``load(...)``-ed runner, ``gather_outputs`` concatenates the per-rank results on every rank (host-side
  all-gather; gloo on CPU tensors, so it also runs without GPUs);
* one process, several contexts: ``ReplicaGroup`` owns one ``CudaReplica`` (context + runner + pinned staging) per
  device, enqueues all replicas from one host thread each before it waits for any of them, and concatenates the
  outputs (through the host, or by peer copies into the first device).

Failure handling is host-side: a replica that raises, returns an error status or misses a deadline is named in a
``ReplicaError``; among processes ``check_all_ranks_ok`` makes every rank learn of a failed rank before the gather.
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
        part = a[tuple(idx)]
        # a slice along the leading axis is contiguous already: keep the view (and with it the page-locked
        # property of an array that came from WebDNNCudaContext.pinned_array)
        out.append(part if part.flags["C_CONTIGUOUS"] else np.ascontiguousarray(part))
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


class ReplicaError(RuntimeError):
    """One or more replicas failed (an error status from the device library, an exception in an operator) or missed
    the deadline.  ``failures`` maps the replica index to the exception (``TimeoutError`` for a missed deadline)."""

    def __init__(self, failures):
        self.failures = dict(failures)
        parts = [f"replica {i}: {type(e).__name__}: {e}" for i, e in sorted(self.failures.items())]
        super().__init__("; ".join(parts))


def check_all_ranks_ok(local_error: Optional[BaseException], group=None) -> None:
    """One process per GPU: every rank reports whether its replica's step succeeded (host-side all-gather of one
    integer) and every rank raises ``ReplicaError`` naming the failed ranks, so that no rank goes on to gather
    slices that do not exist.  A rank that never arrives ends the collective with the process group's timeout,
    which the caller sees as the backend's own exception."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    flags = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(flags, torch.tensor([0 if local_error is None else 1], dtype=torch.int64), group=group)
    failed = [r for r, f in enumerate(flags) if int(f.item()) != 0]
    if failed:
        me = dist.get_rank(group)
        raise ReplicaError({r: (local_error if r == me else RuntimeError("reported a failed step")) for r in failed})


class CudaReplica:
    """One context + runner on one device.  ``start(shard)`` enqueues the replica's whole step without waiting for
    the GPU: the shard is copied into pinned staging memory, moved on the context's copy stream
    (wdc_upload_async) and run (as a replayed CUDA graph from the third step of a given shape on, when
    ``graph_replay``); ``finish()`` waits and returns host arrays; ``finish_on_device()`` returns the device
    tensors for a peer gather.  Steps are queued: ``start_async(shard)`` also enqueues the device-to-host transfer of
    the outputs (on the download stream, into page-locked staging), so that a second step may be started before the
    first is finished; ``finish()`` always answers the oldest step."""

    MAX_IN_FLIGHT = 2          # steps started and not yet finished (staging buffers are double-buffered)

    def __init__(self, source, device: int, graph_replay: bool = True):
        from .backend import WebDNNCudaContext
        from .runner import load
        self.device = device
        self.context = WebDNNCudaContext(device=device)
        self.context.initialize()
        self.runner = load(source, backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": self.context}})
        self.graph_replay = graph_replay
        self._pinned = {}       # (input index, shape, dtype) -> [pinned staging arrays, next index]
        self._captured = {}     # shape signature -> CapturedRun
        self._seen = {}
        self._queue = []        # steps in flight, oldest first

    def _stage(self, j: int, a: np.ndarray):
        from .backend import CPUTensor
        if getattr(a, "_wdc_pinned", False) and a.flags["C_CONTIGUOUS"]:
            # the caller's array is page-locked already (WebDNNCudaContext.pinned_array): transfer straight from it
            return CPUTensor(list(a.shape), "int32" if a.dtype == np.int32 else "float32", a)
        key = (j, a.shape, a.dtype.str)
        ring = self._pinned.setdefault(key, [[], 0])
        if len(ring[0]) < self.MAX_IN_FLIGHT + 1:      # one more than the steps in flight: never the one in transfer
            ring[0].append(self.context.pinned_array(a.shape, a.dtype))
            buf = ring[0][-1]
        else:
            ring[1] = (ring[1] + 1) % len(ring[0])
            buf = ring[0][ring[1]]
        buf[...] = a
        return CPUTensor(list(a.shape), "int32" if a.dtype == np.int32 else "float32", buf)

    def start_async(self, shard: Sequence[np.ndarray]) -> None:
        self.start(shard, download=True)

    def start(self, shard: Sequence[np.ndarray], download: bool = False) -> None:
        ctx = self.context
        if len(self._queue) >= self.MAX_IN_FLIGHT:
            raise RuntimeError(f"replica on device {self.device}: {len(self._queue)} steps in flight already")
        host = [self._stage(j, a if isinstance(a, np.ndarray) else np.asarray(a)) for j, a in enumerate(shard)]
        dev_in = [ctx.prefetch_tensor(t) for t in host]
        sig = tuple((tuple(t.dims), t.data_type) for t in host)
        cap = self._captured.get(sig)
        if cap is None and self.graph_replay and self._seen.get(sig, 0) >= 1:
            try:
                cap = self._captured[sig] = self.runner.capture(dev_in)
            except Exception:      # e.g. a node on the cpu backend: this replica keeps running node by node
                self.graph_replay = False
        self._seen[sig] = self._seen.get(sig, 0) + 1
        if cap is not None:
            for dst, src in zip(cap.inputs, dev_in):
                ctx.wait_upload(src)
                ctx._call("wdc_copy", _vp(dst.ptr), _vp(src.ptr), dst.length * 4)
            # The transfer buffers go back to the arena now, BEFORE the graph is queued: the arena hands a freed block
            # to another stream only behind everything queued up to the free, so a block freed after the launch
            # would make the next step's transfer (copy stream) wait for this step's whole graph.
            for t in dev_in:
                t.dispose()
            dev_in = []
            cap.launch()
            outs, owned = list(cap.outputs), False
        else:
            outs, owned = self.runner.run(dev_in, outputs_on_device=True), True
        # (a captured run's output buffers are written again by the next replay: their transfer is queued now, in
        # stream order, when the caller wants to start another step before finishing this one)
        downloads = [ctx.download_async(o) for o in outs] if download else None
        self._queue.append((dev_in, outs, owned, downloads))

    def finish_on_device(self):
        """(device tensors in canonical layout, release callback)."""
        dev_in, outs, owned, downloads = self._queue.pop(0)
        if downloads is not None:
            raise RuntimeError("this step was started with start_async: finish() has its outputs")
        canon = [self.context.canonical(o) for o in outs]

        def release():
            for c, o in zip(canon, outs):
                if c is not o:
                    c.dispose()
                if owned:
                    o.dispose()
            for t in dev_in:
                t.dispose()
        return canon, release

    def finish(self) -> List[np.ndarray]:
        if self._queue and self._queue[0][3] is not None:
            dev_in, outs, owned, downloads = self._queue.pop(0)
            try:
                return [d.result().reshape(o.dims) for d, o in zip(downloads, outs)]
            finally:
                if owned:
                    for o in outs:
                        o.dispose()
                for t in dev_in:
                    t.dispose()
        canon, release = self.finish_on_device()
        try:
            return [c.get_data().reshape(c.dims) for c in canon]
        finally:
            release()

    def close(self) -> None:
        for cap in self._captured.values():
            cap.dispose()
        self._captured.clear()
        self.runner.dispose()
        self.context.close()


def _vp(ptr: int):
    from ctypes import c_void_p
    return c_void_p(ptr)


class ReplicaGroup:
    """N replicas on N devices inside one process.  ``run`` slices the batch, lets one host thread per replica
    enqueue that replica's step (so the per-node host work of the replicas overlaps; the device library releases the
    interpreter lock inside its calls), then gathers.  ``replicas`` may be given instead of ``source``/``devices``:
    any objects with ``start(shard)``, ``finish() -> [ndarray]`` and ``close()`` (the CPU tests pass stand-ins
    that compute with the oracle, fail, or stall)."""

    def __init__(self, source=None, devices: Sequence[int] = (), batch_axis: int = 0,
                 output_axes: Optional[Sequence[int]] = None, replicas: Optional[Sequence[object]] = None,
                 graph_replay: bool = True):
        self.batch_axis = batch_axis
        self.output_axes = output_axes
        if replicas is not None:
            self.replicas = list(replicas)
        else:
            self.replicas = [CudaReplica(source, d, graph_replay) for d in devices]
        if not self.replicas:
            raise ValueError("ReplicaGroup needs at least one replica")
        self.contexts = [getattr(r, "context", None) for r in self.replicas]
        self.runners = [getattr(r, "runner", None) for r in self.replicas]

    def _on_threads(self, fn, deadline_s: Optional[float]):
        """fn(i, replica) on one thread per replica; collects results, exceptions and missed deadlines."""
        import threading
        import time
        n = len(self.replicas)
        results, errors = [None] * n, {}

        def work(i):
            try:
                results[i] = fn(i, self.replicas[i])
            except BaseException as e:   # reported to the caller with the replica's index
                errors[i] = e

        threads = [threading.Thread(target=work, args=(i,), daemon=True) for i in range(n)]
        t_end = None if deadline_s is None else time.monotonic() + deadline_s
        for t in threads:
            t.start()
        for i, t in enumerate(threads):
            t.join(None if t_end is None else max(t_end - time.monotonic(), 0.0))
            if t.is_alive():
                errors[i] = TimeoutError(f"no answer within {deadline_s} s")
        if errors:
            raise ReplicaError(errors)
        return results

    def run(self, inputs: Sequence[np.ndarray], gather: str = "host", deadline_s: Optional[float] = None) -> List[np.ndarray]:
        """``gather="host"``: every replica copies its output slice to the host.  ``gather="peer"``: the slices are
        first collected on the first device by peer copies over NVLink (batch axis 0 only: a replica's slice is
        then one contiguous range) and leave in one device-to-host transfer.  ``deadline_s`` bounds each of the two
        phases on the host; a replica that fails or stalls raises ``ReplicaError`` naming it (a stalled replica's
        thread is abandoned, the group should then be closed)."""
        if gather not in ("host", "peer"):
            raise ValueError("gather must be 'host' or 'peer'")
        if getattr(self, "_started", 0) != getattr(self, "_finished", 0):
            raise RuntimeError("steps started by run_async are still in flight: take their results first")
        n = len(self.replicas)
        shards = [shard_for_rank(inputs, i, n, self.batch_axis) for i in range(n)]
        self._on_threads(lambda i, r: r.start(shards[i]), deadline_s)      # enqueue everything first
        if gather == "host":
            return self._finish_host(deadline_s)
        pending = [r.finish_on_device() for r in self.replicas]
        n_out = len(pending[0][0])
        axes = self.output_axes or [self.batch_axis] * n_out
        if any(a != 0 for a in axes):
            for _, release in pending:
                release()
            raise ValueError("gather='peer' needs outputs sharded along axis 0")
        ctx0 = self.contexts[0]
        results = []
        for j in range(n_out):
            parts = [canon[j] for canon, _ in pending]
            dims = [sum(p.dims[0] for p in parts)] + list(parts[0].dims[1:])
            whole = ctx0.empty_tensor(dims, parts[0].data_type)
            off = 0
            for ctx, p in zip(self.contexts, parts):
                ctx0.peer_copy_from(whole, off, ctx, p, p.length)
                off += p.length
            results.append(whole.get_data().reshape(dims))
            whole.dispose()
        for _, release in pending:
            release()
        return results

    def run_async(self, inputs: Sequence[np.ndarray], deadline_s: Optional[float] = None) -> "PendingGroupRun":
        """Starts a step on every replica (slice, transfer, run, and the transfer of the outputs back, all queued)
        and returns without waiting for the GPUs; ``PendingGroupRun.result()`` waits and concatenates through the
        host.  Up to two steps may be in flight; their results are taken in the order they were started.  With page-
        locked inputs (``WebDNNCudaContext.pinned_array``) the transfer of step i + 1 overlaps the GPUs' work on
        step i."""
        n = len(self.replicas)
        shards = [shard_for_rank(inputs, i, n, self.batch_axis) for i in range(n)]
        self._on_threads(lambda i, r: getattr(r, "start_async", r.start)(shards[i]), deadline_s)
        self._started = getattr(self, "_started", 0) + 1
        return PendingGroupRun(self, self._started)

    def _finish_host(self, deadline_s: Optional[float]) -> List[np.ndarray]:
        per_replica = self._on_threads(lambda i, r: r.finish(), deadline_s)
        axes = self.output_axes or [self.batch_axis] * len(per_replica[0])
        return [np.concatenate([rep[j] for rep in per_replica], axis=axes[j]) for j in range(len(per_replica[0]))]

    def close(self) -> None:
        for r in self.replicas:
            r.close()


class PendingGroupRun:
    """A step started by ``ReplicaGroup.run_async``."""

    def __init__(self, group: ReplicaGroup, seq: int):
        self.group, self.seq = group, seq

    def result(self, deadline_s: Optional[float] = None) -> List[np.ndarray]:
        g = self.group
        if self.seq != getattr(g, "_finished", 0) + 1:
            raise RuntimeError("results of pipelined steps are taken in the order the steps were started")
        out = g._finish_host(deadline_s)
        g._finished = self.seq
        return out
