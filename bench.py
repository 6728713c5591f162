"""Benchmark of the operator-execution path: ResNet-50 v1.5 fp32 inference through runner.run().

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One "step" is one pass over a GLOBAL batch of B synthetic images (default 256, the configuration the metric is
quoted on).  With N > 1 (launched by torch.distributed.run, one process per GPU) the batch is split: every rank
runs an independent replica on its B/N images (strong scaling; no collective is on the data path, torch.distributed
is used only for the barrier and the max-over-ranks of the timings).  A rank whose share is at most 32 images runs
its step as a replayed CUDA graph (backendOptions.cuda.graphReplay), larger shares run node by node.

Printed keys: `value` = images/s with the input batch already resident in HBM (device time, CUDA events on the
backend's stream); `e2e` = images/s through the public API with the batch in pinned host memory (H2D of the inputs
and D2H of the result inside the timed region); `roofline` = the contraction kernels' algorithmic TFLOP/s, timed per
launch with CUDA events in a second pass over the same steps, against a cuBLAS TF32 matmul measured in the same
process (burst and sustained); `cpu_baseline` = the CPU oracle (a port of the reference's cpu backend) on a bounded
sample, on all host threads and on one; `weak` (N > 1) = the same with B images on every GPU; `one_process`
(N > 1) = the split batch driven by one process through ReplicaGroup.run with outputs gathered by peer copies;
`configs` / `layers` (N = 1) = the other benchmark configurations and the reference's own operator shapes;
`configs_sharded` = configurations 4 and 5 with their batch split over the N ranks (device time, max over ranks).
No explicit L2 flush: every step streams far more than the 126 MB L2 (at 256 images the input alone is 154 MB; at
the 32 images a GPU gets from a batch split eight ways, a step still walks about 300 MB of weights and their split
copies and over 1 GB of activations), so nothing a step reads at its start is still cached from the step before.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "resnet50_fp32_inference_images_per_sec"
# dram__bytes_read.sum + dram__bytes_write.sum of the contraction launches of one batch-256 step, per launch, from one
# ncu capture of this workload (the algorithmic bytes of the same launches are 28.06 GB per step).
CONTRACTION_DRAM_BYTES_PER_STEP_B256 = 25.38e9
GRAPH_MAX_BATCH = 32     # a rank whose share of the batch is at most this runs its step as a replayed CUDA graph


RESULT_OUT = sys.stdout   # where the JSON line goes; main() re-points it at the process's original stdout


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs: NVML queries from a thread of this
    process every 20 ms (read-only), or, where the NVML binding is missing, lines of ``nvidia-smi -lms``.
    (One nvidia-smi process per rank is too slow to report within a 100 ms region on an 8-GPU box.)"""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []          # nvidia-smi lines
        self.sm, self.mx, self.reasons = [], [], set()
        self.proc = None
        self.thread = None
        self.nvml = None
        self.handle = None
        self.stop_flag = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                import torch
                pr = torch.cuda.get_device_properties(gpu_index)
                bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
                self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _sample_nvml(self):
        n = self.nvml
        try:
            self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
            self.mx.append(float(n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)))
            get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
            mask = int(get(self.handle))
            for name, bit in self.BITS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _loop_nvml(self):
        while not self.stop_flag.is_set():
            self._sample_nvml()
            self.stop_flag.wait(0.02)

    def start(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._loop_nvml, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self._sample_nvml()            # one more sample while the GPU is still warm from the region
            self.stop_flag.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None,
                    "sm_max_mhz": max(self.mx) if self.mx else None, "reasons": sorted(self.reasons),
                    "samples": len(self.sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def bind_to_gpu_cpus(gpu_index: int):
    """Multi-GPU runs: keep this rank's threads, and so the pinned host buffers it allocates, on the CPUs NVML lists
    as local to its GPU (same NUMA node and PCIe root), so that eight ranks' input transfers do not cross sockets.
    Reads the topology only; returns the number of CPUs bound to, or None when NVML or the call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def measure_tf32_peak(device: int, sustained_s: float = 0.0):
    """cuBLAS TF32 8192^3 matmul, TFLOP/s: the denominator of the tensor roofline.  Returns (burst, sustained):
    burst = best of 10 single launches; sustained = back-to-back launches for `sustained_s` seconds (None if 0),
    which is what a kernel timed inside a long, power-capped step should be compared with."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    flop = 2 * 8192 ** 3
    with torch.cuda.device(device):
        a = torch.randn(8192, 8192, device=f"cuda:{device}")
        b = torch.randn(8192, 8192, device=f"cuda:{device}")
        for _ in range(3):
            a @ b
        best = 1e9
        for _ in range(10):
            s, e = torch.cuda.Event(True), torch.cuda.Event(True)
            s.record()
            a @ b
            e.record()
            e.synchronize()
            best = min(best, s.elapsed_time(e))
        sustained = None
        if sustained_s > 0:
            n = max(int(sustained_s / (best * 1e-3)), 10)
            s, e = torch.cuda.Event(True), torch.cuda.Event(True)
            s.record()
            for _ in range(n):
                a @ b
            e.record()
            e.synchronize()
            sustained = flop * n / (s.elapsed_time(e) * 1e-3) / 1e12
        del a, b
        torch.cuda.empty_cache()
    return flop / (best * 1e-3) / 1e12, sustained


def cpu_port_images_per_sec(n_images: int, threads: int = 0):
    """Times the CPU oracle (port of the reference's cpu backend) on ResNet-50, batch n_images, on `threads` host
    threads (0 = every thread this process may use)."""
    from oracle import ops, ref_runner
    from webdnn_b200 import zoo
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host thread it can
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    ops.set_threads(threads if threads > 0 else avail)
    model = zoo.resnet50(n_images)
    x = zoo.make_input((n_images, 3, 224, 224))
    t0 = time.perf_counter()
    ref_runner.run_model(model, [x])
    dt = time.perf_counter() - t0
    return n_images / dt, ops.num_threads(), dt


def cpu_port_seconds(model, inputs) -> float:
    """One run of the CPU oracle on a model (all host threads), seconds."""
    from oracle import ops, ref_runner
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    ops.set_threads(avail)
    t0 = time.perf_counter()
    ref_runner.run_model(model, inputs)
    return time.perf_counter() - t0


def workload_name(batch: int, world: int) -> str:
    split = f"split over {world} GPUs ({batch // world} images each)" if world > 1 else "on one GPU"
    return f"ResNet-50 v1.5 [B,3,224,224] fp32 through runner.run(), global batch B={batch} {split}"


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    n = args.ref_images
    vals = []
    for _ in range(args.warmup):
        cpu_port_images_per_sec(1)
    cores = 1
    t_total = 0.0
    for _ in range(args.steps):
        v, cores, dt = cpu_port_images_per_sec(n)
        vals.append(v)
        t_total += dt
    value = n * args.steps / t_total
    sample = f"{args.steps} steps x {n} images of the batch-{args.batch} workload"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.batch, max(args.gpus, 1)) + " (CPU arm: bounded sample on rank 0)",
                   "global_batch": args.batch},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is TypeScript and cannot run here (no Node.js); this is the C restatement of its "
                "cpu backend (oracle/cpu_ops.c), OpenMP over independent outputs",
    }), file=RESULT_OUT, flush=True)


class ReplicaBench:
    """One replica of the network on this rank's GPU at a fixed per-GPU batch: the device-resident step, the
    end-to-end step through the public API, and (node by node only) the per-launch timing of the contractions."""

    def __init__(self, ctx, batch: int, seed: int, graph: bool):
        from webdnn_b200 import zoo
        from webdnn_b200.backend import CPUTensor
        from webdnn_b200.runner import load
        self.ctx, self.batch, self.graph = ctx, batch, graph
        self.model = zoo.resnet50(batch)
        self.flops_per_step = zoo.contraction_flops(self.model, {"input": [batch, 3, 224, 224]})
        self.runner = load(self.model, backend_order=["cuda", "cpu"],
                           backend_options={"cuda": {"context": ctx, "graphReplay": graph}})
        self.plain = self.runner if not graph else load(
            self.model, backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": ctx, "graphReplay": False}})
        x_pinned = ctx.pinned_array((batch, 3, 224, 224), np.float32)
        x_pinned[...] = zoo.make_input((batch, 3, 224, 224), seed=seed)
        self.x_host = CPUTensor([batch, 3, 224, 224], "float32", x_pinned)
        self.x_dev = ctx.move_tensor(self.x_host)
        self.cap = None

    def warm(self, n: int) -> None:
        for _ in range(n):
            self.node_step()
        if self.graph:
            self.cap = self.runner.capture([self.x_host])     # the recorded run of the device-resident step
            for _ in range(n):
                self.cap.launch()
        self.e2e_steps(max(n, 3))                             # (with graphReplay: records its own graph at step 2)
        assert not self.plain.nodes_on("cpu"), self.plain.nodes_on("cpu")

    def node_step(self) -> None:
        for o in self.plain.run([self.x_dev], outputs_on_device=True):
            o.dispose()

    def device_step(self) -> None:
        if self.cap is not None:
            self.cap.launch()
        else:
            self.node_step()

    def e2e_steps(self, n: int):
        """n end-to-end steps through the public API: every step's batch goes host -> device (ctx.prefetch_tensor,
        from pinned memory, on the copy stream) and its result device -> host (runner.run(..., wait=False) queues the
        kernels and the transfer of the outputs; PendingRun.result() waits for them).  The loop is the one a server
        runs: batch i+1 is on its way and step i+1 is queued before the host reads the result of step i, so neither
        the copies nor the host's enqueueing leave the GPU idle.  Every step's result is read inside the region."""
        ctx = self.ctx
        out = None
        pending = None
        nxt = ctx.prefetch_tensor(self.x_host)
        for i in range(n):
            cur = nxt
            nxt = ctx.prefetch_tensor(self.x_host) if i + 1 < n else None
            p = self.runner.run([cur], wait=False)
            cur.dispose()
            if pending is not None:
                out = pending.result()
            pending = p
        out = pending.result()
        return out

    def h2d_only_ms(self, n: int) -> float:
        """Milliseconds per step of the input transfer alone (pinned host -> device, nothing computing): what the
        host link gives this rank while every rank transfers at once."""
        ctx = self.ctx
        ctx.sync()
        t0 = time.perf_counter()
        for _ in range(n):
            t = ctx.prefetch_tensor(self.x_host)
            ctx.wait_upload(t)
            t.dispose()
        ctx.sync()
        return (time.perf_counter() - t0) * 1e3 / n

    def launches_per_step(self) -> int:
        self.ctx.sync()
        before = self.ctx.stats()["launches"]
        self.node_step()
        return int(self.ctx.stats()["launches"] - before)

    def close(self) -> None:
        if self.cap is not None:
            self.cap.dispose()
        self.x_dev.dispose()
        self.runner.dispose()
        if self.plain is not self.runner:
            self.plain.dispose()


def one_process_replicas(world: int, batch: int, steps: int, warmup: int) -> dict:
    """The split batch driven by ONE process: ReplicaGroup.run slices the global batch, one host thread per GPU
    enqueues that GPU's replica, the outputs are gathered on the first GPU by peer copies over NVLink
    (wdc_peer_copy) and leave in one device-to-host transfer.  Wall clock around whole run() calls (host inputs in,
    host outputs out), so it is an end-to-end figure."""
    from webdnn_b200 import zoo
    from webdnn_b200.replicas import ReplicaGroup
    model = zoo.resnet50(batch // world)
    t_load = time.perf_counter()
    # every replica replays a recorded graph whatever its share: one interpreter drives all GPUs here, and node by
    # node its per-node work for N replicas would be longer than the GPUs' step
    group = ReplicaGroup(model, devices=list(range(world)), graph_replay=True)
    t_load = time.perf_counter() - t_load
    # the batch sits in page-locked host memory, as in the other end-to-end figure: each replica transfers its
    # slice straight from it (a pageable array would first be copied into the replica's staging buffer)
    x = group.contexts[0].pinned_array((batch, 3, 224, 224), np.float32)
    x[...] = zoo.make_input((batch, 3, 224, 224), seed=1)
    try:
        ref = None
        res = {}
        for gather in ("peer", "host"):
            for _ in range(max(warmup, 3)):
                (out,) = group.run([x], gather=gather)
            t0 = time.perf_counter()
            for _ in range(steps):
                (out,) = group.run([x], gather=gather)
            dt = time.perf_counter() - t0
            res[gather] = {"images_per_s": batch * steps / dt, "ms_per_step": 1e3 * dt / steps}
            if ref is None:
                ref = out
            else:
                res["peer_equals_host_gather"] = bool(np.array_equal(ref, out))
        # the same call pipelined: step i + 1 is started (slice, transfer, run, result transfer all queued) before
        # the result of step i is taken, so the input transfer of one step overlaps the GPUs' work on the other
        pend = group.run_async([x])
        for _ in range(max(warmup, 3)):
            nxt = group.run_async([x])
            (out,) = pend.result()
            pend = nxt
        t0 = time.perf_counter()
        for _ in range(steps):
            nxt = group.run_async([x])
            (out,) = pend.result()
            pend = nxt
        dt = time.perf_counter() - t0
        (out,) = pend.result()
        res["pipelined"] = {"images_per_s": batch * steps / dt, "ms_per_step": 1e3 * dt / steps,
                            "equals_synchronous": bool(np.array_equal(ref, out))}
        res["output_shape"] = list(ref.shape)
        res["load_s"] = t_load
        res["api"] = ("ReplicaGroup.run(inputs, gather='peer'|'host') and ReplicaGroup.run_async(inputs).result(): one "
                      "process, one host thread per GPU")
        return res
    finally:
        group.close()


def other_configs(ctx, tf32_peak: float) -> list:
    """The other benchmark configurations on this GPU (inputs resident, node by node and graph replay) beside one run
    of the CPU port on the same seeded inputs."""
    import config_report
    from webdnn_b200 import zoo
    rows = []
    for name, factory, shapes, kind, items in config_report.CONFIGS:
        if name.startswith("C3") or name.endswith("B=8"):
            continue           # C3 is the headline of this line; C5 at batch 8 is in config_report.py's own table
        r = config_report.measure(ctx, name, factory, shapes, kind, items, reps=5)
        cpu_s = cpu_port_seconds(factory(), [zoo.make_input(sh, kind) for sh in shapes])
        best = r["ms_graph_replay"] if r["ms_graph_replay"] is not None else r["ms_node_by_node"]
        bound = "latency (launches)" if name.startswith("C1") else "serial dependency (us/step)" if name.startswith("C4") \
            else "tensor"
        rows.append({"name": name, "ms_per_run": best, "ms_node_by_node": r["ms_node_by_node"],
                     "ms_graph_replay": r["ms_graph_replay"], "nodes": r["nodes"], "nodes_on_cpu": r["nodes_on_cpu"],
                     "bound": bound, "contraction_tflops": r["tflops_algorithmic"],
                     "contraction_frac_of_tf32_peak": r["tflops_algorithmic"] / tf32_peak if tf32_peak else None,
                     "cpu_port_s_per_run": cpu_s, "speedup_vs_cpu_port": cpu_s * 1e3 / best})
    return rows


SHARDED_CONFIGS = [
    # name, global batch, model factory (per-GPU batch), input shapes (per-GPU batch)
    ("C4 LSTM seq128 in256 hid512", 64, lambda b: __import__("webdnn_b200.zoo", fromlist=["zoo"]).lstm(batch=b),
     lambda b: [(128, b, 256)]),
    ("C5 DETR-style 800x800", 8, lambda b: __import__("webdnn_b200.zoo", fromlist=["zoo"]).detr(batch=b),
     lambda b: [(b, 3, 800, 800)]),
]


def sharded_configs(ctx, stream, rank: int, world: int, barrier, max_over_ranks, reps: int = 10) -> list:
    """Configurations 4 and 5 with their batch split evenly over the ranks (no exchange between them: every rank
    runs its share as a replayed graph, inputs resident).  Timed on the device, barrier on both sides, max over
    ranks; items/s counts the whole batch.  A batch the ranks cannot split evenly is left out."""
    import torch

    from webdnn_b200 import zoo
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.runner import load
    rows = []
    for name, gbatch, factory, shapes_of in SHARDED_CONFIGS:
        if gbatch % world != 0:
            continue
        b = gbatch // world
        # a rank that fails here still meets the others at the barriers; its time is reported as an error
        err, cap, runner = None, None, None
        try:
            runner = load(factory(b), backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": ctx}})
            host = [CPUTensor.from_array(zoo.make_input(sh, "normal", seed=1 + rank)) for sh in shapes_of(b)]
            cap = runner.capture(host)
            for _ in range(3):
                cap.launch()
        except Exception as e:
            err = f"{type(e).__name__}: {e}"
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        if err is None:
            for _ in range(reps):
                cap.launch()
        ev1.record(stream)
        barrier()
        ms, failed = max_over_ranks(ev0.elapsed_time(ev1) / reps, 0.0 if err is None else 1.0)
        if cap is not None:
            cap.dispose()
        if runner is not None:
            runner.dispose()
        if failed:
            rows.append({"name": name, "global_batch": gbatch, "items_per_gpu": b,
                         "error": err or "another rank failed"})
            continue
        rows.append({"name": name, "global_batch": gbatch, "items_per_gpu": b, "ms_per_run": ms,
                     "items_per_s": gbatch / ms * 1e3, "step": "replayed CUDA graph", "reps": reps})
    return rows


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch

    from webdnn_b200.backend import WebDNNCudaContext

    dist = None
    affinity = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        affinity = bind_to_gpu_cpus(local_rank)
        # NCCL's own log lines (its version banner, NCCL_DEBUG output) go to stderr: stdout carries the JSON line only
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        host_group = dist.new_group(backend="gloo")   # host-side barrier for the phase in which rank 0 drives every GPU

    G = args.batch
    if G % world != 0:
        raise SystemExit(f"--batch {G} is not divisible by {world} GPUs")
    B = G // world                                   # this rank's share of every step
    ctx = WebDNNCudaContext(device=local_rank)
    ctx.initialize()
    stream = torch.cuda.ExternalStream(ctx.stream_handle(), device=f"cuda:{local_rank}")
    warm = max(args.warmup, 3)

    def barrier():
        if dist is not None:
            dist.barrier()
        ctx.sync()
        torch.cuda.synchronize(local_rank)

    def max_over_ranks(*vals):
        if dist is None:
            return list(vals)
        t = torch.tensor(list(vals), device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def timed_pair(rb: "ReplicaBench"):
        """(device-resident ms, end-to-end ms, stats of the end-to-end region, last output) for args.steps steps."""
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            rb.device_step()
        ev1.record(stream)
        barrier()
        dev_ms = ev0.elapsed_time(ev1)
        ctx.reset_stats()
        t0 = time.perf_counter()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record(stream)
        out = rb.e2e_steps(args.steps)
        ev3.record(stream)
        barrier()
        e2e_ms = max((time.perf_counter() - t0) * 1e3, ev2.elapsed_time(ev3))
        return dev_ms, e2e_ms, ctx.stats(), out

    rb = ReplicaBench(ctx, B, seed=1 + rank, graph=B <= GRAPH_MAX_BATCH)
    rb.warm(warm)
    launches_per_step = rb.launches_per_step()

    # bring the GPU to its steady clock before anything is timed: a replica has been idle while the host built the
    # model, and 10 steps of a 2 ms graph are over before the clock governor has reacted
    t_spin = time.perf_counter()
    while time.perf_counter() - t_spin < args.spin_up:
        for _ in range(4):
            rb.device_step()
        ctx.sync()

    sampler = ClockSampler(local_rank)
    sampler.start()
    dev_ms, e2e_ms, st, out = timed_pair(rb)
    clocks = sampler.stop()
    checksum = float(out[0].numpy().sum())
    barrier()
    h2d_ms = rb.h2d_only_ms(args.steps)      # every rank at once: the share of the host link a rank really gets

    # ---- the contraction launches one by one (CUDA events around every wdc_conv2d / wdc_gemm launch), node by node,
    # over the same number of steps: the roofline's `achieved`
    barrier()
    ctx.profile_enable(True)
    for _ in range(args.steps):
        rb.node_step()
    k_ms, k_launches, k_flops = ctx.profile_read()
    ctx.profile_enable(False)
    barrier()
    dev_ms, e2e_ms, h2d_ms = max_over_ranks(dev_ms, e2e_ms, h2d_ms)
    # ---- configurations 4 and 5 with their batch split over the ranks (N = 1: the whole batch, the reference point);
    # before the peak measurement below, for the reason given there
    sharded = None
    if not args.no_extra:
        barrier()
        sharded = sharded_configs(ctx, stream, rank, world, barrier, max_over_ranks)
        barrier()

    # the roofline's denominators, measured AFTER the timed regions: seconds of back-to-back cuBLAS GEMMs pull the
    # clock down under the power cap, and a step timed right behind them would pay for it
    tf32_peak = tf32_sustained = None
    if rank == 0:
        tf32_peak, tf32_sustained = measure_tf32_peak(local_rank, sustained_s=4.0 if world == 1 else 0.0)
    barrier()

    # ---- weak scaling beside it (N > 1): the whole batch on every GPU, (the figure of a replica per GPU with a full batch each)
    weak = None
    if world > 1 and not args.no_weak:
        rb.close()
        rb = None
        wb = ReplicaBench(ctx, G, seed=1 + rank, graph=False)
        wb.warm(warm)
        w_dev, w_e2e, _, _ = timed_pair(wb)
        w_dev, w_e2e = max_over_ranks(w_dev, w_e2e)
        wb.close()
        weak = {"scaling": "weak", "images_per_gpu": G, "value": world * G * args.steps / (w_dev * 1e-3),
                "e2e": world * G * args.steps / (w_e2e * 1e-3), "ms_per_step": w_dev / args.steps, "unit": "images/s"}
    if rb is not None:
        rb.close()

    # ---- one process driving all GPUs (rank 0, while the other ranks wait at the barrier)
    one_proc = None
    if world > 1 and not args.no_one_process:
        barrier()
        if rank == 0:
            try:
                one_proc = one_process_replicas(world, G, args.steps, warm)
            except Exception as e:      # reported, never fatal for the line
                one_proc = {"error": f"{type(e).__name__}: {e}"}
        # the other ranks wait on the host (gloo): an NCCL barrier would keep a kernel spinning on the very GPUs
        # rank 0 is timing
        dist.barrier(group=host_group)

    if rank == 0:
        value = G * args.steps / (dev_ms * 1e-3)
        e2e_value = G * args.steps / (e2e_ms * 1e-3)
        achieved = k_flops / (k_ms * 1e-3) / 1e12 if k_ms > 0 else 0.0
        traffic = CONTRACTION_DRAM_BYTES_PER_STEP_B256 * args.steps / k_launches if (B == 256 and k_launches) else None
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(G, world), "global_batch": G, "images_per_gpu": B, "replicas": world,
                       "step": "replayed CUDA graph" if B <= GRAPH_MAX_BATCH else "node by node",
                       "cpus_per_rank": affinity, "precision": ctx.precision,
                       "l2": "no flush: a step streams > 1 GB of weights and activations through the 126 MB L2"},
            "e2e": {"value": e2e_value, "unit": "images/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": world * (st["h2d_bytes"] // args.steps),
                    "d2h_bytes_per_step": world * (st["d2h_bytes"] // args.steps),
                    "h2d_only_ms_per_step": h2d_ms,
                    "h2d_only_gb_per_s": world * (st["h2d_bytes"] // args.steps) / (h2d_ms * 1e-3) / 1e9,
                    "h2d_note": "the input transfer alone, all ranks at once (max over ranks): where this is close to "
                                "e2e.ms_per_step the end-to-end figure is bound by the host link, not by the GPUs"},
            "gpu_launches": int(launches_per_step * args.steps * 2),
            "gpu_launches_note": f"{launches_per_step} kernel launches per step and rank (counted on a node-by-node "
                                 "step); two timed regions of `steps` steps each; a replayed graph issues the same kernels",
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": achieved / tf32_peak if tf32_peak else None,
                         "peak_sustained": tf32_sustained,
                         "frac_of_sustained": achieved / tf32_sustained if tf32_sustained else None,
                         "issue_frac": 3 * achieved / tf32_peak if tf32_peak else None,
                         "issue_frac_note": "3xTF32 issues three MMAs per algorithmic multiply-add, so `frac` "
                                            "(algorithmic) cannot exceed 1/3; `issue_frac` counts the issued MMAs and "
                                            "is the reading in which a 60% tensor-roofline target can be met",
                         "traffic": traffic,
                         "traffic_unit": "bytes of DRAM read + written per contraction launch (one ncu capture of the "
                                         "batch-256 step, averaged over the step's launches)",
                         "kernel": "Conv/Gemm contraction launches (wdc_conv2d, wdc_gemm: tc_igemm_kernel)",
                         "launches": int(k_launches), "kernel_ms_per_step": k_ms / args.steps,
                         "algorithmic_flops_per_step_per_gpu": k_flops / args.steps,
                         "timed": "per launch, CUDA events, node-by-node pass over the same steps right after the timed region",
                         "peak_source": "cuBLAS TF32 8192^3 torch.matmul measured in this run: best of 10 (peak) and "
                                        "back to back for 4 s (peak_sustained, N = 1 only)"},
            "output_checksum": checksum,
        }
        if world > 1:
            # what stops the split batch from scaling linearly, in the line's own numbers: the step is the same 54
            # contraction launches (plus split passes) whatever the share, and each launch has a floor
            step_ms = dev_ms / args.steps
            n_contr = int(k_launches) // max(args.steps, 1)
            line["strong_scaling_limit"] = {
                "images_per_gpu": B, "ms_per_step": step_ms, "kernel_launches_per_step": launches_per_step,
                "contraction_launches_per_step": n_contr,
                "us_per_contraction_launch": 1e3 * step_ms / max(n_contr, 1),
                "note": "per contraction launch a persistent 148-CTA grid has a fixed cost (launch, pipeline fill, the last "
                        "tile's epilogue: about 5 us) and, at this share, 1-3 waves of tiles per launch, so the cost is not "
                        "amortised as it is at 256 images per GPU; a 218 KB / 512-TMEM-column CTA cannot share its SM with "
                        "the next launch's CTA, so programmatic dependent launch hides the launch latency only"}
        if sharded is not None:
            line["configs_sharded"] = sharded
        if weak is not None:
            line["weak"] = weak
        if one_proc is not None:
            line["one_process"] = one_proc
        if world == 1 and not args.no_cpu:
            v, cores, dt = cpu_port_images_per_sec(args.cpu_images)
            v1, _, dt1 = cpu_port_images_per_sec(2, threads=1)
            line["cpu_baseline"] = {"value": v, "unit": "images/s", "cores": cores, "kind": "port",
                                    "sample": f"{args.cpu_images} images of the same network and init, {dt:.1f} s",
                                    "one_thread": {"value": v1, "cores": 1, "sample": f"2 images, {dt1:.1f} s",
                                                   "note": "the reference's JavaScript cpu backend is single-threaded"}}
        if world == 1 and not args.no_extra:
            import layer_bench
            line["configs"] = other_configs(ctx, tf32_peak)
            line["layers"] = layer_bench.reference_shapes_bench(ctx, 20, tf32_peak, 6542.1)
            line["layers_note"] = ("operator shapes of the reference's benchmark list (batch 1, as there); frac_of_peak is "
                                   "against the TF32 peak above (tensor) or the 6542 GB/s measured HBM copy (hbm)")
        print(json.dumps(line), file=RESULT_OUT, flush=True)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-images", type=int, default=64,
                    help="images in the CPU-baseline sample of the default arm (about 10 s of host work)")
    ap.add_argument("--ref-images", type=int, default=16,
                    help="images per step of the reference arm (13 steps of 16 images are about 35 s of host work)")
    ap.add_argument("--spin-up", type=float, default=0.5,
                    help="seconds of untimed steps after the W warm-up steps, so that the clock has settled")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations and the operator shapes (N = 1)")
    ap.add_argument("--no-weak", action="store_true", help="skip the weak-scaling figure (N > 1)")
    ap.add_argument("--no-one-process", action="store_true", help="skip the one-process ReplicaGroup figure (N > 1)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl != "reference" and world != args.gpus and world == 1 and args.gpus > 1:
        # launched without torchrun: re-exec under it
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    # stdout carries the one JSON line and nothing else: whatever libraries print there from native code (NCCL's
    # version banner, for one) is sent to stderr by pointing descriptor 1 at it; the JSON line goes to a duplicate
    # of the original descriptor
    global RESULT_OUT
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
