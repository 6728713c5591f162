"""Benchmark of the operator-execution path: ResNet-50 v1.5 fp32 inference through runner.run().

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One "step" is one runner.run() over a batch of B synthetic images (default 256, the configuration
the metric is quoted on).  With N > 1 (launched by torch.distributed.run, one process per GPU) every
rank runs an independent replica on its own batch of B images: no collective is on the data path;
torch.distributed is used only for the barrier and the max-over-ranks of the timings.

Printed keys: `value` = images/s with the input batch already resident in HBM (device time, CUDA
events on the backend's stream); `e2e` = images/s through the public API with the batch in pinned
host memory (H2D of the inputs and D2H of the result inside the timed region); `roofline` = the
contraction kernels' algorithmic TFLOP/s against a cuBLAS TF32 matmul measured in the same process;
`cpu_baseline` = the CPU oracle (a port of the reference's cpu backend) on a bounded sample.
Inputs (154 MB per batch) and activations (GBs) exceed the 126 MB L2, so no explicit flush is needed.
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
# dram__bytes_read.sum + dram__bytes_write.sum of the 54 tc_igemm launches of one batch-256 step, divided by 54
# (profiles/resnet50_b256_contraction_dram_traffic.md); the algorithmic bytes of the same launches are 28.06 GB.
CONTRACTION_DRAM_BYTES_PER_LAUNCH_B256 = 25.166e9 / 54


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


def measure_tf32_peak(device: int) -> float:
    """cuBLAS TF32 8192^3 matmul, best of 10, TFLOP/s: the denominator of the tensor roofline."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
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
        del a, b
        torch.cuda.empty_cache()
    return 2 * 8192 ** 3 / (best * 1e-3) / 1e12


def cpu_port_images_per_sec(n_images: int):
    """Times the CPU oracle (port of the reference's cpu backend) on ResNet-50, batch n_images."""
    from oracle import ops, ref_runner
    from webdnn_b200 import zoo
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host thread it can
    ops.set_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    model = zoo.resnet50(n_images)
    x = zoo.make_input((n_images, 3, 224, 224))
    t0 = time.perf_counter()
    ref_runner.run_model(model, [x])
    dt = time.perf_counter() - t0
    return n_images / dt, ops.num_threads(), dt


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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"ResNet-50 v1.5 [B,3,224,224] fp32, B={args.batch} (CPU arm: bounded sample)"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is TypeScript and cannot run here (no Node.js); this is the C restatement of its "
                "cpu backend (oracle/cpu_ops.c), OpenMP over independent outputs",
    }), file=RESULT_OUT, flush=True)


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch

    from webdnn_b200 import zoo
    from webdnn_b200.backend import CPUTensor, WebDNNCudaContext
    from webdnn_b200.runner import load

    dist = None
    affinity = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        affinity = bind_to_gpu_cpus(local_rank)
        # NCCL's own log lines (its version banner, NCCL_DEBUG output) go to stderr: stdout carries the JSON line only
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))

    B = args.batch
    ctx = WebDNNCudaContext(device=local_rank)
    ctx.initialize()
    model = zoo.resnet50(B)
    flops_per_step = zoo.contraction_flops(model, {"input": [B, 3, 224, 224]})
    runner = load(model, backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": ctx}})
    x_pinned = ctx.pinned_array((B, 3, 224, 224), np.float32)
    x_pinned[...] = zoo.make_input((B, 3, 224, 224), seed=1 + rank)
    x_host = CPUTensor([B, 3, 224, 224], "float32", x_pinned)
    x_dev = ctx.move_tensor(x_host)
    stream = torch.cuda.ExternalStream(ctx.stream_handle(), device=f"cuda:{local_rank}")

    def barrier():
        if dist is not None:
            dist.barrier()
        ctx.sync()
        torch.cuda.synchronize(local_rank)

    def device_step():
        outs = runner.run([x_dev], outputs_on_device=True)
        for o in outs:
            o.dispose()

    def e2e_steps(n):
        """n end-to-end steps through the public API: every step's batch goes host -> device
        (ctx.prefetch_tensor, from pinned memory, on the copy stream) and its result device -> host
        (runner.run returns CPU tensors).  The transfer of batch i+1 is queued before the kernels of
        batch i, so the two overlap; nothing is reused between steps."""
        out = None
        nxt = ctx.prefetch_tensor(x_host)
        for i in range(n):
            cur = nxt
            nxt = ctx.prefetch_tensor(x_host) if i + 1 < n else None
            out = runner.run([cur])
            cur.dispose()
        return out

    for _ in range(max(args.warmup, 3)):
        device_step()
    e2e_steps(max(args.warmup, 3))
    assert not runner.nodes_on("cpu"), runner.nodes_on("cpu")

    tf32_peak = measure_tf32_peak(local_rank) if rank == 0 else None

    sampler = ClockSampler(local_rank)
    # ---- device-resident timing (value) with per-launch contraction timing for the roofline
    barrier()
    sampler.start()
    ctx.reset_stats()
    ctx.profile_enable(True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        device_step()
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = ctx.stats()["launches"]
    k_ms, k_launches, k_flops = ctx.profile_read()
    ctx.profile_enable(False)

    # ---- end-to-end timing (e2e): pinned host input -> H2D -> all nodes -> D2H of the softmax
    barrier()
    ctx.reset_stats()
    t0 = time.perf_counter()
    ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev2.record(stream)
    out = e2e_steps(args.steps)
    ev3.record(stream)
    barrier()
    e2e_ms = max((time.perf_counter() - t0) * 1e3, ev2.elapsed_time(ev3))
    st = ctx.stats()
    clocks = sampler.stop()
    checksum = float(out[0].numpy().sum())

    if dist is not None:
        t = torch.tensor([dev_ms, e2e_ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()

    if rank == 0:
        value = world * B * args.steps / (dev_ms * 1e-3)
        e2e_value = world * B * args.steps / (e2e_ms * 1e-3)
        achieved = k_flops / (k_ms * 1e-3) / 1e12 if k_ms > 0 else 0.0
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"ResNet-50 v1.5 [B,3,224,224] fp32 through runner.run(), B={B} per GPU",
                       "global_batch": B * world, "replicas": world, "cpus_per_rank": affinity,
                       "l2": "inputs (154 MB) and activations exceed the 126 MB L2; no flush",
                       "precision": os.environ.get("WDC_PRECISION", "default")},
            "e2e": {"value": e2e_value, "unit": "images/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": st["h2d_bytes"] // args.steps,
                    "d2h_bytes_per_step": st["d2h_bytes"] // args.steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": achieved / tf32_peak if tf32_peak else None,
                         "traffic": CONTRACTION_DRAM_BYTES_PER_LAUNCH_B256 if B == 256 else None,
                         "traffic_unit": "bytes of DRAM read + written per launch, average over the step's 54 "
                                         "contraction launches (one ncu capture at batch 256, see profiles/)",
                         "kernel": "Conv/Gemm contraction launches (wdc_conv2d, wdc_gemm)",
                         "launches": int(k_launches), "kernel_ms_per_step": k_ms / args.steps,
                         "algorithmic_flops_per_step": flops_per_step,
                         "peak_source": "cuBLAS TF32 8192^3 torch.matmul measured in this run (best of 10)"},
            "output_checksum": checksum,
        }
        if world == 1 and not args.no_cpu:
            v, cores, dt = cpu_port_images_per_sec(args.cpu_images)
            line["cpu_baseline"] = {"value": v, "unit": "images/s", "cores": cores, "kind": "port",
                                    "sample": f"{args.cpu_images} images of the same network and init, {dt:.1f} s"}
        print(json.dumps(line), file=RESULT_OUT, flush=True)
    x_dev.dispose()
    runner.dispose()
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
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
