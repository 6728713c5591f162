"""Per-configuration timing table of the cuda backend (the five benchmark configurations).

    python config_report.py [--only C3] [--reps 10]

For every configuration: nodes after the load-time rewrite, nodes placed on the cpu backend (must be
0), milliseconds per ``runner.run()`` with the inputs resident on the device (node by node, host
clock around a synchronised loop), the same as a replayed CUDA graph, host microseconds per node
(node-by-node time minus graph time, divided by the node count), and the contraction launches'
device time (CUDA events around each launch of one node-by-node run, so launch gaps of tiny kernels
are included) with their algorithmic TFLOP/s.  Synthetic seeded inputs; no comparison with
the CPU oracle happens here (the parity tests do that).
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import argparse
import time

from webdnn_b200 import zoo
from webdnn_b200.backend import CPUTensor, WebDNNCudaContext
from webdnn_b200.runner import load

# name, model factory, input shapes (in graph-input order), input kind, items per run
CONFIGS = [
    ("C1 MLP 784-512-512-10 B=64", lambda: zoo.mlp(64), [(64, 784)], "uniform", 64),
    ("C2 Conv3x3+BN+Relu [32,64,56,56]", lambda: zoo.conv_bn_relu(32), [(32, 64, 56, 56)], "normal", 32),
    ("C3 ResNet-50 B=1", lambda: zoo.resnet50(1), [(1, 3, 224, 224)], "normal", 1),
    ("C3 ResNet-50 B=32", lambda: zoo.resnet50(32), [(32, 3, 224, 224)], "normal", 32),
    ("C3 ResNet-50 B=256", lambda: zoo.resnet50(256), [(256, 3, 224, 224)], "normal", 256),
    ("C4 LSTM seq128 B=64 in256 hid512", lambda: zoo.lstm(), [(128, 64, 256)], "normal", 64),
    ("C5 DETR-style 800x800 B=1", lambda: zoo.detr(batch=1), [(1, 3, 800, 800)], "normal", 1),
    ("C5 DETR-style 800x800 B=8", lambda: zoo.detr(batch=8), [(8, 3, 800, 800)], "normal", 8),
]


def _timed(fn, ctx, reps: int) -> float:
    ctx.sync()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    ctx.sync()
    return (time.perf_counter() - t0) / reps * 1e3


def measure(ctx, name, factory, shapes, kind, items, reps: int = 10) -> dict:
    """One configuration on the cuda backend with resident inputs: node-by-node and graph-replay milliseconds per
    run, node counts, the contraction launches' device time and algorithmic TFLOP/s."""
    model = factory()
    runner = load(model, backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": ctx}})
    host = [CPUTensor.from_array(zoo.make_input(s, kind)) for s in shapes]
    dev = [ctx.move_tensor(t) for t in host]

    def step():
        for o in runner.run(dev, outputs_on_device=True):
            o.dispose()

    for _ in range(3):
        step()
    t_node = _timed(step, ctx, reps)
    ctx.profile_enable(True)
    step()
    ctx.sync()
    k_ms, k_launches, k_flops = ctx.profile_read()
    ctx.profile_enable(False)
    n_nodes = len(runner.node_backends)
    n_cpu = sum(1 for _, _, b in runner.node_backends if b != "cuda")
    t_graph = None
    note = None
    try:
        cap = runner.capture(host)
        for _ in range(3):
            cap.launch()
        t_graph = _timed(cap.launch, ctx, reps)
        cap.dispose()
    except Exception as e:   # a run that cannot be recorded is reported node by node only
        note = f"not captured: {e}"
    for t in dev:
        t.dispose()
    runner.dispose()
    best = t_graph if t_graph is not None else t_node
    return {"name": name, "nodes": n_nodes, "nodes_on_cpu": n_cpu, "ms_node_by_node": t_node, "ms_graph_replay": t_graph,
            "items_per_s": items / best * 1e3, "host_us_per_node": (max(t_node - t_graph, 0.0) / n_nodes * 1e3
                                                                    if t_graph is not None else None),
            "contraction_ms": k_ms, "contraction_launches": int(k_launches), "contraction_flops": k_flops,
            "tflops_algorithmic": k_flops / k_ms / 1e9 if k_ms > 0 else 0.0, "note": note}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="comma-separated name prefixes, e.g. C3,C5")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--split-k", type=int, default=1, help="0: never cut a tile's reduction into ranges")
    ap.add_argument("--pdl", type=int, default=1, help="0: plain stream order between contraction launches")
    ap.add_argument("--precision", default="tf32x3", choices=["tf32x3", "tf32x1"])
    args = ap.parse_args()
    only = [s for s in args.only.split(",") if s]
    ctx = WebDNNCudaContext()
    ctx.initialize()
    ctx.set_option("split_k", args.split_k)
    ctx.set_option("pdl", args.pdl)
    ctx.set_precision(args.precision)
    print("| configuration | nodes | on cpu | ms/run node by node | ms/run graph replay | items/s (best) | host us/node | "
          "contraction ms | TFLOP/s algorithmic |")
    print("|---|---:|---:|---:|---:|---:|---:|---:|---:|")
    for name, factory, shapes, kind, items in CONFIGS:
        if only and not any(name.startswith(o) for o in only):
            continue
        r = measure(ctx, name, factory, shapes, kind, items, args.reps)
        if r["note"]:
            print(f"  ({name}: {r['note']})")
        graph_col = f"{r['ms_graph_replay']:.3f}" if r["ms_graph_replay"] is not None else "n/a"
        host_col = f"{r['host_us_per_node']:.1f}" if r["host_us_per_node"] is not None else "n/a"
        print(f"| {name} | {r['nodes']} | {r['nodes_on_cpu']} | {r['ms_node_by_node']:.3f} | {graph_col} | "
              f"{r['items_per_s']:.0f} | {host_col} | {r['contraction_ms']:.3f} | {r['tflops_algorithmic']:.1f} |")
    ctx.close()


if __name__ == "__main__":
    main()
