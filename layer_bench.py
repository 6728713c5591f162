"""Times wdc_conv2d on single convolution shapes (the ResNet-50 layers at a given batch), or
wdc_attention on the attention shapes of the DETR-style configuration.

    python layer_bench.py [--batch 256] [--only l4.c2,l1.c3] [--reps 5]
    python layer_bench.py --attention [--batch 8] [--only enc] [--reps 5]
    python layer_bench.py --streaming [--reps 20]     # HBM-bound operators, GB/s of algorithmic bytes

Prints, per layer, the mean device time of the contraction launch (CUDA events recorded by the
library around each launch), algorithmic TFLOP/s, the tensor-issue rate (3 MMAs per algorithmic
multiply-add) and the bytes the layer has to move.  Used to profile one kernel shape under ncu
without running a whole network.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import argparse

import numpy as np

from webdnn_b200.backend import CPUTensor, WebDNNCudaContext
from ctypes import byref, c_void_p

from webdnn_b200.lib import AttentionDesc, ConvDesc

# name, ch_in, ch_out, input size, kernel, stride, pad, residual, occurrences in ResNet-50 v1.5
LAYERS = [
    ("stem 7x7 3->64 s2", 3, 64, 224, 7, 2, 3, 0, 1),
    ("l1.c1 1x1 64->64", 64, 64, 56, 1, 1, 0, 0, 1),
    ("l1.c2 3x3 64->64", 64, 64, 56, 3, 1, 1, 0, 3),
    ("l1.c3 1x1 64->256 +res", 64, 256, 56, 1, 1, 0, 1, 3),
    ("l1.ds 1x1 64->256", 64, 256, 56, 1, 1, 0, 0, 1),
    ("l1.c1b 1x1 256->64", 256, 64, 56, 1, 1, 0, 0, 2),
    ("l2.c1 1x1 256->128 @56", 256, 128, 56, 1, 1, 0, 0, 1),
    ("l2.c2 3x3 128->128 s2", 128, 128, 56, 3, 2, 1, 0, 1),
    ("l2.c2b 3x3 128->128", 128, 128, 28, 3, 1, 1, 0, 3),
    ("l2.c3 1x1 128->512 +res", 128, 512, 28, 1, 1, 0, 1, 4),
    ("l2.ds 1x1 256->512 s2", 256, 512, 56, 1, 2, 0, 0, 1),
    ("l2.c1b 1x1 512->128", 512, 128, 28, 1, 1, 0, 0, 3),
    ("l3.c1a 1x1 512->256 @28", 512, 256, 28, 1, 1, 0, 0, 1),
    ("l3.c2a 3x3 256->256 s2", 256, 256, 28, 3, 2, 1, 0, 1),
    ("l3.c1 1x1 1024->256", 1024, 256, 14, 1, 1, 0, 0, 5),
    ("l3.c2 3x3 256->256", 256, 256, 14, 3, 1, 1, 0, 5),
    ("l3.c3 1x1 256->1024 +res", 256, 1024, 14, 1, 1, 0, 1, 6),
    ("l3.ds 1x1 512->1024 s2", 512, 1024, 28, 1, 2, 0, 0, 1),
    ("l4.c1a 1x1 1024->512 @14", 1024, 512, 14, 1, 1, 0, 0, 1),
    ("l4.c2a 3x3 512->512 s2", 512, 512, 14, 3, 2, 1, 0, 1),
    ("l4.c1 1x1 2048->512", 2048, 512, 7, 1, 1, 0, 0, 2),
    ("l4.c2 3x3 512->512", 512, 512, 7, 3, 1, 1, 0, 2),
    ("l4.c3 1x1 512->2048 +res", 512, 2048, 7, 1, 1, 0, 1, 3),
    ("l4.ds 1x1 1024->2048 s2", 1024, 2048, 14, 1, 2, 0, 0, 1),
]


# name, query tokens, key tokens, heads, head size, occurrences in the 6 + 6 layer transformer (800x800 input)
ATTENTION = [
    ("enc self 625x625", 625, 625, 8, 32, 6),
    ("dec cross 100x625", 100, 625, 8, 32, 6),
    ("dec self 100x100", 100, 100, 8, 32, 6),
]


def attention_bench(ctx: WebDNNCudaContext, batch: int, only, reps: int) -> None:
    rng = np.random.default_rng(0)
    for name, tq, tk, h, c, count in ATTENTION:
        if only and not any(name.startswith(o) for o in only):
            continue
        dm = h * c
        q, k, v = (ctx.move_tensor(CPUTensor.from_array(rng.standard_normal((batch, t, dm)).astype(np.float32)))
                   for t in (tq, tk, tk))
        y = ctx.empty_tensor([batch, tq, dm])
        d = AttentionDesc(batch=batch, heads=h, tq=tq, tk=tk, dh=c, q_sb=tq * dm, q_sh=c, q_st=dm, k_sb=tk * dm,
                          k_sh=c, k_st=dm, v_sb=tk * dm, v_sh=c, v_st=dm, y_sb=tq * dm, y_sh=c, y_st=dm,
                          scale=c ** -0.5)
        call = lambda: ctx._call("wdc_attention", byref(d), *(c_void_p(t.ptr) for t in (q, k, v, y)))
        for _ in range(2):
            call()
        ctx.profile_enable(True)
        for _ in range(reps):
            call()
        ms, _, fl = ctx.profile_read()
        ctx.profile_enable(False)
        ms /= reps
        flops = fl / reps
        nbytes = 4 * (q.length + k.length + v.length + y.length)
        print(f"{name:22s} batch {batch}: {ms * 1e3:8.1f} us  {flops / ms / 1e9:6.2f} TFLOP/s fp32 algorithmic  "
              f"{nbytes / 1e6:6.1f} MB of operands  x{count}")
        for t in (q, k, v, y):
            t.dispose()


# name, op type, attributes, input shapes, opset, algorithmic bytes as a multiple of the first input's bytes
STREAMING = [
    ("Relu 256 MB", "Relu", {}, [(64, 1024, 1024)], 13, 2.0),
    ("Sigmoid 256 MB", "Sigmoid", {}, [(64, 1024, 1024)], 13, 2.0),
    ("Add 2 x 256 MB", "Add", {}, [(64, 1024, 1024), (64, 1024, 1024)], 13, 3.0),
    ("Add bias [.., 1024] + [1024]", "Add", {}, [(64, 1024, 1024), (1024,)], 13, 2.0),
    ("Softmax rows of 625", "Softmax", {"axis": -1}, [(64, 1000, 625)], 13, 2.0),
    ("Softmax rows of 4096", "Softmax", {"axis": -1}, [(16384, 4096)], 13, 2.0),
    ("LayerNormalization rows of 256", "LayerNormalization", {"axis": -1}, [(262144, 256), (256,), (256,)], 17, 2.0),
    ("LayerNormalization rows of 4096", "LayerNormalization", {"axis": -1}, [(16384, 4096), (4096,), (4096,)], 17, 2.0),
    ("ReduceMean last axis of 1024", "ReduceMean", {"axes": [-1], "keepdims": 1}, [(65536, 1024)], 11, 1.0),
    ("Transpose [64,1024,1024] 0,2,1", "Transpose", {"perm": [0, 2, 1]}, [(64, 1024, 1024)], 13, 2.0),
    ("Transpose heads [8,625,8,32] 0,2,1,3", "Transpose", {"perm": [0, 2, 1, 3]}, [(64, 625, 8, 32)], 13, 2.0),
    ("GlobalAveragePool [256,2048,7,7]", "GlobalAveragePool", {}, [(256, 2048, 7, 7)], 13, 1.0),
]


def streaming_bench(ctx: WebDNNCudaContext, only, reps: int, hbm_peak: float) -> None:
    import time

    from webdnn_b200 import onnx_io
    from webdnn_b200.runner import load
    print("| operator | ms | GB/s of algorithmic bytes | of the measured HBM copy peak |")
    print("|---|---:|---:|---:|")
    for name, op, attrs, shapes, opset, factor in STREAMING:
        if only and not any(name.startswith(o) for o in only):
            continue
        names = [f"in{i}" for i in range(len(shapes))]
        node = onnx_io.make_node(op, names, ["out"], name=op, **attrs)
        g = onnx_io.Graph("g", [node], [], [onnx_io.ValueInfo(n, onnx_io.FLOAT, list(sh)) for n, sh in zip(names, shapes)],
                          [onnx_io.ValueInfo("out", onnx_io.FLOAT, [])])
        runner = load(onnx_io.Model(g, opset_import=[("", opset)]), backend_order=["cuda", "cpu"],
                      backend_options={"cuda": {"context": ctx}})
        dev = []
        for sh in shapes:
            t = ctx.empty_tensor(list(sh))
            ctx._call("wdc_fill_u32", c_void_p(t.ptr), 0x3F000000, t.length)   # 0.5
            dev.append(t)

        def step():
            for o in runner.run(dev, outputs_on_device=True):
                o.dispose()

        for _ in range(3):
            step()
        # a replayed graph where the run can be recorded: short kernels (tens of microseconds) are otherwise timed by
        # the host's per-node work, not by the device
        fn = step
        cap = None
        try:
            cap = runner.capture(dev)
            fn = cap.launch
            for _ in range(3):
                fn()
        except Exception:
            cap = None
        ctx.sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        ctx.sync()
        ms = (time.perf_counter() - t0) / reps * 1e3
        if cap is not None:
            cap.dispose()
        gbs = factor * dev[0].length * 4 / ms / 1e6
        print(f"| {name} | {ms:.3f} | {gbs:.0f} | {gbs / hbm_peak * 100:.0f}% |")
        for t in dev:
            t.dispose()
        runner.dispose()


# The operator shapes of the reference's own benchmark list (example/benchmark/make_models.py:142-162), batch 1
# as there: name, op type, attributes, graph-input shapes, constant (initializer) shapes, opset, algorithmic FLOPs,
# algorithmic bytes (every operand and the result once), bound.
def _conv_ref(cin, cout, k, pad, hw):
    return (f"conv-{cin}-{cout}-{k}-1-{pad} [1,{cin},{hw},{hw}]", "Conv",
            dict(kernel_shape=[k, k], strides=[1, 1], pads=[pad] * 4), [(1, cin, hw, hw)], [(cout, cin, k, k)], 13,
            2 * hw * hw * cout * cin * k * k, 4 * (cin * hw * hw + cout * hw * hw + cout * cin * k * k), "tensor")


def _convt_ref(cin, cout, hw):
    oh = (hw - 1) * 2 + 3
    return (f"convtranspose-{cin}-{cout}-3-2-0 [1,{cin},{hw},{hw}]", "ConvTranspose",
            dict(kernel_shape=[3, 3], strides=[2, 2], pads=[0, 0, 0, 0]), [(1, cin, hw, hw)], [(cin, cout, 3, 3)], 13,
            2 * hw * hw * cin * cout * 9, 4 * (cin * hw * hw + cout * oh * oh + cin * cout * 9), "hbm")


REFERENCE_SHAPES = [
    _conv_ref(64, 64, 3, 1, 56), _conv_ref(256, 64, 1, 0, 56), _conv_ref(128, 128, 3, 1, 28),
    _conv_ref(512, 128, 1, 0, 28), _conv_ref(256, 256, 3, 1, 14), _conv_ref(1024, 256, 1, 0, 14),
    _convt_ref(512, 256, 64), _convt_ref(32, 16, 64),
    ("gemm-1024-2048-4096", "Gemm", {"transB": 1}, [(1024, 4096)], [(2048, 4096), (2048,)], 13,
     2 * 1024 * 2048 * 4096, 4 * (1024 * 4096 + 2048 * 4096 + 1024 * 2048), "tensor"),
    ("gemm-1048576-32-288", "Gemm", {"transB": 1}, [(1048576, 288)], [(32, 288), (32,)], 13,
     2 * 1048576 * 32 * 288, 4 * (1048576 * 288 + 32 * 288 + 1048576 * 32), "hbm"),
    ("matmul-850x1x256-256x2048", "MatMul", {}, [(850, 1, 256), (256, 2048)], [], 13,
     2 * 850 * 256 * 2048, 4 * (850 * 256 + 256 * 2048 + 850 * 2048), "hbm"),
    ("matmul-850x1x2048-2048x256", "MatMul", {}, [(850, 1, 2048), (2048, 256)], [], 13,
     2 * 850 * 256 * 2048, 4 * (850 * 2048 + 256 * 2048 + 850 * 256), "hbm"),
    ("matmul-850x1x2048-c2048x256", "MatMul", {}, [(850, 1, 2048)], [(2048, 256)], 13,
     2 * 850 * 256 * 2048, 4 * (850 * 2048 + 256 * 2048 + 850 * 256), "hbm"),
    ("matmul-8x850x32-8x32x850", "MatMul", {}, [(8, 850, 32), (8, 32, 850)], [], 13,
     2 * 8 * 850 * 850 * 32, 4 * (2 * 8 * 850 * 32 + 8 * 850 * 850), "hbm"),
    ("matmul-8x850x850-8x850x32", "MatMul", {}, [(8, 850, 850), (8, 850, 32)], [], 13,
     2 * 8 * 850 * 850 * 32, 4 * (8 * 850 * 850 + 2 * 8 * 850 * 32), "hbm"),
    ("softmax-8-850-850", "Softmax", {"axis": 2}, [(8, 850, 850)], [], 13, 0, 8 * 8 * 850 * 850, "hbm"),
    ("softmax-8-100-850", "Softmax", {"axis": 2}, [(8, 100, 850)], [], 13, 0, 8 * 8 * 100 * 850, "hbm"),
    ("softmax-8-100-100", "Softmax", {"axis": 2}, [(8, 100, 100)], [], 13, 0, 8 * 8 * 100 * 100, "hbm"),
]


def reference_shapes_bench(ctx: WebDNNCudaContext, reps: int, tf32_peak: float, hbm_peak: float, only=()):
    """Runs every entry of REFERENCE_SHAPES as a one-node model through the runner with resident inputs, node by
    node and as a replayed graph (the better of the two is reported, like the reference's harness reports its
    minimum), and returns one record per entry: microseconds, TFLOP/s, GB/s and the fraction of the bound's peak."""
    import time

    from webdnn_b200 import onnx_io
    from webdnn_b200.runner import load
    rng = np.random.default_rng(0)
    out = []
    for name, op, attrs, in_shapes, const_shapes, opset, flops, nbytes, bound in REFERENCE_SHAPES:
        if only and not any(name.startswith(o) for o in only):
            continue
        in_names = [f"in{i}" for i in range(len(in_shapes))]
        c_names = [f"c{i}" for i in range(len(const_shapes))]
        node = onnx_io.make_node(op, in_names + c_names, ["out"], name=op, **attrs)
        inits = [onnx_io.make_tensor(n, (rng.standard_normal(sh) * 0.05).astype(np.float32))
                 for n, sh in zip(c_names, const_shapes)]
        g = onnx_io.Graph("g", [node], inits, [onnx_io.ValueInfo(n, onnx_io.FLOAT, list(sh)) for n, sh in
                                                zip(in_names, in_shapes)], [onnx_io.ValueInfo("out", onnx_io.FLOAT, [])])
        runner = load(onnx_io.Model(g, opset_import=[("", opset)]), backend_order=["cuda", "cpu"],
                      backend_options={"cuda": {"context": ctx}})
        host = [CPUTensor.from_array(rng.standard_normal(sh).astype(np.float32)) for sh in in_shapes]
        dev = [ctx.move_tensor(t) for t in host]

        def step():
            for o in runner.run(dev, outputs_on_device=True):
                o.dispose()

        def timed(fn):
            for _ in range(3):
                fn()
            ctx.sync()
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            ctx.sync()
            return (time.perf_counter() - t0) / reps * 1e6

        us = timed(step)
        mode = "node by node"
        try:
            cap = runner.capture(host)
            us_g = timed(cap.launch)
            cap.dispose()
            if us_g < us:
                us, mode = us_g, "graph replay"
        except Exception:
            pass
        on_cuda = all(b == "cuda" for _, _, b in runner.node_backends)
        for t in dev:
            t.dispose()
        runner.dispose()
        tf = flops / us / 1e6
        gbs = nbytes / us / 1e3
        frac = tf / tf32_peak if bound == "tensor" else gbs / hbm_peak
        out.append({"name": name, "us": us, "mode": mode, "tflops": tf, "gbs": gbs, "bound": bound, "frac_of_peak": frac,
                    "on_cuda": on_cuda})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=0, help="default 256 (convolutions) or 8 (attention)")
    ap.add_argument("--attention", action="store_true")
    ap.add_argument("--streaming", action="store_true")
    ap.add_argument("--reference-shapes", action="store_true",
                    help="the operator shapes of the reference's benchmark list (example/benchmark/make_models.py)")
    ap.add_argument("--hbm-peak", type=float, default=6542.0, help="GB/s used for the fraction column of --streaming")
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--tf32-peak", type=float, default=752.0, help="TFLOP/s used for the issue-rate column")
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
    if args.attention:
        attention_bench(ctx, args.batch or 8, only, args.reps)
        ctx.close()
        return
    if args.streaming:
        streaming_bench(ctx, only, max(args.reps, 10), args.hbm_peak)
        ctx.close()
        return
    if args.reference_shapes:
        print("| shape | us | mode | TFLOP/s | GB/s | bound | of that peak |")
        print("|---|---:|---|---:|---:|---|---:|")
        for r in reference_shapes_bench(ctx, max(args.reps, 10), args.tf32_peak, args.hbm_peak, only):
            print(f"| {r['name']} | {r['us']:.1f} | {r['mode']} | {r['tflops']:.2f} | {r['gbs']:.0f} | {r['bound']} | "
                  f"{r['frac_of_peak'] * 100:.1f}% |")
        ctx.close()
        return
    B = args.batch or 256
    total = 0.0
    weighted = 0.0
    for name, cin, cout, hw, k, s, pad, res, count in LAYERS:
        if only and not any(name.startswith(o) for o in only):
            continue
        oh = (hw + 2 * pad - k) // s + 1
        x = ctx.empty_tensor([B, cin, hw, hw], layout="nhwc")
        w = ctx.empty_tensor([cout, k, k, cin])
        ctx._call("wdc_fill_u32", x.ptr, 0x3F800000, x.length)   # 1.0
        ctx._call("wdc_fill_u32", w.ptr, 0x3C000000, w.length)   # 2^-7
        sc = ctx.move_tensor(CPUTensor.from_array(np.ones(cout, np.float32)))
        sh = ctx.move_tensor(CPUTensor.from_array(np.zeros(cout, np.float32)))
        y = ctx.empty_tensor([B, cout, oh, oh], layout="nhwc")
        r = ctx.empty_tensor([B, cout, oh, oh], layout="nhwc") if res else None
        d = ConvDesc(batch=B, ch_in=cin, in_h=hw, in_w=hw, ch_out=cout, k_h=k, k_w=k, out_h=oh, out_w=oh,
                     stride_h=s, stride_w=s, pad_t=pad, pad_l=pad, dil_h=1, dil_w=1, group=1, relu=1)
        for _ in range(2):
            ctx.conv2d(d, x, w, sc, sh, r, y)
        ctx.profile_enable(True)
        for _ in range(args.reps):
            ctx.conv2d(d, x, w, sc, sh, r, y)
        ms, _, fl = ctx.profile_read()
        ctx.profile_enable(False)
        ms /= args.reps
        flops = fl / args.reps
        nbytes = 4 * (x.length + y.length * (2 if res else 1) + w.length)
        total += ms
        weighted += ms * count
        print(f"{name:28s} {ms * 1e3:8.1f} us  {flops / ms / 1e9:7.1f} TFLOP/s algorithmic "
              f"({3 * flops / ms / 1e9 / args.tf32_peak * 100:5.1f}% of TF32 issue)  {nbytes / ms / 1e6:7.0f} GB/s "
              f"of algorithmic bytes  x{count}")
        for t in (x, w, sc, sh, y) + ((r,) if r else ()):
            t.dispose()
    print(f"sum {total:.3f} ms; weighted by occurrences in the network {weighted:.3f} ms")
    ctx.close()


if __name__ == "__main__":
    main()
