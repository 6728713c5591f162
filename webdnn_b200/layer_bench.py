"""Times wdc_conv2d on single convolution shapes (the ResNet-50 layers at a given batch), or
wdc_attention on the attention shapes of the DETR-style configuration.

    python -m webdnn_b200.layer_bench [--batch 256] [--only l4.c2,l1.c3] [--reps 5]
    python -m webdnn_b200.layer_bench --attention [--batch 8] [--only enc] [--reps 5]
    python -m webdnn_b200.layer_bench --streaming [--reps 20]     # HBM-bound operators, GB/s of algorithmic bytes

Prints, per layer, the mean device time of the contraction launch (CUDA events recorded by the
library around each launch), algorithmic TFLOP/s, the tensor-issue rate (3 MMAs per algorithmic
multiply-add) and the bytes the layer has to move.  Used to profile one kernel shape under ncu
without running a whole network.
"""
from __future__ import annotations

import argparse

import numpy as np

from .backend import CPUTensor, WebDNNCudaContext
from ctypes import byref, c_void_p

from .lib import AttentionDesc, ConvDesc

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

    from . import onnx_io
    from .runner import load
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
        ctx.sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            step()
        ctx.sync()
        ms = (time.perf_counter() - t0) / reps * 1e3
        gbs = factor * dev[0].length * 4 / ms / 1e6
        print(f"| {name} | {ms:.3f} | {gbs:.0f} | {gbs / hbm_peak * 100:.0f}% |")
        for t in dev:
            t.dispose()
        runner.dispose()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=0, help="default 256 (convolutions) or 8 (attention)")
    ap.add_argument("--attention", action="store_true")
    ap.add_argument("--streaming", action="store_true")
    ap.add_argument("--hbm-peak", type=float, default=6542.0, help="GB/s used for the fraction column of --streaming")
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--tf32-peak", type=float, default=752.0, help="TFLOP/s used for the issue-rate column")
    args = ap.parse_args()
    only = [s for s in args.only.split(",") if s]
    ctx = WebDNNCudaContext()
    ctx.initialize()
    if args.attention:
        attention_bench(ctx, args.batch or 8, only, args.reps)
        ctx.close()
        return
    if args.streaming:
        streaming_bench(ctx, only, max(args.reps, 10), args.hbm_peak)
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
