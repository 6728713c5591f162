"""Helpers shared by the tests: golden-case loading, single-op ONNX models, comparisons."""
from __future__ import annotations

import json
import os

import numpy as np

from webdnn_b200 import onnx_io

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def known_answers():
    with open(os.path.join(GOLDEN_DIR, "reference_known_answers.json")) as f:
        return json.load(f)


_cases = None


def torch_cases():
    """name -> dict(op, attrs, inputs[list], outputs[list]) from tests/golden/torch_cases.npz."""
    global _cases
    if _cases is None:
        z = np.load(os.path.join(GOLDEN_DIR, "torch_cases.npz"))
        meta = json.loads(bytes(z["__meta__"]).decode("utf-8"))
        _cases = {}
        for name, m in meta.items():
            _cases[name] = dict(op=m["op"], attrs=m["attrs"],
                                inputs=[z[f"{name}/in{i}"] for i in range(m["n_in"])],
                                outputs=[z[f"{name}/out{i}"] for i in range(m["n_out"])])
    return _cases


def single_op_model(op, attrs, inputs, n_out=1, n_graph_inputs=None, opset=13):
    """One-node model. The first ``n_graph_inputs`` arrays are graph inputs, the rest initializers
    (int64 initializers for shape-like operands)."""
    attrs = dict(attrs)
    opset = attrs.pop("_opset", opset)
    if n_graph_inputs is None:
        n_graph_inputs = len(inputs)
    names = [f"input_{i}" for i in range(len(inputs))]
    outs = [f"output_{i}" for i in range(n_out)]
    node = onnx_io.make_node(op, names, outs, name=f"{op}_0", **attrs)
    g = onnx_io.Graph("g", [node], [], [], [])
    for i, (n, a) in enumerate(zip(names, inputs)):
        a = np.asarray(a)
        if i < n_graph_inputs:
            et = onnx_io.FLOAT if a.dtype == np.float32 else onnx_io.INT32
            g.input.append(onnx_io.ValueInfo(n, et, list(a.shape)))
        else:
            g.initializer.append(onnx_io.make_tensor(n, a))
    for o in outs:
        g.output.append(onnx_io.ValueInfo(o, onnx_io.FLOAT, []))
    return onnx_io.Model(g, opset_import=[("", opset)])


def max_err_rel_linf(actual, expected) -> float:
    """max |a - e| / ||e||_inf  (the parity metric: <= 1e-4 for float outputs)."""
    a = np.asarray(actual, np.float64).reshape(-1)
    e = np.asarray(expected, np.float64).reshape(-1)
    assert a.shape == e.shape, (a.shape, e.shape)
    if e.size == 0:
        return 0.0
    assert np.array_equal(np.isnan(a), np.isnan(e)), "NaN pattern differs"
    m = ~np.isnan(e)
    if not m.any():
        return 0.0
    inf_e = np.isinf(e[m])
    assert np.array_equal(a[m][inf_e], e[m][inf_e]), "infinities differ"
    fin = ~inf_e
    if not fin.any():
        return 0.0
    scale = np.abs(e[m][fin]).max()
    d = np.abs(a[m][fin] - e[m][fin]).max()
    return float(d / scale) if scale > 0 else float(d)


def run_cuda(model, inputs, ctx, return_runner=False):
    """Run a model through the shipped runner on the cuda backend; returns numpy outputs."""
    from webdnn_b200.backend import CPUTensor
    from webdnn_b200.runner import load
    runner = load(model, backend_order=["cuda", "cpu"], backend_options={"cuda": {"context": ctx}})
    outs = runner.run([CPUTensor.from_array(np.asarray(a)) for a in inputs])
    res = [o.numpy().copy() for o in outs]
    if return_runner:
        return res, runner
    runner.dispose()
    return res
