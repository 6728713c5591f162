"""Load-time graph rewrite for the cuda backend.

``core/modelTransform.ts:7-22`` is the reference's post-decode hook: it receives the backend order,
renames duplicate nodes and carries a TODO for backend-specific transforms.  The cuda backend uses
that hook to fuse epilogues, because ``RunnerImpl.run()`` executes node by node and must stay
unchanged:

* ``Conv`` [+ ``BatchNormalization``] [+ ``Add`` residual] [+ ``Relu``] -> one ``CudaConvFused`` node.
  Bias and the BatchNormalization parameters are folded (in float64, once) into a per-channel
  scale/shift pair stored as new initializers; weights are left untouched.
* ``Gemm`` + ``Relu`` -> ``CudaGemmRelu``.

The private op types are registered like a custom operator (``example/custom_operator/twice.ts``),
the same way the offline WebGL passes rename ``op_type`` to ``ConvReshapeWebGL`` / ``MatMulNT141``.
An intermediate tensor is only fused away when it has exactly one consumer and is not a graph
output.
"""
from __future__ import annotations

import logging
from typing import Dict, List

import numpy as np

from .onnx_io import FLOAT, Model, Node, make_attr, make_tensor
from .operators.base import get_attr_float

logger = logging.getLogger("WebDNN.modelTransform")


def rename_duplicated_node(model: Model) -> None:
    """modelTransform.ts:24-45."""
    used = set()
    for node in model.graph.node:
        orig = node.name or "unnamed"
        if orig in used:
            new = orig + "_"
            while new in used:
                new += "_"
            node.name = new
            used.add(new)
            logger.warning("node name %s is already used: renaming to %s", orig, new)
        else:
            node.name = orig
            used.add(orig)


def find_tensor_release_timing(model: Model, initializer_names) -> Dict[str, List[str]]:
    """modelTransform.ts:52-82: tensor names to dispose right after each node."""
    last: Dict[str, str] = {}
    g = model.graph
    for node in g.node:
        for name in node.input:
            last[name] = node.name
    for name in initializer_names:
        last.pop(name, None)
    for vi in g.input:
        last.pop(vi.name, None)
    for vi in g.output:
        last.pop(vi.name, None)
    timing: Dict[str, List[str]] = {}
    for name, node_name in last.items():
        timing.setdefault(node_name, []).append(name)
    return timing


def _fuse_cuda(model: Model) -> None:
    g = model.graph
    inits = {t.name: t for t in g.initializer}
    graph_outputs = {vi.name for vi in g.output}
    consumers: Dict[str, List[Node]] = {}
    for n in g.node:
        for i in n.input:
            consumers.setdefault(i, []).append(n)

    removed = set()

    def sole_consumer(tensor: str):
        c = consumers.get(tensor, [])
        if len(c) == 1 and tensor not in graph_outputs and id(c[0]) not in removed:
            return c[0]
        return None

    replace_at: Dict[int, Node] = {}  # id(last node of chain) -> fused node
    for n in g.node:
        if id(n) in removed:
            continue
        if n.op_type == "Conv" and len(n.input) >= 2 and n.input[1] in inits:
            if len(n.input) > 2 and n.input[2] not in inits:
                continue
            ch_out = inits[n.input[1]].dims[0]
            bias = inits[n.input[2]].array.astype(np.float64) if len(n.input) > 2 else None
            chain = [n]
            out = n.output[0]
            scale = shift = None
            nxt = sole_consumer(out)
            if (nxt is not None and nxt.op_type == "BatchNormalization" and nxt.input[0] == out
                    and all(p in inits for p in nxt.input[1:5]) and len(nxt.output) == 1):
                gm, bt, mu, var = (inits[p].array.astype(np.float64) for p in nxt.input[1:5])
                eps = float(np.float32(get_attr_float(nxt.attribute, "epsilon", 1e-5)))
                scale = gm / np.sqrt(var + eps)
                shift = bt - mu * scale
                chain.append(nxt)
                out = nxt.output[0]
                nxt = sole_consumer(out)
            if bias is not None:
                shift = bias * scale + shift if scale is not None else bias
            residual = None
            if nxt is not None and nxt.op_type == "Add" and len(nxt.input) == 2 and out in nxt.input:
                other = nxt.input[0] if nxt.input[1] == out else nxt.input[1]
                if other != out and other not in inits:
                    residual = other
                    chain.append(nxt)
                    out = nxt.output[0]
                    nxt = sole_consumer(out)
            relu = False
            if nxt is not None and nxt.op_type == "Relu":
                relu = True
                chain.append(nxt)
                out = nxt.output[0]
            if len(chain) == 1 and bias is None:
                continue  # nothing to fuse
            inputs = [n.input[0], n.input[1]]
            base = n.name or n.output[0]
            if scale is not None:
                nm = f"{base}__cuda_scale"
                g.initializer.append(make_tensor(nm, scale.astype(np.float32).reshape(ch_out)))
                inputs.append(nm)
            if shift is not None:
                nm = f"{base}__cuda_shift"
                g.initializer.append(make_tensor(nm, shift.astype(np.float32).reshape(ch_out)))
                inputs.append(nm)
            if residual is not None:
                inputs.append(residual)
            fused = Node("CudaConvFused", inputs, [out], base,
                         [a for a in n.attribute] + [
                             make_attr("relu", int(relu)), make_attr("has_scale", int(scale is not None)),
                             make_attr("has_shift", int(shift is not None)),
                             make_attr("has_residual", int(residual is not None))])
            for c in chain:
                removed.add(id(c))
            replace_at[id(chain[-1])] = fused
        elif n.op_type == "Gemm":
            nxt = sole_consumer(n.output[0])
            if nxt is not None and nxt.op_type == "Relu":
                fused = Node("CudaGemmRelu", list(n.input), [nxt.output[0]], n.name, list(n.attribute))
                removed.add(id(n))
                removed.add(id(nxt))
                replace_at[id(nxt)] = fused
    new_nodes = []
    for n in g.node:
        if id(n) in replace_at:
            new_nodes.append(replace_at[id(n)])
        elif id(n) not in removed:
            new_nodes.append(n)
    g.node = new_nodes
    # drop initializers nothing references any more (folded bias / BatchNormalization vectors)
    used = {i for n in g.node for i in n.input} | graph_outputs
    g.initializer = [t for t in g.initializer if t.name in used]


def model_transform(model: Model, backend_order) -> None:
    if "cuda" in backend_order:
        _fuse_cuda(model)
    rename_duplicated_node(model)
