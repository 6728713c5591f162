"""Load-time graph rewrite for the cuda backend.

``core/modelTransform.ts:7-22`` is the reference's post-decode hook: it receives the backend order,
renames duplicate nodes and carries a TODO for backend-specific transforms.  The cuda backend uses
that hook to fuse epilogues, because ``RunnerImpl.run()`` executes node by node and must stay
unchanged:

* ``Conv`` [+ ``BatchNormalization``] [+ ``Add`` residual] [+ ``Relu``] -> one ``CudaConvFused`` node.
  Bias and the BatchNormalization parameters are folded (in float64, once) into a per-channel
  scale/shift pair stored as new initializers; weights are left untouched.
* ``Gemm`` + ``Relu`` -> ``CudaGemmRelu``.
* ``MatMul`` by a constant 2-D matrix + ``Add`` of a constant vector [+ ``Relu`` | + ``Add`` of another
  activation] -> ``CudaMatMulBias`` (bias, Relu and the residual sum move into the contraction's epilogue).
* the decomposed LayerNormalization chain over the last axis (``ReduceMean``, ``Sub``, ``Mul``/``Pow``,
  ``ReduceMean``, ``Add`` epsilon, ``Sqrt``, ``Div``, ``Mul`` gamma, ``Add`` beta) -> ``CudaLayerNorm``.
* ``MatMul``(q, ``Transpose``(k)) [-> ``Mul``/``Div`` by a constant scalar] -> ``Softmax`` over the last
  axis -> ``MatMul``(., v) on rank-3 tensors -> ``CudaAttention``; the head split in front of q, k, v
  (``Reshape`` [b, t, h, c] -> ``Transpose`` 0,2,1,3 -> ``Reshape`` [b*h, t, c]) and the head merge behind the
  result are absorbed as strides when their shapes are constants.

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


def _last_axis_mean(n: Node) -> bool:
    axes = [a for a in n.attribute if a.name == "axes"]
    keep = [a for a in n.attribute if a.name == "keepdims"]
    return (n.op_type == "ReduceMean" and len(n.input) == 1 and len(axes) == 1 and list(axes[0].ints) == [-1]
            and (not keep or keep[0].i == 1))


def _match_layernorm(mean_node: Node, inits, consumers, graph_outputs, removed):
    """Matches the opset-13 export of LayerNormalization over the last axis that starts at
    ``mean_node`` and ends with the affine part; returns (chain in graph order, fused node) or None.
    Every intermediate value must have no consumer outside the chain and must not be a graph output."""
    if not _last_axis_mean(mean_node):
        return None

    def users(t):
        seen, out = set(), []
        for c in consumers.get(t, []):   # a node that takes t twice is listed twice
            if id(c) not in removed and id(c) not in seen:
                seen.add(id(c))
                out.append(c)
        return out

    def internal(t, allowed):
        return t not in graph_outputs and all(any(c is a for a in allowed) for c in users(t))

    x = mean_node.input[0]
    mean = mean_node.output[0]
    sub = users(mean)
    if len(sub) != 1 or sub[0].op_type != "Sub" or list(sub[0].input) != [x, mean] or not internal(mean, sub):
        return None
    sub = sub[0]
    xc = sub.output[0]
    xc_users = users(xc)
    sq = [c for c in xc_users if (c.op_type == "Mul" and list(c.input) == [xc, xc]) or
          (c.op_type == "Pow" and c.input[0] == xc and c.input[1] in inits and inits[c.input[1]].array.size == 1
           and float(inits[c.input[1]].array.reshape(-1)[0]) == 2.0)]
    div = [c for c in xc_users if c.op_type == "Div" and c.input[0] == xc]
    if len(sq) != 1 or len(div) != 1 or not internal(xc, [sq[0], div[0]]):
        return None
    sq, div = sq[0], div[0]
    var = users(sq.output[0])
    if len(var) != 1 or not _last_axis_mean(var[0]) or not internal(sq.output[0], var):
        return None
    var = var[0]
    add = users(var.output[0])
    if len(add) != 1 or add[0].op_type != "Add" or not internal(var.output[0], add):
        return None
    add = add[0]
    eps_name = add.input[1] if add.input[0] == var.output[0] else add.input[0]
    if eps_name not in inits or inits[eps_name].array.size != 1:
        return None
    sqrt = users(add.output[0])
    if len(sqrt) != 1 or sqrt[0].op_type != "Sqrt" or not internal(add.output[0], sqrt):
        return None
    sqrt = sqrt[0]
    if list(div.input) != [xc, sqrt.output[0]] or not internal(sqrt.output[0], [div]):
        return None
    mul = users(div.output[0])
    if len(mul) != 1 or mul[0].op_type != "Mul" or not internal(div.output[0], mul):
        return None
    mul = mul[0]
    gamma = mul.input[1] if mul.input[0] == div.output[0] else mul.input[0]
    addb = users(mul.output[0])
    if gamma not in inits or len(addb) != 1 or addb[0].op_type != "Add" or not internal(mul.output[0], addb):
        return None
    addb = addb[0]
    beta = addb.input[1] if addb.input[0] == mul.output[0] else addb.input[0]
    if beta not in inits:
        return None
    gd, bd = list(inits[gamma].dims), list(inits[beta].dims)
    if len(gd) != 1 or gd != bd:
        return None
    eps = float(np.float32(inits[eps_name].array.reshape(-1)[0]))
    fused = Node("CudaLayerNorm", [x, gamma, beta], [addb.output[0]], mean_node.name or mean,
                 [make_attr("axis", -1), make_attr("epsilon", eps)])
    return [mean_node, sub, sq, var, add, sqrt, div, mul, addb], fused


ATTENTION_HEAD_SIZES = (32, 64)   # head sizes of the fused kernel (wdc_attention)


def _const_ints(name, inits):
    t = inits.get(name)
    if t is None:
        return None
    return [int(v) for v in np.asarray(t.array).reshape(-1)]


def _perm(n: Node):
    a = [a for a in n.attribute if a.name == "perm"]
    return list(a[0].ints) if a else None


def _match_attention(softmax: Node, inits, consumers, producers, graph_outputs, removed):
    """Matches scaled-dot-product attention around a last-axis ``Softmax``; returns (nodes to drop,
    last node of the chain, fused node) or None.  Every intermediate value has exactly one consumer
    and is not a graph output."""
    axis = [a for a in softmax.attribute if a.name == "axis"]
    if not axis or axis[0].i != -1 or len(softmax.input) != 1:
        return None   # the default axis flattens instead (opset < 13); -1 means the same in every opset

    def sole(tensor):
        c = [x for x in consumers.get(tensor, []) if id(x) not in removed]
        return c[0] if len(c) == 1 and tensor not in graph_outputs else None

    def prod(tensor):
        n = producers.get(tensor)
        return n if n is not None and id(n) not in removed and sole(tensor) is not None else None

    chain = [softmax]
    scale = 1.0
    up = prod(softmax.input[0])
    if up is not None and up.op_type in ("Mul", "Div") and len(up.input) == 2:
        a, b = up.input
        const = b if b in inits else (a if a in inits and up.op_type == "Mul" else None)
        if const is None or inits[const].array.size != 1 or inits[const].data_type != FLOAT:
            return None
        c = float(np.float32(np.asarray(inits[const].array).reshape(-1)[0]))
        if up.op_type == "Div":
            if c == 0.0:
                return None
            c = float(np.float32(1.0 / c))
        scale = c
        chain.append(up)
        up = prod(a if const == b else b)
    if up is None or up.op_type != "MatMul" or len(up.input) != 2:
        return None
    qk = up
    chain.append(qk)
    kt = prod(qk.input[1])
    if kt is None or kt.op_type != "Transpose" or _perm(kt) != [0, 2, 1]:
        return None
    chain.append(kt)
    pv = sole(softmax.output[0])
    if pv is None or pv.op_type != "MatMul" or len(pv.input) != 2 or pv.input[0] != softmax.output[0]:
        return None
    chain.append(pv)
    srcs = {"q": qk.input[0], "k": kt.input[0], "v": pv.input[1]}
    if any(t in inits for t in srcs.values()):
        return None

    # head split in front of an operand: Reshape [b, t, h, c] -> Transpose 0,2,1,3 -> Reshape [b*h, t, c]
    split = {}
    for key, t in list(srcs.items()):
        r2 = prod(t)
        if r2 is None or r2.op_type != "Reshape" or len(r2.input) != 2:
            continue
        tr = prod(r2.input[0])
        if tr is None or tr.op_type != "Transpose" or _perm(tr) != [0, 2, 1, 3]:
            continue
        r1 = prod(tr.input[0])
        if r1 is None or r1.op_type != "Reshape" or len(r1.input) != 2:
            continue
        s1, s2 = _const_ints(r1.input[1], inits), _const_ints(r2.input[1], inits)
        if (s1 is None or s2 is None or len(s1) != 4 or len(s2) != 3 or min(s1) <= 0
                or s2 != [s1[0] * s1[2], s1[1], s1[3]] or s1[3] not in ATTENTION_HEAD_SIZES):
            continue
        split[key] = (s1, [r1, tr, r2])
    # the three operands must agree on (batch, heads) to be read through strides
    if (len(split) == 3 and len({(v[0][0], v[0][2], v[0][3]) for v in split.values()}) == 1
            and split["k"][0][1] == split["v"][0][1]):
        for key in ("q", "k", "v"):
            srcs[key] = split[key][1][0].input[0]
            chain.extend(split[key][1])
        b, _, h, dh = split["q"][0]
    else:
        split = {}
        b = h = dh = 0

    out = pv.output[0]
    last = pv
    merged = 0
    if split:
        # head merge behind the result: Reshape [b, h, t, c] -> Transpose 0,2,1,3 -> Reshape [b, t, h*c]
        r1 = sole(out)
        tr = sole(r1.output[0]) if r1 is not None and r1.op_type == "Reshape" and len(r1.input) == 2 else None
        r2 = sole(tr.output[0]) if tr is not None and tr.op_type == "Transpose" and _perm(tr) == [0, 2, 1, 3] else None
        if r2 is not None and r2.op_type == "Reshape" and len(r2.input) == 2:
            s1, s2 = _const_ints(r1.input[1], inits), _const_ints(r2.input[1], inits)
            tq, c = split["q"][0][1], split["q"][0][3]
            if s1 == [b, h, tq, c] and s2 == [b, tq, h * c]:
                chain.extend([r1, tr, r2])
                out, last, merged = r2.output[0], r2, 1
    attrs = [make_attr("scale", scale), make_attr("batch", b), make_attr("heads", h), make_attr("head_size", dh),
             make_attr("merge_heads", merged)]
    fused = Node("CudaAttention", [srcs["q"], srcs["k"], srcs["v"]], [out], qk.name or qk.output[0], attrs)
    return chain, last, fused


def _fuse_cuda(model: Model) -> None:
    g = model.graph
    inits = {t.name: t for t in g.initializer}
    graph_outputs = {vi.name for vi in g.output}
    consumers: Dict[str, List[Node]] = {}
    producers: Dict[str, Node] = {}
    for n in g.node:
        for i in n.input:
            consumers.setdefault(i, []).append(n)
        for o in n.output:
            producers[o] = n

    removed = set()

    def sole_consumer(tensor: str):
        c = consumers.get(tensor, [])
        if len(c) == 1 and tensor not in graph_outputs and id(c[0]) not in removed:
            return c[0]
        return None

    replace_at: Dict[int, Node] = {}  # id(last node of chain) -> fused node
    # attention first: its matcher looks at plain MatMul / Reshape / Transpose nodes on both sides
    for n in g.node:
        if n.op_type == "Softmax" and id(n) not in removed:
            m = _match_attention(n, inits, consumers, producers, graph_outputs, removed)
            if m is not None:
                chain, last, fused = m
                for c in chain:
                    removed.add(id(c))
                replace_at[id(last)] = fused
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
        elif n.op_type == "MatMul" and len(n.input) == 2 and n.input[1] in inits and len(inits[n.input[1]].dims) == 2:
            nxt = sole_consumer(n.output[0])
            if nxt is None or nxt.op_type != "Add" or len(nxt.input) != 2:
                continue
            other = nxt.input[0] if nxt.input[1] == n.output[0] else nxt.input[1]
            n_out = inits[n.input[1]].dims[1]
            if other not in inits or other == n.output[0]:
                continue
            bdims = [d for d in inits[other].dims if d != 1]
            if bdims != [n_out] or inits[other].dims[-1] != n_out:
                continue
            chain = [n, nxt]
            out = nxt.output[0]
            relu = False
            nx2 = sole_consumer(out)
            if nx2 is not None and nx2.op_type == "Relu":
                relu = True
                chain.append(nx2)
                out = nx2.output[0]
            inputs = [n.input[0], n.input[1], other]
            residual = 0
            if not relu:
                # x + linear(...) of a residual block: the sum moves into the contraction's epilogue too (the
                # operator checks at run time that the shapes are equal, and adds separately otherwise)
                nx3 = sole_consumer(out)
                if nx3 is not None and nx3.op_type == "Add" and len(nx3.input) == 2 and out in nx3.input:
                    res = nx3.input[0] if nx3.input[1] == out else nx3.input[1]
                    if res != out and res not in inits and res != n.input[0]:
                        inputs.append(res)
                        residual = 1
                        chain.append(nx3)
                        out = nx3.output[0]
            fused = Node("CudaMatMulBias", inputs, [out], n.name or n.output[0],
                         [make_attr("relu", int(relu)), make_attr("has_residual", residual)])
            for c in chain:
                removed.add(id(c))
            replace_at[id(chain[-1])] = fused
        elif n.op_type == "ReduceMean":
            fused_ln = _match_layernorm(n, inits, consumers, graph_outputs, removed)
            if fused_ln is not None:
                chain, fused = fused_ln
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
