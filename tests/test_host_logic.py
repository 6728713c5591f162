"""CPU: host-side logic of the backend mirror (no device): tensors, registry, graph rewrite, runner."""
import numpy as np
import pytest

from webdnn_b200 import onnx_io, zoo
from webdnn_b200.backend import CPUTensor, WebDNNCPUContext
from webdnn_b200.model_transform import find_tensor_release_timing, model_transform
from webdnn_b200.operator_table import OperatorEntry, instantiate_operator, register_operators
from webdnn_b200.operators import base
from webdnn_b200.runner import Runner, load

from util import known_answers, single_op_model


def test_cpu_tensor_semantics_from_reference_unit_test():
    ka = known_answers()["tensor_semantics"]
    t = CPUTensor(ka["dims"], "float32")
    assert t.data.dtype == np.float32 and t.data.size == ka["length"] and not t.data.any()
    assert t.length == ka["length"] and t.ndim == ka["ndim"] and t.strides == ka["strides"]
    buf = np.asarray(ka["data"], np.float32)
    t = CPUTensor(ka["dims"], "float32", buf)
    assert t.use_external_buffer and np.shares_memory(t.data, buf)
    assert t.get_value(ka["get_value"]["index"]) == ka["get_value"]["value"]
    t.set_value(ka["set_value"]["value"], ka["set_value"]["index"])
    assert t.get_value(ka["set_value"]["index"]) == ka["set_value"]["value"]
    assert CPUTensor([2], "int32").data.dtype == np.int32
    assert base.array_prod(known_answers()["array_prod"]["input"]) == known_answers()["array_prod"]["expected"]


def test_shape_math():
    g = base.Gemm("cuda")
    g.initialize([onnx_io.make_attr("transB", 1)])
    assert g.calc_shape([64, 784], [512, 784]) == (64, 512, 784, [784, 1], [1, 784])
    c = base.Conv("cuda")
    c.initialize([onnx_io.make_attr("strides", [2, 2]), onnx_io.make_attr("pads", [3, 3, 3, 3])])
    s = c.calc_shape([1, 3, 224, 224], [64, 3, 7, 7])
    assert s["out_shape"] == [112, 112] and s["kernel_shape"] == [7, 7]
    p = base.MaxPool("cuda")
    p.initialize([onnx_io.make_attr("kernel_shape", [3, 3]), onnx_io.make_attr("strides", [2, 2]),
                  onnx_io.make_attr("ceil_mode", 1)])
    assert p.calc_shape([2, 3, 10, 12])["out_shape"] == [5, 6]
    p.ceil_mode = False
    assert p.calc_shape([2, 3, 10, 12])["out_shape"] == [4, 5]
    m = base.MatMul("cuda")
    r = m.calc_shape([1, 3, 128], [4, 128, 1])
    assert r["result_dims"] == [4, 3, 1] and r["strides_a"][0] == 0
    assert m.calc_shape([128], [128])["result_dims_after_squeeze"] == []
    rs = base.Reshape5("cuda")
    rs.initialize([])
    assert rs.calc_shape(CPUTensor([2, 3, 4]), CPUTensor([3], "int32", np.asarray([0, -1, 2], np.int32))) == [2, 6, 2]
    assert base.squeeze_shape([3, 4, 1, 5, 1, 6], []) == [3, 4, 5, 6]
    assert base.unsqueeze_shape([3, 4], [0, -1]) == [1, 3, 4, 1]
    assert base.broadcast_multi([[2, 3, 10, 12], [1, 3, 1, 12]]) == ([2, 3, 10, 12], [[360, 120, 12, 1], [0, 12, 0, 1]])
    with pytest.raises(ValueError):
        base.broadcast_uni([2, 3], [4])


def test_registry_opset_windows_and_shape_op_placement():
    made = []

    class Op:
        def __init__(self, tag):
            made.append(tag)
            self.tag = tag

    register_operators([
        OperatorEntry("TestSplit", 1, 13, "cuda", lambda: Op("cuda<13")),
        OperatorEntry("TestSplit", 13, None, "cuda", lambda: Op("cuda>=13")),
        OperatorEntry("TestSplit", 1, None, "cpu", lambda: Op("cpu")),
    ])
    assert instantiate_operator("TestSplit", 11, ["cuda", "cpu"], [["cpu"]]).tag == "cuda<13"
    assert instantiate_operator("TestSplit", 13, ["cuda", "cpu"], [["cpu"]]).tag == "cuda>=13"
    assert instantiate_operator("TestSplit", 13, ["cpu"], [["cpu"]]).tag == "cpu"
    assert instantiate_operator("NoSuchOp", 13, ["cuda", "cpu"], [[]]) is None
    # shape-like ops run where the data tensor is; the last backend of the order that holds it wins
    register_operators([OperatorEntry("Pad", 5, None, "cuda", lambda: Op("reshape-cuda")),
                        OperatorEntry("Pad", 5, None, "cpu", lambda: Op("reshape-cpu"))])
    assert instantiate_operator("Pad", 13, ["cuda", "cpu"], [["cuda"], ["cpu"]]).tag == "reshape-cuda"
    assert instantiate_operator("Pad", 13, ["cuda", "cpu"], [["cuda", "cpu"], ["cpu"]]).tag == "reshape-cpu"


def test_cuda_fusion_rewrite_structure_and_numerics():
    m = zoo.resnet50(1, 64, 16, (1, 1, 1, 1), 10)
    n_conv = sum(n.op_type == "Conv" for n in m.graph.node)
    ref = onnx_io.decode_model(onnx_io.encode_model(m))
    model_transform(m, ["cuda", "cpu"])
    types = [n.op_type for n in m.graph.node]
    assert types.count("CudaConvFused") == n_conv
    assert not {"Conv", "BatchNormalization", "Add", "Relu"} & set(types)
    assert types[-4:] == ["GlobalAveragePool", "Flatten", "Gemm", "Softmax"]
    # every input of every node is produced earlier (topological order survives the rewrite)
    known = {vi.name for vi in m.graph.input} | {t.name for t in m.graph.initializer}
    for n in m.graph.node:
        assert all(i in known for i in n.input), n.name
        known.update(n.output)
    # the folded scale/shift equal the BatchNormalization formula
    inits = {t.name: t.array for t in ref.graph.initializer}
    conv0, bn0 = ref.graph.node[0], ref.graph.node[1]
    g, b, mu, var = (inits[x].astype(np.float64) for x in bn0.input[1:5])
    scale = g / np.sqrt(var + float(np.float32(1e-5)))
    new = {t.name: t.array for t in m.graph.initializer}
    fused0 = m.graph.node[0]
    assert np.array_equal(new[fused0.input[2]], scale.astype(np.float32))
    assert np.array_equal(new[fused0.input[3]], (b - mu * scale).astype(np.float32))
    attrs = {a.name: a.i for a in fused0.attribute if a.i is not None}
    assert attrs["relu"] == 1 and attrs["has_scale"] == 1 and attrs["has_residual"] == 0
    res_nodes = [n for n in m.graph.node if n.op_type == "CudaConvFused" and
                 {a.name: a.i for a in n.attribute}.get("has_residual") == 1]
    assert len(res_nodes) == 4  # one residual Add per bottleneck


def test_fusion_respects_graph_outputs_and_fanout():
    m = zoo.conv_bn_relu(1, 8, 6)
    m.graph.output.append(onnx_io.ValueInfo(m.graph.node[0].output[0], onnx_io.FLOAT, []))
    model_transform(m, ["cuda", "cpu"])
    assert [n.op_type for n in m.graph.node] == ["CudaConvFused", "BatchNormalization", "Relu"]  # bias only
    m2 = zoo.conv_bn_relu(1, 8, 6)
    model_transform(m2, ["cpu"])
    assert [n.op_type for n in m2.graph.node] == ["Conv", "BatchNormalization", "Relu"]


def test_release_timing_and_duplicate_names():
    m = zoo.mlp(2)
    m.graph.node[1].name = m.graph.node[0].name
    model_transform(m, ["cpu"])
    names = [n.name for n in m.graph.node]
    assert len(set(names)) == len(names)
    timing = find_tensor_release_timing(m, {t.name for t in m.graph.initializer})
    released = [t for ts in timing.values() for t in ts]
    assert "input" not in released and m.graph.output[0].name not in released
    assert m.graph.node[0].output[0] in timing[m.graph.node[1].name]


def test_runner_on_host_backend_runs_shape_subgraph_and_binds_positionally():
    x = np.zeros((2, 3, 4), np.float32)
    g = onnx_io.Graph("g", [
        onnx_io.make_node("Shape", ["x"], ["s"]),
        onnx_io.make_node("Gather", ["s", "idx"], ["d"], axis=0),
        onnx_io.make_node("Unsqueeze", ["d"], ["d1"], axes=[0]),
        onnx_io.make_node("Concat", ["d1", "minus1"], ["shape"], axis=0),
        onnx_io.make_node("Reshape", ["x", "shape"], ["y"]),
    ], [onnx_io.make_tensor("idx", np.asarray(0, np.int64)), onnx_io.make_tensor("minus1", np.asarray([-1], np.int64))],
        [onnx_io.ValueInfo("x", onnx_io.FLOAT, [2, 3, 4]), onnx_io.ValueInfo("idx", onnx_io.INT64, [])],
        [onnx_io.ValueInfo("y", onnx_io.FLOAT, [2, 12])])
    runner = load(onnx_io.Model(g, opset_import=[("", 11)]), backend_order=["cpu"])
    assert runner.get_input_names() == ["x"]  # initializer-named graph inputs are skipped
    (y,) = runner.run([CPUTensor.from_array(x)])
    assert y.dims == [2, 12] and np.shares_memory(y.data, x) or y.dims == [2, 12]
    assert all(b == "cpu" for _, _, b in runner.node_backends)
    with pytest.raises(ValueError):
        runner.run([])


def test_no_cpu_fallback_for_arithmetic_ops():
    x = np.ones((2, 3), np.float32)
    runner = load(single_op_model("Relu", {}, [x]), backend_order=["cpu"])
    with pytest.raises(RuntimeError, match="does not exist"):
        runner.run([CPUTensor.from_array(x)])


def test_load_without_gpu_reports_no_backend():
    import ctypes
    from webdnn_b200 import lib
    n = ctypes.c_int(0)
    lib.load_library().wdc_device_count(ctypes.byref(n))
    if n.value > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="No backend available"):
        load(zoo.mlp(2), backend_order=["cuda"])


def test_transformer_fusions_layernorm_chain_and_matmul_bias():
    m = zoo.detr(batch=1, size=64, d=32, heads=4, enc_layers=1, dec_layers=1, ffn=64, queries=5, classes=7, width=8,
                 blocks=(1, 1, 1, 1))
    before = [n.op_type for n in m.graph.node]
    n_ln = before.count("Sqrt")                      # one Sqrt per decomposed LayerNormalization
    model_transform(m, ["cuda", "cpu"])
    types = [n.op_type for n in m.graph.node]
    assert types.count("CudaLayerNorm") == n_ln == 5
    assert not {"ReduceMean", "Sub", "Sqrt", "Div"} & set(types)
    # every linear layer (MatMul by a constant + bias) is one node; the FFN's first one carries its Relu
    assert types.count("CudaMatMulBias") == 4 * 3 + 2 * 2 + 1 + 3
    relus = [n for n in m.graph.node if n.op_type == "CudaMatMulBias" and {a.name: a.i for a in n.attribute}["relu"]]
    assert len(relus) == 2 + 2                        # two feed-forward blocks, two hidden layers of the box head
    # the residual sums x + linear(...) in front of each LayerNormalization ride on the linear layer, except the
    # decoder's first, whose other operand is a constant of the graph (the zero target)
    with_res = [n for n in m.graph.node if n.op_type == "CudaMatMulBias"
                and {a.name: a.i for a in n.attribute}["has_residual"]]
    assert len(with_res) == 4 and all(len(n.input) == 4 for n in with_res)
    # the three attention blocks (scores, scale, softmax, context) are one node each; heads of 8 channels are
    # not a size of the fused kernel, so the head split / merge around them stays in the graph
    assert types.count("MatMul") == 0 and types.count("Softmax") == 0 and types.count("CudaAttention") == 3
    att = {a.name: a for a in next(n for n in m.graph.node if n.op_type == "CudaAttention").attribute}
    assert att["heads"].i == 0 and att["merge_heads"].i == 0 and abs(att["scale"].f - 8 ** -0.5) < 1e-7
    assert types.count("Transpose") == 1 + 3 * 4     # token layout + (q, k, v, merge) per attention block
    ln = next(n for n in m.graph.node if n.op_type == "CudaLayerNorm")
    attrs = {a.name: a for a in ln.attribute}
    assert attrs["axis"].i == -1 and abs(attrs["epsilon"].f - 1e-5) < 1e-12 and len(ln.input) == 3
    known = {vi.name for vi in m.graph.input} | {t.name for t in m.graph.initializer}
    for n in m.graph.node:
        assert all(i in known for i in n.input), (n.op_type, n.name)
        known.update(n.output)


def test_attention_rewrite_absorbs_the_head_split_and_merge():
    m = zoo.detr(batch=2, size=64, d=64, heads=2, enc_layers=1, dec_layers=1, ffn=64, queries=5, classes=7, width=8,
                 blocks=(1, 1, 1, 1))
    model_transform(m, ["cuda", "cpu"])
    types = [n.op_type for n in m.graph.node]
    assert types.count("CudaAttention") == 3 and types.count("Transpose") == 1 and types.count("Reshape") == 1
    assert not {"MatMul", "Softmax", "Mul"} & set(types)
    for n in m.graph.node:
        if n.op_type == "CudaAttention":
            att = {a.name: a for a in n.attribute}
            assert (att["batch"].i, att["heads"].i, att["head_size"].i, att["merge_heads"].i) == (2, 2, 32, 1)
            assert abs(att["scale"].f - 32 ** -0.5) < 1e-7 and len(n.input) == 3
    known = {vi.name for vi in m.graph.input} | {t.name for t in m.graph.initializer}
    for n in m.graph.node:
        assert all(i in known for i in n.input), (n.op_type, n.name)
        known.update(n.output)


def test_attention_with_an_outside_consumer_of_the_scores_is_left_alone():
    from webdnn_b200.zoo import _Builder, _Transformer
    b = _Builder(0)
    t = _Transformer(b, 1, 64, 2, 16)
    y = t.attention("x", "x", "x", 5, 5)
    probs = next(n.output[0] for n in b.nodes if n.op_type == "Softmax")
    m = b.model([("x", [1, 5, 64])], [(y, [1, 5, 64]), (probs, [2, 5, 5])])
    model_transform(m, ["cuda", "cpu"])
    types = [n.op_type for n in m.graph.node]
    assert "CudaAttention" not in types and types.count("MatMul") == 2 and types.count("Softmax") == 1


def test_layernorm_chain_with_an_outside_consumer_is_left_alone():
    from webdnn_b200.zoo import _Builder, _Transformer
    b = _Builder(0)
    t = _Transformer(b, 1, 8, 2, 16)
    y = t.layer_norm("x")
    # the centred value (output of Sub) is also a graph output: the chain must stay
    sub_out = next(n.output[0] for n in b.nodes if n.op_type == "Sub")
    m = b.model([("x", [1, 3, 8])], [(y, [1, 3, 8]), (sub_out, [1, 3, 8])])
    model_transform(m, ["cuda", "cpu"])
    types = [n.op_type for n in m.graph.node]
    assert "CudaLayerNorm" not in types and types.count("ReduceMean") == 2


def test_lstm_rejects_what_the_kernels_do_not_implement():
    """Non-default activations, clip, layout=1, input_forget and a reverse direction must raise at initialize():
    the kernels compute the operator's defaults only and would otherwise return the default's numbers."""
    from webdnn_b200.operators.cuda import CudaLSTM
    ok = onnx_io.make_node("LSTM", ["x", "w", "r"], ["y"], hidden_size=8, direction="forward",
                           activations=["Sigmoid", "Tanh", "Tanh"])
    CudaLSTM().initialize(ok.attribute)
    for bad in (dict(activations=["Relu", "Tanh", "Tanh"]), dict(clip=3.0), dict(layout=1), dict(input_forget=1),
                dict(direction="reverse"), dict(activation_alpha=[0.5])):
        node = onnx_io.make_node("LSTM", ["x", "w", "r"], ["y"], hidden_size=8, **bad)
        with pytest.raises(ValueError):
            CudaLSTM().initialize(node.attribute)
    # the attribute list survives the wire format
    rt = onnx_io.decode_model(onnx_io.encode_model(onnx_io.Model(onnx_io.Graph("g", [ok], [], [], []))))
    acts = [a for a in rt.graph.node[0].attribute if a.name == "activations"][0]
    assert [s.decode() for s in acts.strings] == ["Sigmoid", "Tanh", "Tanh"]


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` times the CPU restatement of the reference's cpu backend (no GPU involved) and
    prints one JSON line with the keys the benchmark contract names; here on a one-image sample."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--ref-images", "1"], capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "resnet50_fp32_inference_images_per_sec"
    assert d["unit"] == "images/s" and d["higher_is_better"] is True and d["value"] > 0
    assert d["steps"] == 1 and d["n_gpus"] == 1 and d["dtype"] == "f32" and d["data"] == "synthetic"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]
