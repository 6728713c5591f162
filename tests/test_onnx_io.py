"""CPU: the wire-format ONNX reader/writer against the reference's only committed model."""
import base64

import numpy as np

from webdnn_b200 import onnx_io, zoo

from util import known_answers


def test_minimum_model_decodes_like_the_reference_fixture():
    ka = known_answers()["minimum_model"]
    raw = base64.b64decode(ka["base64"])
    assert len(raw) == 104
    m = onnx_io.decode_model(raw)
    assert m.ir_version == ka["ir_version"]
    assert m.producer_name == ka["producer_name"] and m.producer_version == ka["producer_version"]
    assert m.opset_import == [("", ka["opset"])]
    (node,) = m.graph.node
    assert (node.name, node.op_type, node.input, node.output) == (
        ka["node"]["name"], ka["node"]["op_type"], ka["node"]["input"], ka["node"]["output"])
    assert m.graph.input[0].shape == ka["io_shape"] and m.graph.output[0].shape == ka["io_shape"]
    assert m.graph.input[0].elem_type == onnx_io.FLOAT


def test_round_trip_preserves_graph():
    m = zoo.conv_bn_relu(2, 8, 6)
    m2 = onnx_io.decode_model(onnx_io.encode_model(m))
    assert [n.op_type for n in m2.graph.node] == ["Conv", "BatchNormalization", "Relu"]
    for a, b in zip(m.graph.initializer, m2.graph.initializer):
        assert a.name == b.name and a.dims == b.dims and np.array_equal(a.array.reshape(-1), b.array.reshape(-1))
    conv = m2.graph.node[0]
    attrs = {a.name: a for a in conv.attribute}
    assert attrs["pads"].ints == [1, 1, 1, 1] and attrs["group"].i == 1
    assert abs({a.name: a for a in m2.graph.node[1].attribute}["epsilon"].f - 1e-5) < 1e-12


def test_int64_is_saturated_like_cliplong():
    assert onnx_io.clip_long(2 ** 40) == 2 ** 31 - 1
    assert onnx_io.clip_long(-2 ** 40) == -2 ** 31
    assert onnx_io.clip_long(-10) == -10
    n = onnx_io.make_node("Reshape", ["a", "s"], ["b"], axis=-(2 ** 40))
    m = onnx_io.Model(onnx_io.Graph("g", [n]))
    back = onnx_io.decode_model(onnx_io.encode_model(m)).graph.node[0].attribute[0]
    assert back.i == -(2 ** 40)  # the wire keeps 64 bits; narrowing happens in the attribute getters


def test_resnet50_graph_shape():
    m = zoo.resnet50(1)
    ops_ = [n.op_type for n in m.graph.node]
    assert ops_.count("Conv") == 53 and ops_.count("BatchNormalization") == 53
    assert ops_.count("Relu") == 49 and ops_.count("Add") == 16 and ops_.count("Gemm") == 1
    assert zoo.contraction_flops(m, {"input": [1, 3, 224, 224]}) == 8178368512
