"""WDN2 tensor container: reader, writer and 8-bit codec against fixtures made from the reference
checkout (tests/golden/make_wdn2_golden.py) and against round trips; runner loading of external
weights.  CPU only."""
import base64
import json
import os

import numpy as np
import pytest

from webdnn_b200 import onnx_io, tensor_export, tensor_loader, zoo
from webdnn_b200.runner import load

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "wdn2_golden.json")))


def test_decode_levels_match_the_reference_table():
    assert tensor_loader.EIGHTBIT_TABLE.tolist() == GOLDEN["table"]


@pytest.mark.parametrize("case", GOLDEN["eightbit_cases"], ids=lambda c: c["name"])
def test_eightbit_decode_of_reference_encoded_bodies(case):
    blob = base64.b64decode(case["blob"])
    rec = tensor_loader.TensorRecord("t", [len(case["values"])], onnx_io.FLOAT, 1, blob)
    got = tensor_loader.decode(rec)
    assert got.view(np.uint32).tolist() == case["expected_bits"]
    # and our encoder produces the reference encoder's bytes
    assert tensor_export.compress_tensor_eightbit(np.array(case["values"], np.float32)) == blob


def test_container_built_from_the_reference_layout(tmp_path):
    p = tmp_path / "weights.bin"
    p.write_bytes(base64.b64decode(GOLDEN["container"]))
    tensors = tensor_loader.TensorLoader(str(p)).load_all()
    assert list(tensors) == ["a", "b", "c8"]
    assert tensors["a"].dims == [2, 3] and tensors["a"].data_type == "float32"
    assert tensors["a"].numpy().tolist() == GOLDEN["container_a"]
    assert tensors["b"].data_type == "int32" and tensors["b"].numpy().tolist() == GOLDEN["container_b_clipped"]
    c8 = np.array(GOLDEN["container_c8"], np.float32)
    got = tensors["c8"].numpy()
    assert got.shape == (4, 5)
    # the 8-bit grid is coarse: a few percent of the tensor's largest magnitude
    assert np.max(np.abs(got - c8)) <= 0.04 * np.max(np.abs(c8))


def test_writer_reader_round_trip_raw_split_and_progress(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"w": rng.standard_normal((3, 4, 5)).astype(np.float32), "i": np.arange(-3, 4, dtype=np.int32),
               "l": np.array([5, -(2 ** 35)], np.int64), "s": np.float32(2.5).reshape(())}
    paths = tensor_export.serialize_tensors(str(tmp_path / "w-{}.bin"), tensors, split_size=64)
    assert len(paths) > 1
    seen = []
    got = tensor_loader.TensorLoader(paths).load_all(seen.append)
    assert seen[0] == 0 and seen[-1] == sum(os.path.getsize(p) for p in paths)
    assert np.array_equal(got["w"].numpy(), tensors["w"])
    assert np.array_equal(got["i"].numpy(), tensors["i"])
    assert got["l"].numpy().tolist() == [5, -(2 ** 31)]
    assert got["s"].dims == [] and got["s"].numpy() == np.float32(2.5)


def test_eightbit_round_trip_is_idempotent(tmp_path):
    """decode(encode(x)) lies on the grid, so encoding it again reproduces the same codes."""
    x = (np.random.default_rng(1).standard_normal(4000) * 0.05).astype(np.float32)
    (p,) = tensor_export.serialize_tensors(str(tmp_path / "w.bin"), {"x": x}, compression_algorithm=1)
    y = tensor_loader.TensorLoader(p).load_all()["x"].numpy()
    (p2,) = tensor_export.serialize_tensors(str(tmp_path / "w2.bin"), {"x": y}, compression_algorithm=1)
    z = tensor_loader.TensorLoader(p2).load_all()["x"].numpy()
    assert np.array_equal(y, z)
    assert np.max(np.abs(y - x)) <= 0.04 * np.max(np.abs(x))


def test_bad_containers_are_rejected(tmp_path):
    with pytest.raises(ValueError, match="signature"):
        tensor_loader.parse_container(b"XXXX")
    with pytest.raises(ValueError, match="EOF"):
        tensor_loader.parse_container(b"WDN2TENS")
    chunk = tensor_export.make_tensor_chunk("t", np.zeros(3, np.float32))
    with pytest.raises(ValueError, match="EOF"):
        tensor_loader.parse_container(b"WDN2" + chunk[:-2])
    bad = bytearray(chunk)
    bad[8] = 7  # unknown compression algorithm
    with pytest.raises(ValueError, match="compression"):
        tensor_loader.decode(tensor_loader.parse_container(b"WDN2" + bytes(bad) + b"CLOS\0\0\0\0")[0])


def _externalise(model, directory, compression):
    """Moves every initializer of a zoo model into weight files beside model.onnx, the way the
    reference's optimizer exports a model (metadata key WebDNN2.WeightPaths)."""
    tensors = {t.name: np.asarray(t.array).reshape(t.dims) for t in model.graph.initializer}
    paths = tensor_export.serialize_tensors(os.path.join(directory, "weight-{}.bin"), tensors, split_size=1 << 16,
                                            compression_algorithm=compression)
    del model.graph.initializer[:]
    model.metadata_props["WebDNN2.WeightPaths"] = ":".join(os.path.basename(p) for p in paths)
    onnx_io.save_model(model, os.path.join(directory, "model.onnx"))


@pytest.mark.parametrize("compression", [0, 1])
def test_runner_reads_external_weights(tmp_path, compression):
    """load_model resolves WebDNN2.WeightPaths: every initializer of the exported model is back, raw
    ones bit for bit, 8-bit ones on the codec's grid; with the cuda backend in the order, large 8-bit
    tensors stay as codes for the device (nothing here touches a GPU)."""
    from webdnn_b200.backend import EightbitCPUTensor, WebDNNCPUContext
    from webdnn_b200.runner import Runner
    model = zoo.mlp(4)
    originals = {t.name: np.asarray(t.array).reshape(t.dims) for t in model.graph.initializer}
    _externalise(model, str(tmp_path), compression)
    for order in (["cpu"], ["cuda", "cpu"]):
        r = Runner(order, {"cpu": WebDNNCPUContext()})
        r.load_model(str(tmp_path))
        assert set(r.initializer_tensors) == set(originals)
        assert [vi.name for vi in r.inputs_without_initializer] == ["input"]
        for name, want in originals.items():
            t = r.initializer_tensors[name]
            lazy = isinstance(t, EightbitCPUTensor)
            assert lazy == (compression == 1 and order[0] == "cuda" and want.size >= Runner.DEVICE_DECODE_MIN_ELEMENTS)
            got = t.numpy()
            assert list(got.shape) == list(want.shape)
            if compression == 0:
                assert np.array_equal(got, want)
            else:
                assert np.max(np.abs(got - want)) <= 0.04 * np.max(np.abs(want)) + 1e-12


def test_offline_optimizer_bundle(tmp_path):
    """optimize_model writes the rewritten graph without constants, the weight files and the
    reference's metadata keys; loading the bundle gives back exactly the constants of a load-time
    rewrite of the original model, and rewrites nothing a second time."""
    from webdnn_b200 import optimize_model
    from webdnn_b200.backend import WebDNNCPUContext
    from webdnn_b200.runner import Runner
    src = tmp_path / "src.onnx"
    onnx_io.save_model(zoo.conv_bn_relu(2, 8, 6), str(src))
    optimize_model.main([str(src), str(tmp_path / "out")])
    bundle = onnx_io.load_model(str(tmp_path / "out" / "model-cuda.onnx"))
    assert [n.op_type for n in bundle.graph.node] == ["CudaConvFused"]
    assert not bundle.graph.initializer
    paths = bundle.metadata_props["WebDNN2.WeightPaths"].split(":")
    sizes = [int(v) for v in bundle.metadata_props["WebDNN2.WeightSizes"].split(":")]
    assert sizes == [os.path.getsize(tmp_path / "out" / p) for p in paths]
    assert json.loads(bundle.metadata_props["WebDNN2.TensorMoveOptions"]) == {}
    direct = Runner(["cuda", "cpu"], {"cpu": WebDNNCPUContext()})
    direct.load_model(zoo.conv_bn_relu(2, 8, 6))
    loaded = Runner(["cuda", "cpu"], {"cpu": WebDNNCPUContext()})
    loaded.load_model(str(tmp_path / "out"), "model-cuda.onnx")
    assert [n.op_type for n in loaded.model.graph.node] == ["CudaConvFused"]
    assert [vi.name for vi in loaded.inputs_without_initializer] == ["input"]
    assert set(loaded.initializer_tensors) == set(direct.initializer_tensors)
    for name, t in direct.initializer_tensors.items():
        assert np.array_equal(loaded.initializer_tensors[name].numpy(), t.numpy())
