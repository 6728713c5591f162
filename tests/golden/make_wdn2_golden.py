"""Regenerates tests/golden/wdn2_golden.json from a checkout of the reference:

    python tests/golden/make_wdn2_golden.py <path to the mil-tokyo/webdnn checkout>


What is taken from the reference itself:
  * the 128 decode levels, parsed out of core/tensorDecoder/decodeTensorEightbit.ts;
  * 8-bit tensor bodies produced by the reference's own encoder
    (graph_transpiler/webdnn/constant_codec_eightbit.py, imported by path: it needs only numpy);
  * the container layout constants of graph_transpiler/webdnn/tensor_export.py, by building a
    container byte by byte from the struct formats that file uses.
The expected decoded values are level * scale evaluated in double and rounded to float32, which is
what decodeTensorEightbit.ts:52-58 does.
"""
import base64
import importlib.util
import json
import os
import re
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    if len(sys.argv) != 2 or not os.path.isdir(sys.argv[1]):
        raise SystemExit(__doc__)
    REF = sys.argv[1]
    ts = open(os.path.join(REF, "src/descriptor_runner/core/tensorDecoder/decodeTensorEightbit.ts")).read()
    body = ts[ts.index("const decodeTable = ["):ts.index("];")]
    table = [float(x) for x in re.findall(r"[0-9]+\.[0-9]+(?:e-?[0-9]+)?", body)]
    assert len(table) == 128 and table[0] == 0.0 and table[-1] == 1.0
    spec = importlib.util.spec_from_file_location(
        "ref_codec", os.path.join(REF, "src/graph_transpiler/webdnn/constant_codec_eightbit.py"))
    codec = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(codec)
    rng = np.random.default_rng(20)
    cases = []
    for name, arr in [
        ("normal", (rng.standard_normal(300) * 0.2).astype(np.float32)),
        ("with_zeros_and_extremes", np.array([0.0, -0.0, 1.0, -1.0, 1e-7, -3e-6, 0.5, -0.25, 0.999, 2.0], np.float32)),
        ("all_zero", np.zeros(7, np.float32)),
    ]:
        blob = codec.compress_tensor_eightbit(arr)
        code_len, scale = struct.unpack_from("<If", blob, 0)
        import zlib
        codes = np.frombuffer(zlib.decompress(blob[8:8 + code_len]), np.uint8)
        levels = np.array(table, np.float64)
        expected = (levels[codes & 127] * float(scale) * np.where(codes < 128, 1.0, -1.0)).astype(np.float32)
        cases.append(dict(name=name, values=arr.tolist(), blob=base64.b64encode(blob).decode(),
                          expected_bits=expected.view(np.uint32).tolist()))
    # one container, assembled field by field: a raw float tensor, a raw int64 tensor, an 8-bit tensor
    def chunk(name, arr, comp, body, dtype_code):
        nb = name.encode()
        c = struct.pack("<BIBB", comp, len(body), dtype_code, arr.ndim) + struct.pack("<" + "I" * arr.ndim, *arr.shape)
        c += struct.pack("<I", len(nb)) + nb + struct.pack("<I", 0) + body
        return b"TENS" + struct.pack("<I", len(c)) + c
    a = np.arange(6, dtype=np.float32).reshape(2, 3) - 2.5
    b = np.array([1, -2, 2 ** 40, -(2 ** 40)], np.int64)
    c8 = (rng.standard_normal((4, 5)) * 0.1).astype(np.float32)
    container = b"WDN2" + chunk("a", a, 0, a.tobytes(), 1) + chunk("b", b, 0, b.tobytes(), 7) \
        + chunk("c8", c8, 1, codec.compress_tensor_eightbit(c8), 1) + b"CLOS" + b"\0\0\0\0"
    out = dict(table=table, eightbit_cases=cases, container=base64.b64encode(container).decode(),
               container_a=a.tolist(), container_b_clipped=[1, -2, 2 ** 31 - 1, -(2 ** 31)], container_c8=c8.tolist())
    with open(os.path.join(HERE, "wdn2_golden.json"), "w") as f:
        json.dump(out, f)
    print("wrote", os.path.join(HERE, "wdn2_golden.json"), os.path.getsize(os.path.join(HERE, "wdn2_golden.json")), "bytes")


if __name__ == "__main__":
    main()
