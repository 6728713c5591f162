"""Offline optimizer for the cuda backend: ``python -m webdnn_b200.optimize_model model.onnx dst_dir``.

The counterpart of ``graph_transpiler/webdnn/optimize_model.py:14-48`` for one more backend name:
the backend's graph passes run once, ahead of time, and the result is written the way the
reference writes its per-backend bundles:

* ``model-cuda.onnx``  the rewritten graph without initializers.  The passes are the same rewrite the
  runner applies at load time (``model_transform``: Conv [+ BatchNormalization] [+ Add] [+ Relu] ->
  ``CudaConvFused`` with the folded per-channel scale/shift as new constants, Gemm + Relu ->
  ``CudaGemmRelu``); applied to an already rewritten graph they change nothing, so loading the bundle
  costs no second fold.
* ``weight-cuda-<i>.bin``  every constant in one WDN2 container cut into 4 MiB files
  (``tensor_export``), optionally with the 8-bit codec (``--compression 1``; like the reference it
  then codes every float32 constant, the folded scale/shift included).
* metadata ``WebDNN2.WeightPaths`` / ``WebDNN2.WeightSizes`` (colon-separated basenames and byte
  sizes) and ``WebDNN2.TensorMoveOptions`` (empty: the cuda backend has no texture layouts to plan).

``load(dst_dir, onnx_basename="model-cuda.onnx")`` runs the bundle.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List

import numpy as np

from . import onnx_io
from .model_transform import model_transform
from .tensor_export import serialize_tensors

SPLIT_SIZE = 4 * 1024 * 1024
BACKEND = "cuda"


def optimize(model: onnx_io.Model, dst_dir: str, compression: int = 0) -> Dict[str, object]:
    """Rewrites ``model`` in place and writes the bundle; returns what was written."""
    os.makedirs(dst_dir, exist_ok=True)
    before = [n.op_type for n in model.graph.node]
    model_transform(model, [BACKEND, "cpu"])
    tensors = {t.name: np.asarray(t.array).reshape(t.dims) for t in model.graph.initializer}
    init_names = set(tensors)
    del model.graph.initializer[:]
    # graph inputs that only declared an initializer's shape would now look like run-time inputs
    model.graph.input[:] = [vi for vi in model.graph.input if vi.name not in init_names]
    paths = serialize_tensors(os.path.join(dst_dir, f"weight-{BACKEND}-{{}}.bin"), tensors, SPLIT_SIZE, compression)
    model.metadata_props["WebDNN2.WeightPaths"] = ":".join(os.path.basename(p) for p in paths)
    model.metadata_props["WebDNN2.WeightSizes"] = ":".join(str(os.path.getsize(p)) for p in paths)
    model.metadata_props["WebDNN2.TensorMoveOptions"] = json.dumps({})
    model_path = os.path.join(dst_dir, f"model-{BACKEND}.onnx")
    onnx_io.save_model(model, model_path)
    return dict(model=model_path, weights=paths, nodes_before=len(before), nodes_after=len(model.graph.node),
                constants=len(tensors))


def main(argv: List[str] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("onnx_model")
    ap.add_argument("dst_dir")
    ap.add_argument("--compression", type=int, default=0, help="compression algorithm number (0 = raw, 1 = 8-bit)")
    args = ap.parse_args(argv)
    info = optimize(onnx_io.load_model(args.onnx_model), args.dst_dir, args.compression)
    print(json.dumps(info))


if __name__ == "__main__":
    main()
