"""Writer of the WDN2 tensor container (the format ``tensor_loader`` reads).

Follows ``graph_transpiler/webdnn/tensor_export.py:36-81`` (container and TENS chunk layout, optional
split into fixed-size files) and ``constant_codec_eightbit.py:33-65`` (8-bit codec: scale = max |x|,
level = position of |x| / scale among the midpoints of neighbouring decode levels, sign in bit 7,
codes deflated at level 9).  Only float32 tensors are ever 8-bit coded; other dtypes stay raw.
"""
from __future__ import annotations

import struct
import zlib
from typing import Dict, List

import numpy as np

from .onnx_io import FLOAT, INT32, INT64
from .tensor_loader import EIGHTBIT_TABLE, SIGNATURE_CLOSE, SIGNATURE_FILE, SIGNATURE_TENSOR

_DTYPE_CODE = {np.dtype(np.float32): FLOAT, np.dtype(np.int32): INT32, np.dtype(np.int64): INT64}


def eightbit_thresholds() -> np.ndarray:
    """127 decision thresholds between the 128 levels: 1.5e-6 below the first non-zero level, the
    midpoints of neighbouring levels, and 0.995703 below the level 1.0."""
    levels = EIGHTBIT_TABLE[1:127]  # the 126 levels strictly between 0 and 1
    th = [1.5e-6]
    for i in range(1, 126):
        th.append((levels[i] + levels[i - 1]) / 2.0)
    th.append(0.995703)
    return np.array(th, dtype=np.float32)


def compress_tensor_eightbit(data: np.ndarray) -> bytes:
    if data.dtype != np.float32:
        raise TypeError("8-bit coding takes float32")
    maxval = np.maximum(np.max(np.abs(data)) if data.size else np.float32(0), 1e-20)  # avoid dividing by zero
    scaled = np.abs(data) / maxval
    code = np.searchsorted(eightbit_thresholds(), scaled)
    code = code + (data < 0.0).astype(np.int64) * 128
    code_bytes = zlib.compress(code.astype(np.uint8).tobytes("C"), 9)
    return struct.pack("<If", len(code_bytes), maxval) + code_bytes


def make_tensor_chunk(name: str, data: np.ndarray, compression_algorithm: int = 0) -> bytes:
    data = np.asarray(data)
    if data.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {data.dtype}")
    if data.dtype != np.float32:
        compression_algorithm = 0
    if compression_algorithm == 0:
        body = np.ascontiguousarray(data).astype(data.dtype.newbyteorder("<")).tobytes()
    elif compression_algorithm == 1:
        body = compress_tensor_eightbit(np.ascontiguousarray(data))
    else:
        raise ValueError("unknown compression algorithm")
    name_bytes = name.encode("utf-8")
    chunk = struct.pack("<BIBB", compression_algorithm, len(body), _DTYPE_CODE[data.dtype], data.ndim)
    chunk += struct.pack("<" + "I" * data.ndim, *data.shape)
    chunk += struct.pack("<I", len(name_bytes)) + name_bytes
    chunk += struct.pack("<I", 0)  # no extra data
    chunk += body
    return SIGNATURE_TENSOR + struct.pack("<I", len(chunk)) + chunk


def serialize_tensors(path_template: str, tensors: Dict[str, np.ndarray], split_size: int = 0,
                      compression_algorithm: int = 0) -> List[str]:
    """Writes one container; with ``split_size`` > 0 it is cut into files ``path_template.format(i)``."""
    chunks = [SIGNATURE_FILE]
    for name, data in tensors.items():
        chunks.append(make_tensor_chunk(name, data, compression_algorithm))
    chunks.append(SIGNATURE_CLOSE + b"\0\0\0\0")
    full = b"".join(chunks)
    if split_size <= 0:
        with open(path_template, "wb") as f:
            f.write(full)
        return [path_template]
    paths = []
    for i in range((len(full) + split_size - 1) // split_size):
        p = path_template.format(i)
        with open(p, "wb") as f:
            f.write(full[i * split_size:(i + 1) * split_size])
        paths.append(p)
    return paths
