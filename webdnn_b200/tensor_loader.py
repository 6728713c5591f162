"""Reader of the WDN2 tensor container (weights stored beside an optimized model).

File layout (little endian), as written by ``graph_transpiler/webdnn/tensor_export.py:8-81`` and read
by ``core/tensorLoaderImpl.ts:10-208``: the 4-byte signature ``WDN2``, then chunks of
``signature(4) | body length(u32) | body``.  A ``TENS`` body is ``compression algorithm(u8) |
compressed length(u32) | ONNX data type(u8) | ndim(u8) | dims(u32 * ndim) | name length(u32) | name
(utf-8) | extra length(u32) | extra | compressed data``; ``CLOS`` ends the file.  A container may
be split over several files, which are concatenated before parsing.

Compression 0 is the raw little-endian array (float32, int32, or int64 saturated to int32 like
``decodeTensorRaw.ts:21-33``).  Compression 1 is the 8-bit codec of
``tensorDecoder/decodeTensorEightbit.ts:36-61``: ``code length(u32) | scale(f32) | zlib stream`` of
one byte per element; byte b decodes to ``table[b & 127] * scale`` with the sign from bit 7, where
``table`` is the 128-level non-uniform grid of the format (from "8-Bit Approximations for
Parallelism in Deep Learning", Dettmers 2016; the values below are the format's constants, also
pinned by ``tests/golden/wdn2_golden.json``).

``load_all`` returns CPU tensors like the reference's loader.  ``load_all_device`` keeps 8-bit
tensors compressed on the host side of the bus: the inflated codes (1 byte per element) are
uploaded and expanded to float32 on the GPU by ``wdc_decode_eightbit``.
"""
from __future__ import annotations

import struct
import zlib
from typing import Callable, Dict, List, Optional, Sequence, Union

import numpy as np

from .backend import CPUTensor, WebDNNCPUContext
from .onnx_io import FLOAT, INT32, INT64

SIGNATURE_FILE = b"WDN2"
SIGNATURE_TENSOR = b"TENS"
SIGNATURE_CLOSE = b"CLOS"

# decode levels 0..127 (level 0 is exactly zero, level 127 exactly one)
EIGHTBIT_TABLE = np.array([
    0.0, 2.750000021e-6, 7.249999726e-6, 1.875000089e-5, 3.624999954e-5, 5.874999624e-5, 8.624999464e-5,
    1.437500032e-4, 2.312500001e-4, 3.187500115e-4, 4.062500084e-4, 5.187499919e-4, 6.562499912e-4,
    7.937499322e-4, 9.312499315e-4, 1.218750025e-3, 1.65624998e-3, 2.093750052e-3, 2.531250007e-3,
    2.968749963e-3, 3.406249918e-3, 3.843750106e-3, 4.281249829e-3, 4.843750037e-3, 5.531250034e-3,
    6.218749564e-3, 6.90624956e-3, 7.593749557e-3, 8.281249553e-3, 8.968749084e-3, 9.656248614e-3,
    1.109374966e-2, 1.328125037e-2, 1.546875015e-2, 1.765624993e-2, 1.98437497e-2, 2.203124948e-2,
    2.421874925e-2, 2.640625089e-2, 2.859375067e-2, 3.078125045e-2, 3.296874836e-2, 3.515625e-2,
    3.734375164e-2, 3.953124955e-2, 4.171875119e-2, 4.390624911e-2, 4.671875015e-2, 5.01562506e-2,
    5.359374732e-2, 5.703124776e-2, 6.046874821e-2, 6.390624493e-2, 6.734374911e-2, 7.078124583e-2,
    7.421874255e-2, 7.765624672e-2, 8.109374344e-2, 8.453124017e-2, 8.796874434e-2, 9.140624106e-2,
    9.484373778e-2, 9.828124195e-2, 1.0546875e-1, 1.16406247e-1, 1.27343744e-1, 1.38281256e-1, 1.49218753e-1,
    1.6015625e-1, 1.71093747e-1, 1.82031244e-1, 1.92968756e-1, 2.03906253e-1, 2.1484375e-1, 2.25781247e-1,
    2.36718744e-1, 2.47656256e-1, 2.585937381e-1, 2.6953125e-1, 2.804687619e-1, 2.91406244e-1, 3.02343756e-1,
    3.132812381e-1, 3.2421875e-1, 3.351562619e-1, 3.46093744e-1, 3.57031256e-1, 3.679687381e-1, 3.7890625e-1,
    3.898437619e-1, 4.00781244e-1, 4.11718756e-1, 4.226562381e-1, 4.3359375e-1, 4.445312619e-1, 4.58593756e-1,
    4.757812321e-1, 4.929687381e-1, 5.101562142e-1, 5.2734375e-1, 5.445312262e-1, 5.617187023e-1,
    5.789062381e-1, 5.960937142e-1, 6.1328125e-1, 6.304687262e-1, 6.476562023e-1, 6.648437381e-1,
    6.820312142e-1, 6.992186904e-1, 7.164062262e-1, 7.335937023e-1, 7.507811785e-1, 7.679687142e-1,
    7.851561904e-1, 8.023436666e-1, 8.195312023e-1, 8.367186785e-1, 8.539061546e-1, 8.710936904e-1,
    8.882811666e-1, 9.054686427e-1, 9.226561785e-1, 9.398436546e-1, 9.570311308e-1, 9.742186666e-1,
    9.914061427e-1, 1.0,
], dtype=np.float64)


def scaled_table(scale: float) -> np.ndarray:
    """The 256-entry float32 table of one tensor: JS computes ``table[i & 127] * scale * (+-1)`` in
    double and stores it into a Float32Array (decodeTensorEightbit.ts:52-55)."""
    s = float(np.float32(scale))
    pos = EIGHTBIT_TABLE * s
    return np.concatenate([pos, -pos]).astype(np.float32)


class TensorRecord:
    """One parsed TENS chunk before decoding."""

    __slots__ = ("name", "dims", "data_type", "compression", "body")

    def __init__(self, name: str, dims: List[int], data_type: int, compression: int, body: bytes):
        self.name, self.dims, self.data_type, self.compression, self.body = name, dims, data_type, compression, body

    @property
    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n


def parse_container(data: bytes) -> List[TensorRecord]:
    if data[:4] != SIGNATURE_FILE:
        raise ValueError("Unexpected file signature")
    offset = 4
    out: List[TensorRecord] = []
    while True:
        if len(data) - offset < 8:
            raise ValueError("Unexpected EOF")
        sig = data[offset:offset + 4]
        (body_len,) = struct.unpack_from("<I", data, offset + 4)
        body_off = offset + 8
        if len(data) - body_off < body_len:
            raise ValueError("Unexpected EOF")
        if sig == SIGNATURE_TENSOR:
            out.append(_parse_tensor_chunk(data, body_off))
        elif sig == SIGNATURE_CLOSE:
            return out
        offset = body_off + body_len  # unknown chunk types are skipped like tensorLoaderImpl.ts:47-63


def _parse_tensor_chunk(data: bytes, ofs: int) -> TensorRecord:
    compression, comp_len, data_type, ndim = struct.unpack_from("<BIBB", data, ofs)
    ofs += 7
    dims = list(struct.unpack_from("<" + "I" * ndim, data, ofs))
    ofs += 4 * ndim
    (name_len,) = struct.unpack_from("<I", data, ofs)
    ofs += 4
    name = data[ofs:ofs + name_len].decode("utf-8")
    ofs += name_len
    (extra_len,) = struct.unpack_from("<I", data, ofs)
    ofs += 4 + extra_len
    return TensorRecord(name, dims, data_type, compression, data[ofs:ofs + comp_len])


def decode_raw(rec: TensorRecord) -> np.ndarray:
    n = rec.numel
    if rec.data_type == FLOAT:
        return np.frombuffer(rec.body, dtype="<f4", count=n).copy()
    if rec.data_type == INT32:
        return np.frombuffer(rec.body, dtype="<i4", count=n).copy()
    if rec.data_type == INT64:
        v = np.frombuffer(rec.body, dtype="<i8", count=n)
        return np.clip(v, -(2 ** 31), 2 ** 31 - 1).astype(np.int32)
    raise ValueError("Unsupported DataType")


def eightbit_codes(rec: TensorRecord) -> "tuple[np.ndarray, float]":
    """(codes uint8 [numel], scale) of an 8-bit tensor body."""
    if rec.data_type != FLOAT:
        raise ValueError("Unsupported DataType")
    code_len, scale = struct.unpack_from("<If", rec.body, 0)
    codes = np.frombuffer(zlib.decompress(rec.body[8:8 + code_len]), dtype=np.uint8)
    if codes.size < rec.numel:
        raise ValueError("8-bit tensor body is shorter than the tensor")
    return codes[:rec.numel], scale


def decode_eightbit(rec: TensorRecord) -> np.ndarray:
    codes, scale = eightbit_codes(rec)
    return scaled_table(scale)[codes]


def decode(rec: TensorRecord) -> np.ndarray:
    if rec.compression == 0:
        return decode_raw(rec)
    if rec.compression == 1:
        return decode_eightbit(rec)
    raise ValueError("Unexpected compression algorithm")


def _data_type_name(data_type: int) -> str:
    if data_type == FLOAT:
        return "float32"
    if data_type in (INT32, INT64):
        return "int32"
    raise ValueError("Unsupported DataType")


class TensorLoader:
    """``TensorLoaderImpl`` (core/tensorLoaderImpl.ts:14-66): ``paths`` are the parts of one container."""

    def __init__(self, paths: Union[str, Sequence[str]], cpu_context: Optional[WebDNNCPUContext] = None):
        self.paths = [paths] if isinstance(paths, str) else list(paths)
        self.cpu_context = cpu_context or WebDNNCPUContext()

    def _fetch_all(self, progress: Optional[Callable[[int], object]]) -> bytes:
        parts = []
        loaded = 0
        if progress:
            progress(loaded)
        for p in self.paths:
            with open(p, "rb") as f:
                b = f.read()
            parts.append(b)
            loaded += len(b)
            if progress:
                progress(loaded)
        return b"".join(parts)

    def records(self, progress: Optional[Callable[[int], object]] = None) -> List[TensorRecord]:
        return parse_container(self._fetch_all(progress))

    def load_all(self, progress: Optional[Callable[[int], object]] = None) -> Dict[str, CPUTensor]:
        out: Dict[str, CPUTensor] = {}
        for rec in self.records(progress):
            out[rec.name] = self.cpu_context.empty_tensor(rec.dims, _data_type_name(rec.data_type), decode(rec))
        return out

    def load_all_device(self, cuda_context, progress: Optional[Callable[[int], object]] = None) -> Dict[str, object]:
        """Tensors on the cuda backend.  8-bit float tensors cross the bus as codes (a quarter of the
        bytes) and are expanded by the GPU; the result is bit-identical to ``load_all`` + move."""
        out: Dict[str, object] = {}
        for rec in self.records(progress):
            dtype = _data_type_name(rec.data_type)
            if rec.compression == 1 and rec.numel > 0:
                codes, scale = eightbit_codes(rec)
                out[rec.name] = cuda_context.decode_eightbit(codes, scale, rec.dims)
            else:
                out[rec.name] = cuda_context.move_tensor(self.cpu_context.empty_tensor(rec.dims, dtype, decode(rec)))
        return out
