"""Minimal ONNX model reader/writer on the protobuf wire format.

WebDNN decodes ``model.onnx`` with protobufjs bindings generated from ``scripts/onnx.proto``
(``core/runnerImpl.ts:88-134``).  Only the messages the runner touches are handled here:
ModelProto, OperatorSetIdProto, StringStringEntryProto, GraphProto, NodeProto, AttributeProto,
TensorProto, ValueInfoProto, TypeProto.Tensor and TensorShapeProto.  Field numbers follow
``scripts/onnx.proto`` (:122-184 attribute, :208-230 node, :357-400 model, :456-490 graph,
:499-657 tensor, :687-790 shape/type/opset).  Unknown fields are skipped on read.

Integer narrowing follows the runner: int64 attribute values and int64 tensors are saturated to
the int32 range (``util.ts:73-81``), float tensors stay float32.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

# TensorProto.DataType
FLOAT, UINT8, INT32, INT64, BOOL = 1, 2, 6, 7, 9
# AttributeProto.AttributeType
A_FLOAT, A_INT, A_STRING, A_TENSOR, A_FLOATS, A_INTS, A_STRINGS = 1, 2, 3, 4, 6, 7, 8

INT32_MIN, INT32_MAX = -(2 ** 31), 2 ** 31 - 1


def clip_long(v: int) -> int:
    """Saturate a signed 64-bit value to int32 (``util.ts:73-81``)."""
    return INT32_MIN if v < INT32_MIN else INT32_MAX if v > INT32_MAX else int(v)


# ------------------------------------------------------------------ wire primitives
def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    result = 0
    shift = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise ValueError("varint too long")


def _signed64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _fields(buf: bytes):
    """Yield (field_number, wire_type, value) over one message body."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _read_varint(buf, pos)
        fno, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _read_varint(buf, pos)
        elif wt == 1:
            v = buf[pos:pos + 8]
            pos += 8
        elif wt == 2:
            ln, pos = _read_varint(buf, pos)
            v = buf[pos:pos + ln]
            if len(v) != ln:
                raise ValueError("truncated length-delimited field")
            pos += ln
        elif wt == 5:
            v = buf[pos:pos + 4]
            pos += 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        yield fno, wt, v


def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(fno: int, wt: int) -> bytes:
    return _varint((fno << 3) | wt)


def _ld(fno: int, payload: bytes) -> bytes:
    return _key(fno, 2) + _varint(len(payload)) + payload


def _packed_varints(buf: bytes) -> List[int]:
    out, pos = [], 0
    while pos < len(buf):
        v, pos = _read_varint(buf, pos)
        out.append(_signed64(v))
    return out


# ------------------------------------------------------------------ data model
@dataclass
class Tensor:
    name: str
    dims: List[int]
    data_type: int
    array: np.ndarray  # float32 / int32 / int64 as stored


@dataclass
class Attribute:
    name: str
    type: int = 0
    f: Optional[float] = None
    i: Optional[int] = None
    s: Optional[bytes] = None
    t: Optional[Tensor] = None
    floats: List[float] = field(default_factory=list)
    ints: List[int] = field(default_factory=list)
    strings: List[bytes] = field(default_factory=list)


@dataclass
class Node:
    op_type: str
    input: List[str]
    output: List[str]
    name: str = ""
    attribute: List[Attribute] = field(default_factory=list)
    domain: str = ""


@dataclass
class ValueInfo:
    name: str
    elem_type: int = FLOAT
    shape: List[Any] = field(default_factory=list)  # ints or dim_param strings


@dataclass
class Graph:
    name: str = "graph"
    node: List[Node] = field(default_factory=list)
    initializer: List[Tensor] = field(default_factory=list)
    input: List[ValueInfo] = field(default_factory=list)
    output: List[ValueInfo] = field(default_factory=list)


@dataclass
class Model:
    graph: Graph
    ir_version: int = 7
    opset_import: List[Tuple[str, int]] = field(default_factory=lambda: [("", 13)])
    producer_name: str = ""
    producer_version: str = ""
    metadata_props: Dict[str, str] = field(default_factory=dict)


# ------------------------------------------------------------------ decode
def _decode_tensor(buf: bytes) -> Tensor:
    dims: List[int] = []
    dt = 0
    name = ""
    raw = None
    floats: List[float] = []
    i32: List[int] = []
    i64: List[int] = []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            dims += _packed_varints(v) if wt == 2 else [_signed64(v)]
        elif fno == 2:
            dt = v
        elif fno == 8:
            name = v.decode("utf-8")
        elif fno == 9:
            raw = bytes(v)
        elif fno == 4:
            if wt == 2:
                floats += list(struct.unpack(f"<{len(v) // 4}f", v))
            else:
                floats.append(struct.unpack("<f", v)[0])
        elif fno == 5:
            i32 += _packed_varints(v) if wt == 2 else [_signed64(v)]
        elif fno == 7:
            i64 += _packed_varints(v) if wt == 2 else [_signed64(v)]
    if dt == FLOAT:
        arr = np.frombuffer(raw, dtype="<f4").copy() if raw else np.asarray(floats, dtype=np.float32)
    elif dt == INT64:
        arr = np.frombuffer(raw, dtype="<i8").copy() if raw else np.asarray(i64, dtype=np.int64)
    elif dt == INT32:
        arr = np.frombuffer(raw, dtype="<i4").copy() if raw else np.asarray(i32, dtype=np.int32)
    else:
        arr = np.frombuffer(raw or b"", dtype=np.uint8).copy()
    return Tensor(name, dims, dt, arr)


def _decode_attribute(buf: bytes) -> Attribute:
    a = Attribute("")
    for fno, wt, v in _fields(buf):
        if fno == 1:
            a.name = v.decode("utf-8")
        elif fno == 20:
            a.type = v
        elif fno == 2:
            a.f = struct.unpack("<f", v)[0]
        elif fno == 3:
            a.i = _signed64(v)
        elif fno == 4:
            a.s = bytes(v)
        elif fno == 5:
            a.t = _decode_tensor(v)
        elif fno == 7:
            if wt == 2:
                a.floats += list(struct.unpack(f"<{len(v) // 4}f", v))
            else:
                a.floats.append(struct.unpack("<f", v)[0])
        elif fno == 8:
            a.ints += _packed_varints(v) if wt == 2 else [_signed64(v)]
        elif fno == 9:
            a.strings.append(bytes(v))
    return a


def _decode_node(buf: bytes) -> Node:
    n = Node("", [], [])
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            n.input.append(v.decode("utf-8"))
        elif fno == 2:
            n.output.append(v.decode("utf-8"))
        elif fno == 3:
            n.name = v.decode("utf-8")
        elif fno == 4:
            n.op_type = v.decode("utf-8")
        elif fno == 5:
            n.attribute.append(_decode_attribute(v))
        elif fno == 7:
            n.domain = v.decode("utf-8")
    return n


def _decode_value_info(buf: bytes) -> ValueInfo:
    vi = ValueInfo("")
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            vi.name = v.decode("utf-8")
        elif fno == 2:  # TypeProto
            for f2, _w2, v2 in _fields(v):
                if f2 == 1:  # tensor_type
                    for f3, _w3, v3 in _fields(v2):
                        if f3 == 1:
                            vi.elem_type = v3
                        elif f3 == 2:  # TensorShapeProto
                            for f4, _w4, v4 in _fields(v3):
                                if f4 == 1:  # Dimension
                                    dim: Any = 0
                                    for f5, _w5, v5 in _fields(v4):
                                        if f5 == 1:
                                            dim = _signed64(v5)
                                        elif f5 == 2:
                                            dim = v5.decode("utf-8")
                                    vi.shape.append(dim)
    return vi


def _decode_graph(buf: bytes) -> Graph:
    g = Graph()
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            g.node.append(_decode_node(v))
        elif fno == 2:
            g.name = v.decode("utf-8")
        elif fno == 5:
            g.initializer.append(_decode_tensor(v))
        elif fno == 11:
            g.input.append(_decode_value_info(v))
        elif fno == 12:
            g.output.append(_decode_value_info(v))
    return g


def decode_model(buf: bytes) -> Model:
    m = Model(Graph(), ir_version=0, opset_import=[])
    for fno, _wt, v in _fields(buf):
        if fno == 1:
            m.ir_version = v
        elif fno == 2:
            m.producer_name = v.decode("utf-8")
        elif fno == 3:
            m.producer_version = v.decode("utf-8")
        elif fno == 7:
            m.graph = _decode_graph(v)
        elif fno == 8:
            dom, ver = "", 0
            for f2, _w2, v2 in _fields(v):
                if f2 == 1:
                    dom = v2.decode("utf-8")
                elif f2 == 2:
                    ver = _signed64(v2)
            m.opset_import.append((dom, ver))
        elif fno == 14:
            k = val = ""
            for f2, _w2, v2 in _fields(v):
                if f2 == 1:
                    k = v2.decode("utf-8")
                elif f2 == 2:
                    val = v2.decode("utf-8")
            m.metadata_props[k] = val
    return m


def load_model(path: str) -> Model:
    with open(path, "rb") as f:
        return decode_model(f.read())


# ------------------------------------------------------------------ encode
def _encode_tensor(t: Tensor) -> bytes:
    out = b""
    if t.dims:
        out += _ld(1, b"".join(_varint(d) for d in t.dims))
    out += _key(2, 0) + _varint(t.data_type)
    out += _ld(8, t.name.encode("utf-8"))
    arr = np.ascontiguousarray(t.array)
    out += _ld(9, arr.tobytes())
    return out


def _encode_attribute(a: Attribute) -> bytes:
    out = _ld(1, a.name.encode("utf-8"))
    if a.f is not None:
        out += _key(2, 5) + struct.pack("<f", a.f)
    if a.i is not None:
        out += _key(3, 0) + _varint(a.i)
    if a.s is not None:
        out += _ld(4, a.s)
    if a.t is not None:
        out += _ld(5, _encode_tensor(a.t))
    if a.floats:
        out += _ld(7, struct.pack(f"<{len(a.floats)}f", *a.floats))
    if a.ints:
        out += _ld(8, b"".join(_varint(v) for v in a.ints))
    for s in a.strings:
        out += _ld(9, s)
    out += _key(20, 0) + _varint(a.type)
    return out


def _encode_node(n: Node) -> bytes:
    out = b""
    for s in n.input:
        out += _ld(1, s.encode("utf-8"))
    for s in n.output:
        out += _ld(2, s.encode("utf-8"))
    out += _ld(3, n.name.encode("utf-8"))
    out += _ld(4, n.op_type.encode("utf-8"))
    for a in n.attribute:
        out += _ld(5, _encode_attribute(a))
    if n.domain:
        out += _ld(7, n.domain.encode("utf-8"))
    return out


def _encode_value_info(vi: ValueInfo) -> bytes:
    dims = b""
    for d in vi.shape:
        if isinstance(d, str):
            dims += _ld(1, _ld(2, d.encode("utf-8")))
        else:
            dims += _ld(1, _key(1, 0) + _varint(int(d)))
    tensor_type = _key(1, 0) + _varint(vi.elem_type) + _ld(2, dims)
    return _ld(1, vi.name.encode("utf-8")) + _ld(2, _ld(1, tensor_type))


def encode_model(m: Model) -> bytes:
    g = m.graph
    gb = b""
    for n in g.node:
        gb += _ld(1, _encode_node(n))
    gb += _ld(2, g.name.encode("utf-8"))
    for t in g.initializer:
        gb += _ld(5, _encode_tensor(t))
    for vi in g.input:
        gb += _ld(11, _encode_value_info(vi))
    for vi in g.output:
        gb += _ld(12, _encode_value_info(vi))
    out = _key(1, 0) + _varint(m.ir_version)
    if m.producer_name:
        out += _ld(2, m.producer_name.encode("utf-8"))
    if m.producer_version:
        out += _ld(3, m.producer_version.encode("utf-8"))
    out += _ld(7, gb)
    for dom, ver in m.opset_import:
        ob = (_ld(1, dom.encode("utf-8")) if dom else b"") + _key(2, 0) + _varint(ver)
        out += _ld(8, ob)
    for k, v in m.metadata_props.items():
        out += _ld(14, _ld(1, k.encode("utf-8")) + _ld(2, v.encode("utf-8")))
    return out


def save_model(m: Model, path: str) -> None:
    with open(path, "wb") as f:
        f.write(encode_model(m))


# ------------------------------------------------------------------ builders
def make_tensor(name: str, array: np.ndarray) -> Tensor:
    array = np.asarray(array)
    if array.dtype == np.float32:
        dt = FLOAT
    elif array.dtype == np.int64:
        dt = INT64
    elif array.dtype == np.int32:
        dt = INT32
    else:
        raise TypeError(f"unsupported initializer dtype {array.dtype}")
    return Tensor(name, list(array.shape), dt, array)


def make_attr(name: str, value: Any) -> Attribute:
    if isinstance(value, bool):
        return Attribute(name, A_INT, i=int(value))
    if isinstance(value, int):
        return Attribute(name, A_INT, i=value)
    if isinstance(value, float):
        return Attribute(name, A_FLOAT, f=value)
    if isinstance(value, str):
        return Attribute(name, A_STRING, s=value.encode("utf-8"))
    if isinstance(value, Tensor):
        return Attribute(name, A_TENSOR, t=value)
    if isinstance(value, (list, tuple)):
        if value and all(isinstance(v, (str, bytes)) for v in value):
            return Attribute(name, A_STRINGS, strings=[v.encode("utf-8") if isinstance(v, str) else v for v in value])
        if all(isinstance(v, int) for v in value):
            return Attribute(name, A_INTS, ints=list(value))
        if all(isinstance(v, (int, float)) for v in value):
            return Attribute(name, A_FLOATS, floats=[float(v) for v in value])
    raise TypeError(f"unsupported attribute value for {name}: {value!r}")


def make_node(op_type: str, inputs: List[str], outputs: List[str], name: str = "", **attrs) -> Node:
    return Node(op_type, list(inputs), list(outputs), name or f"{op_type}_{outputs[0]}",
                [make_attr(k, v) for k, v in attrs.items()])
