"""Tensors and backend contexts of the Python host mirror.

Mirrors the reference's L1 layer:

* ``TensorImpl`` (``core/tensorImpl.ts:4-36``): dims, ndim, length, row-major strides.
* ``CPUTensor`` (``backend/cpu/cpuTensorImpl.ts:14-89``): a typed array plus dims; the I/O type of
  ``runner.run()``.
* ``CudaTensor``: modelled on ``WebGPUTensorImpl`` (``backend/webgpu/webgpuTensorImpl.ts:6-75``) with
  the refcounted shared buffer and ``alias()`` of ``WasmTensorImpl``
  (``backend/wasm/wasmTensorImpl.ts:16-52,77-85``).  Supports float32 and int32.  Carries a
  ``layout`` tag the way ``WebGLTensor`` carries its texture shape: a 4-D tensor may be stored
  channels-last ("nhwc") because the convolution kernels want the reduction axis contiguous;
  ``dims`` always stay the logical NCHW dims.
* ``WebDNNCudaContext``: ``BackendContext`` (``interface/core/backendContext.ts:4-8``) with
  ``emptyTensor`` / ``moveTensor`` plus typed kernel launchers.

Nothing here computes on the CPU: every method either moves bytes or enqueues a kernel of
libwebdnn_cuda.so on the context's stream.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_void_p
from typing import Dict, List, Optional, Sequence

import numpy as np

from .lib import (DTYPE_CODE, ConvDesc, CudaBackendError, GemmDesc, Library, PoolDesc, i64_array)

NP_DTYPE = {"float32": np.float32, "int32": np.int32, "bool": np.uint8}


def calc_strides(dims: Sequence[int]) -> List[int]:
    strides: List[int] = []
    length = 1
    for d in reversed(dims):
        strides.insert(0, length)
        length *= d
    return strides


class TensorImpl:
    backend = "cpu"

    def __init__(self, dims: Sequence[int], data_type: str, backend: str):
        self.dims = [int(d) for d in dims]
        self.ndim = len(self.dims)
        self.data_type = data_type
        self.backend = backend
        self.strides = calc_strides(self.dims)
        length = 1
        for d in self.dims:
            length *= d
        self.length = length


class CPUTensor(TensorImpl):
    """Host tensor: a flat numpy array of ``length`` elements plus dims."""

    def __init__(self, dims: Sequence[int], data_type: str = "float32", data: Optional[np.ndarray] = None):
        super().__init__(dims, data_type, "cpu")
        if data is None:
            self.data = np.zeros(self.length, dtype=NP_DTYPE[data_type])
            self.use_external_buffer = False
        else:
            arr = np.asarray(data)
            if arr.dtype != NP_DTYPE[data_type]:
                raise TypeError(f"CPUTensor: data dtype {arr.dtype} does not match {data_type}")
            self.data = arr.reshape(-1)
            if self.data.size != self.length:
                raise ValueError("CPUTensor: data length does not match dims")
            self.use_external_buffer = True

    @classmethod
    def from_array(cls, arr: np.ndarray) -> "CPUTensor":
        arr = np.asarray(arr)
        if not arr.flags.c_contiguous:
            arr = arr.copy(order="C")  # (np.ascontiguousarray would turn a 0-d array into 1-d)
        dt = {np.dtype(np.float32): "float32", np.dtype(np.int32): "int32", np.dtype(np.uint8): "bool"}[arr.dtype]
        return cls(arr.shape, dt, arr.reshape(-1))

    def get_data(self) -> np.ndarray:
        return self.data

    def set_data(self, data: np.ndarray) -> None:
        self.data[:] = np.asarray(data).reshape(-1)

    def get_value(self, idxs: Sequence[int]):
        return self.data[sum(i * s for i, s in zip(idxs, self.strides))]

    def set_value(self, value, idxs: Sequence[int]) -> None:
        self.data[sum(i * s for i, s in zip(idxs, self.strides))] = value

    def numpy(self) -> np.ndarray:
        return self.data.reshape(self.dims)

    def dispose(self) -> None:
        pass


class EightbitCPUTensor(CPUTensor):
    """A float32 initializer still held as the 8-bit codes of a WDN2 container.  On the host it decodes
    itself at first access; a cuda context moves it by uploading the codes and decoding on the
    device (``WebDNNCudaContext.move_tensor``)."""

    def __init__(self, dims: Sequence[int], codes: np.ndarray, scale: float):
        TensorImpl.__init__(self, dims, "float32", "cpu")
        self.codes = np.ascontiguousarray(codes, dtype=np.uint8)
        if self.codes.size != self.length:
            raise ValueError("EightbitCPUTensor: code count does not match dims")
        self.scale = float(scale)
        self._decoded: Optional[np.ndarray] = None
        self.use_external_buffer = False

    @property
    def data(self) -> np.ndarray:
        if self._decoded is None:
            from .tensor_loader import scaled_table
            self._decoded = scaled_table(self.scale)[self.codes]
        return self._decoded


class CudaSharedBuffer:
    """Refcounted device allocation shared by aliases of one tensor."""

    def __init__(self, context: "WebDNNCudaContext", byte_length: int):
        self.context = context
        self.byte_length = byte_length
        self.ptr = context._alloc(byte_length)
        self.ref_count = 1

    def incr_ref(self) -> None:
        self.ref_count += 1

    def dispose(self) -> None:
        self.ref_count -= 1
        if self.ref_count == 0 and self.ptr is not None:
            self.context._free(self.ptr)
            self.ptr = None


class CudaTensor(TensorImpl):
    def __init__(self, context: "WebDNNCudaContext", dims: Sequence[int], data_type: str = "float32",
                 shared_buffer: Optional[CudaSharedBuffer] = None, layout: str = "nchw"):
        super().__init__(dims, data_type, "cuda")
        if data_type not in ("float32", "int32"):
            raise TypeError(f"CudaTensor: dataType {data_type} is not supported")
        self.context = context
        self.byte_length = max(self.length * 4, 4)
        self.shared_buffer = shared_buffer or CudaSharedBuffer(context, self.byte_length)
        if layout == "nhwc" and self.ndim != 4:
            raise ValueError("channels-last layout needs a 4-D tensor")
        self.layout = layout
        self.aux: Dict[str, "CudaTensor"] = {}  # derived device data that lives and dies with this tensor
        self.upload_ticket: Optional[int] = None  # pending transfer on the copy stream (prefetch_tensor)
        self.disposed = False

    @property
    def ptr(self) -> int:
        if self.disposed or self.shared_buffer.ptr is None:
            raise CudaBackendError(1, "CudaTensor used after dispose")
        return self.shared_buffer.ptr

    def alias(self, dims: Sequence[int]) -> "CudaTensor":
        """New dims over the same device memory (Reshape/Flatten/Squeeze/Unsqueeze)."""
        self.shared_buffer.incr_ref()
        return CudaTensor(self.context, dims, self.data_type, self.shared_buffer)

    def get_data(self) -> np.ndarray:
        """D2H of the canonical (NCHW row-major) contents; waits for the stream."""
        src = self.context.canonical(self)
        out = np.empty(self.length, dtype=NP_DTYPE[self.data_type])
        if self.length:
            self.context._download(out, src.ptr, self.length * 4)
        if src is not self:
            src.dispose()
        return out

    def set_data(self, data: np.ndarray) -> None:
        arr = np.ascontiguousarray(np.asarray(data).reshape(-1), dtype=NP_DTYPE[self.data_type])
        if arr.size != self.length:
            raise ValueError("CudaTensor.set_data: length mismatch")
        if self.layout != "nchw":
            raise ValueError("set_data writes canonical tensors only")
        if self.length:
            self.context._upload(self.ptr, arr)

    def dispose(self) -> None:
        if self.disposed:
            return
        for t in self.aux.values():
            t.dispose()
        self.aux.clear()
        self.shared_buffer.dispose()
        self.disposed = True

    # physical element strides of the logical (n, c, h, w) axes
    def nchw_strides(self) -> List[int]:
        n, c, h, w = self.dims
        if self.layout == "nhwc":
            return [h * w * c, 1, w * c, c]
        return [c * h * w, h * w, w, 1]


class WebDNNCPUContext:
    backend = "cpu"

    def empty_tensor(self, dims: Sequence[int], data_type: str = "float32", data=None) -> CPUTensor:
        return CPUTensor(dims, data_type, data)

    def move_tensor(self, tensor, option=None) -> CPUTensor:
        # backend/cpu/cpuContextImpl.ts:42-49
        return CPUTensor(tensor.dims, tensor.data_type, tensor.get_data())

    @staticmethod
    def is_cpu_tensor(t) -> bool:
        return isinstance(t, CPUTensor)

    def asserts_cpu_tensor_array(self, tensors) -> None:
        for t in tensors:
            if not isinstance(t, CPUTensor):
                raise TypeError("tensor is not CPUTensor")


class PendingDownload:
    """A device-to-host transfer in flight (WebDNNCudaContext.download_async)."""

    def __init__(self, context, tensor, source, host, ticket):
        self.context, self.tensor, self.source, self.host, self.ticket = context, tensor, source, host, ticket

    def result(self) -> np.ndarray:
        """Waits for the transfer and returns a copy of the data (the staging buffer is reused by later transfers)."""
        self.context._call("wdc_wait_download", self.ticket)
        out = np.array(self.host[:self.tensor.length], copy=True)
        if self.source is not self.tensor:
            self.source.dispose()
        self.source = None
        return out


class WebDNNCudaContext:
    """Owns one device context (stream + arena) of libwebdnn_cuda.so."""

    backend = "cuda"

    def __init__(self, cpu_context: Optional[WebDNNCPUContext] = None, device: int = 0,
                 arena_bytes: int = 0):
        self.cpu_context = cpu_context or WebDNNCPUContext()
        self.device = device
        self.arena_bytes = arena_bytes
        self._L = None
        self.handle = None
        self.precision = "tf32x3"
        self.profile = False      # backendOptions.cuda.profile: NVTX range "name(opType)" around every node

    # --- lifecycle
    def initialize(self) -> None:
        self._L = Library()
        if self._L.device_count() <= self.device:
            raise CudaBackendError(2, f"no CUDA device {self.device} available")
        h = c_void_p()
        st = self._L.lib.wdc_create(self.device, self.arena_bytes, byref(h))
        self._L.check(None, st)
        self.handle = h

    def close(self) -> None:
        if self.handle is not None:
            self._L.lib.wdc_destroy(self.handle)
            self.handle = None

    def _call(self, name: str, *args) -> None:
        st = getattr(self._L.lib, name)(self.handle, *args)
        if st != 0:
            self._L.check(self.handle, st)

    # --- raw memory
    def _alloc(self, nbytes: int) -> int:
        p = c_void_p()
        self._call("wdc_alloc", nbytes, byref(p))
        return p.value

    def _free(self, ptr: int) -> None:
        if self.handle is not None:
            self._call("wdc_free", c_void_p(ptr))

    def _upload(self, ptr: int, arr: np.ndarray) -> None:
        # cudaMemcpyAsync from pageable memory returns once the source has been staged, so the
        # caller may release `arr` right away; pinned sources must outlive the copy
        self._call("wdc_upload", c_void_p(ptr), arr.ctypes.data_as(c_void_p), arr.nbytes)

    def _download(self, out: np.ndarray, ptr: int, nbytes: int) -> None:
        self._call("wdc_download", out.ctypes.data_as(c_void_p), c_void_p(ptr), nbytes)

    def sync(self) -> None:
        self._call("wdc_sync")

    def stream_handle(self) -> int:
        return self._L.lib.wdc_stream(self.handle)

    def stats(self, device_memory: bool = False) -> Dict[str, int]:
        """Arena and traffic counters; with device_memory also the GPU's free / total bytes (cudaMemGetInfo)."""
        n = 11 if device_memory else 9
        out = (ctypes.c_int64 * n)()
        self._call("wdc_stats", out, n)
        keys = ["bytes_in_use", "high_water_bytes", "reserved_bytes", "allocs", "frees", "launches",
                "h2d_bytes", "d2h_bytes", "tensor_core_launches", "device_free_bytes", "device_total_bytes"]
        return dict(zip(keys[:n], list(out)))

    def reset_stats(self) -> None:
        self._call("wdc_reset_stats")

    PRECISIONS = {"tf32x3": 0, "tf32x1": 1}

    def set_option(self, name: str, value: int) -> None:
        """wdc_set_option: "precision" (0 tf32x3 / 1 tf32x1), "split_k", "pdl", "nvtx"."""
        self._call("wdc_set_option", name.encode("utf-8"), int(value))

    def set_precision(self, precision: str) -> None:
        """backendOptions.cuda.precision: "tf32x3" (default, fp32-class accuracy) or "tf32x1"."""
        if precision not in self.PRECISIONS:
            raise ValueError(f"precision must be one of {sorted(self.PRECISIONS)}, not {precision!r}")
        self.set_option("precision", self.PRECISIONS[precision])
        self.precision = precision

    def range_push(self, name: str) -> None:
        self._call("wdc_range_push", name.encode("utf-8"))

    def range_pop(self) -> None:
        self._call("wdc_range_pop")

    def profile_enable(self, on: bool) -> None:
        self._call("wdc_profile_enable", int(on))

    def profile_read(self):
        """(milliseconds, launches, algorithmic FLOPs) of the contraction kernels since the last read."""
        ms, n, fl = ctypes.c_double(), ctypes.c_int64(), ctypes.c_double()
        self._call("wdc_profile_read", 0, byref(ms), byref(n), byref(fl))
        return ms.value, n.value, fl.value

    def pinned_array(self, shape, dtype=np.float32) -> np.ndarray:
        """numpy view of page-locked host memory (kept alive by the context)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = c_void_p()
        self._call("wdc_host_alloc", n, byref(p))
        buf = (ctypes.c_char * max(n, 1)).from_address(p.value)

        class _Pinned(np.ndarray):
            _wdc_pinned = True

        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape).view(_Pinned)
        return arr

    # --- BackendContext
    def is_cuda_tensor(self, t) -> bool:
        return isinstance(t, CudaTensor)

    def asserts_cuda_tensor(self, t) -> None:
        if not isinstance(t, CudaTensor):
            raise TypeError("tensor is not CudaTensor")
        if t.context is not self:
            # another context's arena (possibly another GPU): its memory is not ordered with this stream
            raise TypeError("CudaTensor belongs to another cuda context")

    def asserts_cuda_tensor_array(self, tensors) -> None:
        for t in tensors:
            self.asserts_cuda_tensor(t)

    def empty_tensor(self, dims: Sequence[int], data_type: str = "float32", layout: str = "nchw") -> CudaTensor:
        return CudaTensor(self, dims, data_type, layout=layout)

    def move_tensor(self, tensor, option=None) -> CudaTensor:
        if isinstance(tensor, EightbitCPUTensor):
            return self.decode_eightbit(tensor.codes, tensor.scale, tensor.dims)
        dst = CudaTensor(self, tensor.dims, tensor.data_type)
        dst.set_data(tensor.get_data())
        return dst

    def decode_eightbit(self, codes: np.ndarray, scale: float, dims: Sequence[int]) -> CudaTensor:
        """float32 tensor from the 8-bit codes of a WDN2 container: the codes (1 byte per element)
        are uploaded and expanded on the device."""
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        dst = CudaTensor(self, dims, "float32")
        if dst.length != codes.size:
            raise ValueError("decode_eightbit: code count does not match dims")
        if codes.size:
            staging = self._alloc(codes.size)
            try:
                self._upload(staging, codes)
                self._call("wdc_decode_eightbit", c_void_p(staging), c_void_p(dst.ptr), codes.size,
                           ctypes.c_float(scale))
            finally:
                self._free(staging)  # stream-ordered: reused only by work queued after the decode
        return dst

    def prefetch_tensor(self, tensor: CPUTensor) -> CudaTensor:
        """Like move_tensor, but the transfer runs on the context's copy stream, so that it overlaps
        the kernels already queued (the next batch moves while the current one is computed).  The
        source array should be pinned (pinned_array) and must stay unchanged until the tensor has
        been used; Runner.run orders its first kernel after the transfer."""
        dst = CudaTensor(self, tensor.dims, tensor.data_type)
        arr = np.ascontiguousarray(np.asarray(tensor.data).reshape(-1), dtype=NP_DTYPE[tensor.data_type])
        ticket = ctypes.c_int64()
        # (dst was allocated two lines up: nothing queued touches it, so the transfer need not wait for queued runs)
        self._call("wdc_upload_fresh_async", c_void_p(dst.ptr), arr.ctypes.data_as(c_void_p), arr.nbytes, byref(ticket))
        dst.upload_ticket = ticket.value
        dst._prefetch_source = arr  # keeps the host memory alive until the tensor goes away
        return dst

    # --- capture of a run into a CUDA graph
    def capture_begin(self) -> None:
        self._call("wdc_capture_begin")

    def capture_end(self) -> int:
        g = c_void_p()
        self._call("wdc_capture_end", byref(g))
        return g.value

    def graph_launch(self, graph: int) -> None:
        self._call("wdc_graph_launch", c_void_p(graph))

    def graph_destroy(self, graph: int) -> None:
        if self.handle is not None:
            self._call("wdc_graph_destroy", c_void_p(graph))

    def peer_copy_from(self, dst: CudaTensor, dst_offset: int, src_context: "WebDNNCudaContext", src: CudaTensor,
                       n_elements: int) -> None:
        """dst[dst_offset : dst_offset + n] <- src[0 : n] across devices (NVLink peer copy, ordered after
        the work queued on the source's stream and before later work on this context's stream)."""
        if dst.data_type != src.data_type:
            raise TypeError("peer_copy_from: dtype mismatch")
        if dst_offset < 0 or n_elements < 0 or dst_offset + n_elements > dst.length or n_elements > src.length:
            raise ValueError("peer_copy_from: range out of bounds")
        st = self._L.lib.wdc_peer_copy(self.handle, c_void_p(dst.ptr + 4 * dst_offset), src_context.handle,
                                       c_void_p(src.ptr), 4 * n_elements)
        if st != 0:
            self._L.check(self.handle, st)

    def download_async(self, t: CudaTensor) -> "PendingDownload":
        """Starts the device-to-host transfer of a tensor's (canonical) contents on the download stream and returns at
        once; ``PendingDownload.result()`` waits for it.  Work queued on the context after this call does not delay
        the transfer and is not delayed by it."""
        src = self.canonical(t)
        n = max(t.length, 1)
        host = self._download_buffer(n, t.data_type)
        ticket = ctypes.c_int64()
        self._call("wdc_download_async", host.ctypes.data_as(c_void_p), c_void_p(src.ptr), t.length * 4, byref(ticket))
        return PendingDownload(self, t, src, host, ticket.value)

    def _download_buffer(self, n: int, data_type: str) -> np.ndarray:
        """A pinned staging array of at least n elements, reused round-robin (pinned allocations are slow)."""
        pool = self.__dict__.setdefault("_dl_pool", {})
        key = (n, data_type)
        ring = pool.setdefault(key, {"bufs": [], "next": 0})
        if len(ring["bufs"]) < 4:
            ring["bufs"].append(self.pinned_array((n,), NP_DTYPE[data_type]))
            return ring["bufs"][-1]
        ring["next"] = (ring["next"] + 1) % len(ring["bufs"])
        return ring["bufs"][ring["next"]]

    def wait_upload(self, t: CudaTensor) -> None:
        """Compute stream waits (on the device, not the host) for the tensor's pending transfer."""
        if t.upload_ticket is not None:
            self._call("wdc_wait_upload", t.upload_ticket)
            t.upload_ticket = None

    # --- layout helpers
    def canonical(self, t: CudaTensor) -> CudaTensor:
        """Return ``t`` itself if it is stored row-major, else a converted copy."""
        if t.layout == "nchw":
            return t
        n, c, h, w = t.dims
        if c == 1 or h * w == 1:
            t.shared_buffer.incr_ref()
            return CudaTensor(self, t.dims, t.data_type, t.shared_buffer)
        out = CudaTensor(self, t.dims, t.data_type)
        self.strided_copy(t, out, t.dims, t.nchw_strides(), 0, out.strides, 0)
        return out

    def channels_last(self, t: CudaTensor) -> CudaTensor:
        if t.layout == "nhwc":
            return t
        n, c, h, w = t.dims
        if c == 1 or h * w == 1:
            t.shared_buffer.incr_ref()
            return CudaTensor(self, t.dims, t.data_type, t.shared_buffer, layout="nhwc")
        out = CudaTensor(self, t.dims, t.data_type, layout="nhwc")
        # iterate destination in (n, h, w, c) order
        self.strided_copy(t, out, [n, h, w, c], [c * h * w, w, 1, h * w], 0, [h * w * c, w * c, c, 1], 0)
        return out

    # --- kernel launchers (one per C entry point)
    def strided_copy(self, src: CudaTensor, dst: CudaTensor, dims, sstr, soff, dstr, doff) -> None:
        self._call("wdc_strided_copy", c_void_p(src.ptr), c_void_p(dst.ptr), len(dims), i64_array(dims),
                   i64_array(sstr), soff, i64_array(dstr), doff)

    def unary(self, op: int, src: CudaTensor, dst: CudaTensor, p0: float = 0.0, p1: float = 0.0) -> None:
        self._call("wdc_unary", op, DTYPE_CODE[src.data_type], c_void_p(src.ptr), c_void_p(dst.ptr),
                   src.length, p0, p1)

    def binary(self, op: int, a: CudaTensor, b: CudaTensor, out: CudaTensor, dims, sa, sb) -> None:
        self._call("wdc_binary", op, DTYPE_CODE[a.data_type], c_void_p(a.ptr), c_void_p(b.ptr),
                   c_void_p(out.ptr), len(dims), i64_array(dims), i64_array(sa), i64_array(sb))

    def gemm(self, desc: GemmDesc, a: CudaTensor, b: CudaTensor, c: Optional[CudaTensor], y: CudaTensor) -> None:
        self._call("wdc_gemm", byref(desc), c_void_p(a.ptr), c_void_p(b.ptr),
                   c_void_p(c.ptr) if c is not None else None, c_void_p(y.ptr))

    def conv2d(self, desc: ConvDesc, x, w, scale, shift, residual, y) -> None:
        def p(t):
            return c_void_p(t.ptr) if t is not None else None
        self._call("wdc_conv2d", byref(desc), p(x), p(w), p(scale), p(shift), p(residual), p(y))

    def pool(self, kind: str, desc: PoolDesc, x: CudaTensor, y: CudaTensor) -> None:
        self._call("wdc_maxpool2d" if kind == "max" else "wdc_avgpool2d", byref(desc), c_void_p(x.ptr),
                   c_void_p(y.ptr))
