"""ctypes binding of libwebdnn_cuda.so (the C ABI declared in include/webdnn_cuda.h).

This is the Python stand-in for the N-API shim a Node.js host would use: it adds nothing to the
ABI, converts status codes into exceptions (as the wasm context turns worker errors into JS
errors, ``backend/wasm/wasmContextImpl.ts:57-62``) and never computes anything on the CPU.
If the shared library is missing the import fails loudly; there is no fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libwebdnn_cuda.so")

WDC_OK, WDC_ERR_INVALID, WDC_ERR_CUDA, WDC_ERR_OOM, WDC_ERR_UNSUPPORTED, WDC_ERR_DEVICE_WAIT = range(6)
STATUS_NAMES = ["ok", "invalid argument", "cuda error", "out of memory", "unsupported", "device wait expired"]

DTYPE_CODE = {"float32": 0, "int32": 1, "bool": 2}

UNARY_OPS = {
    "Abs": 0, "Acos": 1, "Acosh": 2, "Asin": 3, "Asinh": 4, "Atan": 5, "Atanh": 6, "Ceil": 7, "Cos": 8,
    "Cosh": 9, "Exp": 10, "Floor": 11, "HardSwish": 12, "Log": 13, "Neg": 14, "Reciprocal": 15,
    "Relu": 16, "Round": 17, "Sigmoid": 18, "Sign": 19, "Sin": 20, "Softplus": 21, "Softsign": 22,
    "Sqrt": 23, "Tan": 24, "Tanh": 25, "Elu": 32, "HardSigmoid": 33, "LeakyRelu": 34, "Selu": 35,
    "ThresholdedRelu": 36, "Clip": 40, "Identity": 41,
}
BINARY_OPS = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3, "Pow": 4, "Max": 5, "Min": 6}
REDUCE_KINDS = {"ReduceSum": 0, "ReduceMean": 1, "ReduceMax": 2, "ReduceMin": 3, "ReduceProd": 4,
                "ReduceL1": 5, "ReduceL2": 6, "ReduceLogSum": 7, "ReduceLogSumExp": 8,
                "ReduceSumSquare": 9}


class CudaBackendError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"webdnn cuda backend: {STATUS_NAMES[status] if 0 <= status < 6 else status}: {message}")
        self.status = status


class GemmDesc(Structure):
    _fields_ = [("batch", c_int64), ("m", c_int64), ("n", c_int64), ("k", c_int64),
                ("sab", c_int64), ("sa0", c_int64), ("sa1", c_int64),
                ("sbb", c_int64), ("sb0", c_int64), ("sb1", c_int64),
                ("sc0", c_int64), ("sc1", c_int64),
                ("alpha", c_float), ("beta", c_float), ("relu", c_int)]


class ConvDesc(Structure):
    _fields_ = [(n, c_int64) for n in (
        "batch", "ch_in", "in_h", "in_w", "ch_out", "k_h", "k_w", "out_h", "out_w",
        "stride_h", "stride_w", "pad_t", "pad_l", "dil_h", "dil_w", "group")] + [("relu", c_int), ("x_nchw", c_int)]


class ConvTransposeDesc(Structure):
    _fields_ = [(n, c_int64) for n in ("batch", "ch_in", "in_h", "in_w", "ch_out_per_group", "group", "k_h", "k_w",
                                       "out_h", "out_w", "stride_h", "stride_w", "pad_t", "pad_l", "dil_h", "dil_w",
                                       "w_layout")]


class AttentionDesc(Structure):
    _fields_ = [(n, c_int64) for n in ("batch", "heads", "tq", "tk", "dh", "q_sb", "q_sh", "q_st", "k_sb", "k_sh",
                                       "k_st", "v_sb", "v_sh", "v_st", "y_sb", "y_sh", "y_st")] + [("scale", c_float)]


class PoolDesc(Structure):
    _fields_ = [(n, c_int64) for n in (
        "batch", "ch", "in_h", "in_w", "out_h", "out_w", "k_h", "k_w", "stride_h", "stride_w",
        "pad_t", "pad_l", "dil_h", "dil_w", "xs_n", "xs_c", "xs_h", "xs_w",
        "ys_n", "ys_c", "ys_h", "ys_w")] + [("count_include_pad", c_int)]


I64P = POINTER(c_int64)

# name -> (restype, argtypes); every function include/webdnn_cuda.h declares
SIGNATURES = {
    "wdc_device_count": (c_int, [POINTER(c_int)]),
    "wdc_create": (c_int, [c_int, c_int64, POINTER(c_void_p)]),
    "wdc_destroy": (c_int, [c_void_p]),
    "wdc_last_error": (c_char_p, [c_void_p]),
    "wdc_alloc": (c_int, [c_void_p, c_int64, POINTER(c_void_p)]),
    "wdc_free": (c_int, [c_void_p, c_void_p]),
    "wdc_host_alloc": (c_int, [c_void_p, c_int64, POINTER(c_void_p)]),
    "wdc_host_free": (c_int, [c_void_p, c_void_p]),
    "wdc_upload": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "wdc_conv_transpose2d": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "wdc_instance_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                  ctypes.c_double]),
    "wdc_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "wdc_decode_eightbit": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_float]),
    "wdc_capture_begin": (c_int, [c_void_p]),
    "wdc_capture_end": (c_int, [c_void_p, POINTER(c_void_p)]),
    "wdc_graph_launch": (c_int, [c_void_p, c_void_p]),
    "wdc_graph_destroy": (c_int, [c_void_p, c_void_p]),
    "wdc_upload_async": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, POINTER(c_int64)]),
    "wdc_upload_fresh_async": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, POINTER(c_int64)]),
    "wdc_wait_upload": (c_int, [c_void_p, c_int64]),
    "wdc_download_async": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, POINTER(c_int64)]),
    "wdc_wait_download": (c_int, [c_void_p, c_int64]),
    "wdc_download": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "wdc_copy": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "wdc_fill_u32": (c_int, [c_void_p, c_void_p, c_uint32, c_int64]),
    "wdc_sync": (c_int, [c_void_p]),
    "wdc_stream": (c_void_p, [c_void_p]),
    "wdc_stats": (c_int, [c_void_p, I64P, c_int]),
    "wdc_reset_stats": (c_int, [c_void_p]),
    "wdc_profile_enable": (c_int, [c_void_p, c_int]),
    "wdc_profile_read": (c_int, [c_void_p, c_int, POINTER(ctypes.c_double), POINTER(c_int64), POINTER(ctypes.c_double)]),
    "wdc_peer_copy": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64]),
    "wdc_unary": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_float, c_float]),
    "wdc_binary": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P]),
    "wdc_cast": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64]),
    "wdc_channel_affine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int]),
    "wdc_gemm": (c_int, [c_void_p, POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p]),
    "wdc_conv2d": (c_int, [c_void_p, POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "wdc_pack_conv_weight": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64]),
    "wdc_maxpool2d": (c_int, [c_void_p, POINTER(PoolDesc), c_void_p, c_void_p]),
    "wdc_avgpool2d": (c_int, [c_void_p, POINTER(PoolDesc), c_void_p, c_void_p]),
    "wdc_global_avgpool": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64]),
    "wdc_softmax": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64]),
    "wdc_reduce_axis": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64]),
    "wdc_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float]),
    "wdc_argmax": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int]),
    "wdc_strided_copy": (c_int, [c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, c_int64, I64P, c_int64]),
    "wdc_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64]),
    "wdc_lstm": (c_int, [c_void_p] + [c_void_p] * 9 + [c_int64] * 4),
    "wdc_lstm_static": (c_int, [c_void_p] + [c_void_p] * 9 + [c_int64] * 4),
    "wdc_selftest_device_wait": (c_int, [c_void_p, c_int64]),
    "wdc_set_option": (c_int, [c_void_p, c_char_p, c_int64]),
    "wdc_range_push": (c_int, [c_void_p, c_char_p]),
    "wdc_range_pop": (c_int, [c_void_p]),
}

_lib = None


def load_library() -> ctypes.CDLL:
    """Load the shared library and bind every declared entry point; raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m webdnn_b200.build` "
            "(the cuda backend has no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def i64_array(values) -> ctypes.Array:
    return (c_int64 * max(len(values), 1))(*[int(v) for v in values])


class Library:
    """Thin checked-call wrapper bound to one context handle."""

    def __init__(self):
        self.lib = load_library()

    def check(self, ctx, status: int) -> None:
        if status != WDC_OK:
            msg = self.lib.wdc_last_error(ctx)
            raise CudaBackendError(status, msg.decode("utf-8", "replace") if msg else "")

    def device_count(self) -> int:
        n = c_int(0)
        st = self.lib.wdc_device_count(byref(n))
        return n.value if st == WDC_OK else 0
