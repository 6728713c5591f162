"""CPU: the C-ABI library loads and exports every function include/webdnn_cuda.h declares, and the
ctypes binding covers exactly that set (no compute calls: there is no GPU here)."""
import ctypes
import os
import re

from webdnn_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    with open(os.path.join(ROOT, "include", "webdnn_cuda.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(wdc_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_functions()
    assert len(names) >= 30
    for must in ("wdc_create", "wdc_alloc", "wdc_upload", "wdc_download", "wdc_gemm", "wdc_conv2d", "wdc_lstm"):
        assert must in names


def test_library_exports_every_declared_symbol():
    so = ctypes.CDLL(lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(so, name), f"{name} declared in include/webdnn_cuda.h but not exported"


def test_binding_matches_header():
    assert sorted(lib.SIGNATURES) == declared_functions()
    lib.load_library()


def test_calls_without_a_gpu_fail_with_status_not_crash():
    so = lib.load_library()
    n = ctypes.c_int(-1)
    st = so.wdc_device_count(ctypes.byref(n))
    if st != 0 or n.value == 0:
        h = ctypes.c_void_p()
        assert so.wdc_create(0, 0, ctypes.byref(h)) != 0
        assert so.wdc_last_error(None)
    assert so.wdc_sync(None) == lib.WDC_ERR_INVALID
    assert so.wdc_free(None, None) == lib.WDC_ERR_INVALID


def test_struct_layouts_match_header_field_counts():
    assert len(lib.GemmDesc._fields_) == 15 and ctypes.sizeof(lib.GemmDesc) == 12 * 8 + 3 * 4 + 4
    assert len(lib.ConvDesc._fields_) == 18 and ctypes.sizeof(lib.ConvDesc) == 16 * 8 + 8
    assert len(lib.PoolDesc._fields_) == 23 and ctypes.sizeof(lib.PoolDesc) == 22 * 8 + 8
    assert len(lib.ConvTransposeDesc._fields_) == 17 and ctypes.sizeof(lib.ConvTransposeDesc) == 17 * 8
    assert len(lib.AttentionDesc._fields_) == 18 and ctypes.sizeof(lib.AttentionDesc) == 17 * 8 + 8
