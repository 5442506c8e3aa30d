"""The public C boundary (libclDNN64.so, include/cldnn_c_api.h) against the reference's own api/C headers -- no GPU needed.

* binary layout: the probe tests/api_cpp/abi_probe.cpp compiled against include/cldnn_c_api.h prints exactly what it printed
  when compiled against the reference's headers (golden text made by tests/golden/make_c_abi_layout.py); with the clDNN
  tree at hand (CLDNN_REFERENCE_ROOT) the golden text itself is re-derived and compared;
* exports: every CLDNN_API function the header declares is exported by the library;
* error convention: without a CUDA device cldnn_create_engine returns NULL with CLDNN_DEVICE_ERROR and a message --
  there is no CPU fallback behind this boundary; a primitive type the path does not implement is refused, not emulated.
"""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "cldnn_c_api.h")
LIB = os.path.join(ROOT, "cldnn_b200", "libclDNN64.so")
GOLDEN = os.path.join(ROOT, "tests", "golden", "cldnn_c_abi_layout.txt")
PROBE = os.path.join(ROOT, "tests", "api_cpp", "abi_probe.cpp")


def test_header_has_the_layout_of_the_reference_headers(tmp_path):
    exe = str(tmp_path / "probe")
    subprocess.check_call(["g++", "-std=c++14", "-I" + os.path.join(ROOT, "include"), "-o", exe, PROBE])
    mine = subprocess.check_output([exe]).decode()
    assert mine == open(GOLDEN).read()
    assert len(mine.splitlines()) > 150


def test_golden_layout_matches_the_reference_tree_when_present():
    import ref_lib
    ref = ref_lib.REFERENCE_ROOT
    if not os.path.isfile(os.path.join(ref, "api", "C", "cldnn.h")):
        pytest.skip("clDNN tree not at hand (CLDNN_REFERENCE_ROOT)")
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_c_abi_layout
    assert make_c_abi_layout.layout_from_reference(ref) == open(GOLDEN).read()


def _declared():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"CLDNN_API[^;(]*?\b(cldnn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_entry_point():
    names = _declared()
    assert len(names) >= 65 and "cldnn_add_primitive" in names and "cldnn_fused_conv_eltwise_type_id" in names
    lib = C.CDLL(LIB)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_status_convention_without_a_device_and_for_unknown_primitives():
    lib = C.CDLL(LIB)
    lib.cldnn_get_last_error_message.restype = C.c_char_p
    lib.cldnn_create_topology.restype = C.c_void_p
    lib.cldnn_create_engine.restype = C.c_void_p
    st = C.c_int32(123)
    topo = lib.cldnn_create_topology(C.byref(st))
    assert topo and st.value == 0
    # a descriptor whose type is not one of this library's primitive types
    class Head(C.Structure):
        _fields_ = [("type", C.c_void_p), ("id", C.c_char_p), ("in_data", C.c_void_p), ("in_size", C.c_size_t), ("rest", C.c_char * 160)]
    bogus_type = C.create_string_buffer(64)
    d = Head(C.cast(bogus_type, C.c_void_p), b"mystery", None, 0)
    lib.cldnn_add_primitive(C.c_void_p(topo), C.byref(d), C.byref(st))
    assert st.value == -6                                         # CLDNN_UNSUPPORTED_FORMAT
    assert b"mystery" in lib.cldnn_get_last_error_message()
    lib.cldnn_add_primitive(C.c_void_p(topo), None, C.byref(st))
    assert st.value == -1 and b"should not be null" in lib.cldnn_get_last_error_message()
    lib.cldnn_release_topology(C.c_void_p(topo), C.byref(st))
    assert st.value == 0
    import torch
    if not torch.cuda.is_available():
        eng = lib.cldnn_create_engine(0, 0, None, C.byref(st))
        assert not eng and st.value == -4                         # CLDNN_DEVICE_ERROR: no CPU fallback
        assert b"no CUDA device" in lib.cldnn_get_last_error_message() or b"CPU fallback" in lib.cldnn_get_last_error_message()
    # half-precision helpers (src/half.cpp) are pure host code
    lib.cldnn_float_to_half.restype = C.c_uint16
    lib.cldnn_float_to_half.argtypes = [C.c_float, C.POINTER(C.c_int32)]
    lib.cldnn_half_to_float.restype = C.c_float
    lib.cldnn_half_to_float.argtypes = [C.c_uint16, C.POINTER(C.c_int32)]
    import numpy as np
    for v in (0.0, 1.0, -2.5, 65504.0, 1e-7, 6.1e-5, 0.333251953125, 1e9, -1e-9):
        want = np.float32(v).astype(np.float16)
        got = lib.cldnn_float_to_half(v, None)
        assert got == int(want.view(np.uint16)), v
        assert lib.cldnn_half_to_float(got, None) == float(want) or (np.isinf(float(want)) and np.isinf(lib.cldnn_half_to_float(got, None)))
