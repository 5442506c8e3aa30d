"""Loader for oracle/_ref: the reference's own reference convolution kernel (its .cl source compiled as C++ by
oracle/ref_build/build_variant.py).  A missing variant is built on the spot when the clDNN tree is present; machines
without the tree use the prebuilt files.  Test infrastructure."""
import ctypes as C
import importlib.util
import os

import numpy as np

from cldnn_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
def _reference_root():
    """The clDNN source tree: CLDNN_REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    env = os.environ.get("CLDNN_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(ROOT), "reference")


REFERENCE_ROOT = _reference_root()
_T = {abi.I8: "c", abi.U8: "uc", abi.F32: "f"}
_libs = {}


def _builder():
    spec = importlib.util.spec_from_file_location("build_variant", os.path.join(ROOT, "oracle", "ref_build", "build_variant.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def variant_of(p):
    if p.in_.dtype not in _T or p.out.dtype not in _T or p.groups < 1:
        return None
    bias = {abi.NONE: "n", abi.I32: "i", abi.F32: "f"}.get(p.bias_dtype)
    if bias is None:
        return None
    e = _T.get(p.eltw.dtype, "c") if p.fused_eltw else "c"
    return "%s_%s_%s_b%s_q%dc%do%d_f%dn%de%d" % (_T[p.in_.dtype], _T[p.out.dtype], e, bias, p.quantization, p.calibration, p.has_o_qf,
                                                 p.fused_eltw, p.has_non_conv_scale if p.fused_eltw else 0, p.eltw_calibration if p.fused_eltw else 0)


def available(p):
    name = variant_of(p)
    if name is None or p.in_out_opt:
        return False
    return os.path.exists(os.path.join(REF_DIR, "clref_%s.so" % name)) or os.path.isdir(os.path.join(REFERENCE_ROOT, "kernel_selector"))


def _load(name):
    if name not in _libs:
        so = os.path.join(REF_DIR, "clref_%s.so" % name)
        if not os.path.exists(so):
            _builder().build(REFERENCE_ROOT, name)
        lib = C.CDLL(so)
        lib.clref_run.argtypes = [C.POINTER(abi.ConvParams), C.POINTER(abi.Args), C.c_long, C.c_long, C.c_int]
        _libs[name] = lib
    return _libs[name]


def conv(p, inp, w, bias=None, quant=None, calib=None, eltw=None, eltw_calib=None, threads=1, out=None):
    """Same calling convention as oracle_lib.conv; runs the reference's kernel source."""
    lib = _load(variant_of(p))
    if out is None:
        n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
        out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    ptr = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
    a = abi.Args()
    a.input0, a.input1, a.output, a.weights, a.bias = ptr(inp), ptr(eltw), ptr(out), ptr(w), ptr(bias)
    a.weights_quantization_factors, a.output_calibration_factors, a.eltw_output_calibration_factors = ptr(quant), ptr(calib), ptr(eltw_calib)
    assert lib.clref_run(C.byref(p), C.byref(a), 0, p.out.b * p.out.f, threads) == 0
    return out
