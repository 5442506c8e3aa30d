"""Loader and thin numpy front-end for the CPU oracle (oracle/libcldnn_oracle.so).

Test infrastructure: imported only by tests, the smoke entry and the bench's
CPU-baseline leg.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from cldnn_b200 import abi

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_ROOT, "oracle", "libcldnn_oracle.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(_ROOT, "oracle", "cldnn_oracle.c")
        if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", os.path.join(_ROOT, "oracle"), "libcldnn_oracle.so"],
                                  stdout=subprocess.DEVNULL)
        _lib = C.CDLL(_SO)
        _lib.oracle_conv.argtypes = [C.POINTER(abi.ConvParams), C.POINTER(abi.Args), C.c_int32]
        _lib.oracle_conv_range.argtypes = [C.POINTER(abi.ConvParams), C.POINTER(abi.Args), C.c_int64, C.c_int64, C.c_int32]
        _lib.oracle_pooling.argtypes = [C.POINTER(abi.PoolParams), C.c_void_p, C.c_void_p, C.c_int32]
        _lib.oracle_fc.argtypes = [C.POINTER(abi.FcParams), C.POINTER(abi.Args), C.c_int32, C.POINTER(C.c_int64)]
        _lib.oracle_softmax.argtypes = [C.POINTER(abi.SoftmaxParams), C.c_void_p, C.c_void_p]
        _lib.oracle_eltwise.argtypes = [C.POINTER(abi.EltwiseParams), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.oracle_reorder.argtypes = [C.POINTER(abi.ReorderParams), C.c_void_p, C.c_void_p]
        _lib.oracle_lrn.argtypes = [C.POINTER(abi.LrnParams), C.c_void_p, C.c_void_p]
        _lib.oracle_activation.argtypes = [C.POINTER(abi.ActivationParams), C.c_void_p, C.c_void_p]
        _lib.oracle_conv_out_size.argtypes = [C.c_int32] * 5
        _lib.oracle_pool_out_size.argtypes = [C.c_int32] * 4
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads():
    return lib().oracle_num_threads()


def conv(p, inp, w, bias=None, quant=None, calib=None, eltw=None, eltw_calib=None, out=None, threads=0):
    """Run the oracle convolution. Arrays are flat buffers laid out as `p` says.
    Returns the flat output buffer."""
    if out is None:
        n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
        out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    a = abi.Args()
    a.input0, a.input1, a.output, a.weights = _ptr(inp), _ptr(eltw), _ptr(out), _ptr(w)
    a.bias, a.weights_quantization_factors = _ptr(bias), _ptr(quant)
    a.output_calibration_factors, a.eltw_output_calibration_factors = _ptr(calib), _ptr(eltw_calib)
    st = lib().oracle_conv(C.byref(p), C.byref(a), threads or num_threads())
    assert st == 0, st
    return out


def pooling(p, inp, out=None, threads=0):
    if out is None:
        n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
        out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    assert lib().oracle_pooling(C.byref(p), _ptr(inp), _ptr(out), threads or num_threads()) == 0
    return out


def fc(p, inp, w, bias=None, quant=None, calib=None, out=None, threads=0):
    if out is None:
        n = max(p.out.b * p.out.pb, p.out.f * p.out.pf) + p.out.offset
        out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    a = abi.Args()
    a.input0, a.output, a.weights, a.bias = _ptr(inp), _ptr(out), _ptr(w), _ptr(bias)
    a.weights_quantization_factors, a.output_calibration_factors = _ptr(quant), _ptr(calib)
    oor = C.c_int64(0)
    assert lib().oracle_fc(C.byref(p), C.byref(a), threads or num_threads(), C.byref(oor)) == 0
    return out, oor.value


def softmax(p, inp):
    n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
    out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    assert lib().oracle_softmax(C.byref(p), _ptr(inp), _ptr(out)) == 0
    return out


def eltwise(p, in0, in1, calib=None):
    n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
    out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    assert lib().oracle_eltwise(C.byref(p), _ptr(in0), _ptr(in1), _ptr(calib), _ptr(out)) == 0
    return out


def reorder(p, inp):
    n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
    out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    assert lib().oracle_reorder(C.byref(p), _ptr(inp), _ptr(out)) == 0
    return out


def lrn(p, inp):
    n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
    out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    assert lib().oracle_lrn(C.byref(p), _ptr(inp), _ptr(out)) == 0
    return out


def activation(p, inp):
    n = max(p.out.b * p.out.pb, p.out.f * p.out.pf, p.out.y * p.out.py, p.out.x * p.out.px) + p.out.offset
    out = np.zeros(int(n), dtype=abi.np_dtype_of(p.out.dtype))
    assert lib().oracle_activation(C.byref(p), _ptr(inp), _ptr(out)) == 0
    return out


def conv_out_size(n, k, offset, stride, dil=1):
    return lib().oracle_conv_out_size(n, k, offset, stride, dil)


def pool_out_size(n, k, offset, stride):
    return lib().oracle_pool_out_size(n, k, offset, stride)
