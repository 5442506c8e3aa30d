"""ctypes mirror of include/cldnn_b200.h.

Field order and types follow the header exactly; `tests/test_abi_layout.py`
checks the sizes against the compiled library.  Nothing here computes: the
structures only describe tensors and launch constants to the C ABI.
"""
import ctypes as C

import numpy as np

SUCCESS = 0
ERROR = -1
INVALID_ARG = -2
OUT_OF_RESOURCES = -3
DEVICE_ERROR = -4
UNSUPPORTED_SIZE = -5
UNSUPPORTED_FORMAT = -6
DIMENSION_MISMATCH = -7

I8, U8, I32, F16, F32, NONE = 0x01, 0x41, 0x04, 0x82, 0x84, 0x00

ACT_NONE, ACT_RELU, ACT_RELU_NEGATIVE_SLOPE, ACT_CLAMP = 0, 1, 2, 3
EPILOGUE_REF, EPILOGUE_MMAD, EPILOGUE_IMAD = 0, 1, 2       # cldnn_b200_conv_params.epilogue_order
ACT_LOGISTIC, ACT_TANH, ACT_ABS, ACT_LINEAR, ACT_SQUARE, ACT_SQRT, ACT_ELU = 4, 5, 6, 7, 8, 9, 10

POOL_MAX, POOL_AVG = 0, 1
DIV_FIXED, DIV_DYNAMIC, DIV_DYNAMIC_WITH_PADDING = 0, 1, 2
ELTW_SUM, ELTW_SUB, ELTW_MAX, ELTW_PROD, ELTW_MIN = 0, 1, 2, 3, 4

_NP2DT = {np.dtype(np.int8): I8, np.dtype(np.uint8): U8, np.dtype(np.int32): I32,
          np.dtype(np.float16): F16, np.dtype(np.float32): F32}
_DT2NP = {v: k for k, v in _NP2DT.items()}


def dtype_of(np_dtype):
    return _NP2DT[np.dtype(np_dtype)]


def np_dtype_of(dt):
    return _DT2NP[dt]


def dtype_size(dt):
    return dt & 0x0F


class Tensor(C.Structure):
    _fields_ = [("dtype", C.c_int32),
                ("b", C.c_int32), ("f", C.c_int32), ("y", C.c_int32), ("x", C.c_int32),
                ("pb", C.c_int64), ("pf", C.c_int64), ("py", C.c_int64), ("px", C.c_int64),
                ("offset", C.c_int64)]

    def shape(self):
        return (self.b, self.f, self.y, self.x)


class ConvParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor), ("eltw", Tensor),
                ("w_dtype", C.c_int32), ("ofm", C.c_int32), ("ifm", C.c_int32),
                ("kh", C.c_int32), ("kw", C.c_int32),
                ("w_po", C.c_int64), ("w_pi", C.c_int64), ("w_py", C.c_int64), ("w_px", C.c_int64),
                ("w_offset", C.c_int64),
                ("stride_x", C.c_int32), ("stride_y", C.c_int32),
                ("pad_x", C.c_int32), ("pad_y", C.c_int32),
                ("dil_x", C.c_int32), ("dil_y", C.c_int32),
                ("groups", C.c_int32), ("bias_dtype", C.c_int32),
                ("quantization", C.c_int32), ("i_qf", C.c_float),
                ("calibration", C.c_int32), ("has_o_qf", C.c_int32), ("o_qf", C.c_float),
                ("act", C.c_int32), ("act_m", C.c_float), ("act_n", C.c_float),
                ("fused_eltw", C.c_int32),
                ("has_non_conv_scale", C.c_int32), ("non_conv_scale", C.c_float),
                ("eltw_act", C.c_int32), ("eltw_m", C.c_float), ("eltw_n", C.c_float),
                ("eltw_calibration", C.c_int32),
                ("eltw_stride_x", C.c_int32), ("eltw_stride_y", C.c_int32),
                ("in_out_opt", C.c_int32),
                ("tune", C.c_int32), ("epilogue_order", C.c_int32), ("reserved", C.c_int32 * 6)]


class Args(C.Structure):
    _fields_ = [("input0", C.c_void_p), ("input1", C.c_void_p), ("output", C.c_void_p),
                ("weights", C.c_void_p), ("bias", C.c_void_p),
                ("weights_quantization_factors", C.c_void_p),
                ("output_calibration_factors", C.c_void_p),
                ("eltw_output_calibration_factors", C.c_void_p),
                ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t)]


class PoolParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor),
                ("mode", C.c_int32), ("div_mode", C.c_int32),
                ("size_x", C.c_int32), ("size_y", C.c_int32),
                ("stride_x", C.c_int32), ("stride_y", C.c_int32),
                ("pad_x", C.c_int32), ("pad_y", C.c_int32),
                ("act", C.c_int32), ("act_m", C.c_float), ("act_n", C.c_float),
                ("reserved", C.c_int32 * 4)]


class FcParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor),
                ("w_dtype", C.c_int32),
                ("w_po", C.c_int64), ("w_pi", C.c_int64), ("w_py", C.c_int64), ("w_px", C.c_int64),
                ("w_offset", C.c_int64),
                ("bias_dtype", C.c_int32),
                ("quantization", C.c_int32), ("i_qf", C.c_float),
                ("calibration", C.c_int32), ("o_qf", C.c_float),
                ("act", C.c_int32), ("act_m", C.c_float), ("act_n", C.c_float),
                ("reserved", C.c_int32 * 4)]


class SoftmaxParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor), ("dimension", C.c_int32), ("reserved", C.c_int32 * 3)]


SOFTMAX_F, SOFTMAX_X, SOFTMAX_Y, SOFTMAX_FYX = 0, 1, 2, 3


class EltwiseParams(C.Structure):
    _fields_ = [("in0", Tensor), ("in1", Tensor), ("out", Tensor),
                ("mode", C.c_int32),
                ("stride_x0", C.c_int32), ("stride_y0", C.c_int32),
                ("stride_x1", C.c_int32), ("stride_y1", C.c_int32),
                ("quantization", C.c_int32), ("calibration", C.c_int32), ("o_qf", C.c_float),
                ("act", C.c_int32), ("act_m", C.c_float), ("act_n", C.c_float),
                ("reserved", C.c_int32 * 4)]


class ReorderParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor),
                ("has_mean", C.c_int32), ("mean", C.c_float * 4),
                ("reserved", C.c_int32 * 4)]


class LrnParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor),
                ("size", C.c_int32), ("k", C.c_float), ("alpha", C.c_float), ("beta", C.c_float),
                ("reserved", C.c_int32 * 4)]


class ActivationParams(C.Structure):
    _fields_ = [("in_", Tensor), ("out", Tensor),
                ("act", C.c_int32), ("act_m", C.c_float), ("act_n", C.c_float),
                ("reserved", C.c_int32 * 4)]


class EngineInfo(C.Structure):
    _fields_ = [("cores_count", C.c_uint32), ("core_frequency", C.c_uint32),
                ("max_alloc_mem_size", C.c_uint64), ("max_global_mem_size", C.c_uint64),
                ("max_local_mem_size", C.c_uint64), ("max_work_group_size", C.c_uint32),
                ("supports_fp16", C.c_uint32), ("supports_imad", C.c_uint32), ("supports_immad", C.c_uint32),
                ("compute_major", C.c_uint32), ("compute_minor", C.c_uint32),
                ("name", C.c_char * 64)]


# ---- tensor descriptors for the clDNN activation formats ---------------------
def tensor(dtype, b, f, y, x, fmt="bfyx", f_align=1, pad_lo=(0, 0), pad_hi=(0, 0)):
    """Descriptor of a dense tensor in a clDNN format (api/CPP/tensor.hpp:81-195).

    fmt: "bfyx" (NCHW), "byxf" (NHWC) or "yxfb".  f_align pads the stored
    feature count (byxf_af32-style).  pad_lo/pad_hi = (y, x) spatial padding
    kept in the buffer around the data (cldnn::padding).
    Returns (Tensor, element_count_of_buffer).
    """
    fs = -(-f // f_align) * f_align
    ys = y + pad_lo[0] + pad_hi[0]
    xs = x + pad_lo[1] + pad_hi[1]
    t = Tensor()
    t.dtype, t.b, t.f, t.y, t.x = dtype, b, f, y, x
    if fmt == "bfyx":
        t.px, t.py, t.pf, t.pb = 1, xs, xs * ys, xs * ys * fs
    elif fmt == "byxf":
        t.pf, t.px, t.py, t.pb = 1, fs, fs * xs, fs * xs * ys
    elif fmt == "yxfb":
        t.pb, t.pf, t.px, t.py = 1, b, b * fs, b * fs * xs
    else:
        raise ValueError("unknown format " + fmt)
    t.offset = pad_lo[0] * t.py + pad_lo[1] * t.px
    return t, b * fs * ys * xs


def to_layout(arr_bfyx, fmt="bfyx", f_align=1):
    """Lay a logical [b,f,y,x] numpy array out in `fmt`; returns a flat array."""
    b, f, y, x = arr_bfyx.shape
    fs = -(-f // f_align) * f_align
    if fs != f:
        padded = np.zeros((b, fs, y, x), dtype=arr_bfyx.dtype)
        padded[:, :f] = arr_bfyx
        arr_bfyx = padded
    if fmt == "bfyx":
        return np.ascontiguousarray(arr_bfyx).reshape(-1)
    if fmt == "byxf":
        return np.ascontiguousarray(arr_bfyx.transpose(0, 2, 3, 1)).reshape(-1)
    if fmt == "yxfb":
        return np.ascontiguousarray(arr_bfyx.transpose(2, 3, 1, 0)).reshape(-1)
    raise ValueError(fmt)


def from_layout(flat, shape_bfyx, fmt="bfyx", f_align=1):
    """Inverse of to_layout: returns the logical [b,f,y,x] array."""
    b, f, y, x = shape_bfyx
    fs = -(-f // f_align) * f_align
    if fmt == "bfyx":
        return flat.reshape(b, fs, y, x)[:, :f]
    if fmt == "byxf":
        return flat.reshape(b, y, x, fs).transpose(0, 3, 1, 2)[:, :f]
    if fmt == "yxfb":
        return flat.reshape(y, x, fs, b).transpose(3, 2, 0, 1)[:, :f]
    raise ValueError(fmt)


def set_weights(p, w_dtype, groups, ofm, ifm, kh, kw, layout="oiyx", i_align=1):
    """Fill the weights part of a ConvParams. layout "oiyx" (bfyx weights) or
    "oyxi" (input features innermost, padded to i_align)."""
    p.w_dtype, p.groups, p.ofm, p.ifm, p.kh, p.kw = w_dtype, groups, ofm, ifm, kh, kw
    if layout == "oiyx":
        p.w_px, p.w_py, p.w_pi, p.w_po = 1, kw, kw * kh, kw * kh * ifm
    elif layout == "oyxi":
        istore = -(-ifm // i_align) * i_align
        p.w_pi, p.w_px, p.w_py, p.w_po = 1, istore, istore * kw, istore * kw * kh
    else:
        raise ValueError(layout)
    p.w_offset = 0
