"""Seeded synthetic convolution cases shared by the CPU and GPU tests.

Value distributions follow the benchmark configuration: u8 activations uniform
in [0,255] (i8: [-128,127]), i8 weights uniform in [-127,127], i32 bias uniform
in [-4096,4096], per-output-channel f32 scales uniform in [2^-14, 2^-10].
"""
import ctypes as C

import numpy as np

from cldnn_b200 import abi


class ConvCase:
    """Holds the launch constants plus host arrays already laid out as the constants say."""

    def __init__(self):
        self.p = abi.ConvParams()
        self.inp = self.w = self.bias = self.quant = self.calib = self.eltw = self.ecal = None
        self.out_elems = 0
        self.out_fmt = "bfyx"
        self.out_f_align = 1


def conv_out(n, k, pad, stride, dil=1):
    return (n + 2 * pad - ((k - 1) * dil + 1)) // stride + 1


def make_conv_case(seed, N, C, K, H, W, kh=3, kw=3, stride=1, pad=1, dil=1,
                   in_dtype=np.uint8, out_dtype=np.int8, fmt="byxf", f_align=32,
                   bias="i32", quant=True, calib=False, act=abi.ACT_RELU,
                   fused=False, eltw_dtype=None, eltw_calib=False, non_conv_scale=1.0,
                   eltw_act=abi.ACT_RELU, in_out_opt=False, eltw_stride=1,
                   i_qf=1.0, o_qf=1.0, scale_lo=2.0 ** -14, scale_hi=2.0 ** -10,
                   w_layout=None, groups=1, w_range=127, out_fmt=None):
    rng = np.random.default_rng(seed)
    c = ConvCase()
    p = c.p
    P, Q = conv_out(H, kh, pad, stride, dil), conv_out(W, kw, pad, stride, dil)
    in_dtype, out_dtype = np.dtype(in_dtype), np.dtype(out_dtype)
    p.in_, _ = abi.tensor(abi.dtype_of(in_dtype), N, C, H, W, fmt, f_align)
    ofmt = out_fmt or fmt
    o_align = 32 if (ofmt == "byxf" and (out_fmt or f_align > 1)) else 1
    if ofmt == "byxf" and not out_fmt:
        o_align = f_align
    p.out, c.out_elems = abi.tensor(abi.dtype_of(out_dtype), N, K, P, Q, ofmt, o_align)
    c.out_fmt, c.out_f_align = ofmt, o_align
    if in_dtype == np.uint8:
        x = rng.integers(0, 256, size=(N, C, H, W), dtype=np.int64).astype(np.uint8)
    elif in_dtype == np.int8:
        x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int64).astype(np.int8)
    else:
        x = rng.standard_normal((N, C, H, W)).astype(in_dtype)
    c.x_logical = x
    c.inp = abi.to_layout(x, fmt, f_align)
    ifm = C // groups
    ofm = K // groups
    if in_dtype.kind in "iu":
        w = rng.integers(-w_range, w_range + 1, size=(K, ifm, kh, kw), dtype=np.int64).astype(np.int8)
    else:
        w = (rng.standard_normal((K, ifm, kh, kw)) * np.sqrt(2.0 / (ifm * kh * kw))).astype(in_dtype)
    c.w_logical = w
    if w_layout is None:
        w_layout = "oyxi" if fmt == "byxf" else "oiyx"
    if w_layout == "oyxi":
        cs = -(-ifm // f_align) * f_align
        wp = np.zeros((K, kh, kw, cs), dtype=w.dtype)
        wp[..., :ifm] = w.transpose(0, 2, 3, 1)
        c.w = wp.reshape(-1)
        abi.set_weights(p, abi.dtype_of(w.dtype), groups, ofm, ifm, kh, kw, "oyxi", f_align)
    else:
        c.w = np.ascontiguousarray(w).reshape(-1)
        abi.set_weights(p, abi.dtype_of(w.dtype), groups, ofm, ifm, kh, kw, "oiyx")
    p.stride_x = p.stride_y = stride
    p.pad_x = p.pad_y = pad
    p.dil_x = p.dil_y = dil
    if bias == "i32":
        c.bias = rng.integers(-4096, 4097, size=K, dtype=np.int64).astype(np.int32)
        p.bias_dtype = abi.I32
    elif bias == "f32":
        c.bias = rng.uniform(-8.0, 8.0, size=K).astype(np.float32)
        p.bias_dtype = abi.F32
    else:
        p.bias_dtype = abi.NONE
    p.quantization = int(quant)
    if quant:
        c.quant = rng.uniform(scale_lo, scale_hi, size=K).astype(np.float32)
    p.calibration = int(calib)
    if calib:
        c.calib = rng.uniform(0.5, 2.0, size=K).astype(np.float32)
    p.i_qf, p.o_qf = i_qf, o_qf
    p.has_o_qf = int(o_qf != 1.0 or (fused and quant))
    p.act = act
    p.act_m, p.act_n = 0.0, 6.0
    p.eltw_stride_x = p.eltw_stride_y = eltw_stride
    p.eltw_m, p.eltw_n = 0.0, 6.0
    if fused:
        p.fused_eltw = 1
        edt = np.dtype(eltw_dtype or out_dtype)
        p.in_out_opt = int(in_out_opt)
        if edt == np.uint8:
            e = rng.integers(0, 256, size=(N, K, P * eltw_stride, Q * eltw_stride), dtype=np.int64).astype(np.uint8)
        elif edt == np.int8:
            e = rng.integers(-128, 128, size=(N, K, P * eltw_stride, Q * eltw_stride), dtype=np.int64).astype(np.int8)
        else:
            e = rng.standard_normal((N, K, P * eltw_stride, Q * eltw_stride)).astype(edt)
        p.eltw, _ = abi.tensor(abi.dtype_of(edt), N, K, P * eltw_stride, Q * eltw_stride, ofmt, c.out_f_align)
        c.eltw = abi.to_layout(e, ofmt, c.out_f_align)
        p.has_non_conv_scale = int(non_conv_scale != 1.0)
        p.non_conv_scale = non_conv_scale
        p.eltw_act = eltw_act
        p.eltw_calibration = int(eltw_calib)
        if eltw_calib:
            c.ecal = rng.uniform(0.25, 1.0, size=K).astype(np.float32)
    c.shape_out = (N, K, P, Q)
    return c


def copy_params(p):
    q = type(p)()
    C.memmove(C.byref(q), C.byref(p), C.sizeof(p))
    return q


def run_oracle(case, threads=0):
    import oracle_lib
    out = None
    if case.p.in_out_opt:
        out = case.eltw.astype(abi.np_dtype_of(case.p.out.dtype)).copy()
    return oracle_lib.conv(case.p, case.inp, case.w, case.bias, case.quant, case.calib,
                           None if case.p.in_out_opt else case.eltw, case.ecal, out=out, threads=threads)


def run_gpu(engine, case, kernel="conv_i8_tc", tune=0):
    """Launch through the C ABI and return the flat output buffer."""
    from cldnn_b200 import engine as eng
    p = copy_params(case.p)
    p.tune = tune
    mems = {k: (engine.upload(v) if v is not None else None)
            for k, v in dict(inp=case.inp, w=case.w, bias=case.bias, quant=case.quant, calib=case.calib,
                             eltw=case.eltw, ecal=case.ecal).items()}
    out_dt = abi.np_dtype_of(p.out.dtype)
    if p.in_out_opt:
        out = engine.upload(case.eltw.astype(out_dt))
    else:
        out = engine.alloc(case.out_elems * out_dt.itemsize)
    import ctypes as _C
    k = engine.kernel(kernel)
    sb = _C.c_size_t()
    engine.lib.cldnn_b200_kernel_scratch_bytes(k.handle, _C.byref(p), _C.sizeof(p), _C.byref(sb))
    scratch = engine.alloc(sb.value) if sb.value else None
    mems["scratch"] = scratch
    args = eng.make_args(input0=mems["inp"], input1=None if p.in_out_opt else mems["eltw"], output=out, weights=mems["w"],
                         bias=mems["bias"], quant=mems["quant"], calib=mems["calib"], eltw_calib=mems["ecal"], scratch=scratch)
    engine.kernel(kernel).launch(p, args)
    engine.sync()
    res = out.read(out_dt, case.out_elems)
    status = engine.device_status()
    for m in list(mems.values()) + [out]:
        if m is not None:
            m.free()
    assert status == 0, "device status word 0x%x" % status
    return res


def logical_out(case, flat):
    return abi.from_layout(flat[:case.out_elems], case.shape_out, case.out_fmt, case.out_f_align)
