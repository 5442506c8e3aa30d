"""The MMAD / IMAD epilogue orders of the oracle against the reference's own kernel text, and against the reference order.

oracle/_ref/clref_epilogues.so holds the epilogue lines of convolution_gpu_mmad.cl (:105-128) and
fused_conv_eltwise_gpu_imad.cl (:171-205) compiled as C++ where they lie in the clDNN tree (oracle/ref_build/build_epilogues.py).
Each output value of a small quantised convolution run on the oracle in that order must equal what those lines compute from
the same accumulator, bit for bit -- including values outside the 8-bit range, where the lines do not saturate.  With ReLU,
positive factors and in-range values the three orders must agree with each other.
"""
import ctypes as C
import os

import numpy as np
import pytest

import cases
from cldnn_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "oracle", "_ref", "clref_epilogues.so")


class EpiIn(C.Structure):
    _fields_ = [("acc", C.c_int), ("q", C.c_float), ("iqf", C.c_float), ("bias", C.c_float), ("scale", C.c_float), ("act", C.c_int), ("m", C.c_float),
                ("n", C.c_float), ("eltw", C.c_int), ("ecal", C.c_float), ("eltw_act", C.c_int), ("em", C.c_float), ("en", C.c_float)]


def _case(seed, order, fused=False, calib=False, act=abi.ACT_RELU, eltw_act=abi.ACT_RELU, scale_lo=2.0 ** -9, scale_hi=2.0 ** -7, o_qf=1.0):
    c = cases.make_conv_case(seed, N=2, C=8, K=16, H=6, W=6, kh=1, kw=1, pad=0, in_dtype=np.int8, out_dtype=np.int8, fmt="bfyx", f_align=1, bias="f32",
                             calib=calib, act=act, fused=fused, eltw_dtype=np.int8, eltw_calib=fused, eltw_act=eltw_act, scale_lo=scale_lo, scale_hi=scale_hi,
                             o_qf=o_qf)
    c.p.epilogue_order = order
    return c


def _accumulators(c):
    x = c.x_logical.astype(np.int64)                       # [N, C, H, W]
    w = c.w_logical.astype(np.int64)[:, :, 0, 0]           # [K, C]
    return np.einsum("nchw,kc->nkhw", x, w)


@pytest.mark.parametrize("variant", ["mmad_oqf", "mmad_calibrated", "imad_oqf", "imad_calibrated", "imad_fused_calibrated"])
@pytest.mark.parametrize("act", [abi.ACT_NONE, abi.ACT_RELU, abi.ACT_CLAMP])
def test_oracle_order_equals_the_reference_epilogue_text(variant, act):
    if not os.path.exists(SHIM):
        pytest.skip("oracle/_ref/clref_epilogues.so not built (needs the clDNN tree)")
    lib = C.CDLL(SHIM)
    fn = getattr(lib, "clref_" + variant)
    fn.argtypes = [C.POINTER(EpiIn)]
    fn.restype = C.c_int
    order = abi.EPILOGUE_MMAD if variant.startswith("mmad") else abi.EPILOGUE_IMAD
    fused = "fused" in variant
    calib = "calibrated" in variant
    # scales large enough that part of the values leaves the 8-bit range: the conversion there must match too
    c = _case(71, order, fused=fused, calib=calib, act=act, eltw_act=act, scale_lo=2.0 ** -8, scale_hi=2.0 ** -5, o_qf=1.0 if calib else 0.75)
    c.p.act_m, c.p.act_n, c.p.eltw_m, c.p.eltw_n = -20.0, 90.0, -20.0, 90.0
    got = cases.logical_out(c, cases.run_oracle(c))
    acc = _accumulators(c)
    e_log = abi.from_layout(c.eltw, c.shape_out, "bfyx", 1) if fused else None
    N, K, H, W = got.shape
    wrapped = 0
    for n in range(N):
        for k in range(K):
            for y in range(H):
                for x in range(W):
                    e = EpiIn(int(acc[n, k, y, x]), float(c.quant[k]), 1.0, float(c.bias[k]), float(c.calib[k]) if calib else float(c.p.o_qf), act, -20.0, 90.0,
                              int(e_log[n, k, y, x]) if fused else 0, float(c.ecal[k]) if fused else 1.0, act, -20.0, 90.0)
                    want = C.c_int8(fn(C.byref(e))).value
                    assert int(got[n, k, y, x]) == want, (variant, n, k, y, x, int(acc[n, k, y, x]))
                    t = (np.float32(acc[n, k, y, x]) * np.float32(c.quant[k]) + np.float32(c.bias[k])) * np.float32(e.scale)
                    wrapped += abs(float(t)) > 128
    assert wrapped > 10                                    # the non-saturating conversion was exercised


def test_the_three_orders_agree_on_in_range_values():
    outs = {}
    for order in (abi.EPILOGUE_REF, abi.EPILOGUE_MMAD, abi.EPILOGUE_IMAD):
        c = _case(72, order, calib=True, scale_lo=2.0 ** -12, scale_hi=2.0 ** -10)
        outs[order] = cases.run_oracle(c)
        assert np.abs(outs[order].astype(np.int32)).max() < 127 and len(np.unique(outs[order])) > 8
    assert np.array_equal(outs[abi.EPILOGUE_REF], outs[abi.EPILOGUE_MMAD])
    assert np.array_equal(outs[abi.EPILOGUE_REF], outs[abi.EPILOGUE_IMAD])


def test_orders_are_refused_where_the_reference_kernels_have_no_meaning():
    import oracle_lib
    c = cases.make_conv_case(73, N=1, C=8, K=8, H=4, W=4, kh=1, kw=1, pad=0, fmt="bfyx", f_align=1)      # i32 bias
    c.p.epilogue_order = abi.EPILOGUE_MMAD
    a = abi.Args()
    assert oracle_lib.lib().oracle_conv(C.byref(c.p), C.byref(a), 1) == abi.UNSUPPORTED_FORMAT
