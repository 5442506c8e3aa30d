"""The C oracle against the reference's own kernel source (fused_conv_eltwise_gpu_ref.cl compiled as C++, oracle/_ref):
bit-exact on the literal KATs and on seeded random cases covering layouts, strides, padding, dilation, groups, every
epilogue form.  Skipped where neither the clDNN tree nor a prebuilt variant exists."""
import numpy as np
import pytest

import cases
import oracle_lib
import ref_lib
from cldnn_b200 import abi
from golden import kat_conv_quantized, kat_fused_conv_eltwise
from test_oracle_kat import build_kat_conv


def _both(case):
    p = case.p
    if not ref_lib.available(p):
        pytest.skip("no reference tree and no prebuilt oracle/_ref variant")
    want = ref_lib.conv(p, case.inp, case.w, case.bias, case.quant, case.calib, case.eltw, case.ecal)
    got = cases.run_oracle(case, threads=1)
    n = case.out_elems
    if want.dtype.kind in "iu":
        assert np.array_equal(want[:n], got[:n]), "%d differ" % int((want[:n] != got[:n]).sum())
    else:
        np.testing.assert_array_equal(want[:n], got[:n])
    return want


RANDOM = {
    "config1": dict(N=1, C=128, K=128, H=28, W=28, fmt="bfyx", f_align=1),
    "byxf_3x3": dict(N=2, C=32, K=48, H=9, W=11),
    "yxfb_stride2": dict(N=3, C=8, K=8, H=11, W=9, stride=2, fmt="yxfb", f_align=1),
    "dilated": dict(N=1, C=16, K=16, H=12, W=12, dil=2, pad=2, fmt="bfyx", f_align=1),
    "depthwise": dict(N=2, C=16, K=16, H=9, W=9, groups=16, fmt="bfyx", f_align=1),
    "grouped4": dict(N=1, C=16, K=32, H=7, W=7, groups=4, fmt="bfyx", f_align=1),
    "7x7_stride2_c3": dict(N=1, C=3, K=16, H=33, W=31, kh=7, kw=7, stride=2, pad=3, fmt="bfyx", f_align=1),
    "u8_out": dict(N=1, C=32, K=32, H=8, W=8, out_dtype=np.uint8),
    "i8_in_float_out": dict(N=1, C=32, K=32, H=8, W=8, in_dtype=np.int8, out_dtype=np.float32),
    "float_bias_calibrated": dict(N=1, C=32, K=32, H=8, W=8, bias="f32", calib=True),
    "o_qf_i_qf": dict(N=1, C=32, K=32, H=8, W=8, o_qf=0.75, i_qf=0.5),
    "leaky": dict(N=1, C=32, K=32, H=8, W=8, act=abi.ACT_RELU_NEGATIVE_SLOPE),
    "clamp": dict(N=1, C=32, K=32, H=8, W=8, act=abi.ACT_CLAMP, scale_lo=2.0 ** -13, scale_hi=2.0 ** -12),
    "fused_u8_residual": dict(N=2, C=32, K=64, H=7, W=7, kh=1, kw=1, pad=0, fused=True, out_dtype=np.uint8),
    "fused_i8_residual_scaled_calibrated": dict(N=2, C=32, K=32, H=7, W=7, fused=True, out_dtype=np.uint8, eltw_dtype=np.int8,
                                                non_conv_scale=1.0 / 3.0, eltw_calib=True),
    "fused_int_domain": dict(N=1, C=32, K=32, H=6, W=6, fused=True, quant=False, in_dtype=np.int8, out_dtype=np.uint8, eltw_dtype=np.int8,
                             eltw_calib=True, w_range=2),
    "fp32": dict(N=1, C=8, K=8, H=6, W=6, in_dtype=np.float32, out_dtype=np.float32, bias="none", quant=False, fmt="bfyx", f_align=1),
}


@pytest.mark.parametrize("name", sorted(RANDOM))
def test_oracle_equals_reference_kernel_source(name):
    kw = dict(RANDOM[name])
    case = cases.make_conv_case(101, **kw)
    if name == "leaky":
        case.p.act_m = 0.125
    want = _both(case)
    assert (want != 0).any()


@pytest.mark.parametrize("name", sorted(kat_conv_quantized.CASES))
def test_reference_kernel_source_passes_its_own_kats(name):
    """Pins the shim itself: the reference kernel, compiled here, reproduces the reference test-suite's expectations."""
    case = kat_conv_quantized.CASES[name]
    in_dt, out_dt = np.dtype(case["in_dtype"]), np.dtype(case["out_dtype"])
    feats = case["features"]
    p, inp, w, bias = build_kat_conv(feats, in_dt.type, out_dt.type)
    p.quantization, p.act = 1, abi.ACT_RELU
    if not ref_lib.available(p):
        pytest.skip("no reference tree and no prebuilt oracle/_ref variant")
    quant = np.array([f[3] for f in feats], dtype=np.float32)
    out = ref_lib.conv(p, inp.reshape(-1), w.reshape(-1), bias, quant).reshape(len(feats), 2)
    pre = np.array([f[4] for f in feats])
    info = np.iinfo(out_dt) if out_dt.kind in "iu" else np.finfo(out_dt)
    exp = np.minimum(info.max, np.maximum(info.min, np.maximum(0, pre)))
    if out_dt.kind in "iu":
        assert np.array_equal(out.astype(np.int64), exp.astype(np.int64))
    else:
        np.testing.assert_allclose(out, exp, atol=1e-3)
