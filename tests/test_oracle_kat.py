"""The CPU oracle against the reference's own literal known-answer tests.

Every case here is data from the clDNN test-suite (see tests/golden/kat_*.py
for file:line); the expectations are the reference's, not ours.
"""
import numpy as np
import pytest

import oracle_lib
from cldnn_b200 import abi
from golden import kat_conv_quantized, kat_fused_conv_eltwise


def _clamp_expected(pre_relu, out_dtype):
    info = np.iinfo(out_dtype) if np.issubdtype(out_dtype, np.integer) else np.finfo(out_dtype)
    return np.minimum(info.max, np.maximum(info.min, np.maximum(0, pre_relu)))


def build_kat_conv(features, in_dtype, out_dtype, bias_dtype=np.int32, fmt="bfyx"):
    """The tensors ConvQuantizedTest::do_test builds: 1 x n x 1 x 4 input, diagonal filter."""
    n = len(features)
    inp = np.array([f[0] for f in features], dtype=in_dtype).reshape(1, n, 1, 4)
    w = np.zeros((n, n, 1, 3), dtype=np.float32 if in_dtype == np.float32 else np.int8)
    for i, f in enumerate(features):
        w[i, i, 0, :] = f[1]
    bias = np.array([f[2] for f in features], dtype=bias_dtype)
    p = abi.ConvParams()
    p.in_, _ = abi.tensor(abi.dtype_of(in_dtype), 1, n, 1, 4, fmt)
    p.out, _ = abi.tensor(abi.dtype_of(out_dtype), 1, n, 1, 2, fmt)
    abi.set_weights(p, abi.dtype_of(w.dtype), 1, n, n, 1, 3)
    p.stride_x = p.stride_y = p.dil_x = p.dil_y = 1
    p.bias_dtype = abi.dtype_of(bias_dtype)
    p.i_qf = p.o_qf = 1.0
    p.eltw_stride_x = p.eltw_stride_y = 1
    return p, inp, w, bias


@pytest.mark.parametrize("name", sorted(kat_conv_quantized.CASES))
@pytest.mark.parametrize("fmt", ["bfyx", "byxf", "yxfb"])
def test_conv_quantized_kat(name, fmt):
    case = kat_conv_quantized.CASES[name]
    in_dt, out_dt = np.dtype(case["in_dtype"]), np.dtype(case["out_dtype"])
    feats = case["features"]
    p, inp, w, bias = build_kat_conv(feats, in_dt.type, out_dt.type, fmt=fmt)
    quant = np.array([f[3] for f in feats], dtype=np.float32)
    p.quantization = 1
    p.act = abi.ACT_RELU
    out = oracle_lib.conv(p, abi.to_layout(inp, fmt), w.reshape(-1), bias, quant)
    got = abi.from_layout(out, (1, len(feats), 1, 2), fmt)[0, :, 0, :]
    pre = np.array([f[4] for f in feats])
    if np.issubdtype(out_dt, np.integer):
        np.testing.assert_array_equal(got.astype(np.int64), _clamp_expected(pre, out_dt).astype(np.int64))
    else:
        np.testing.assert_allclose(got, _clamp_expected(pre, out_dt), atol=1e-3)


@pytest.mark.parametrize("name", sorted(kat_fused_conv_eltwise.CASES))
def test_fused_conv_eltwise_kat(name):
    case = kat_fused_conv_eltwise.CASES[name]
    in_dt, out_dt = np.dtype(case["in_dtype"]), np.dtype(case["out_dtype"])
    feats = case["features"]
    is_float = in_dt == np.float32
    p, inp, w, bias = build_kat_conv(feats, in_dt.type, out_dt.type,
                                     bias_dtype=np.float32 if is_float else np.int32)
    n = len(feats)
    nan = float("nan")
    quant = np.array([nan if f[3] is None else f[3] for f in feats], dtype=np.float32)
    calib = np.array([nan if f[4] is None else f[4] for f in feats], dtype=np.float32)
    eltw = np.array([f[5] for f in feats], dtype=in_dt).reshape(1, n, 1, 2)
    ecal = np.array([nan if f[6] is None else f[6] for f in feats], dtype=np.float32)
    p.eltw, _ = abi.tensor(abi.dtype_of(in_dt), 1, n, 1, 2)
    p.fused_eltw = 1
    p.quantization = int(case["use_quant"])
    p.calibration = int(case["use_conv_calib"])
    p.eltw_calibration = int(case["use_eltw_calib"])
    p.i_qf = case["conv_i_qf"]
    # fused_conv_eltwise_kernel_base.cpp:139-151: O_QF is always emitted under quantisation
    p.has_o_qf = int(case["use_quant"])
    p.o_qf = 1.0
    p.has_non_conv_scale = int(case["non_conv_scale"] != 1.0)      # fused_conv_eltwise_kernel_ref.cpp:92-94
    p.non_conv_scale = case["non_conv_scale"]
    p.act = abi.ACT_NONE
    p.eltw_act = abi.ACT_RELU
    out = oracle_lib.conv(p, inp.reshape(-1), w.reshape(-1), bias,
                          quant if case["use_quant"] else None,
                          calib if case["use_conv_calib"] else None,
                          eltw.reshape(-1), ecal if case["use_eltw_calib"] else None)
    got = out.reshape(n, 2)
    pre = np.array([f[7] for f in feats])
    if np.issubdtype(out_dt, np.integer):
        np.testing.assert_array_equal(got.astype(np.int64), _clamp_expected(pre, out_dt).astype(np.int64))
    else:
        np.testing.assert_allclose(got, _clamp_expected(pre, out_dt), atol=1e-3)


# ---- int8 pooling and fully_connected KATs (through the oracle's reorder, like the reference's topologies) -------------
from golden import kat_tail_int8


def _reorder(arr, out_dtype, fmt_in="bfyx", fmt_out="bfyx"):
    b, f, y, x = arr.shape
    rp = abi.ReorderParams()
    rp.in_, _ = abi.tensor(abi.dtype_of(arr.dtype), b, f, y, x, fmt_in)
    rp.out, _ = abi.tensor(abi.dtype_of(np.dtype(out_dtype)), b, f, y, x, fmt_out)
    return oracle_lib.reorder(rp, np.ascontiguousarray(arr).reshape(-1)).reshape(arr.shape)


def _pool_3x3(x_i8, mode):
    pp = abi.PoolParams()
    pp.in_, _ = abi.tensor(abi.I8, 1, 1, 3, 3, "bfyx")
    pp.out, _ = abi.tensor(abi.I8, 1, 1, 1, 1, "bfyx")
    pp.size_x = pp.size_y = 3
    pp.stride_x = pp.stride_y = 1
    pp.mode, pp.div_mode = mode, abi.DIV_FIXED
    return oracle_lib.pooling(pp, x_i8.reshape(-1)).reshape(1, 1, 1, 1)


def test_pooling_int8_kats():
    k = kat_tail_int8.POOL_MAX_INT8
    x = _reorder(np.array(k["input_f32"], dtype=np.float32).reshape(1, 1, 3, 3), np.int8, fmt_in="byxf")
    got = _reorder(_pool_3x3(x, abi.POOL_MAX), np.float32)
    assert got.reshape(-1).tolist() == k["expected_f32"]
    k = kat_tail_int8.POOL_AVG_INT8
    vals = np.array(k["input_f32"], dtype=np.float32)
    expected = float(np.int8(np.trunc(np.trunc(vals).astype(np.int8).astype(np.float32).sum() / vals.size)))
    x = _reorder(vals.reshape(1, 1, 3, 3), np.int8, fmt_in="byxf")
    got = _reorder(_pool_3x3(x, abi.POOL_AVG), np.float32)
    assert got.reshape(-1).tolist() == [expected]


def test_fully_connected_int8_kat():
    k = kat_tail_int8.FC_NO_BIAS_INT8
    x = _reorder(np.array(k["input_f32"], dtype=np.float32).reshape(1, 1, 1, 3), np.int8)
    w = np.array(k["weights_i8"], dtype=np.int8)
    fp = abi.FcParams()
    fp.in_, _ = abi.tensor(abi.I8, 1, 1, 1, 3, "bfyx")
    fp.out, _ = abi.tensor(abi.I8, 1, 4, 1, 1, "bfyx")
    fp.w_dtype = abi.I8
    fp.w_px, fp.w_py, fp.w_pi, fp.w_po = 1, 3, 3, 3
    fp.bias_dtype = abi.NONE
    fp.i_qf = fp.o_qf = 1.0
    out, oor = oracle_lib.fc(fp, x.reshape(-1), w.reshape(-1))
    got = _reorder(out.reshape(1, 4, 1, 1), np.float32)
    assert got.reshape(-1).tolist() == k["expected_f32"]


def _softmax_scope(dimension, x_bfyx):
    from golden import kat_softmax  # noqa: F401
    sp = abi.SoftmaxParams()
    N, F, Y, X = x_bfyx.shape
    sp.in_, n = abi.tensor(abi.F32, N, F, Y, X, "bfyx", 1)
    sp.out, _ = abi.tensor(abi.F32, N, F, Y, X, "bfyx", 1)
    sp.dimension = dimension
    return sp, n


def softmax_scope_checks(run):
    """Shared by the oracle and the GPU test: `run(params, flat input) -> flat output`."""
    from golden import kat_softmax as K
    x = np.array(K.VALUES_BATCH_WISE["input"], dtype=np.float32).reshape(1, 10, 1, 1)
    for dim in (abi.SOFTMAX_F, abi.SOFTMAX_FYX):
        sp, n = _softmax_scope(dim, x)
        got = run(sp, x.reshape(-1))
        assert np.allclose(got, np.array(K.VALUES_BATCH_WISE["expected"], dtype=np.float32), rtol=1e-5, atol=1e-7)
    x = np.array(K.SCOPES_INPUT_BFYX, dtype=np.float32).reshape(2, 3, 2, 2)
    for dim, expected, axes in ((abi.SOFTMAX_FYX, K.EXPECTED_MAX_FYX, (1, 2, 3)), (abi.SOFTMAX_Y, K.EXPECTED_MAX_Y, (2,)), (abi.SOFTMAX_F, K.EXPECTED_MAX_F, (1,))):
        sp, n = _softmax_scope(dim, x)
        got = run(sp, x.reshape(-1)).reshape(x.shape)
        assert np.allclose(got.sum(axis=axes), 1.0, atol=1e-5)
        mx = got.max(axis=axes).reshape(-1)                          # remaining axes in b, f, y, x order: the reference's walk
        assert np.allclose(mx, np.array(expected, dtype=np.float32), rtol=1e-5, atol=1e-6), (dim, mx, expected)
    sp, n = _softmax_scope(abi.SOFTMAX_X, x)                         # no literal vector in the reference: sums and a numpy restatement
    got = run(sp, x.reshape(-1)).reshape(x.shape)
    e = np.exp(x - x.max(axis=3, keepdims=True))
    assert np.allclose(got, e / e.sum(axis=3, keepdims=True), rtol=1e-5, atol=1e-7)


def test_softmax_reference_kats_all_scopes():
    softmax_scope_checks(lambda sp, x: oracle_lib.softmax(sp, x))
