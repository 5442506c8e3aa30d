"""The bandwidth-bound tail kernels (pooling, fully_connected, softmax) through the C ABI against the CPU oracle and the
reference's known-answer vectors.  8-bit results are bit-exact; softmax is compared within 1e-5 relative (the device's
expf and the summation order differ from the host's in the last bits)."""
import numpy as np
import pytest

import oracle_lib
from cldnn_b200 import abi
from golden import kat_tail_int8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from cldnn_b200 import engine
    e = engine.Engine(0)
    yield e
    e.close()


def _run(eng, kernel, params, out_elems, out_dtype, **bufs):
    from cldnn_b200 import engine as E
    mems = {k: eng.upload(v) for k, v in bufs.items() if v is not None}
    out = eng.alloc(out_elems * np.dtype(out_dtype).itemsize)
    k = eng.kernel(kernel)
    assert k.supports(params), kernel
    k.launch(params, E.make_args(output=out, **mems))
    eng.sync()
    res = out.read(np.dtype(out_dtype), out_elems)
    assert eng.device_status() == 0
    for m in list(mems.values()) + [out]:
        m.free()
    return res


def _pool_params(dtype, N, C, H, W, size, stride, pad, mode, div=abi.DIV_FIXED, act=abi.ACT_NONE, out_dtype=None, fmt="byxf", f_align=32):
    P = (H + 2 * pad - size) // stride + 1
    Q = (W + 2 * pad - size) // stride + 1
    pp = abi.PoolParams()
    pp.in_, n_in = abi.tensor(abi.dtype_of(np.dtype(dtype)), N, C, H, W, fmt, f_align)
    pp.out, n_out = abi.tensor(abi.dtype_of(np.dtype(out_dtype or dtype)), N, C, P, Q, fmt, f_align)
    pp.size_x = pp.size_y = size
    pp.stride_x = pp.stride_y = stride
    pp.pad_x = pp.pad_y = pad
    pp.mode, pp.div_mode, pp.act = mode, div, act
    return pp, n_in, n_out


POOLS = {
    "resnet_pool1_max3x3s2_u8": dict(dtype=np.uint8, N=2, C=64, H=33, W=35, size=3, stride=2, pad=0, mode=abi.POOL_MAX),
    "max3x3s2_pad1_s8": dict(dtype=np.int8, N=2, C=32, H=14, W=15, size=3, stride=2, pad=1, mode=abi.POOL_MAX),
    "max2x2s2_s8_relu": dict(dtype=np.int8, N=1, C=48, H=8, W=8, size=2, stride=2, pad=0, mode=abi.POOL_MAX, act=abi.ACT_RELU),
    "global_avg_7x7_u8_to_s8": dict(dtype=np.uint8, N=3, C=64, H=7, W=7, size=7, stride=1, pad=0, mode=abi.POOL_AVG, out_dtype=np.int8),
    "avg3x3s1_pad1_s8_dynamic": dict(dtype=np.int8, N=1, C=16, H=6, W=7, size=3, stride=1, pad=1, mode=abi.POOL_AVG, div=abi.DIV_DYNAMIC),
    # windows inside the input: the average summed in 16-bit lanes
    "global_avg_7x7_s8_relu": dict(dtype=np.int8, N=2, C=96, H=7, W=7, size=7, stride=1, pad=0, mode=abi.POOL_AVG, act=abi.ACT_RELU),
    "avg4x4s2_u8": dict(dtype=np.uint8, N=2, C=32, H=10, W=12, size=4, stride=2, pad=0, mode=abi.POOL_AVG),
    # more items than one pass of the grid: every thread walks several (batch, y, x, feature vector) items
    "max3x3s2_u8_many_items": dict(dtype=np.uint8, N=24, C=64, H=225, W=227, size=3, stride=2, pad=0, mode=abi.POOL_MAX),
    "avg3x3s2_s8_many_items": dict(dtype=np.int8, N=40, C=48, H=113, W=225, size=3, stride=2, pad=1, mode=abi.POOL_AVG),
}


@pytest.mark.parametrize("name", sorted(POOLS))
@pytest.mark.parametrize("kernel", ["pooling_i8_byxf", "pooling_ref"])
def test_pooling_int8_matches_oracle(eng, name, kernel):
    pp, n_in, n_out = _pool_params(**POOLS[name])
    dt = np.dtype(POOLS[name]["dtype"])
    rng = np.random.default_rng(61)
    x = rng.integers(np.iinfo(dt).min, np.iinfo(dt).max + 1, size=n_in, dtype=np.int64).astype(dt)
    odt = abi.np_dtype_of(pp.out.dtype)
    want = oracle_lib.pooling(pp, x)
    got = _run(eng, kernel, pp, n_out, odt, input0=x)
    assert np.array_equal(want[:n_out], got), "%d differ" % int((want[:n_out] != got).sum())
    assert len(np.unique(got)) > 8


def test_pooling_and_fc_reference_kats_on_gpu(eng):
    k = kat_tail_int8.POOL_MAX_INT8
    x = np.trunc(np.array(k["input_f32"], dtype=np.float32)).astype(np.int8)
    pp, n_in, n_out = _pool_params(np.int8, 1, 1, 3, 3, 3, 1, 0, abi.POOL_MAX, fmt="bfyx", f_align=1)
    assert _run(eng, "pooling_ref", pp, 1, np.int8, input0=x).astype(np.float32).tolist() == k["expected_f32"]
    k = kat_tail_int8.FC_NO_BIAS_INT8
    x = np.trunc(np.array(k["input_f32"], dtype=np.float32)).astype(np.int8)
    w = np.array(k["weights_i8"], dtype=np.int8).reshape(-1)
    fp = abi.FcParams()
    fp.in_, _ = abi.tensor(abi.I8, 1, 1, 1, 3, "bfyx")
    fp.out, _ = abi.tensor(abi.I8, 1, 4, 1, 1, "bfyx")
    fp.w_dtype = abi.I8
    fp.w_px, fp.w_py, fp.w_pi, fp.w_po = 1, 3, 3, 3
    fp.bias_dtype = abi.NONE
    fp.i_qf = fp.o_qf = 1.0
    assert _run(eng, "fc_ref", fp, 4, np.int8, input0=x, weights=w).astype(np.float32).tolist() == k["expected_f32"]


@pytest.mark.parametrize("features", [40, 1000, 2048])
def test_softmax_matches_oracle(eng, features):
    """40 features: one warp per row; 1000 / 2048: one block per row."""
    sp = abi.SoftmaxParams()
    sp.in_, n = abi.tensor(abi.F32, 5, features, 1, 1, "bfyx")
    sp.out, _ = abi.tensor(abi.F32, 5, features, 1, 1, "bfyx")
    x = (np.random.default_rng(62).standard_normal(n) * 4.0).astype(np.float32)
    want = oracle_lib.softmax(sp, x)
    got = _run(eng, "softmax", sp, n, np.float32, input0=x)
    np.testing.assert_allclose(got, want[:n], rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(got.reshape(5, features).sum(1), 1.0, rtol=1e-5)


F16_POOLS = {
    "alexnet_max3x3s2": dict(dtype=np.float16, N=2, C=96, H=27, W=27, size=3, stride=2, pad=0, mode=abi.POOL_MAX, f_align=8),
    "vgg_max2x2s2": dict(dtype=np.float16, N=2, C=64, H=14, W=16, size=2, stride=2, pad=0, mode=abi.POOL_MAX, f_align=16),
    "max3x3s1_pad1_relu": dict(dtype=np.float16, N=1, C=40, H=9, W=7, size=3, stride=1, pad=1, mode=abi.POOL_MAX, act=abi.ACT_RELU, f_align=8),
    "global_avg_7x7": dict(dtype=np.float16, N=3, C=256, H=7, W=7, size=7, stride=1, pad=0, mode=abi.POOL_AVG, f_align=32),
    "avg3x3s2_pad1_dynamic": dict(dtype=np.float16, N=2, C=24, H=11, W=12, size=3, stride=2, pad=1, mode=abi.POOL_AVG, div=abi.DIV_DYNAMIC, f_align=8),
    # more items than one pass of the grid: every thread walks several (batch, y, x, feature vector) items
    "max2x2s2_many_items": dict(dtype=np.float16, N=40, C=72, H=113, W=115, size=2, stride=2, pad=0, mode=abi.POOL_MAX, f_align=8),
}


@pytest.mark.parametrize("name", sorted(F16_POOLS))
@pytest.mark.parametrize("kernel", ["pooling_f16_byxf", "pooling_ref"])
def test_pooling_fp16_matches_oracle(eng, name, kernel):
    """fp16 pooling in the feature-innermost layout: the maximum is exact, the average within fp16 rounding (1e-3 relative)."""
    pp, n_in, n_out = _pool_params(**F16_POOLS[name])
    rng = np.random.default_rng(62)
    x = rng.standard_normal(n_in).astype(np.float16)
    want = oracle_lib.pooling(pp, x).astype(np.float32)
    got = _run(eng, kernel, pp, n_out, np.float16, input0=x).astype(np.float32)
    if F16_POOLS[name]["mode"] == abi.POOL_MAX:
        assert np.array_equal(want[:n_out], got)
    else:
        assert np.abs(want[:n_out] - got).max() <= 2e-3 * max(1.0, float(np.abs(want).max()))
    assert len(np.unique(got)) > 8


@pytest.mark.parametrize("kernel", ["lrn_f16_byxf", "lrn_ref"])
@pytest.mark.parametrize("shape", [(2, 96, 13, 14), (1, 256, 5, 6), (3, 8, 4, 4), (24, 96, 55, 54)])   # the last: several items per thread
def test_lrn_fp16_across_channels_matches_oracle(eng, kernel, shape):
    """AlexNet's local response normalisation (window 5, k = 1, alpha = 1e-4, beta = 0.75; and a strong alpha so the
    neighbours matter) in the feature-innermost layout; 2e-3 relative to the output scale (fp16 output, device pow)."""
    N, C, H, W = shape
    for alpha in (1e-4, 0.5):
        lp = abi.LrnParams()
        lp.in_, n = abi.tensor(abi.F16, N, C, H, W, "byxf", 8)
        lp.out, _ = abi.tensor(abi.F16, N, C, H, W, "byxf", 8)
        lp.size, lp.k, lp.alpha, lp.beta = 5, 1.0, alpha, 0.75
        x = (np.random.default_rng(63).standard_normal(n) * 3).astype(np.float16)
        want = oracle_lib.lrn(lp, x).astype(np.float32)
        got = _run(eng, kernel, lp, n, np.float16, input0=x).astype(np.float32)
        assert np.abs(want - got).max() <= 2e-3 * float(np.abs(want).max())
        assert float(np.abs(want).max()) > 0.5


def test_softmax_reference_kats_all_scopes_on_gpu(eng):
    """The reference's softmax vectors for normalize_f / _y / _fyx (and normalize_x against numpy) through the GPU kernel."""
    from test_oracle_kat import softmax_scope_checks
    softmax_scope_checks(lambda sp, x: _run(eng, "softmax", sp, x.size, np.float32, input0=x))


def test_softmax_whole_image_scope_matches_oracle(eng):
    """normalize_fyx on a feature-innermost fp16 tensor: one set of f*y*x values per batch."""
    sp = abi.SoftmaxParams()
    sp.in_, n = abi.tensor(abi.F16, 3, 21, 9, 7, "byxf", 8)
    sp.out, _ = abi.tensor(abi.F32, 3, 21, 9, 7, "bfyx", 1)
    sp.dimension = abi.SOFTMAX_FYX
    x = (np.random.default_rng(64).standard_normal(n) * 2).astype(np.float16)
    want = oracle_lib.softmax(sp, x)
    got = _run(eng, "softmax", sp, 3 * 21 * 9 * 7, np.float32, input0=x)
    assert np.allclose(got, want[:got.size], rtol=1e-4, atol=1e-8)
    assert np.allclose(got.reshape(3, -1).sum(axis=1), 1.0, atol=1e-4)


def _eltwise_params(dtype0, dtype1, out_dtype, shape, fmt, f_align, mode, quant, calib, o_qf, act):
    N, C, H, W = shape
    ep = abi.EltwiseParams()
    ep.in0, n = abi.tensor(abi.dtype_of(np.dtype(dtype0)), N, C, H, W, fmt, f_align)
    ep.in1, _ = abi.tensor(abi.dtype_of(np.dtype(dtype1)), N, C, H, W, fmt, f_align)
    ep.out, _ = abi.tensor(abi.dtype_of(np.dtype(out_dtype)), N, C, H, W, fmt, f_align)
    ep.mode = mode
    ep.stride_x0 = ep.stride_y0 = ep.stride_x1 = ep.stride_y1 = 1
    ep.quantization, ep.calibration, ep.o_qf, ep.act = int(quant), int(calib), o_qf, act
    return ep, n


ELTWISE = {
    # the requantising 8-bit form (generic_eltwise_ref.cl with QUANTIZATION_TERM) and the floating form, on padded byxf and on bfyx
    "sum_s8_s8_oqf_byxf": dict(d0=np.int8, d1=np.int8, out=np.int8, fmt="byxf", f_align=32, mode=abi.ELTW_SUM, quant=True, calib=False, o_qf=0.5, act=abi.ACT_NONE),
    "sum_u8_s8_to_u8_relu_byxf": dict(d0=np.uint8, d1=np.int8, out=np.uint8, fmt="byxf", f_align=32, mode=abi.ELTW_SUM, quant=True, calib=False, o_qf=1.0, act=abi.ACT_RELU),
    "max_s8_calibrated_byxf": dict(d0=np.int8, d1=np.int8, out=np.int8, fmt="byxf", f_align=32, mode=abi.ELTW_MAX, quant=True, calib=True, o_qf=1.0, act=abi.ACT_NONE),
    "prod_s8_oqf_bfyx": dict(d0=np.int8, d1=np.int8, out=np.int8, fmt="bfyx", f_align=1, mode=abi.ELTW_PROD, quant=True, calib=False, o_qf=0.01, act=abi.ACT_RELU),
    "sum_f16_relu_byxf": dict(d0=np.float16, d1=np.float16, out=np.float16, fmt="byxf", f_align=32, mode=abi.ELTW_SUM, quant=False, calib=False, o_qf=1.0, act=abi.ACT_RELU),
    "sub_f16_bfyx": dict(d0=np.float16, d1=np.float16, out=np.float16, fmt="bfyx", f_align=1, mode=abi.ELTW_SUB, quant=False, calib=False, o_qf=1.0, act=abi.ACT_NONE),
}


@pytest.mark.parametrize("name", sorted(ELTWISE))
@pytest.mark.parametrize("kernel", ["eltwise_byxf", "eltwise_ref"])
@pytest.mark.parametrize("shape", [(3, 48, 9, 16), (40, 96, 57, 56)])          # the second: several vectors per thread
def test_eltwise_matches_oracle(eng, name, kernel, shape):
    c = ELTWISE[name]
    ep, n = _eltwise_params(c["d0"], c["d1"], c["out"], shape, c["fmt"], c["f_align"], c["mode"], c["quant"], c["calib"], c["o_qf"], c["act"])
    rng = np.random.default_rng(5)

    def values(dt):
        dt = np.dtype(dt)
        logical = rng.standard_normal(shape).astype(dt) if dt.kind == "f" else rng.integers(np.iinfo(dt).min, np.iinfo(dt).max + 1, size=shape).astype(dt)
        return abi.to_layout(logical, c["fmt"], c["f_align"])
    a, b = values(c["d0"]), values(c["d1"])
    calib = rng.uniform(0.25, 1.5, size=shape[1]).astype(np.float32) if c["calib"] else None
    want = oracle_lib.eltwise(ep, a, b, calib)
    got = _run(eng, kernel, ep, n, c["out"], input0=a, input1=b, calib=calib)
    real = abi.from_layout(want[:n], shape, c["fmt"], c["f_align"]), abi.from_layout(got[:n], shape, c["fmt"], c["f_align"])
    if np.dtype(c["out"]).kind == "f":
        np.testing.assert_array_equal(real[0].view(np.uint16), real[1].view(np.uint16))
    else:
        assert np.array_equal(real[0], real[1])
    assert len(np.unique(real[0])) > 8
