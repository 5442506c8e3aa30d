"""Parity of the CUDA convolution kernels with the CPU oracle, through the C ABI.
Integer outputs must be bit-exact."""
import numpy as np
import pytest

import cases
from cldnn_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from cldnn_b200 import engine
    e = engine.Engine(0)
    yield e
    e.close()


def _exact(eng, case, kernel, tune=0):
    want = cases.run_oracle(case)
    got = cases.run_gpu(eng, case, kernel, tune)
    n = case.out_elems
    if want.dtype.kind in "iu":
        bad = np.flatnonzero(want[:n] != got[:n])
        assert bad.size == 0, "%d of %d differ; first at %d: want %d got %d" % (bad.size, n, bad[0], want[bad[0]], got[bad[0]])
    else:
        np.testing.assert_allclose(got[:n], want[:n], rtol=1e-6, atol=1e-6)
    return want


GEOMS = {
    # the reference's own CPU-runnable int8 layer case: N=1, C=128 -> K=128, 28x28, 3x3 stride 1 pad 1, u8 in, s8 out, ReLU
    "config1": dict(N=1, C=128, K=128, H=28, W=28),
    "1x1": dict(N=2, C=64, K=256, H=56, W=56, kh=1, kw=1, pad=0),
    "1x1_stride2": dict(N=2, C=256, K=128, H=28, W=28, kh=1, kw=1, pad=0, stride=2),
    "c64_56": dict(N=2, C=64, K=64, H=56, W=56),
    "ragged_c32_k48": dict(N=3, C=32, K=48, H=9, W=11),
    "c96_k40": dict(N=1, C=96, K=40, H=7, W=7),
    "stride2_3x3": dict(N=10, C=64, K=64, H=15, W=15, stride=2),
    "dilation2": dict(N=1, C=32, K=32, H=12, W=12, dil=2, pad=2),
    "c512_7x7map": dict(N=4, C=512, K=512, H=7, W=7),
    "5x5": dict(N=1, C=32, K=32, H=10, W=10, kh=5, kw=5, pad=2),
    "1x1_map1": dict(N=5, C=2048, K=1000, H=1, W=1, kh=1, kw=1, pad=0),
    "nopad": dict(N=1, C=32, K=32, H=6, W=6, pad=0),
}


@pytest.mark.parametrize("name", sorted(GEOMS))
def test_conv_ref_kernel_matches_oracle(eng, name):
    _exact(eng, cases.make_conv_case(1, **GEOMS[name]), "conv_ref")


@pytest.mark.parametrize("name", sorted(GEOMS))
def test_conv_i8_tc_matches_oracle(eng, name):
    case = cases.make_conv_case(2, **GEOMS[name])
    k = eng.kernel("conv_i8_tc")
    assert k.supports(case.p)
    want = _exact(eng, case, "conv_i8_tc")
    assert (want != 0).any() and (want != 127).any()      # the comparison is not on a saturated constant


@pytest.mark.parametrize("name", sorted(GEOMS))
def test_conv_i8_tc_every_tuning_variant(eng, name):
    """All addressing modes (flat / TMA im2col / tiled box) and feature tiles give the same bits."""
    k = eng.kernel("conv_i8_tc")
    case = cases.make_conv_case(3, **GEOMS[name])
    want = cases.run_oracle(case)
    ran = 0
    for tune in range(1, k.tune_count(case.p)):
        p = cases.copy_params(case.p)
        p.tune = tune
        if not k.supports(p):
            continue
        got = cases.run_gpu(eng, case, "conv_i8_tc", tune)
        assert np.array_equal(want[:case.out_elems], got[:case.out_elems]), "tune %d" % tune
        ran += 1
    assert ran >= 4


EPILOGUES = {
    "fused_residual_calibrated": dict(fused=True, out_dtype=np.uint8, eltw_calib=True, non_conv_scale=0.5),
    "fused_residual_plain": dict(fused=True, out_dtype=np.uint8),
    "fused_residual_in_place": dict(fused=True, out_dtype=np.uint8, in_out_opt=True),
    "fused_i8_residual": dict(fused=True, out_dtype=np.int8, eltw_dtype=np.int8, non_conv_scale=1.0 / 3.0),
    "float_bias_and_calibration": dict(bias="f32", calib=True),
    "i8_in_float_out": dict(in_dtype=np.int8, out_dtype=np.float32),
    "u8_out": dict(out_dtype=np.uint8),
    "no_bias": dict(bias="none"),
    "no_activation": dict(act=abi.ACT_NONE),
    "relu6_clamp": dict(act=abi.ACT_CLAMP, scale_lo=2.0 ** -13, scale_hi=2.0 ** -12),
    "leaky": dict(act=abi.ACT_RELU_NEGATIVE_SLOPE),
    "o_qf": dict(o_qf=0.75),
    "i_qf": dict(i_qf=0.5),
    "int_domain_fused": dict(fused=True, quant=False, in_dtype=np.int8, out_dtype=np.uint8, eltw_dtype=np.int8,
                             eltw_calib=True, w_range=2),
}


@pytest.mark.parametrize("name", sorted(EPILOGUES))
@pytest.mark.parametrize("kernel", ["conv_ref", "conv_i8_tc"])
def test_epilogue_variants(eng, name, kernel):
    kw = dict(EPILOGUES[name])
    case = cases.make_conv_case(4, N=2, C=64, K=64, H=14, W=14, **kw)
    if name == "leaky":
        case.p.act_m = 0.125
    assert eng.kernel(kernel).supports(case.p)
    _exact(eng, case, kernel)


# The specialised kernels behind conv_i8_tc (per-channel dequantisation only, NONE / ReLU, 8-bit output):
# every epilogue variant they are compiled for, on every feature tile, and the float-domain path they
# fall back to when a feature's value range could leave the integer-exact range.
FAST_VARIANTS = {
    "plain_u8_none": dict(out_dtype=np.uint8, act=abi.ACT_NONE),
    "plain_u8_relu": dict(out_dtype=np.uint8),
    "plain_s8_none": dict(act=abi.ACT_NONE),
    "plain_s8_relu": dict(),
    "plain_s8_in": dict(in_dtype=np.int8, act=abi.ACT_NONE),
    "sum_u8_none_relu": dict(fused=True, out_dtype=np.uint8, act=abi.ACT_NONE),                       # the ResNet block tail
    "sum_u8_relu_none": dict(fused=True, out_dtype=np.uint8, eltw_act=abi.ACT_NONE),
    "sum_u8_none_none_s8res": dict(fused=True, out_dtype=np.uint8, act=abi.ACT_NONE, eltw_act=abi.ACT_NONE, eltw_dtype=np.int8),
    "sum_s8_none_none_s8res": dict(fused=True, out_dtype=np.int8, act=abi.ACT_NONE, eltw_act=abi.ACT_NONE, eltw_dtype=np.int8),
    "sum_s8_none_relu_s8res": dict(fused=True, out_dtype=np.int8, act=abi.ACT_NONE, eltw_dtype=np.int8),
    "sum_s8_relu_relu_u8res": dict(fused=True, out_dtype=np.int8, eltw_dtype=np.uint8),
    "sum_s8_relu_none_u8res": dict(fused=True, out_dtype=np.int8, eltw_act=abi.ACT_NONE, eltw_dtype=np.uint8),
    "sum_in_place": dict(fused=True, out_dtype=np.uint8, act=abi.ACT_NONE, in_out_opt=True),
    "sum_no_bias": dict(fused=True, out_dtype=np.uint8, act=abi.ACT_NONE, bias="none"),
}


@pytest.mark.parametrize("name", sorted(FAST_VARIANTS))
@pytest.mark.parametrize("wide", [False, True])
def test_conv_i8_tc_fast_variants(eng, name, wide):
    k = eng.kernel("conv_i8_tc")
    case = cases.make_conv_case(11, N=12, C=64, K=256, H=14, W=14, scale_lo=2.0 ** -13, scale_hi=2.0 ** -11, **FAST_VARIANTS[name])
    if wide:
        case.quant[7] = 0.75          # one feature whose values can exceed 2^22: its tile takes the float-domain path
        case.quant[200] = -3.0
    want = cases.run_oracle(case)
    n = case.out_elems
    assert len(np.unique(want[:n])) > 64
    # automatic, tiled box with 64 / 128 / 256 features per tile, TMA im2col with 128, then the same with four epilogue groups,
    # then CTA pairs (im2col and tiled, 128 and 256 features; the 19 pixel tiles of this case leave a phantom twentieth)
    for tune in (0, 10, 11, 12, 7, 38, 39, 35, 47, 48, 49, 50):
        p = cases.copy_params(case.p)
        p.tune = tune
        assert k.supports(p)
        got = cases.run_gpu(eng, case, "conv_i8_tc", tune)
        bad = np.flatnonzero(want[:n] != got[:n])
        assert bad.size == 0, "tune %d: %d of %d differ; first at %d: want %d got %d" % (tune, bad.size, n, bad[0], want[bad[0]], got[bad[0]])


REQUANT = {
    # a uniform O_QF behind the per-feature scale (MobileNet's layers), on feature counts that do not fill the tiles
    "relu6_requantised_u8": dict(out_dtype=np.uint8, act=abi.ACT_CLAMP, o_qf=42.5),
    "linear_s8_oqf16": dict(act=abi.ACT_NONE, o_qf=16.0),
    "relu_u8_oqf": dict(out_dtype=np.uint8, o_qf=2.5),
    "sum_s8_oqf16": dict(fused=True, act=abi.ACT_NONE, eltw_act=abi.ACT_NONE, eltw_dtype=np.int8, o_qf=16.0),
    "sum_u8_oqf_relu_after": dict(fused=True, out_dtype=np.uint8, act=abi.ACT_NONE, o_qf=4.0),
    "clamp_not_subsumed": dict(out_dtype=np.uint8, act=abi.ACT_CLAMP, o_qf=20.0),
    "relu_s8_oqf": dict(o_qf=8.0),                                                            # s8 after ReLU with O_QF: general kernel
}


@pytest.mark.parametrize("name", sorted(REQUANT))
@pytest.mark.parametrize("features", [16, 24, 96, 144, 320])
def test_conv_i8_tc_requantised_ragged_features(eng, name, features):
    k = eng.kernel("conv_i8_tc")
    case = cases.make_conv_case(12, N=5, C=64, K=features, H=14, W=14, kh=1, kw=1, pad=0, scale_lo=2.0 ** -13, scale_hi=2.0 ** -11, **REQUANT[name])
    want = cases.run_oracle(case)
    n = case.out_elems
    assert len(np.unique(want[:n])) > 32
    ran = 0
    # automatic; flat with 64 / 128 / 256 features per tile; tiled 64 / 128; im2col 128; general kernel; four epilogue groups
    for tune in (0, 2, 3, 4, 10, 11, 7, 15, 30, 31, 39):
        p = cases.copy_params(case.p)
        p.tune = tune
        if not k.supports(p):
            continue
        got = cases.run_gpu(eng, case, "conv_i8_tc", tune)
        bad = np.flatnonzero(want[:n] != got[:n])
        assert bad.size == 0, "tune %d: %d of %d differ; first at %d: want %d got %d" % (tune, bad.size, n, bad[0], want[bad[0]], got[bad[0]])
        ran += 1
    assert ran >= 5


def test_conv_i8_tc_requantised_3x3_and_wide(eng):
    k = eng.kernel("conv_i8_tc")
    for name in ("relu6_requantised_u8", "linear_s8_oqf16", "sum_s8_oqf16"):
        for wide in (False, True):
            case = cases.make_conv_case(13, N=3, C=32, K=96, H=15, W=13, scale_lo=2.0 ** -13, scale_hi=2.0 ** -11, **REQUANT[name])
            if wide:
                case.quant[70] = 0.5
            want = cases.run_oracle(case)
            n = case.out_elems
            for tune in (0, 10, 11, 6, 26, 38, 42):
                p = cases.copy_params(case.p)
                p.tune = tune
                if not k.supports(p):
                    continue
                got = cases.run_gpu(eng, case, "conv_i8_tc", tune)
                assert np.array_equal(want[:n], got[:n]), "%s wide=%s tune %d" % (name, wide, tune)


FIRST_LAYER = {
    # ResNet-50 conv1: 3 -> 64, 7x7 stride 2 pad 3, planar u8 image in, byxf out
    "resnet_conv1": dict(N=2, C=3, K=64, H=224, W=224, kh=7, kw=7, stride=2, pad=3),
    "ragged_image": dict(N=3, C=3, K=32, H=37, W=45, kh=7, kw=7, stride=2, pad=3),
    "stride1_5x5": dict(N=1, C=4, K=64, H=20, W=33, kh=5, kw=5, stride=1, pad=2),
    "one_feature_3x3": dict(N=2, C=1, K=96, H=17, W=18, kh=3, kw=3, stride=1, pad=1),
    "no_pad_stride3": dict(N=1, C=3, K=128, H=30, W=31, kh=4, kw=6, stride=3, pad=0),
}


@pytest.mark.parametrize("name", sorted(FIRST_LAYER))
@pytest.mark.parametrize("variant", ["relu_u8", "signed_in_calibrated"])
def test_conv_i8_first_matches_oracle(eng, name, variant):
    kw = dict(FIRST_LAYER[name])
    if variant == "relu_u8":
        case = cases.make_conv_case(21, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, **kw)
    else:
        case = cases.make_conv_case(22, fmt="bfyx", f_align=1, out_fmt="byxf", in_dtype=np.int8, out_dtype=np.int8, bias="f32", calib=True,
                                    act=abi.ACT_NONE, **kw)
    assert eng.kernel("conv_i8_first").supports(case.p)
    want = _exact(eng, case, "conv_i8_first")
    assert (want != 0).any()
    _exact(eng, case, "conv_i8_first", tune=1)       # one CTA per SM, double-buffered epilogue
    _exact(eng, case, "conv_i8_first", tune=2)       # as many CTAs per SM as fit, at most two
    _exact(eng, case, "conv_i8_first", tune=3)       # up to three CTAs per SM


def test_conv_i8_first_requantised(eng):
    """MobileNet's stem: 3x3 stride 2, ReLU6 folded in front of a requantisation by 255/6 (conversion-free with a uniform O_QF),
    a linear s8 output with O_QF, and a clamp the saturation does not subsume."""
    geom = dict(N=3, C=3, K=32, H=65, W=71, kh=3, kw=3, stride=2, pad=1)
    for extra in (dict(out_dtype=np.uint8, act=abi.ACT_CLAMP, o_qf=42.5), dict(act=abi.ACT_NONE, o_qf=16.0), dict(out_dtype=np.uint8, act=abi.ACT_CLAMP, o_qf=20.0)):
        for kernel in ("conv_i8_first", "conv_first_tc"):
            case = cases.make_conv_case(24, fmt="bfyx", f_align=1, out_fmt="byxf", scale_lo=2.0 ** -13, scale_hi=2.0 ** -11, **geom, **extra)
            assert eng.kernel(kernel).supports(case.p)
            want = _exact(eng, case, kernel)
            assert len(np.unique(want[:case.out_elems])) > 16
            if kernel == "conv_i8_first":
                for tune in (1, 2, 3):
                    _exact(eng, case, kernel, tune=tune)


def test_conv_i8_first_plain_variants(eng):
    """The conversion-free epilogue variants of the first-layer kernel (u8 / s8 / s8 after ReLU), the float-domain
    path a large scale forces, and more tiles than CTAs so the operand pipeline wraps several times."""
    geom = dict(N=6, C=3, K=64, H=97, W=131, kh=7, kw=7, stride=2, pad=3)
    for out_dtype, act in ((np.uint8, abi.ACT_RELU), (np.uint8, abi.ACT_NONE), (np.int8, abi.ACT_NONE), (np.int8, abi.ACT_RELU)):
        for wide in (False, True):
            case = cases.make_conv_case(23, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=out_dtype, act=act,
                                        scale_lo=2.0 ** -12, scale_hi=2.0 ** -10, **geom)
            if wide:
                case.quant[5] = 900.0
            for tune in (0, 1, 3):
                _exact(eng, case, "conv_i8_first", tune=tune)


ROW_FORM = {
    # geometries the row form of the first-layer kernel takes: stride 2, 64 output features, 16-byte aligned row pitch
    "resnet_conv1": dict(N=2, C=3, K=64, H=224, W=224, kh=7, kw=7, stride=2, pad=3),
    "odd_height_many_tiles": dict(N=9, C=3, K=64, H=97, W=144, kh=7, kw=7, stride=2, pad=3),     # more tiles than a CTA's rings hold
    "two_row_tiles": dict(N=2, C=3, K=64, H=300, W=64, kh=7, kw=7, stride=2, pad=3),               # 150 output rows: two tiles of 128
    "four_features_5x5": dict(N=2, C=4, K=64, H=40, W=48, kh=5, kw=5, stride=2, pad=2),
    "stem_3x3": dict(N=3, C=3, K=64, H=66, W=80, kh=3, kw=3, stride=2, pad=1),
    "no_pad_4x6": dict(N=1, C=3, K=64, H=30, W=32, kh=4, kw=6, stride=2, pad=0),
    "one_feature": dict(N=2, C=1, K=64, H=33, W=32, kh=7, kw=7, stride=2, pad=3),
    "stem_32_features": dict(N=5, C=3, K=32, H=66, W=80, kh=3, kw=3, stride=2, pad=1),              # x-blocks of eight columns
    "32_features_5x5": dict(N=2, C=3, K=32, H=50, W=112, kh=5, kw=5, stride=2, pad=3),
}


@pytest.mark.parametrize("name", sorted(ROW_FORM))
def test_conv_i8_first_row_form_matches_oracle(eng, name):
    """Tuning variant 4 of conv_i8_first (output rows as GEMM rows, the raw image rows as the TMA-loaded operand, the filter
    as banded matrices): every conversion-free epilogue variant, a signed image, a uniform O_QF, and the float-domain path."""
    geom = ROW_FORM[name]
    k = eng.kernel("conv_i8_first")
    variants = [dict(out_dtype=np.uint8), dict(out_dtype=np.uint8, act=abi.ACT_NONE), dict(act=abi.ACT_NONE), dict(),
                dict(in_dtype=np.int8, out_dtype=np.uint8), dict(out_dtype=np.uint8, o_qf=2.5), dict(act=abi.ACT_NONE, o_qf=16.0),
                dict(out_dtype=np.uint8, bias="none")]
    for i, extra in enumerate(variants):
        case = cases.make_conv_case(80 + i, fmt="bfyx", f_align=1, out_fmt="byxf", scale_lo=2.0 ** -13, scale_hi=2.0 ** -10, **geom, **extra)
        p = cases.copy_params(case.p); p.tune = 4
        assert k.supports(p), (name, extra)
        want = _exact(eng, case, "conv_i8_first", tune=4)
        _exact(eng, case, "conv_i8_first", tune=5)           # four epilogue groups: two share a tile by column halves
        assert len(np.unique(want[:case.out_elems])) > 16
    wide = cases.make_conv_case(90, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, scale_lo=2.0 ** -12, scale_hi=2.0 ** -10, **geom)
    wide.quant[5] = 900.0
    _exact(eng, wide, "conv_i8_first", tune=4)
    _exact(eng, wide, "conv_i8_first", tune=5)
    assert eng.device_status() == 0


def test_conv_i8_first_row_form_reads_a_padded_image(eng):
    """The image inside a larger buffer (cldnn::padding around the data: row pitch and offset beyond the image, garbage in the
    margin): the TMA boxes of the row form go by the pitches, and what lies outside the image counts as zero, as in the reference."""
    geom = dict(N=3, C=3, K=64, H=62, W=64, kh=7, kw=7, stride=2, pad=3)
    case = cases.make_conv_case(96, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, **geom)
    t, n = abi.tensor(abi.U8, geom["N"], geom["C"], geom["H"], geom["W"], "bfyx", 1, pad_lo=(1, 16), pad_hi=(2, 16))
    buf = np.random.default_rng(97).integers(1, 256, size=n, dtype=np.int64).astype(np.uint8)
    buf.reshape(geom["N"], geom["C"], geom["H"] + 3, geom["W"] + 32)[:, :, 1:1 + geom["H"], 16:16 + geom["W"]] = case.x_logical
    case.p.in_ = t
    case.inp = buf
    k = eng.kernel("conv_i8_first")
    for tune in (3, 4, 5):
        p = cases.copy_params(case.p); p.tune = tune
        assert k.supports(p), tune
        _exact(eng, case, "conv_i8_first", tune=tune)


def test_conv_i8_first_row_form_refusals(eng):
    """What the row form does not take is refused by `supports` (the tuner then never offers it): other strides, feature counts,
    row pitches that are not a multiple of 16 bytes, epilogues outside the conversion-free set."""
    k = eng.kernel("conv_i8_first")
    def sup(**kw):
        geom = dict(N=1, C=3, K=64, H=64, W=64, kh=7, kw=7, stride=2, pad=3)
        extra = {}
        for key, val in kw.items():
            (geom if key in geom else extra)[key] = val
        case = cases.make_conv_case(95, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=extra.pop("out_dtype", np.uint8), **geom, **extra)
        p = cases.copy_params(case.p); p.tune = 4
        return k.supports(p)
    assert sup()
    assert not sup(stride=1)                 # 8-bit x-blocks of four columns at stride 1 step by 8 bytes, TMA needs 16
    assert not sup(stride=3)
    assert sup(K=32, kh=3, kw=3, pad=1)      # 32 features: x-blocks of eight columns, a 3-wide filter still fits the window
    assert not sup(K=32)                     # ... a 7-wide one does not
    assert not sup(K=96)
    assert not sup(W=72)                     # 72-byte rows
    assert not sup(C=4)                      # 4 x 7 filter rows: more than shared memory holds
    assert not sup(bias="f32")
    assert not sup(calib=True)
    assert not sup(act=abi.ACT_CLAMP)
    assert not sup(kw=14)                    # the window of four outputs no longer fits 32 columns


def test_conv_ref_layouts_and_groups(eng):
    _exact(eng, cases.make_conv_case(5, 1, 128, 128, 28, 28, fmt="bfyx", f_align=1), "conv_ref")
    _exact(eng, cases.make_conv_case(6, 2, 16, 24, 9, 9, fmt="yxfb", f_align=1), "conv_ref")
    _exact(eng, cases.make_conv_case(7, 2, 32, 32, 9, 9, fmt="bfyx", f_align=1, groups=32), "conv_ref")   # depthwise
    _exact(eng, cases.make_conv_case(8, 2, 32, 64, 9, 9, fmt="bfyx", f_align=1, groups=4), "conv_ref")
    _exact(eng, cases.make_conv_case(9, 1, 16, 16, 8, 8, in_dtype=np.float32, out_dtype=np.float32, bias="none",
                                     quant=False, fmt="bfyx", f_align=1), "conv_ref")


def test_reference_kats_on_gpu(eng):
    """The reference's own literal quantised-convolution vectors through the CUDA reference-order kernel."""
    from golden import kat_conv_quantized
    from test_oracle_kat import build_kat_conv, _clamp_expected
    from cldnn_b200 import engine as E
    for name, case in kat_conv_quantized.CASES.items():
        in_dt, out_dt = np.dtype(case["in_dtype"]), np.dtype(case["out_dtype"])
        feats = case["features"]
        p, inp, w, bias = build_kat_conv(feats, in_dt.type, out_dt.type)
        p.quantization, p.act = 1, abi.ACT_RELU
        quant = np.array([f[3] for f in feats], dtype=np.float32)
        m = [eng.upload(a) for a in (inp.reshape(-1), w.reshape(-1), bias, quant)]
        out = eng.alloc(len(feats) * 2 * out_dt.itemsize)
        eng.kernel("conv_ref").launch(p, E.make_args(input0=m[0], weights=m[1], bias=m[2], quant=m[3], output=out))
        got = out.read(out_dt).reshape(len(feats), 2)
        pre = np.array([f[4] for f in feats])
        if out_dt.kind in "iu":
            np.testing.assert_array_equal(got.astype(np.int64), _clamp_expected(pre, out_dt).astype(np.int64), err_msg=name)
        else:
            np.testing.assert_allclose(got, _clamp_expected(pre, out_dt), atol=1e-3)


def test_unsupported_parameters_are_refused_not_emulated(eng):
    from cldnn_b200 import engine as E
    case = cases.make_conv_case(10, 1, 16, 16, 8, 8, fmt="bfyx", f_align=1)     # bfyx is not a tensor-core layout
    k = eng.kernel("conv_i8_tc")
    assert not k.supports(case.p)
    with pytest.raises(E.EngineError) as e:
        cases.run_gpu(eng, case, "conv_i8_tc")
    assert e.value.status == abi.UNSUPPORTED_FORMAT


DEPTHWISE = {
    # MobileNet-v2 style: 3x3 depthwise, stride 1 and 2, ReLU6 (CLAMP 0..6 in the dequantised domain)
    "dw3x3_c32": dict(N=2, C=32, K=32, H=28, W=28, groups=32),
    "dw3x3_stride2_c96": dict(N=2, C=96, K=96, H=29, W=31, groups=96, stride=2),
    "dw5x5_dilated_c16": dict(N=1, C=16, K=16, H=13, W=12, groups=16, kh=5, kw=5, pad=4, dil=2),
    "dw3x3_c960_7x7": dict(N=3, C=960, K=960, H=7, W=7, groups=960),
    # more strips of rows than one pass of the grid: the threads of the column-walk kernel take several items
    "dw3x3_c144_many_items": dict(N=96, C=144, K=144, H=56, W=56, groups=144),
}


@pytest.mark.parametrize("name", sorted(DEPTHWISE))
@pytest.mark.parametrize("variant", ["relu6_u8", "signed_calibrated"])
def test_conv_i8_dw_matches_oracle(eng, name, variant):
    kw = dict(DEPTHWISE[name])
    if variant == "relu6_u8":
        case = cases.make_conv_case(51, out_dtype=np.uint8, act=abi.ACT_CLAMP, scale_lo=2.0 ** -12, scale_hi=2.0 ** -10, **kw)
    else:
        case = cases.make_conv_case(52, in_dtype=np.int8, out_dtype=np.int8, bias="f32", calib=True, act=abi.ACT_NONE,
                                    scale_lo=2.0 ** -11, scale_hi=2.0 ** -9, **kw)
    k = eng.kernel("conv_i8_dw")
    assert k.supports(case.p)
    # tune 0 (and 2): the column-walk kernel for 3x3 filters (the 16-feature kernel otherwise), tune 1: the 16-feature kernel
    assert k.tune_count(case.p) == (3 if kw.get("kh", 3) == 3 else 1)
    for tune in range(k.tune_count(case.p)):
        case.p.tune = tune
        want = _exact(eng, case, "conv_i8_dw")
        assert len(np.unique(want)) > 4
    case.p.tune = 0
    _exact(eng, case, "conv_ref")


DW_FAST = {
    # the configurations the conversion-free epilogue of the 16-feature kernel covers
    "relu6_requantised_u8": dict(out_dtype=np.uint8, act=abi.ACT_CLAMP, o_qf=42.5),          # clamp(0, 6) * 255/6: the saturation subsumes it
    "relu_u8": dict(out_dtype=np.uint8),
    "none_s8": dict(act=abi.ACT_NONE),
    "relu_s8": dict(),
    "none_s8_oqf16": dict(act=abi.ACT_NONE, o_qf=16.0),
    "s8_in_none_u8": dict(in_dtype=np.int8, out_dtype=np.uint8, act=abi.ACT_NONE, o_qf=3.0),
    "clamp_not_subsumed": dict(out_dtype=np.uint8, act=abi.ACT_CLAMP, o_qf=20.0),             # 6 * 20 < 255: the clamp stays (general path)
}


@pytest.mark.parametrize("name", sorted(DW_FAST))
@pytest.mark.parametrize("wide", [False, True])
def test_conv_i8_dw_conversion_free_variants(eng, name, wide):
    for geom in (dict(N=3, C=48, K=48, H=17, W=19, groups=48), dict(N=2, C=144, K=144, H=15, W=14, groups=144, stride=2)):
        case = cases.make_conv_case(54, scale_lo=2.0 ** -11, scale_hi=2.0 ** -9, **geom, **DW_FAST[name])
        if wide:
            case.quant[5] = 700.0          # a feature whose values can exceed 2^22: the CTA takes the float-domain path
        for tune in (0, 1):
            case.p.tune = tune
            want = _exact(eng, case, "conv_i8_dw")
            assert len(np.unique(want[:case.out_elems])) > 8


def test_conv_i8_dw_refuses_dense_and_grouped(eng):
    k = eng.kernel("conv_i8_dw")
    assert not k.supports(cases.make_conv_case(53, N=1, C=32, K=32, H=8, W=8).p)
    assert not k.supports(cases.make_conv_case(53, N=1, C=32, K=32, H=8, W=8, groups=4).p)


def _prepare_on_gpu(eng, case, kernel, tune=0):
    """Prepared launch + its buffers for `case`; the caller runs it and reads `out`."""
    import ctypes as C
    from cldnn_b200 import engine as E
    p = cases.copy_params(case.p)
    p.tune = tune
    k = eng.kernel(kernel)
    mems = [eng.upload(v) if v is not None else None for v in (case.inp, case.w, case.bias, case.quant, case.calib)]
    out_dt = abi.np_dtype_of(p.out.dtype)
    out = eng.alloc(case.out_elems * out_dt.itemsize)
    sb = C.c_size_t()
    eng.lib.cldnn_b200_kernel_scratch_bytes(k.handle, C.byref(p), C.sizeof(p), C.byref(sb))
    scratch = eng.alloc(sb.value) if sb.value else None
    args = E.make_args(input0=mems[0], weights=mems[1], bias=mems[2], quant=mems[3], calib=mems[4], output=out, scratch=scratch)
    return k.prepare(p, args), out, out_dt, mems + [scratch]


@pytest.mark.parametrize("kernel", ["conv_i8_first", "conv_first_tc"])
def test_two_prepared_launches_with_different_shared_memory_needs(eng, kernel):
    """The dynamic shared-memory limit is a property of the kernel function, not of one prepared launch: preparing a
    small shape after a large one must leave the large one runnable (both stay alive, as two networks of a process do)."""
    big = cases.make_conv_case(71, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, **FIRST_LAYER["resnet_conv1"])
    small = cases.make_conv_case(72, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, **FIRST_LAYER["one_feature_3x3"])
    for c in (big, small):
        assert eng.kernel(kernel).supports(c.p)
    pa, out_a, dt_a, keep_a = _prepare_on_gpu(eng, big, kernel)
    pb, out_b, dt_b, keep_b = _prepare_on_gpu(eng, small, kernel)
    pa.run()
    pb.run()
    pa.run()
    eng.sync()
    assert eng.device_status() == 0
    for case, out, dt in ((big, out_a, dt_a), (small, out_b, dt_b)):
        want = cases.run_oracle(case)
        got = out.read(dt, case.out_elems)
        assert np.array_equal(want[:case.out_elems], got[:case.out_elems])
    pa.destroy()
    pb.destroy()


@pytest.mark.parametrize("order", ["mmad", "imad", "imad_fused"])
@pytest.mark.parametrize("kernel", ["conv_ref", "conv_i8_tc"])
def test_alternative_epilogue_orders_match_oracle(eng, order, kernel):
    """The operation orders of the reference's optimised int8 kernels (convolution_gpu_mmad.cl:105-128,
    fused_conv_eltwise_gpu_imad.cl:171-205) as selectable epilogue modes, on the generic kernel and on the tensor cores;
    scales chosen so that part of the values leaves the 8-bit range, where those orders wrap instead of saturating."""
    fused = order == "imad_fused"
    for calib, act in ((False, abi.ACT_RELU), (True, abi.ACT_NONE), (True, abi.ACT_CLAMP)):
        case = cases.make_conv_case(81, N=3, C=64, K=96, H=9, W=11, in_dtype=np.int8, out_dtype=np.int8, bias="f32", calib=calib, act=act,
                                    fused=fused, eltw_dtype=np.int8, eltw_calib=fused, eltw_act=act, scale_lo=2.0 ** -12, scale_hi=2.0 ** -9,
                                    o_qf=1.0 if calib else 0.75)
        case.p.act_m, case.p.act_n, case.p.eltw_m, case.p.eltw_n = -20.0, 90.0, -20.0, 90.0
        case.p.epilogue_order = abi.EPILOGUE_MMAD if order == "mmad" else abi.EPILOGUE_IMAD
        assert eng.kernel(kernel).supports(case.p)
        want = _exact(eng, case, kernel)
        assert len(np.unique(want[:case.out_elems])) > 64
    # the orders exist for a float bias and a signed 8-bit output only
    bad = cases.make_conv_case(82, N=1, C=32, K=32, H=6, W=6)
    bad.p.epilogue_order = abi.EPILOGUE_IMAD
    assert not eng.kernel(kernel).supports(bad.p)
    assert not eng.kernel("conv_i8_dw").supports(bad.p)
