"""Parity of the general first-layer tensor-core convolution (conv_first_tc: few input features, K = C*kh filter rows padded to
whole 16-byte core rows, planar input read in place) with the CPU oracle, through the C ABI: bit-exact for the 8-bit form, 1e-2 relative to the
output scale for fp16 (the reference accumulates fp16 in half precision with device-defined rounding)."""
import numpy as np
import pytest

import cases
from cldnn_b200 import abi

pytestmark = pytest.mark.gpu

RTOL = 1e-2


@pytest.fixture(scope="module")
def eng():
    from cldnn_b200 import engine
    e = engine.Engine(0)
    yield e
    e.close()


GEOMS = {
    # VGG16 conv1_1: 3 -> 64, 3x3 pad 1; AlexNet conv1: 3 -> 96, 11x11 stride 4 (227 -> 55); ragged and odd shapes
    "vgg_conv1_1": dict(N=2, C=3, K=64, H=64, W=64),
    "alexnet_conv1": dict(N=2, C=3, K=96, H=227, W=227, kh=11, kw=11, stride=4, pad=0),
    "alexnet_conv1_padded": dict(N=3, C=3, K=96, H=43, W=51, kh=11, kw=11, stride=4, pad=2),
    "one_feature_5x5": dict(N=3, C=1, K=32, H=19, W=23, kh=5, kw=5, pad=2),
    "four_features_dilated": dict(N=1, C=4, K=128, H=21, W=20, kh=3, kw=3, dil=2, pad=2),
    "many_tiles": dict(N=9, C=3, K=64, H=93, W=101, stride=2),
    "less_than_one_tile": dict(N=1, C=3, K=256, H=5, W=6, kh=3, kw=3, pad=1),
}


def _f16_case(seed, **kw):
    kw.setdefault("bias", "f32")
    return cases.make_conv_case(seed, fmt="bfyx", f_align=1, out_fmt="byxf", in_dtype=np.float16, out_dtype=np.float16, quant=False, **kw)


def _close(eng, case, tune=0):
    want = cases.run_oracle(case).astype(np.float32)
    got = cases.run_gpu(eng, case, "conv_first_tc", tune).astype(np.float32)
    n = case.out_elems
    scale = float(np.abs(want[:n]).max())
    assert scale > 0
    err = np.abs(got[:n] - want[:n])
    bad = np.flatnonzero(err > RTOL * np.maximum(np.abs(want[:n]), 0.05 * scale))
    assert bad.size == 0, "%d of %d beyond %.0e relative; worst %.4g vs %.4g" % (bad.size, n, RTOL, got[bad[0]], want[bad[0]])
    return want


def _exact(eng, case):
    want = cases.run_oracle(case)
    got = cases.run_gpu(eng, case, "conv_first_tc")
    n = case.out_elems
    bad = np.flatnonzero(want[:n] != got[:n])
    assert bad.size == 0, "%d of %d differ; first at %d: want %d got %d" % (bad.size, n, bad[0], want[bad[0]], got[bad[0]])
    return want


@pytest.mark.parametrize("name", sorted(GEOMS))
def test_conv_first_tc_f16_matches_oracle(eng, name):
    case = _f16_case(51, **GEOMS[name])
    assert eng.kernel("conv_first_tc").supports(case.p)
    want = _close(eng, case)
    assert (want != 0).any()


@pytest.mark.parametrize("name", sorted(GEOMS))
@pytest.mark.parametrize("variant", ["relu_u8", "signed_in_calibrated"])
def test_conv_first_tc_i8_bit_exact(eng, name, variant):
    kw = dict(GEOMS[name])
    if variant == "relu_u8":
        case = cases.make_conv_case(52, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, **kw)
    else:
        case = cases.make_conv_case(53, fmt="bfyx", f_align=1, out_fmt="byxf", in_dtype=np.int8, out_dtype=np.int8, bias="f32", calib=True,
                                    act=abi.ACT_NONE, **kw)
    assert eng.kernel("conv_first_tc").supports(case.p)
    want = _exact(eng, case)
    assert len(np.unique(want[:case.out_elems])) > 16


def test_conv_first_tc_f16_epilogues(eng):
    for extra in (dict(bias="none"), dict(act=abi.ACT_NONE), dict(act=abi.ACT_CLAMP), dict(act=abi.ACT_RELU_NEGATIVE_SLOPE)):
        case = _f16_case(54, N=2, C=3, K=64, H=30, W=31, kh=5, kw=5, pad=2, **extra)
        if extra.get("act") == abi.ACT_RELU_NEGATIVE_SLOPE:
            case.p.act_m = 0.125
        _close(eng, case)


ROW_FORM_F16 = {
    # what the row form (tuning variants 2 / 3: output rows as GEMM rows, image rows by TMA, banded filter matrices) takes in fp16:
    # stride 1 or 2, 64 output features (eight columns of 32 features do not fit a 16-column window), row pitch a multiple of 16 bytes
    "vgg_conv1_1": dict(N=2, C=3, K=64, H=64, W=64),
    "vgg_conv1_1_two_row_tiles": dict(N=3, C=3, K=64, H=224, W=48),
    "many_tiles_stride2": dict(N=9, C=3, K=64, H=93, W=104, stride=2),
    "one_feature_5x5": dict(N=3, C=1, K=64, H=19, W=24, kh=5, kw=5, pad=2),
}


@pytest.mark.parametrize("name", sorted(ROW_FORM_F16))
def test_conv_first_tc_row_form_f16_matches_oracle(eng, name):
    k = eng.kernel("conv_first_tc")
    for i, extra in enumerate((dict(), dict(bias="none", act=abi.ACT_NONE), dict(act=abi.ACT_CLAMP))):
        case = _f16_case(60 + i, **ROW_FORM_F16[name], **extra)
        for tune in (2, 3):
            p = cases.copy_params(case.p); p.tune = tune
            assert k.supports(p), (name, tune)
            want = _close(eng, case, tune)
            assert (want != 0).any()


def test_conv_first_tc_row_form_refusals(eng):
    k = eng.kernel("conv_first_tc")
    def sup(**kw):
        geom = dict(N=1, C=3, K=64, H=32, W=32)
        geom.update(kw)
        p = cases.copy_params(_f16_case(69, **geom).p); p.tune = 2
        return k.supports(p)
    assert sup()
    assert not sup(W=36)                     # 72-byte rows
    assert not sup(K=96)
    assert not sup(K=32)
    assert not sup(stride=4, kh=11, kw=11, pad=0, H=67, W=64)
    assert not sup(kh=3, kw=9, pad=1)        # four outputs' taps no longer fit sixteen columns
    case = cases.make_conv_case(70, fmt="bfyx", f_align=1, out_fmt="byxf", out_dtype=np.uint8, N=1, C=3, K=64, H=32, W=32)
    p = cases.copy_params(case.p); p.tune = 2
    assert not k.supports(p)                 # the 8-bit row form is reached through conv_i8_first


def test_conv_first_tc_reads_any_input_pitches(eng):
    """The gather goes through a table of element offsets, so a feature-innermost (byxf) input works as well."""
    case = cases.make_conv_case(55, N=2, C=4, K=64, H=18, W=18, fmt="byxf", f_align=4, w_layout="oiyx", in_dtype=np.float16, out_dtype=np.float16,
                                quant=False, bias="f32", out_fmt="byxf")
    assert eng.kernel("conv_first_tc").supports(case.p)
    _close(eng, case)


def test_conv_first_tc_refusals(eng):
    k = eng.kernel("conv_first_tc")
    assert not k.supports(_f16_case(56, N=1, C=128, K=64, H=8, W=8).p)              # 384 filter rows: more cores than the gather table holds
    assert not k.supports(_f16_case(56, N=1, C=3, K=40, H=8, W=8).p)                # output features not a multiple of 32
    assert not k.supports(cases.make_conv_case(56, N=1, C=3, K=64, H=8, W=8, fmt="bfyx", f_align=1, out_dtype=np.uint8).p)   # planar output
