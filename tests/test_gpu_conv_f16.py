"""Parity of the fp16 tensor-core convolution with the CPU oracle, through the C ABI.
The reference accumulates fp16 convolutions in half precision with device-defined rounding of mad(), so its own
tests compare against a wide-accumulator helper with a tolerance; the bar here is 1e-2 relative to the output scale."""
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


def _close(eng, case, kernel, tune=0, floor=0.05):
    want = cases.run_oracle(case).astype(np.float32)
    got = cases.run_gpu(eng, case, kernel, tune).astype(np.float32)
    n = case.out_elems
    scale = float(np.abs(want[:n]).max())
    assert scale > 0
    err = np.abs(got[:n] - want[:n])
    # relative to each value, with a floor of `floor` x the output scale under which the error is judged absolutely
    bad = np.flatnonzero(err > RTOL * np.maximum(np.abs(want[:n]), floor * scale))
    assert bad.size == 0, "%d of %d beyond %.0e relative; worst %.4g vs %.4g" % (bad.size, n, RTOL, got[bad[0]], want[bad[0]])
    return want


F16 = dict(in_dtype=np.float16, out_dtype=np.float16, quant=False, bias="f32", f_align=16)

GEOMS = {
    # VGG16-like 3x3 layers at reduced size, the 1x1 / strided / ragged cases of the 8-bit suite
    "vgg_64_64": dict(N=2, C=64, K=64, H=56, W=56),
    "vgg_128_256": dict(N=2, C=128, K=256, H=28, W=28),
    "vgg_512_512": dict(N=3, C=512, K=512, H=14, W=14),
    "first_layer_c3": dict(N=2, C=3, K=64, H=40, W=40),
    "1x1": dict(N=2, C=64, K=256, H=28, W=28, kh=1, kw=1, pad=0),
    "1x1_stride2": dict(N=2, C=256, K=128, H=28, W=28, kh=1, kw=1, pad=0, stride=2),
    "ragged_c48_k40": dict(N=3, C=48, K=40, H=9, W=11),
    "stride2_3x3": dict(N=10, C=64, K=96, H=15, W=15, stride=2),
    "dilation2": dict(N=1, C=32, K=32, H=12, W=12, dil=2, pad=2),
    "5x5": dict(N=1, C=16, K=32, H=10, W=10, kh=5, kw=5, pad=2),
}


@pytest.mark.parametrize("name", sorted(GEOMS))
def test_conv_f16_tc_matches_oracle(eng, name):
    case = cases.make_conv_case(31, **GEOMS[name], **F16)
    k = eng.kernel("conv_f16_tc")
    assert k.supports(case.p)
    want = _close(eng, case, "conv_f16_tc")
    assert (want != 0).any()


@pytest.mark.parametrize("name", ["vgg_128_256", "1x1", "ragged_c48_k40", "stride2_3x3"])
def test_conv_f16_tc_every_tuning_variant(eng, name):
    k = eng.kernel("conv_f16_tc")
    case = cases.make_conv_case(32, **GEOMS[name], **F16)
    ran = 0
    for tune in range(1, k.tune_count(case.p)):
        p = cases.copy_params(case.p)
        p.tune = tune
        if not k.supports(p):
            continue
        _close(eng, case, "conv_f16_tc", tune)
        ran += 1
    assert ran >= 3


PATCH_MODE = {
    # geometries the patch mode takes (stride 1, one feature tile, weights within 80 KiB): tunes 10 / 11 / 12
    "vgg_conv1_2": dict(N=2, C=64, K=64, H=56, W=56),
    "many_tiles_per_cta": dict(N=40, C=64, K=64, H=56, W=56),                 # ~1000 tiles: every ring wraps several times
    "ragged_map_32_features": dict(N=3, C=32, K=40, H=19, W=23),
    "5x5_16_features": dict(N=2, C=16, K=32, H=21, W=20, kh=5, kw=5, pad=2),
    "no_padding_k128": dict(N=2, C=32, K=128, H=17, W=18, pad=0),
}


@pytest.mark.parametrize("name", sorted(PATCH_MODE))
def test_conv_f16_tc_patch_mode(eng, name):
    """Resident weights, one activation patch per filter column (tunes 10..12), plain and with a fused residual."""
    k = eng.kernel("conv_f16_tc")
    for extra in (dict(), dict(fused=True, act=abi.ACT_NONE)):
        kw = dict(F16); kw.update(extra)
        case = cases.make_conv_case(35, **PATCH_MODE[name], **kw)
        ran = 0
        for tune in (10, 11, 12):
            p = cases.copy_params(case.p); p.tune = tune
            if not k.supports(p):
                continue
            _close(eng, case, "conv_f16_tc", tune)
            ran += 1
        assert ran >= 1, name
    assert eng.device_status() == 0


def test_conv_f16_tc_patch_mode_refusals(eng):
    k = eng.kernel("conv_f16_tc")
    def sup(**geom):
        p = cases.copy_params(cases.make_conv_case(36, **geom, **F16).p); p.tune = 10
        return k.supports(p)
    assert sup(N=1, C=64, K=64, H=28, W=28)
    assert not sup(N=1, C=64, K=128, H=28, W=28)              # two feature tiles of 64
    assert not sup(N=1, C=64, K=64, H=28, W=28, stride=2)
    assert not sup(N=1, C=64, K=64, H=28, W=28, kh=1, kw=1, pad=0)
    assert not sup(N=1, C=256, K=64, H=14, W=14)              # 9 x 256 x 64 halves exceed the resident budget


EPILOGUES = {
    "no_bias": dict(bias="none"),
    "no_activation": dict(act=abi.ACT_NONE),
    "relu6_clamp": dict(act=abi.ACT_CLAMP),
    "leaky": dict(act=abi.ACT_RELU_NEGATIVE_SLOPE),
    "residual_sum": dict(fused=True, act=abi.ACT_NONE),
    "residual_sum_in_place": dict(fused=True, in_out_opt=True),
}


@pytest.mark.parametrize("name", sorted(EPILOGUES))
def test_conv_f16_tc_epilogues(eng, name):
    kw = dict(F16); kw.update(EPILOGUES[name])
    case = cases.make_conv_case(33, N=2, C=64, K=128, H=14, W=14, **kw)
    if name == "leaky":
        case.p.act_m = 0.125
    assert eng.kernel("conv_f16_tc").supports(case.p)
    _close(eng, case, "conv_f16_tc")


def test_conv_f16_ref_kernel_agrees(eng):
    """The generic reference-order kernel on the same fp16 case (any layout): the selector's fallback."""
    case = cases.make_conv_case(34, N=2, C=32, K=48, H=9, W=9, **F16)
    _close(eng, case, "conv_ref")


WINOGRAD = {
    "vgg_64_64": dict(N=2, C=64, K=64, H=56, W=56),
    "vgg_256_256": dict(N=2, C=256, K=256, H=28, W=28),
    "vgg_512_512": dict(N=3, C=512, K=512, H=14, W=14),
    "first_layer_c3": dict(N=2, C=3, K=64, H=40, W=40),
    "odd_map_ragged_features": dict(N=3, C=48, K=40, H=9, W=11),
    "no_padding": dict(N=2, C=32, K=32, H=12, W=13, pad=0),
}


@pytest.mark.parametrize("name", sorted(WINOGRAD))
def test_conv_f16_winograd_matches_oracle(eng, name):
    """Winograd F(2x2, 3x3) against the direct-form oracle.  The reference pins nothing here (it has no Winograd test), so the
    bar is this repository's own: 1e-2 relative to each value, and for values below a tenth of the output scale an absolute
    1e-3 of the scale.  Measured on these geometries the largest absolute error is 5.4e-4 .. 6.7e-4 of the scale -- the final
    rounding to fp16 at the top of the range, as for the direct kernel; the fp16 transforms add nothing visible beyond it --
    and 1.9e-3 relative among values above a quarter of the scale."""
    case = cases.make_conv_case(41, **WINOGRAD[name], **F16)
    k = eng.kernel("conv_f16_winograd")
    assert k.supports(case.p)
    _close(eng, case, "conv_f16_winograd", floor=0.1)


def test_conv_f16_winograd_epilogue_and_refusals(eng):
    k = eng.kernel("conv_f16_winograd")
    for extra in (dict(bias="none"), dict(act=abi.ACT_NONE), dict(act=abi.ACT_CLAMP)):
        kw = dict(F16); kw.update(extra)
        _close(eng, cases.make_conv_case(42, N=2, C=32, K=64, H=14, W=14, **kw), "conv_f16_winograd", floor=0.1)
    assert not k.supports(cases.make_conv_case(43, N=1, C=32, K=32, H=8, W=8, stride=2, **F16).p)
    assert not k.supports(cases.make_conv_case(43, N=1, C=32, K=32, H=8, W=8, kh=1, kw=1, pad=0, **F16).p)
    assert not k.supports(cases.make_conv_case(43, N=1, C=32, K=32, H=8, W=8).p)            # 8-bit
