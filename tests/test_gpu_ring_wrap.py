"""Parity of the persistent tensor-core kernels in the regime throughput runs use: many tiles per CTA.

The kernels launch min(SM count, tiles) persistent CTAs; each keeps a ring of operand stages, a ring of NBUF accumulators
in tensor memory (8 / 4 / 2 for 64 / 128 / 256-feature tiles) and a ring of staging tiles, all indexed by the CTA's
running tile count and its parity.  Small cases stop inside the first lap of those rings.  The cases here give every
CTA of a 148-SM device at least 4 x NBUF tiles, in every addressing mode (flat 1x1, TMA im2col, tiled box, patch), with
every feature tile, plain and with the fused residual sum, on the specialised and on the general kernel; each feature
range is visited by several CTAs and most cases cross from one feature tile to the next inside a CTA's walk.
Integer outputs must be bit-exact (arithmetic: fused_conv_eltwise_gpu_ref.cl:65-234), fp16 within 1e-2.
"""
import numpy as np
import pytest

import cases
from cldnn_b200 import abi

pytestmark = pytest.mark.gpu

SMS = 148


@pytest.fixture(scope="module")
def eng():
    from cldnn_b200 import engine
    e = engine.Engine(0)
    yield e
    e.close()


def _nbuf(bn):
    return 2 if bn >= 256 else (4 if bn >= 128 else 8)


def _tiles(case, bn):
    n, k, p, q = case.shape_out
    # flat / im2col tiles hold 128 consecutive pixels; boxed tiles never hold more
    return -(-n * p * q // 128) * -(-k // bn)


SUM = dict(fused=True, out_dtype=np.uint8, act=abi.ACT_NONE)      # the ResNet block tail: conv + residual, then ReLU, u8

# tune index of conv_i8_tc: 1 + 4 * mode + {32, 64, 128, 256}[i] with mode flat / im2col / tiled; +12 = the general kernel;
# 25..28 patch mode; +28 (29..40, and 41..44 for the patch mode) = the specialised kernel with four epilogue warp groups
# (feature tiles of 64 and 128 only: the rings must hold a multiple of the group count);
# 45..50 = CTA pairs (cta_group::2): 45 + 2 * mode + {128, 256}[i]
I8_CASES = {
    # name: (geometry, epilogue, [(tune, feature tile)])
    "3x3_k64_plain": (dict(N=200, C=32, K=64, H=56, W=56), dict(),
                      [(6, 64), (10, 64), (26, 64), (18, 64), (22, 64), (34, 64), (38, 64), (42, 64)]),
    "3x3_k256_sum": (dict(N=50, C=32, K=256, H=56, W=56), SUM,
                     [(7, 128), (11, 128), (27, 128), (8, 256), (12, 256), (28, 256), (19, 128), (24, 256), (35, 128), (39, 128), (43, 128),
                      (47, 128), (48, 256), (49, 128), (50, 256)]),
    # long reduction into 256-feature tiles without a residual: the output goes out by 128-feature units through one buffer
    "3x3_k256_plain_u8": (dict(N=50, C=32, K=256, H=56, W=56), dict(out_dtype=np.uint8),
                          [(8, 256), (12, 256), (48, 256), (50, 256), (7, 128)]),
    "1x1_k128_sum": (dict(N=200, C=32, K=128, H=56, W=56, kh=1, kw=1, pad=0), SUM,
                     [(2, 64), (3, 128), (14, 64), (15, 128), (30, 64), (31, 128), (45, 128)]),
    "1x1_k512_sum_s8res": (dict(N=256, C=64, K=512, H=28, W=28, kh=1, kw=1, pad=0),
                           dict(fused=True, out_dtype=np.int8, act=abi.ACT_NONE, eltw_dtype=np.int8),
                           [(3, 128), (4, 256), (16, 256), (31, 128), (45, 128), (46, 256)]),
    "1x1_k256_plain_u8": (dict(N=100, C=64, K=256, H=56, W=56, kh=1, kw=1, pad=0), dict(out_dtype=np.uint8),
                          [(2, 64), (4, 256), (12, 256), (30, 64), (39, 128), (46, 256), (50, 256)]),
}


@pytest.mark.parametrize("name", sorted(I8_CASES))
def test_conv_i8_tc_many_tiles_per_cta(eng, name):
    geom, epi, tunes = I8_CASES[name]
    case = cases.make_conv_case(61, scale_lo=2.0 ** -13, scale_hi=2.0 ** -11, **geom, **epi)
    want = cases.run_oracle(case)
    n = case.out_elems
    assert len(np.unique(want[:n])) > 64                    # not a saturated constant
    k = eng.kernel("conv_i8_tc")
    for tune, bn in tunes:
        assert _tiles(case, bn) >= 4 * _nbuf(bn) * SMS, "tune %d: the case does not wrap the rings four times" % tune
        p = cases.copy_params(case.p)
        p.tune = tune
        assert k.supports(p), "tune %d" % tune
        got = cases.run_gpu(eng, case, "conv_i8_tc", tune)
        bad = np.flatnonzero(want[:n] != got[:n])
        assert bad.size == 0, "tune %d: %d of %d differ; first at %d: want %d got %d" % (tune, bad.size, n, bad[0], want[bad[0]], got[bad[0]])


F16 = dict(in_dtype=np.float16, out_dtype=np.float16, quant=False, bias="f32", f_align=16)

# tune index of conv_f16_tc: 1 + 3 * mode + {64, 128, 256}[i] with mode flat / im2col / tiled
F16_CASES = {
    "3x3_k64_plain": (dict(N=200, C=16, K=64, H=56, W=56), dict(), [(4, 64), (7, 64)]),
    "3x3_k256_sum": (dict(N=50, C=16, K=256, H=56, W=56), dict(fused=True, act=abi.ACT_NONE), [(5, 128), (6, 256), (8, 128), (9, 256)]),
    "1x1_k128_sum": (dict(N=200, C=16, K=128, H=56, W=56, kh=1, kw=1, pad=0), dict(fused=True), [(1, 64), (2, 128)]),
    "1x1_k512_plain": (dict(N=256, C=32, K=512, H=28, W=28, kh=1, kw=1, pad=0), dict(), [(3, 256), (2, 128)]),
}


@pytest.mark.parametrize("name", sorted(F16_CASES))
def test_conv_f16_tc_many_tiles_per_cta(eng, name):
    geom, epi, tunes = F16_CASES[name]
    kw = dict(F16)
    kw.update(epi)
    case = cases.make_conv_case(62, **geom, **kw)
    want = cases.run_oracle(case).astype(np.float32)
    n = case.out_elems
    scale = float(np.abs(want[:n]).max())
    assert scale > 0
    k = eng.kernel("conv_f16_tc")
    for tune, bn in tunes:
        assert _tiles(case, bn) >= 4 * _nbuf(bn) * SMS
        p = cases.copy_params(case.p)
        p.tune = tune
        assert k.supports(p), "tune %d" % tune
        got = cases.run_gpu(eng, case, "conv_f16_tc", tune).astype(np.float32)
        # 1e-2 relative to each value; values below 5 % of the output scale are judged against that floor
        err = np.abs(got[:n] - want[:n])
        bad = np.flatnonzero(err > 1e-2 * np.maximum(np.abs(want[:n]), 0.05 * scale))
        assert bad.size == 0, "tune %d: %d of %d beyond 1e-2; first at %d: want %.4g got %.4g" % (tune, bad.size, n, bad[0], want[bad[0]], got[bad[0]])
