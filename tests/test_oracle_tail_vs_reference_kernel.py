"""The oracle's pooling, fully_connected and softmax against the reference's own kernel sources.

oracle/_ref/clref_tail.so holds pooling_gpu_int8_ref.cl, fully_connected_gpu_bfyx_ref.cl and softmax_gpu_ref.cl compiled
as C++ where they lie in the clDNN tree (oracle/ref_build/build_tail.py).  On seeded random inputs in bfyx, byxf and
padded layouts the C restatement must give the same bits.  The dynamic-divider branch of the reference's 8-bit pooling
kernel does not compile (unbalanced parenthesis in its source), so only the fixed divider has a reference to be pinned to.
"""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib
from cldnn_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "oracle", "_ref", "clref_tail.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(SO):
        pytest.skip("oracle/_ref/clref_tail.so not built (needs the clDNN tree)")
    lib = C.CDLL(SO)
    lib.clref_pooling.argtypes = [C.POINTER(abi.PoolParams), C.c_void_p, C.c_void_p]
    lib.clref_fc.argtypes = [C.POINTER(abi.FcParams), C.POINTER(abi.Args)]
    lib.clref_softmax.argtypes = [C.POINTER(abi.SoftmaxParams), C.c_void_p, C.c_void_p]
    return lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


POOL_CASES = [
    # dtype, mode, fmt, (b, f, y, x), size, stride, pad, act
    (np.uint8, abi.POOL_MAX, "byxf", (2, 32, 13, 13), 3, 2, 0, abi.ACT_NONE),
    (np.uint8, abi.POOL_MAX, "bfyx", (2, 5, 12, 11), 3, 2, 1, abi.ACT_NONE),
    (np.int8, abi.POOL_MAX, "byxf", (1, 16, 9, 9), 2, 2, 0, abi.ACT_RELU),
    (np.int8, abi.POOL_MAX, "bfyx", (2, 3, 8, 8), 3, 1, 1, abi.ACT_NONE),
    (np.uint8, abi.POOL_AVG, "byxf", (2, 64, 7, 7), 7, 1, 0, abi.ACT_NONE),
    (np.int8, abi.POOL_AVG, "bfyx", (2, 4, 10, 10), 3, 2, 1, abi.ACT_NONE),
    (np.int8, abi.POOL_AVG, "byxf", (1, 32, 6, 6), 2, 2, 0, abi.ACT_RELU),
    (np.uint8, abi.POOL_AVG, "bfyx", (1, 7, 9, 9), 3, 3, 0, abi.ACT_NONE),
]


@pytest.mark.parametrize("case", range(len(POOL_CASES)))
def test_pooling_equals_the_reference_kernel_source(ref, case):
    dtype, mode, fmt, (b, f, y, x), size, stride, pad, act = POOL_CASES[case]
    rng = np.random.default_rng(300 + case)
    dt = abi.U8 if dtype == np.uint8 else abi.I8
    info = np.iinfo(dtype)
    logical = rng.integers(info.min, info.max + 1, size=(b, f, y, x)).astype(dtype)
    oy = oracle_lib.pool_out_size(y, size, -pad, stride)
    ox = oracle_lib.pool_out_size(x, size, -pad, stride)
    p = abi.PoolParams()
    p.in_, _ = abi.tensor(dt, b, f, y, x, fmt)
    p.out, n_out = abi.tensor(dt, b, f, oy, ox, fmt)
    p.mode, p.div_mode = mode, abi.DIV_FIXED
    p.size_x = p.size_y = size
    p.stride_x = p.stride_y = stride
    p.pad_x = p.pad_y = pad
    p.act = act
    flat = abi.to_layout(logical, fmt)
    want = np.full(n_out, 0x55, dtype=dtype)
    assert ref.clref_pooling(C.byref(p), _ptr(flat), _ptr(want)) == 0
    got = np.full(n_out, 0x55, dtype=dtype)
    oracle_lib.pooling(p, flat, out=got, threads=1)
    assert np.array_equal(got, want)
    assert len(np.unique(want)) > 8


@pytest.mark.parametrize("calib", [False, True])
@pytest.mark.parametrize("fmt", ["bfyx", "byxf"])
def test_quantised_fully_connected_equals_the_reference_kernel_source(ref, calib, fmt):
    rng = np.random.default_rng(410 + calib)
    b, f, y, x, ofm = 3, 8, 3, 3, 24
    inp = rng.integers(-128, 128, size=(b, f, y, x)).astype(np.int8)
    w = rng.integers(-128, 128, size=(ofm, f, y, x)).astype(np.int8)
    bias = rng.uniform(-20, 20, size=ofm).astype(np.float32)
    quant = rng.uniform(2.0 ** -12, 2.0 ** -10, size=ofm).astype(np.float32)
    cal = rng.uniform(0.5, 1.5, size=ofm).astype(np.float32)
    p = abi.FcParams()
    p.in_, _ = abi.tensor(abi.I8, b, f, y, x, fmt)
    p.out, n_out = abi.tensor(abi.I8, b, ofm, 1, 1, "bfyx")
    p.w_dtype = abi.I8
    p.w_px, p.w_py, p.w_pi, p.w_po, p.w_offset = 1, x, x * y, x * y * f, 0
    p.bias_dtype, p.quantization, p.i_qf, p.calibration, p.o_qf = abi.F32, 1, 0.75, int(calib), 1.25
    p.act = abi.ACT_RELU
    flat = abi.to_layout(inp, fmt)
    got, oor = oracle_lib.fc(p, flat, w.reshape(-1), bias, quant, cal if calib else None, threads=1)
    assert oor == 0                                  # in range: the reference's plain (char) cast is defined there
    want = np.zeros(n_out, dtype=np.int8)
    a = abi.Args()
    a.input0, a.output, a.weights, a.bias = _ptr(flat), _ptr(want), _ptr(w), _ptr(bias)
    a.weights_quantization_factors = _ptr(quant)
    if calib:
        a.output_calibration_factors = _ptr(cal)
    assert ref.clref_fc(C.byref(p), C.byref(a)) == 0
    assert np.array_equal(got, want)
    assert len(np.unique(want)) > 8


def test_float_fully_connected_equals_the_reference_kernel_source(ref):
    rng = np.random.default_rng(420)
    b, f, y, x, ofm = 2, 6, 2, 2, 10
    inp = rng.standard_normal((b, f, y, x)).astype(np.float32)
    w = rng.standard_normal((ofm, f, y, x)).astype(np.float32)
    bias = rng.standard_normal(ofm).astype(np.float32)
    p = abi.FcParams()
    p.in_, _ = abi.tensor(abi.F32, b, f, y, x, "bfyx")
    p.out, n_out = abi.tensor(abi.F32, b, ofm, 1, 1, "bfyx")
    p.w_dtype = abi.F32
    p.w_px, p.w_py, p.w_pi, p.w_po, p.w_offset = 1, x, x * y, x * y * f, 0
    p.bias_dtype, p.act = abi.F32, abi.ACT_RELU
    flat = inp.reshape(-1)
    got, _ = oracle_lib.fc(p, flat, w.reshape(-1), bias, threads=1)
    want = np.zeros(n_out, dtype=np.float32)
    a = abi.Args()
    a.input0, a.output, a.weights, a.bias = _ptr(flat), _ptr(want), _ptr(w), _ptr(bias)
    assert ref.clref_fc(C.byref(p), C.byref(a)) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dim", [abi.SOFTMAX_F, abi.SOFTMAX_X, abi.SOFTMAX_Y, abi.SOFTMAX_FYX])
@pytest.mark.parametrize("fmt", ["bfyx", "byxf"])
def test_softmax_equals_the_reference_kernel_source(ref, dim, fmt):
    rng = np.random.default_rng(430 + dim)
    b, f, y, x = 3, 10, 4, 5
    logical = (rng.standard_normal((b, f, y, x)) * 3).astype(np.float32)
    if dim == abi.SOFTMAX_FYX and fmt != "bfyx":
        pytest.skip("normalize_fyx reaches the reference kernel as a flattened bfyx feature axis")
    p = abi.SoftmaxParams()
    p.in_, _ = abi.tensor(abi.F32, b, f, y, x, fmt)
    p.out, n_out = abi.tensor(abi.F32, b, f, y, x, fmt)
    p.dimension = dim
    flat = abi.to_layout(logical, fmt)
    got = oracle_lib.softmax(p, flat)
    want = np.zeros(n_out, dtype=np.float32)
    q = abi.SoftmaxParams()
    if dim == abi.SOFTMAX_FYX:
        # what src/gpu/softmax_gpu.cpp:42-63 hands the kernel: one class axis of f*y*x values
        q.in_, _ = abi.tensor(abi.F32, b, f * y * x, 1, 1, "bfyx")
        q.out, _ = abi.tensor(abi.F32, b, f * y * x, 1, 1, "bfyx")
        q.dimension = abi.SOFTMAX_F
    else:
        q.in_, q.out, q.dimension = p.in_, p.out, dim
    assert ref.clref_softmax(C.byref(q), _ptr(flat), _ptr(want)) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    sums = abi.from_layout(want, (b, f, y, x), fmt).sum(axis={abi.SOFTMAX_F: 1, abi.SOFTMAX_X: 3, abi.SOFTMAX_Y: 2, abi.SOFTMAX_FYX: (1, 2, 3)}[dim])
    assert np.allclose(sums, 1.0, atol=1e-5)
