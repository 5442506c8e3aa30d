"""The allocation-free first-layer entry point, cldnn_b200_conv_first_noalloc.

It exists for embedders that may not allocate device memory while they run (a fixed memory budget handed out by another
allocator, or a section that cannot afford cudaMalloc's device-wide synchronisation): the packed-weights workspace that
"conv_i8_first" takes from its caller sits in a fixed array inside the library instead.  The test calls it through the C ABI
twice in a row, with different shapes so the second call finds the first call's leftovers in the shared array, and requires
the bits of the regular entry point (prepare + run with caller-provided scratch) each time.  Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

import cases
from cldnn_b200 import abi

pytestmark = pytest.mark.gpu


def _run_noalloc(eng, case):
    from cldnn_b200 import engine as E
    p = cases.copy_params(case.p)
    mems = [eng.upload(v) if v is not None else None for v in (case.inp, case.w, case.bias, case.quant, case.calib)]
    out_dt = abi.np_dtype_of(p.out.dtype)
    out = eng.alloc(case.out_elems * out_dt.itemsize)
    args = E.make_args(input0=mems[0], weights=mems[1], bias=mems[2], quant=mems[3], calib=mems[4], output=out)
    st = eng.lib.cldnn_b200_conv_first_noalloc(eng.handle, C.byref(p), C.byref(args))
    assert st == abi.SUCCESS, eng.lib.cldnn_b200_last_error().decode()
    eng.sync()
    res = out.read(out_dt, case.out_elems)
    assert eng.device_status() == 0
    return res


def test_no_alloc_entry_point_matches_regular_one_twice_in_a_row():
    from cldnn_b200 import engine as E
    eng = E.Engine(0)
    try:
        # call 1: a wide weights image (128 features x 160 bytes of K); call 2: ResNet's conv1, smaller, other strides
        first = cases.make_conv_case(31, N=2, C=4, K=128, H=21, W=30, kh=5, kw=5, stride=1, pad=2, fmt="bfyx", f_align=1,
                                     out_fmt="byxf", out_dtype=np.uint8)
        second = cases.make_conv_case(32, N=2, C=3, K=64, H=64, W=64, kh=7, kw=7, stride=2, pad=3, fmt="bfyx", f_align=1,
                                      out_fmt="byxf", in_dtype=np.int8, out_dtype=np.int8, bias="f32", calib=True, act=abi.ACT_NONE)
        for case in (first, second):
            want = cases.run_gpu(eng, case, "conv_i8_first")            # existing entry point, scratch allocated by the caller
            got = _run_noalloc(eng, case)
            n = case.out_elems
            assert np.array_equal(want[:n], got[:n]), "%d outputs differ" % int((want[:n] != got[:n]).sum())
            assert (want[:n] != 0).any()
            # and both equal the CPU oracle (bit-exact: integer outputs)
            assert np.array_equal(cases.run_oracle(case)[:n], got[:n])
        # a weights image beyond the built-in 32 KiB is refused before anything is launched
        big = cases.make_conv_case(33, N=1, C=4, K=256, H=16, W=16, kh=8, kw=8, stride=1, pad=0, fmt="bfyx", f_align=1,
                                   out_fmt="byxf", out_dtype=np.uint8)
        p = cases.copy_params(big.p)
        dummy = eng.alloc(big.out_elems)
        src = [eng.upload(v) for v in (big.inp, big.w, big.bias, big.quant)]
        args = E.make_args(input0=src[0], weights=src[1], bias=src[2], quant=src[3], output=dummy)
        assert eng.lib.cldnn_b200_conv_first_noalloc(eng.handle, C.byref(p), C.byref(args)) == abi.UNSUPPORTED_SIZE
        assert b"32768" in eng.lib.cldnn_b200_last_error()
        # a shape the kernel itself cannot run comes back with the code the regular entry point gives it, whatever its size
        p.ofm = 512
        p.out.f = 512
        assert eng.lib.cldnn_b200_conv_first_noalloc(eng.handle, C.byref(p), C.byref(args)) == abi.UNSUPPORTED_FORMAT
    finally:
        eng.close()
