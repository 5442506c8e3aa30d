#!/usr/bin/env python
"""Compiles the epilogues of the reference's optimised int8 kernels as C++ into oracle/_ref/clref_epilogues.so, so that
the MMAD / IMAD epilogue orders of the oracle (and through it of the CUDA kernels) are pinned to the reference's own text:

  * convolution_gpu_mmad.cl, from the `#if BIAS_TERM` behind the accumulation loops to the store (lines 105-128 of the
    clDNN tree this was written against),
  * fused_conv_eltwise_gpu_imad.cl, the body of the output loop from `int dotProd = out[...]` to the store (lines 171-205).

Both kernels read their operands with sub-group intrinsics and cannot be compiled whole for the host; their epilogues are
plain OpenCL C.  The lines are found by their first and last statements, cut into a scratch file under oracle/_ref at build
time, #included into a wrapper function that supplies the variables and JIT macros the lines refer to, compiled, and the
scratch files removed: nothing of the reference is kept in this repository.  TEST INFRASTRUCTURE.

usage: build_epilogues.py <reference root>
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "_ref")


def cut(path, first_stmt, last_stmt_before_endif):
    """Lines from the last line containing `first_stmt` to the first `#endif` after the line containing `last_stmt_before_endif`."""
    lines = open(path).read().split("\n")
    start = max(i for i, l in enumerate(lines) if first_stmt in l)
    last = min(i for i, l in enumerate(lines) if i > start and last_stmt_before_endif in l)
    end = min(i for i, l in enumerate(lines) if i > last and l.strip().startswith("#endif"))
    return "\n".join(lines[start:end + 1]) + "\n"


WRAPPER = r'''
#include "%(shim)s"
// operands of one output value; `scale` is calibrations[f] or O_QF
struct EpiIn { int acc; float q, iqf, bias, scale; int act; float m, n; int eltw; float ecal; int eltw_act; float em, en; };
// ACTIVATION on the 8-bit unit type (MakeActivationJitConstants, jitter.cpp:366-397, typed for char): 0 none, 1 relu, 3 clamp
static inline char act8(int fn, char v, float m, float n)
{
    if (fn == 1) return (char)max((int)0, (int)v);
    if (fn == 3) return (char)max((int)(char)m, min((int)(char)n, (int)v));
    return v;
}
#define UNIT_TYPE char
#define BIAS_TERM 1
#define BIAS_PER_OUTPUT 0
#define BIAS_PER_OFM 1
#define QUANTIZATION_TERM 1
#define I_QF (E->iqf)
#define NL_M (E->m)
#define NL_N (E->n)
#define NL_M_ELTW (E->em)
#define NL_N_ELTW (E->en)
#define ACTIVATION(v, m, n) act8(E->act, (v), (m), (n))
#define GET_DATA_INDEX(...) 0
#define OUTPUT_FEATURE_PITCH 0
#define OUTPUT_FEATURE_NUM 0
#define TO_UNIT_TYPE(v) convert_char(v)
#define TO_UNIT_TYPE_SAT(v) convert_char_sat(v)
#define OUT_BLOCK_WIDTH 1

#define MMAD_BODY(NAME)                                                                                  \
extern "C" int NAME(const EpiIn* E)                                                                      \
{                                                                                                        \
    int dotProd = E->acc; const uint f = 0, b = 0, y = 0, x = 0, split_idx = 0; (void)b; (void)y; (void)x; \
    const float quantizations[1] = {E->q}, biases[1] = {E->bias}, calibrations[1] = {E->scale}; (void)calibrations; \
    char output[1];

#define IMAD_BODY(NAME)                                                                                  \
extern "C" int NAME(const EpiIn* E)                                                                      \
{                                                                                                        \
    const int out[1] = {E->acc}; const int r = 0, c = 0; const uint f = 0, out_idx = 0, eltw_idx = 0; (void)eltw_idx; \
    const float quantizations[1] = {E->q}, biases[1] = {E->bias}, calibrations[1] = {E->scale}, eltw_calibrations[1] = {E->ecal}; \
    (void)calibrations; (void)eltw_calibrations;                                                         \
    const char eltw_input[1] = {(char)E->eltw}; (void)eltw_input;                                        \
    char output[1];

// ---- convolution_gpu_mmad.cl epilogue, per-feature calibration and uniform O_QF
#define CALIBRATION_TERM 1
MMAD_BODY(clref_mmad_calibrated)
#include "%(mmad)s"
    return output[0]; }
#undef CALIBRATION_TERM
#define CALIBRATION_TERM 0
#define O_QF (E->scale)
MMAD_BODY(clref_mmad_oqf)
#include "%(mmad)s"
    return output[0]; }

// ---- fused_conv_eltwise_gpu_imad.cl epilogue: plain convolution, then fused with the residual sum
IMAD_BODY(clref_imad_oqf)
#include "%(imad)s"
    return output[0]; }
#undef CALIBRATION_TERM
#undef O_QF
#define CALIBRATION_TERM 1
IMAD_BODY(clref_imad_calibrated)
#include "%(imad)s"
    return output[0]; }
#define ACTIVATION_ELTW(v, m, n) act8(E->eltw_act, (v), (m), (n))
IMAD_BODY(clref_imad_fused_calibrated)
#include "%(imad)s"
    return output[0]; }
'''


def build(ref):
    kdir = os.path.join(ref, "kernel_selector", "core", "cl_kernels")
    os.makedirs(OUT, exist_ok=True)
    mmad = os.path.join(OUT, "_mmad_epilogue.inc")
    imad = os.path.join(OUT, "_imad_epilogue.inc")
    src = os.path.join(OUT, "clref_epilogues.cpp")
    so = os.path.join(OUT, "clref_epilogues.so")
    open(mmad, "w").write(cut(os.path.join(kdir, "convolution_gpu_mmad.cl"), "#if BIAS_TERM", "output[dst_index] = ACTIVATION(dotProd, NL_M, NL_N);"))
    open(imad, "w").write(cut(os.path.join(kdir, "fused_conv_eltwise_gpu_imad.cl"), "int dotProd = out[r * OUT_BLOCK_WIDTH + c];", "output[out_idx] = after_activation;"))
    open(src, "w").write(WRAPPER % dict(shim=os.path.join(HERE, "cl_shim.h"), mmad=mmad, imad=imad))
    try:
        subprocess.check_call(["/usr/bin/g++", "-O1", "-std=c++14", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-w", "-o", so, src])
    finally:
        for f in (mmad, imad, src):
            if os.path.exists(f):
                os.remove(f)
    return so


if __name__ == "__main__":
    print(build(sys.argv[1]))
