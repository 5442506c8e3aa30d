#!/usr/bin/env python
"""Compiles the reference's own OpenCL reference kernels of the network tail as C++ into oracle/_ref/clref_tail.so:

  * pooling_gpu_int8_ref.cl   (8-bit max / average pooling with the fixed divider),
  * fully_connected_gpu_bfyx_ref.cl (quantised with calibration or O_QF, and float),
  * softmax_gpu_ref.cl        (float).

The sources are taken where they lie in the reference tree and are not copied.  Each is #included several times inside a
namespace-free wrapper with a different set of compile-time switches (the `#if`s of the kernel); sizes, pitches and
factors are read at run time from the cldnn_b200_{pool,fc,softmax}_params block the oracle functions take, which stands
for the JIT "#define" block the reference's host code would emit (kernel_selector/core/common/jitter.cpp:186-639,
actual_kernels/pooling/pooling_kernel_base.cpp, fully_connected_kernel_base.cpp, softmax_kernel_base.cpp).
TEST INFRASTRUCTURE: used to cross-check oracle/cldnn_oracle.c.

usage: build_tail.py <reference root>
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "_ref")

TENSOR = """
#define {pre}_SIZE_X (g->{t}.x)
#define {pre}_SIZE_Y (g->{t}.y)
#define {pre}_FEATURE_NUM (g->{t}.f)
#define {pre}_BATCH_NUM (g->{t}.b)
#define {pre}_X_PITCH ((uint)g->{t}.px)
#define {pre}_Y_PITCH ((uint)g->{t}.py)
#define {pre}_FEATURE_PITCH ((uint)g->{t}.pf)
#define {pre}_BATCH_PITCH ((uint)g->{t}.pb)
#define {pre}_OFFSET ((uint)g->{t}.offset)
"""
UNDEF_TENSOR = "".join("#undef {pre}_%s\n" % s for s in ("SIZE_X", "SIZE_Y", "FEATURE_NUM", "BATCH_NUM", "X_PITCH", "Y_PITCH", "FEATURE_PITCH", "BATCH_PITCH", "OFFSET"))

# ACTIVATION on the kernel's value type: none / relu / clamp are what the tail of the five networks uses (jitter.cpp:366-397)
PRELUDE = r'''
#include "%(shim)s"
#include "%(abi)s"
static inline float max(float a, float b) { return a < b ? b : a; }
template <class T> static inline T tail_act(int fn, T v, float m, float n)
{
    if (fn == 1) return v > (T)0 ? v : (T)0;
    if (fn == 3) { const T lo = (T)m, hi = (T)n; return v < lo ? lo : (v > hi ? hi : v); }
    return v;
}
#define ACTIVATION(v, m, n) tail_act(g->act, (v), (m), (n))
#define NL_M (g->act_m)
#define NL_N (g->act_n)
'''


def pooling_variant(kernel, name, in_t, out_t, mode, div):
    d = ["namespace %s {" % name, "static thread_local const cldnn_b200_pool_params* g;"]
    d.append(TENSOR.format(pre="INPUT0", t="in")); d.append(TENSOR.format(pre="OUTPUT", t="out"))
    d.append("#define INPUT0_TYPE %s\n#define OUTPUT_TYPE %s\n#define TO_OUTPUT_TYPE(v) convert_%s(v)" % (in_t, out_t, out_t))
    d.append("#define OUTPUT_LAYOUT_BFYX 1\n#define %s 1\n#define CHECK_BOUNDRY 1" % ("MAX_POOLING" if mode == "max" else "AVG_POOLING"))
    if div == "dynamic":
        d.append("#define DYNAMIC_KERNEL_DIVIDER 1")
    elif div == "padding":
        d.append("#define DYNAMIC_WITH_PADDING_KERNEL_DIVIDER 1")
    d.append("#define STRIDE_SIZE_X (g->stride_x)\n#define STRIDE_SIZE_Y (g->stride_y)\n#define PADDING_SIZE_X (g->pad_x)\n#define PADDING_SIZE_Y (g->pad_y)")
    d.append("#define POOL_SIZE_X (g->size_x)\n#define POOL_SIZE_Y (g->size_y)")
    d.append('#include "%s"' % kernel)
    d.append("static void run(const cldnn_b200_pool_params* p, const void* in, void* out) {")
    d.append("    g = p;")
    d.append("    for (long bf = 0; bf < (long)p->out.b * p->out.f; ++bf) for (int y = 0; y < p->out.y; ++y) for (int x = 0; x < p->out.x; ++x) {")
    d.append("        cl_gid[0] = x; cl_gid[1] = y; cl_gid[2] = bf; pooling_gpu_int8_ref((const INPUT0_TYPE*)in, (OUTPUT_TYPE*)out); }")
    d.append("}")
    for m in ("INPUT0_TYPE", "OUTPUT_TYPE", "TO_OUTPUT_TYPE", "OUTPUT_LAYOUT_BFYX", "MAX_POOLING", "AVG_POOLING", "CHECK_BOUNDRY", "DYNAMIC_KERNEL_DIVIDER",
              "DYNAMIC_WITH_PADDING_KERNEL_DIVIDER", "STRIDE_SIZE_X", "STRIDE_SIZE_Y", "PADDING_SIZE_X", "PADDING_SIZE_Y", "POOL_SIZE_X", "POOL_SIZE_Y"):
        d.append("#undef " + m)
    d.append(UNDEF_TENSOR.format(pre="INPUT0")); d.append(UNDEF_TENSOR.format(pre="OUTPUT"))
    d.append("}")
    return "\n".join(d)


def fc_variant(kernel, name, quant, calib):
    t = "char" if quant else "float"
    d = ["namespace %s {" % name, "static thread_local const cldnn_b200_fc_params* g;"]
    d.append(TENSOR.format(pre="INPUT0", t="in")); d.append(TENSOR.format(pre="OUTPUT", t="out"))
    d.append("#define FILTER_X_PITCH ((uint)g->w_px)\n#define FILTER_Y_PITCH ((uint)g->w_py)\n#define FILTER_IFM_PITCH ((uint)g->w_pi)\n"
             "#define FILTER_OFM_PITCH ((uint)g->w_po)\n#define FILTER_OFFSET ((uint)g->w_offset)")
    d.append("#define INPUT0_TYPE %s\n#define OUTPUT_TYPE %s\n#define FILTER_TYPE %s\n#define BIAS_TYPE float\n#define UNIT_TYPE %s" % (t, t, t, t))
    d.append("#define BIAS_TERM 1\n#define QUANTIZATION_TERM %d\n#define CALIBRATION_TERM %d\n#define I_QF (g->i_qf)\n#define O_QF (g->o_qf)" % (quant, calib))
    d.append('#include "%s"' % kernel)
    args = "(const INPUT0_TYPE*)a->input0, (OUTPUT_TYPE*)a->output, (const FILTER_TYPE*)a->weights, (const BIAS_TYPE*)a->bias"
    if quant:
        args += ", a->weights_quantization_factors"
    if calib:
        args += ", a->output_calibration_factors"
    d.append("static void run(const cldnn_b200_fc_params* p, const cldnn_b200_args* a) {")
    d.append("    g = p;")
    d.append("    for (int b = 0; b < p->out.b; ++b) for (int o = 0; o < p->out.f; ++o) { cl_gid[0] = o; cl_gid[1] = b; cl_gid[2] = 0; fc(%s); }" % args)
    d.append("}")
    for m in ("FILTER_X_PITCH", "FILTER_Y_PITCH", "FILTER_IFM_PITCH", "FILTER_OFM_PITCH", "FILTER_OFFSET", "INPUT0_TYPE", "OUTPUT_TYPE", "FILTER_TYPE", "BIAS_TYPE",
              "UNIT_TYPE", "BIAS_TERM", "QUANTIZATION_TERM", "CALIBRATION_TERM", "I_QF", "O_QF"):
        d.append("#undef " + m)
    d.append(UNDEF_TENSOR.format(pre="INPUT0")); d.append(UNDEF_TENSOR.format(pre="OUTPUT"))
    d.append("}")
    return "\n".join(d)


def softmax_variant(kernel):
    # the class axis and the two "other" axes as softmax_items_class_kernel_base.cpp:45-99 names them for each dimension;
    # normalize_fyx reaches the kernel as a flattened feature axis (src/gpu/softmax_gpu.cpp:42-63) and is prepared by the caller
    d = ["namespace softmax_f32 {", "struct Axes { int cls, o0, o1; long p_cls, p_o0, p_o1, q_cls, q_o0, q_o1; };",
         "static thread_local const cldnn_b200_softmax_params* g; static thread_local Axes ax;"]
    d.append("#define INPUT0_TYPE float\n#define OUTPUT_TYPE float\n#define UNIT_TYPE float\n#define UNIT_VAL_MIN (-3.402823466e38f)")
    d.append("#define INPUT0_CLASS_NUM (ax.cls)\n#define INPUT0_CLASS_PITCH ((uint)ax.p_cls)\n#define INPUT0_OTHER0_PITCH ((uint)ax.p_o0)\n#define INPUT0_OTHER1_PITCH ((uint)ax.p_o1)")
    d.append("#define OUTPUT_CLASS_PITCH ((uint)ax.q_cls)\n#define OUTPUT_OTHER0_PITCH ((uint)ax.q_o0)\n#define OUTPUT_OTHER1_PITCH ((uint)ax.q_o1)")
    d.append("#define INPUT0_BATCH_PITCH ((uint)g->in.pb)\n#define OUTPUT_BATCH_PITCH ((uint)g->out.pb)\n#define INPUT0_OFFSET ((uint)g->in.offset)\n#define OUTPUT_OFFSET ((uint)g->out.offset)")
    d.append("#undef ACTIVATION\n#define ACTIVATION(v, m, n) (v)")
    d.append("#define __attribute__(x)")
    d.append('#include "%s"' % kernel)
    d.append("#undef __attribute__")
    d.append("static int run(const cldnn_b200_softmax_params* p, const void* in, void* out) {")
    d.append("    g = p; const cldnn_b200_tensor &i = p->in, &o = p->out;")
    d.append("    switch (p->dimension) {")
    d.append("    case 0: ax = {i.f, i.x, i.y, i.pf, i.px, i.py, o.pf, o.px, o.py}; break;")
    d.append("    case 1: ax = {i.x, i.y, i.f, i.px, i.py, i.pf, o.px, o.py, o.pf}; break;")
    d.append("    case 2: ax = {i.y, i.x, i.f, i.py, i.px, i.pf, o.py, o.px, o.pf}; break;")
    d.append("    default: return 1; }")
    d.append("    const int n0 = p->dimension == 0 ? i.x : (p->dimension == 1 ? i.y : i.x), n1 = p->dimension == 0 ? i.y : i.f;")
    d.append("    for (int b = 0; b < i.b; ++b) for (int a1 = 0; a1 < n1; ++a1) for (int a0 = 0; a0 < n0; ++a0) {")
    d.append("        cl_gid[0] = a0; cl_gid[1] = a1; cl_gid[2] = b; softmax((float*)in, (float*)out); }")
    d.append("    return 0;")
    d.append("}")
    d.append("}")
    return "\n".join(d)


def build(ref):
    kdir = os.path.join(ref, "kernel_selector", "core", "cl_kernels")
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(OUT, "clref_tail.cpp")
    so = os.path.join(OUT, "clref_tail.so")
    pool = os.path.join(kdir, "pooling_gpu_int8_ref.cl")
    fc = os.path.join(kdir, "fully_connected_gpu_bfyx_ref.cl")
    sm = os.path.join(kdir, "softmax_gpu_ref.cl")
    parts = [PRELUDE % dict(shim=os.path.join(HERE, "cl_shim.h"), abi=os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "cldnn_b200.h"))]
    pools = []
    for t in ("char", "uchar"):
        for mode in ("max", "avg"):
            for div in ("fixed", "dynamic", "padding"):
                # only the fixed divider: the dynamic-divider branch of the reference kernel (its line 123) has an unbalanced
                # parenthesis and compiles under no compiler, so there is no reference behaviour to pin for it
                if div != "fixed":
                    continue
                name = "pool_%s_%s_%s" % (t, mode, div)
                parts.append(pooling_variant(pool, name, t, t, mode, div))
                pools.append((name, t, mode, div))
    parts.append(fc_variant(fc, "fc_q_calib", 1, 1))
    parts.append(fc_variant(fc, "fc_q_oqf", 1, 0))
    parts.append(fc_variant(fc, "fc_f32", 0, 0))
    parts.append(softmax_variant(sm))
    d = ['extern "C" int clref_pooling(const cldnn_b200_pool_params* p, const void* in, void* out)', "{",
         "    if (p->in.dtype != p->out.dtype) return 1;"]
    for name, t, mode, div in pools:
        dt = "CLDNN_B200_I8" if t == "char" else "CLDNN_B200_U8"
        dm = {"fixed": "CLDNN_B200_DIV_FIXED", "dynamic": "CLDNN_B200_DIV_DYNAMIC", "padding": "CLDNN_B200_DIV_DYNAMIC_WITH_PADDING"}[div]
        cond = "p->in.dtype == %s && p->mode == %s" % (dt, "CLDNN_B200_POOL_MAX" if mode == "max" else "CLDNN_B200_POOL_AVG")
        if mode == "avg":
            cond += " && p->div_mode == " + dm
        d.append("    if (%s) { %s::run(p, in, out); return 0; }" % (cond, name))
    d += ["    return 1;", "}",
          'extern "C" int clref_fc(const cldnn_b200_fc_params* p, const cldnn_b200_args* a)', "{",
          "    if (p->bias_dtype != CLDNN_B200_F32) return 1;",
          "    if (p->quantization && p->in.dtype == CLDNN_B200_I8 && p->out.dtype == CLDNN_B200_I8) { if (p->calibration) fc_q_calib::run(p, a); else fc_q_oqf::run(p, a); return 0; }",
          "    if (!p->quantization && p->in.dtype == CLDNN_B200_F32 && p->out.dtype == CLDNN_B200_F32) { fc_f32::run(p, a); return 0; }",
          "    return 1;", "}",
          'extern "C" int clref_softmax(const cldnn_b200_softmax_params* p, const void* in, void* out)', "{",
          "    if (p->in.dtype != CLDNN_B200_F32 || p->out.dtype != CLDNN_B200_F32) return 1;",
          "    return softmax_f32::run(p, in, out);", "}"]
    parts.append("\n".join(d))
    open(src, "w").write("\n".join(parts) + "\n")
    try:
        subprocess.check_call(["/usr/bin/g++", "-O1", "-std=c++14", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-w",
                               "-I", kdir, "-o", so, src])
    finally:
        if os.path.exists(src) and not os.environ.get("CLREF_KEEP_SOURCE"):
            os.remove(src)
    return so


if __name__ == "__main__":
    print(build(sys.argv[1]))
