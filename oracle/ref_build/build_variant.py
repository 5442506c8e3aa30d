#!/usr/bin/env python
"""Compiles one specialisation of the reference's own OpenCL reference convolution kernel
(kernel_selector/core/cl_kernels/fused_conv_eltwise_gpu_ref.cl in the clDNN tree) as C++ into oracle/_ref/.

The kernel source is taken where it lies in the reference tree and is not copied.  What the reference's host code would
emit as a JIT "#define" block (kernel_selector/core/common/jitter.cpp:186-639, actual_kernels/convolution/
convolution_kernel_base.cpp:51-127, fused_conv_eltwise_kernel_base.cpp:122-190) is written here: the compile-time
switches (#if'd in the kernel) select the variant, sizes / pitches / factors are read at run time from the
cldnn_b200_conv_params block.  TEST INFRASTRUCTURE: used to cross-check oracle/cldnn_oracle.c and as a CPU baseline.

usage: build_variant.py <reference root> <variant name>
variant name: <in>_<out>_<eltw>_b<bias>_q<0|1>c<0|1>o<0|1>_f<0|1>n<0|1>e<0|1>   types: c (i8), uc (u8), f (f32);
              bias: n (none), i (i32), f (f32); eltw type is ignored when f0.
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "_ref")
CT = {"c": "char", "uc": "uchar", "f": "float"}


def parse(name):
    m = re.fullmatch(r"(c|uc|f)_(c|uc|f)_(c|uc|f)_b(n|i|f)_q([01])c([01])o([01])_f([01])n([01])e([01])", name)
    if not m:
        raise SystemExit("bad variant name " + name)
    i, o, e, b, q, c, oq, f, n, ec = m.groups()
    return dict(i=i, o=o, e=e, b=b, q=int(q), c=int(c), oq=int(oq), f=int(f), n=int(n), ec=int(ec))


def variant_name(in_t, out_t, eltw_t, bias, q, c, oq, fused, ncs, ecal):
    return "%s_%s_%s_b%s_q%dc%do%d_f%dn%de%d" % (in_t, out_t, eltw_t, bias, q, c, oq, fused, ncs, ecal)


def source(ref, v):
    kernel = os.path.join(ref, "kernel_selector", "core", "cl_kernels", "fused_conv_eltwise_gpu_ref.cl")
    d = []
    A = d.append
    A('#include "%s"' % os.path.join(HERE, "cl_shim.h"))
    A('#include "%s"' % os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "cldnn_b200.h"))
    A("static thread_local const cldnn_b200_conv_params* g;")
    # tensors: MakeJitConstant(DataTensor), jitter.cpp:229-262
    for pre, t in (("INPUT0", "in"), ("OUTPUT", "out"), ("INPUT1", "eltw")):
        A("#define %s_SIZE_X (g->%s.x)" % (pre, t)); A("#define %s_SIZE_Y (g->%s.y)" % (pre, t))
        A("#define %s_FEATURE_NUM (g->%s.f)" % (pre, t)); A("#define %s_BATCH_NUM 2" % pre if pre == "OUTPUT" else "#define %s_BATCH_NUM (g->%s.b)" % (pre, t))
        A("#define %s_X_PITCH ((uint)g->%s.px)" % (pre, t)); A("#define %s_Y_PITCH ((uint)g->%s.py)" % (pre, t))
        A("#define %s_FEATURE_PITCH ((uint)g->%s.pf)" % (pre, t)); A("#define %s_BATCH_PITCH ((uint)g->%s.pb)" % (pre, t))
        A("#define %s_OFFSET ((uint)g->%s.offset)" % (pre, t))
    # weights: MakeJitConstant(WeightsTensor), jitter.cpp:286-300
    A("#define FILTER_SIZE_X (g->kw)"); A("#define FILTER_SIZE_Y (g->kh)"); A("#define FILTER_IFM_NUM (g->ifm)"); A("#define FILTER_OFM_NUM (g->ofm)")
    A("#define FILTER_X_PITCH ((uint)g->w_px)"); A("#define FILTER_Y_PITCH ((uint)g->w_py)"); A("#define FILTER_IFM_PITCH ((uint)g->w_pi)")
    A("#define FILTER_OFM_PITCH ((uint)g->w_po)"); A("#define FILTER_OFFSET ((uint)g->w_offset)")
    A("#define GET_FILTER_INDEX_DUMMY 0")
    # convolution constants, convolution_kernel_base.cpp:51-127
    A("#define STRIDE_SIZE_X (g->stride_x)"); A("#define STRIDE_SIZE_Y (g->stride_y)"); A("#define PADDING_SIZE_X (g->pad_x)"); A("#define PADDING_SIZE_Y (g->pad_y)")
    A("#define DILATION_SIZE_X (g->dil_x)"); A("#define DILATION_SIZE_Y (g->dil_y)")
    A("#define DEPTHWISE_SEPARABLE_OPT 1")      # all groups in one launch: in_split_offset = (f / FILTER_OFM_NUM) * pitch * IFM
    A("#define GROUPED 0")
    A("#define QUANTIZATION_TERM %d" % v["q"]); A("#define CALIBRATION_TERM %d" % v["c"])
    A("#define I_QF (g->i_qf)")
    if v["oq"]:
        A("#define O_QF (g->o_qf)")
    A("#define BIAS_TERM %d" % (v["b"] != "n")); A("#define BIAS_PER_OFM 1"); A("#define BIAS_PER_OUTPUT 0")
    if v["q"] and v["b"] == "f":
        A("#define DONT_DEQUANTIZE_BIAS 1")      # convolution_kernel_ref.cpp:89-91
    else:
        A("#define DONT_DEQUANTIZE_BIAS 0")
    A("#define INPUT0_TYPE %s" % CT[v["i"]]); A("#define OUTPUT_TYPE %s" % CT[v["o"]]); A("#define INPUT1_TYPE %s" % CT[v["e"]])
    A("#define FILTER_TYPE %s" % ("float" if v["i"] == "f" else "char")); A("#define BIAS_TYPE %s" % {"n": "int", "i": "int", "f": "float"}[v["b"]])
    A("#define OUTPUT_IS_FP %d" % (v["o"] == "f"))
    A("#define INT8_UNIT_USED %d" % (v["i"] == "c")); A("#define UINT8_UNIT_USED %d" % (v["i"] == "uc"))
    # type macros, MakeTypeJitConstants, jitter.cpp:462-585
    A("#define TO_INPUT0_TYPE(v) convert_%s(v)" % CT[v["i"]])
    A("#define TO_OUTPUT_TYPE_SAT(v) %s(v)" % ("convert_float" if v["o"] == "f" else "convert_%s_sat" % CT[v["o"]]))
    A("#define float_VAL_ZERO 0.0f"); A("#define float_VAL_ONE 1.0f"); A("#define float_MAX_FUNC fmax"); A("#define float_MIN_FUNC fmin")
    A("#define TO_float_TYPE(v) convert_float(v)"); A("#define TO_float_TYPE_SAT(v) convert_float(v)")
    A("#define int_VAL_ZERO (int) 0"); A("#define int_VAL_ONE (int) 1"); A("#define int_MAX_FUNC max"); A("#define int_MIN_FUNC min")
    A("#define TO_int_TYPE(v) convert_int(v)"); A("#define TO_int_TYPE_SAT(v) convert_int_sat(v)")
    # the convolution's own float type when the input is float ("INPUT0" base name)
    A("#define INPUT0_VAL_ZERO 0.0f"); A("#define INPUT0_VAL_ONE 1.0f"); A("#define INPUT0_MAX_FUNC fmax"); A("#define INPUT0_MIN_FUNC fmin")
    A("#define TO_INPUT0_TYPE_SAT(v) convert_float(v)")
    # activation macros, MakeActivationJitConstants, jitter.cpp:313-445 (typed form); the function is chosen at run time
    act = ("((fn) == 1 ? (CAT(jit_type, _MAX_FUNC)(CAT(jit_type, _VAL_ZERO), input)) : "
           "(fn) == 2 ? (isinf(CAT(CAT(TO_, jit_type), _TYPE)(m)) ? ((input >= CAT(jit_type, _VAL_ZERO)) ? input : -CAT(CAT(TO_, jit_type), _TYPE)(m)) : "
           "(CAT(jit_type, _MAX_FUNC)(input, CAT(jit_type, _VAL_ZERO)) + (CAT(CAT(TO_, jit_type), _TYPE)(m) * CAT(jit_type, _MIN_FUNC)(input, CAT(jit_type, _VAL_ZERO))))) : "
           "(fn) == 3 ? (CAT(jit_type, _MAX_FUNC)(CAT(CAT(TO_, jit_type), _TYPE)(m), CAT(jit_type, _MIN_FUNC)(n, input))) : input)")
    A("#define ACT_SWITCH(fn, jit_type, input, m, n) " + act)
    A("#define ACTIVATION_TYPED(jit_type, input, m, n) ACT_SWITCH(g->act, jit_type, input, m, n)")
    A("#define NL_M (g->act_m)"); A("#define NL_N (g->act_n)")
    if v["f"]:
        A("#define ACTIVATION_ELTW_TYPED(jit_type, input, m, n) ACT_SWITCH(g->eltw_act, jit_type, input, m, n)")
        A("#define NL_M_ELTW (g->eltw_m)"); A("#define NL_N_ELTW (g->eltw_n)")
        A("#define ELTW_CALIBRATION_TERM %d" % v["ec"]); A("#define IN_OUT_OPT 0")
        A("#define ELTW_STRIDE_X (g->eltw_stride_x)"); A("#define ELTW_STRIDE_Y (g->eltw_stride_y)")
        if v["n"]:
            A("#define NON_CONV_SCALE (g->non_conv_scale)")
    A('#include "%s"' % kernel)
    # driver: the NDRange of convolution_kernel_ref.cpp:110-121, gws = {X, Y, F*B}
    args = ["(const INPUT0_TYPE*)a->input0", "(OUTPUT_TYPE*)a->output", "(const FILTER_TYPE*)a->weights"]
    if v["b"] != "n":
        args.append("(const BIAS_TYPE*)a->bias")
    if v["q"]:
        args.append("a->weights_quantization_factors")
    if v["c"]:
        args.append("a->output_calibration_factors")
    args.append("0u")
    if v["f"]:
        args.append("(const INPUT1_TYPE*)a->input1")
        if v["ec"]:
            args.append("a->eltw_output_calibration_factors")
    A('extern "C" int clref_run(const cldnn_b200_conv_params* p, const cldnn_b200_args* a, long bf_begin, long bf_end, int threads)')
    A("{")
    A("    const long total = (long)p->out.b * p->out.f; if (bf_end > total) bf_end = total;")
    A("    #pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)")
    A("    for (long bf = bf_begin; bf < bf_end; ++bf) {")
    A("        g = p;")
    A("        for (int y = 0; y < p->out.y; ++y) for (int x = 0; x < p->out.x; ++x) {")
    A("            cl_gid[0] = x; cl_gid[1] = y; cl_gid[2] = bf;")
    A("            kernel_name(%s);" % ", ".join(args))
    A("        }")
    A("    }")
    A("    return 0;")
    A("}")
    return "\n".join(d) + "\n"


def build(ref, name):
    v = parse(name)
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(OUT, "clref_%s.cpp" % name)
    so = os.path.join(OUT, "clref_%s.so" % name)
    open(src, "w").write(source(ref, v))
    cmd = ["/usr/bin/g++", "-O2", "-std=c++14", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-w",
           "-I", os.path.join(ref, "kernel_selector", "core", "cl_kernels"), "-o", so, src]
    subprocess.check_call(cmd)
    os.remove(src)
    return so


if __name__ == "__main__":
    print(build(sys.argv[1], sys.argv[2]))
