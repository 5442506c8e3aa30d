/*
 * cldnn_oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C, CPU restatement of the arithmetic of clDNN's reference OpenCL
 * kernels for the convolution hot path.  It is the checker used by tests/,
 * by the smoke entry and by the bench's CPU-baseline leg; nothing in the
 * shipped library includes, links or calls it.
 *
 * Parity status: PINNED.  Checked against the literal known-answer vectors of
 * the reference's own tests (ConvQuantizedTest_*: tests/test_cases/
 * convolution_gpu_test.cpp:3971-4197; FusedConvTest_*: tests/test_cases/
 * fused_conv_eltwise_gpu_test.cpp:117-499; pooling, fully_connected and
 * softmax literals) and, when the reference tree is available, against the
 * reference's own .cl sources compiled as C++ (see ref_build/).
 *
 * Floating point is evaluated un-contracted (build with -ffp-contract=off):
 * every multiply and add rounds separately to binary32, as an OpenCL device
 * that does not fuse would.
 *
 * Each function names the reference source it follows
 * (paths relative to the clDNN tree).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <limits.h>
#include "../include/cldnn_b200.h"

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- element access ------------------------------------------------------ */
static float half_to_float(uint16_t h)
{
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1f, m = h & 0x3ff, u;
    if (e == 0) {
        if (m == 0) u = s;
        else { int k = 0; while (!(m & 0x400)) { m <<= 1; ++k; } m &= 0x3ff; u = s | ((uint32_t)(127 - 15 - k + 1) << 23) | (m << 13); }
    } else if (e == 31) u = s | 0x7f800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}

static uint16_t float_to_half(float f)   /* round to nearest even */
{
    uint32_t u; memcpy(&u, &f, 4);
    uint32_t s = (u >> 16) & 0x8000u; int32_t e = (int32_t)((u >> 23) & 0xff) - 127 + 15; uint32_t m = u & 0x7fffffu;
    if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0));
    if (e >= 31) return (uint16_t)(s | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        m |= 0x800000u; int sh = 14 - e; uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return (uint16_t)(s | r);
    }
    uint32_t r = (uint32_t)(e << 10) | (m >> 13), rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return (uint16_t)(s | r);
}

static double load_elem(const void* p, int32_t dtype, int64_t i)
{
    switch (dtype) {
    case CLDNN_B200_I8:  return ((const int8_t*)p)[i];
    case CLDNN_B200_U8:  return ((const uint8_t*)p)[i];
    case CLDNN_B200_I32: return ((const int32_t*)p)[i];
    case CLDNN_B200_F16: return half_to_float(((const uint16_t*)p)[i]);
    case CLDNN_B200_F32: return ((const float*)p)[i];
    }
    return 0.0;
}
static int32_t load_int(const void* p, int32_t dtype, int64_t i)
{
    switch (dtype) {
    case CLDNN_B200_I8:  return ((const int8_t*)p)[i];
    case CLDNN_B200_U8:  return ((const uint8_t*)p)[i];
    case CLDNN_B200_I32: return ((const int32_t*)p)[i];
    }
    return (int32_t)load_elem(p, dtype, i);
}
static int is_int8(int32_t dt) { return dt == CLDNN_B200_I8 || dt == CLDNN_B200_U8; }
static int is_fp(int32_t dt) { return dt == CLDNN_B200_F16 || dt == CLDNN_B200_F32; }

/* OpenCL convert_<t>_sat(float): NaN -> 0, clamp, truncate toward zero. */
static int32_t sat_from_float(float v, int32_t lo, int32_t hi)
{
    if (v != v) return 0;
    if (v <= (float)lo) return lo;
    if (v >= (float)hi) return hi;
    return (int32_t)v;
}
static int32_t sat_from_int(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* TO_OUTPUT_TYPE_SAT (jitter.cpp:477-560). */
static void store_sat_float(void* p, int32_t dtype, int64_t i, float v)
{
    switch (dtype) {
    case CLDNN_B200_I8:  ((int8_t*)p)[i]  = (int8_t)sat_from_float(v, -128, 127); break;
    case CLDNN_B200_U8:  ((uint8_t*)p)[i] = (uint8_t)sat_from_float(v, 0, 255); break;
    case CLDNN_B200_I32: ((int32_t*)p)[i] = v != v ? 0 : (v >= 2147483648.0f ? INT_MAX : (v <= -2147483648.0f ? INT_MIN : (int32_t)v)); break;
    case CLDNN_B200_F16: ((uint16_t*)p)[i] = float_to_half(v); break;
    case CLDNN_B200_F32: ((float*)p)[i] = v; break;
    }
}
static void store_sat_int(void* p, int32_t dtype, int64_t i, int32_t v)
{
    switch (dtype) {
    case CLDNN_B200_I8:  ((int8_t*)p)[i]  = (int8_t)sat_from_int(v, -128, 127); break;
    case CLDNN_B200_U8:  ((uint8_t*)p)[i] = (uint8_t)sat_from_int(v, 0, 255); break;
    case CLDNN_B200_I32: ((int32_t*)p)[i] = v; break;
    case CLDNN_B200_F16: ((uint16_t*)p)[i] = float_to_half((float)v); break;
    case CLDNN_B200_F32: ((float*)p)[i] = (float)v; break;
    }
}

/* ACTIVATION_TYPED(float, ...) -- MakeActivationJitConstants, jitter.cpp:313-445
 * with the float type macros (fmax/fmin, 0.0f/1.0f). */
static float act_float(int32_t fn, float x, float m, float n)
{
    switch (fn) {
    case CLDNN_B200_ACT_RELU: return fmaxf(0.0f, x);
    case CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE:
        if (isinf(m)) return x >= 0.0f ? x : -m;
        return fmaxf(x, 0.0f) + m * fminf(x, 0.0f);
    case CLDNN_B200_ACT_CLAMP: return fmaxf(m, fminf(n, x));
    case CLDNN_B200_ACT_LOGISTIC: return 1.0f / (1.0f + expf(-x));
    case CLDNN_B200_ACT_TANH: return tanhf(x);
    case CLDNN_B200_ACT_ABS: return fabsf(x);
    case CLDNN_B200_ACT_LINEAR: return m * x + n;
    case CLDNN_B200_ACT_SQUARE: return x * x;
    case CLDNN_B200_ACT_SQRT: return sqrtf(x);
    case CLDNN_B200_ACT_ELU: return fmaxf(x, 0.0f) + m * (expf(fminf(x, 0.0f)) - 1.0f);
    }
    return x;
}
/* ACTIVATION_TYPED(int, ...): the same macros instantiated with the int type
 * constants (max/min, (int)0, convert_int(m)). */
static int32_t act_int(int32_t fn, int32_t x, float m, float n)
{
    switch (fn) {
    case CLDNN_B200_ACT_RELU: return x > 0 ? x : 0;
    case CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE: {
        int32_t s = (int32_t)m;
        return (x > 0 ? x : 0) + s * (x < 0 ? x : 0);
    }
    case CLDNN_B200_ACT_CLAMP: { int32_t lo = (int32_t)m; float t = fminf(n, (float)x); int32_t ti = (int32_t)t; return lo > ti ? lo : ti; }
    case CLDNN_B200_ACT_ABS: return x < 0 ? -x : x;
    }
    return x;
}

static int64_t tidx(const cldnn_b200_tensor* t, int64_t b, int64_t f, int64_t y, int64_t x)
{
    return t->offset + x * t->px + y * t->py + f * t->pf + b * t->pb;   /* fetch.cl:19-24 */
}

/*
 * Convolution and fused convolution+eltwise.
 * Follows KERNEL(fused_conv_eltwise_gpu_ref),
 * kernel_selector/core/cl_kernels/fused_conv_eltwise_gpu_ref.cl:65-234, with
 * the type selection of :18-57.  One call computes every output element;
 * `f_begin..f_end` restricts the (batch*feature) range so callers can shard.
 */
static void conv_one(const cldnn_b200_conv_params* p, const cldnn_b200_args* a,
                     int b, int fg, int y, int x)
{
    const int g = fg / p->ofm;                        /* group of this output feature */
    const int in_x0 = x * p->stride_x - p->pad_x;     /* :105-106 */
    const int in_y0 = y * p->stride_y - p->pad_y;
    const int quant_path = p->quantization || p->calibration || p->has_o_qf;          /* :18 */
    const int int_path = !quant_path && p->fused_eltw && is_int8(p->in.dtype);        /* :35 */
    const int64_t w_base = p->w_offset + (int64_t)fg * p->w_po;
    const int64_t dst = tidx(&p->out, b, fg, y, x);

    int32_t acc_i = 0; float acc_f = 0.0f; double acc_d = 0.0; int8_t acc_c = 0; uint8_t acc_uc = 0;
    const int int_acc = quant_path || int_path;
    const int in_int8 = is_int8(p->in.dtype);

    for (int k = 0; k < p->ifm; ++k) {                /* :113-146 */
        const int fin = g * p->ifm + k;
        for (int j = 0; j < p->kh; ++j) {
            const int iy = in_y0 + j * p->dil_y;
            if (iy < 0 || iy >= p->in.y) continue;
            for (int i = 0; i < p->kw; ++i) {
                const int ix = in_x0 + i * p->dil_x;
                if (ix < 0 || ix >= p->in.x) continue;
                const int64_t ii = tidx(&p->in, b, fin, iy, ix);
                const int64_t wi = w_base + k * p->w_pi + j * p->w_py + i * p->w_px;
                if (int_acc) {
                    acc_i += load_int(a->input0, p->in.dtype, ii) * load_int(a->weights, p->w_dtype, wi);
                } else if (in_int8) {
                    /* ACCUMULATOR_TYPE = INPUT0_TYPE (:44-45): 8-bit wrap-around */
                    int32_t prod = (int32_t)(int8_t)load_int(a->input0, p->in.dtype, ii);
                    if (p->in.dtype == CLDNN_B200_U8) {
                        acc_uc = (uint8_t)(acc_uc + (uint8_t)load_int(a->input0, p->in.dtype, ii) * (uint8_t)load_int(a->weights, p->w_dtype, wi));
                    } else {
                        acc_c = (int8_t)(acc_c + (int8_t)prod * (int8_t)load_int(a->weights, p->w_dtype, wi));
                    }
                } else if (p->in.dtype == CLDNN_B200_F32) {
                    acc_f += (float)load_elem(a->input0, p->in.dtype, ii) * (float)load_elem(a->weights, p->w_dtype, wi);
                } else {
                    /* fp16: the reference accumulates in half with device-specific
                     * contraction; parity there is tolerance-based, so use a wide
                     * accumulator as the reference's own test helper does
                     * (tests/test_cases/convolution_gpu_test.cpp:62-97). */
                    acc_d += load_elem(a->input0, p->in.dtype, ii) * load_elem(a->weights, p->w_dtype, wi);
                }
            }
        }
    }

    const int dont_dequantize_bias = p->quantization && p->bias_dtype == CLDNN_B200_F32;   /* convolution_kernel_ref.cpp:89-91 */

    if (int_acc) {
        if (p->bias_dtype != CLDNN_B200_NONE && !dont_dequantize_bias)                     /* :160-162 */
            acc_i += (int32_t)load_elem(a->bias, p->bias_dtype, fg);
    }

    if (quant_path && p->epilogue_order != CLDNN_B200_EPILOGUE_REF) {
        /* The optimised int8 kernels' own orders: convolution_gpu_mmad.cl:106-132 (MMAD) and
         * fused_conv_eltwise_gpu_imad.cl:171-207 (IMAD).  Both need QUANTIZATION_TERM with a float bias. */
        float t = (float)acc_i * a->weights_quantization_factors[fg];                      /* mmad :110-113, imad :180 */
        t = t * p->i_qf;
        t = t + ((const float*)a->bias)[fg];
        t = roundf(t * (p->calibration ? a->output_calibration_factors[fg] : p->o_qf));   /* mmad :111/:113, imad :191-194 */
        /* (UNIT_TYPE) / convert_char / TO_UNIT_TYPE of the rounded value: not saturating; the low 8 bits are kept */
        const int32_t r = (int32_t)t;
        int32_t a8 = p->out.dtype == CLDNN_B200_U8 ? (int32_t)(uint8_t)r : (int32_t)(int8_t)r;
        a8 = act_int(p->act, a8, p->act_m, p->act_n);                                      /* mmad :126, imad :199 */
        if (p->epilogue_order == CLDNN_B200_EPILOGUE_MMAD || !p->fused_eltw) { store_sat_int(a->output, p->out.dtype, dst, a8); return; }
        const void* esrc = p->in_out_opt ? a->output : a->input1;
        const int32_t edt = p->in_out_opt ? p->out.dtype : p->eltw.dtype;
        const int64_t ei = p->in_out_opt ? dst : tidx(&p->eltw, b, fg, (int64_t)y * p->eltw_stride_y, (int64_t)x * p->eltw_stride_x);
        const float s = roundf((float)(a8 + load_int(esrc, edt, ei)) * a->eltw_output_calibration_factors[fg]);   /* imad :201-203 */
        int32_t o = p->out.dtype == CLDNN_B200_U8 ? (s < 0.0f ? 0 : (s > 255.0f ? 255 : (int32_t)s)) : (s < -128.0f ? -128 : (s > 127.0f ? 127 : (int32_t)s));
        o = act_int(p->eltw_act, o, p->eltw_m, p->eltw_n);
        store_sat_int(a->output, p->out.dtype, dst, o);
        return;
    }

    if (quant_path) {
        float deq = (float)acc_i;                                                          /* :165-171 */
        if (p->quantization) { deq = deq * a->weights_quantization_factors[fg]; deq = deq * p->i_qf; }
        if (dont_dequantize_bias) deq += ((const float*)a->bias)[fg];                      /* :173-179 */
        float v = act_float(p->act, deq, p->act_m, p->act_n);                              /* :181-182 */
        if (p->calibration) v = v * a->output_calibration_factors[fg];                     /* :184-190 */
        else v = v * p->o_qf;
        const int round_conv = p->fused_eltw || !is_fp(p->out.dtype);                      /* :27-34 */
        if (round_conv) v = roundf(v);                                                     /* :192 */
        if (!p->fused_eltw) { store_sat_float(a->output, p->out.dtype, dst, v); return; }  /* :198 */

        const void* esrc = p->in_out_opt ? a->output : a->input1;                          /* :201-205 */
        const int32_t edt = p->in_out_opt ? p->out.dtype : p->eltw.dtype;
        const int64_t ei = p->in_out_opt ? dst : tidx(&p->eltw, b, fg, (int64_t)y * p->eltw_stride_y, (int64_t)x * p->eltw_stride_x);
        float e = (float)load_elem(esrc, edt, ei);
        if (p->has_non_conv_scale) e = e * p->non_conv_scale;                              /* :207-214 */
        float s = v + e;                                                                   /* :217 */
        s = act_float(p->eltw_act, s, p->eltw_m, p->eltw_n);                               /* :218-223 */
        if (p->eltw_calibration) s = s * a->eltw_output_calibration_factors[fg];           /* :225-230 */
        if (!is_fp(p->out.dtype)) s = roundf(s);
        store_sat_float(a->output, p->out.dtype, dst, s);                                  /* :232 */
        return;
    }

    if (int_path) {                                                                        /* :35-42 */
        int32_t v = act_int(p->act, acc_i, p->act_m, p->act_n);
        const void* esrc = p->in_out_opt ? a->output : a->input1;
        const int32_t edt = p->in_out_opt ? p->out.dtype : p->eltw.dtype;
        const int64_t ei = p->in_out_opt ? dst : tidx(&p->eltw, b, fg, (int64_t)y * p->eltw_stride_y, (int64_t)x * p->eltw_stride_x);
        int32_t s;
        if (p->has_non_conv_scale) {
            float e = (float)load_elem(esrc, edt, ei) * p->non_conv_scale;                 /* :208 */
            s = (int32_t)((float)v + e);                                                   /* :217, int = int + float */
        } else {
            s = v + load_int(esrc, edt, ei);                                               /* :213 convert_int_sat of an 8-bit value */
        }
        s = act_int(p->eltw_act, s, p->eltw_m, p->eltw_n);
        if (p->eltw_calibration) {
            float t = (float)s * a->eltw_output_calibration_factors[fg];
            if (!is_fp(p->out.dtype)) t = roundf(t);
            if (is_fp(p->out.dtype)) { store_sat_float(a->output, p->out.dtype, dst, t); return; }
            s = (int32_t)t;
        }
        store_sat_int(a->output, p->out.dtype, dst, s);
        return;
    }

    /* plain path: accumulate and activate in the input type (:43-49) */
    if (in_int8) {
        int32_t v = p->in.dtype == CLDNN_B200_U8 ? (int32_t)acc_uc : (int32_t)acc_c;
        if (p->bias_dtype != CLDNN_B200_NONE) {
            int32_t bv = (int32_t)load_elem(a->bias, p->bias_dtype, fg);
            v = p->in.dtype == CLDNN_B200_U8 ? (int32_t)(uint8_t)(v + bv) : (int32_t)(int8_t)(v + bv);
        }
        v = act_int(p->act, v, p->act_m, p->act_n);
        store_sat_int(a->output, p->out.dtype, dst, v);
        return;
    }
    float v;
    if (p->in.dtype == CLDNN_B200_F32) {
        if (p->bias_dtype != CLDNN_B200_NONE) acc_f += (float)load_elem(a->bias, p->bias_dtype, fg);
        v = acc_f;
    } else {
        if (p->bias_dtype != CLDNN_B200_NONE) acc_d += load_elem(a->bias, p->bias_dtype, fg);
        v = (float)acc_d;
    }
    v = act_float(p->act, v, p->act_m, p->act_n);
    if (p->fused_eltw) {
        const void* esrc = p->in_out_opt ? a->output : a->input1;
        const int32_t edt = p->in_out_opt ? p->out.dtype : p->eltw.dtype;
        const int64_t ei = p->in_out_opt ? dst : tidx(&p->eltw, b, fg, (int64_t)y * p->eltw_stride_y, (int64_t)x * p->eltw_stride_x);
        float e = (float)load_elem(esrc, edt, ei);
        if (p->has_non_conv_scale) e = e * p->non_conv_scale;
        float s = v + e;
        s = act_float(p->eltw_act, s, p->eltw_m, p->eltw_n);
        if (p->eltw_calibration) s = s * a->eltw_output_calibration_factors[fg];
        if (!is_fp(p->out.dtype)) s = roundf(s);
        store_sat_float(a->output, p->out.dtype, dst, s);
        return;
    }
    store_sat_float(a->output, p->out.dtype, dst, v);
}

/* bf_begin/bf_end: half-open range over b*F+f (the NDRange z dimension,
 * convolution_kernel_ref.cpp:110-121); threads>1 splits that range. */
int32_t oracle_conv_range(const cldnn_b200_conv_params* p, const cldnn_b200_args* a,
                          int64_t bf_begin, int64_t bf_end, int32_t threads)
{
    const int F = p->ofm * p->groups;
    if (F != p->out.f) return CLDNN_B200_DIMENSION_MISMATCH;
    if (p->epilogue_order != CLDNN_B200_EPILOGUE_REF) {
        /* the MMAD / IMAD orders: quantised, f32 bias, char output; IMAD's fused form needs eltwise calibration factors */
        if ((p->epilogue_order != CLDNN_B200_EPILOGUE_MMAD && p->epilogue_order != CLDNN_B200_EPILOGUE_IMAD) || !p->quantization ||
            p->bias_dtype != CLDNN_B200_F32 || p->out.dtype != CLDNN_B200_I8) return CLDNN_B200_UNSUPPORTED_FORMAT;
        if (p->fused_eltw && (p->epilogue_order == CLDNN_B200_EPILOGUE_MMAD || !p->eltw_calibration || p->has_non_conv_scale)) return CLDNN_B200_UNSUPPORTED_FORMAT;
    }
    if (bf_begin < 0) bf_begin = 0;
    if (bf_end > (int64_t)p->out.b * F) bf_end = (int64_t)p->out.b * F;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
#endif
    for (int64_t bf = bf_begin; bf < bf_end; ++bf) {
        const int b = (int)(bf / F), f = (int)(bf % F);
        for (int y = 0; y < p->out.y; ++y)
            for (int x = 0; x < p->out.x; ++x)
                conv_one(p, a, b, f, y, x);
    }
    (void)threads;
    return CLDNN_B200_SUCCESS;
}

int32_t oracle_conv(const cldnn_b200_conv_params* p, const cldnn_b200_args* a, int32_t threads)
{
    return oracle_conv_range(p, a, 0, (int64_t)p->out.b * p->out.f, threads);
}

/*
 * Pooling.  int8/u8: KERNEL(pooling_gpu_int8_ref), cl_kernels/
 * pooling_gpu_int8_ref.cl:35-131 (i32 accumulate, max starts at CHAR_MIN,
 * average = convert_int(round((float)sum / n)), TO_OUTPUT_TYPE without
 * saturation).  float: KERNEL(pooling_gpu), cl_kernels/pooling_gpu_ref.cl:36-201.
 * The divider follows src/gpu/pooling_gpu.cpp:122-130.
 */
int32_t oracle_pooling(const cldnn_b200_pool_params* p, const void* in, void* out, int32_t threads)
{
    const int int_in = is_int8(p->in.dtype);
    const int64_t BF = (int64_t)p->out.b * p->out.f;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int64_t bf = 0; bf < BF; ++bf) {
        const int b = (int)(bf / p->out.f), f = (int)(bf % p->out.f);
        for (int y = 0; y < p->out.y; ++y)
            for (int x = 0; x < p->out.x; ++x) {
                const int ox = x * p->stride_x - p->pad_x, oy = y * p->stride_y - p->pad_y;
                int32_t ri = p->mode == CLDNN_B200_POOL_MAX ? -128 : 0;
                float rf = p->mode == CLDNN_B200_POOL_MAX ? (p->in.dtype == CLDNN_B200_F16 ? -65504.0f : -3.402823466e38f) : 0.0f;
                uint32_t n = 0;
                if (ox + p->size_x < 0 || ox >= p->in.x || oy + p->size_y < 0 || oy >= p->in.y) continue;  /* CHECK_BOUNDRY early return */
                for (int j = 0; j < p->size_y; ++j) {
                    const int iy = oy + j; if (iy < 0 || iy >= p->in.y) continue;
                    for (int i = 0; i < p->size_x; ++i) {
                        const int ix = ox + i; if (ix < 0 || ix >= p->in.x) continue;
                        const int64_t ii = tidx(&p->in, b, f, iy, ix);
                        if (int_in) { int32_t v = load_int(in, p->in.dtype, ii); ri = p->mode == CLDNN_B200_POOL_MAX ? (v > ri ? v : ri) : ri + v; }
                        else { float v = (float)load_elem(in, p->in.dtype, ii); rf = p->mode == CLDNN_B200_POOL_MAX ? fmaxf(rf, v) : rf + v; }
                        ++n;
                    }
                }
                uint32_t div;
                if (p->div_mode == CLDNN_B200_DIV_DYNAMIC) div = n ? n : 1;
                else if (p->div_mode == CLDNN_B200_DIV_DYNAMIC_WITH_PADDING) {
                    int hend = oy + p->size_y < p->in.y + p->pad_y ? oy + p->size_y : p->in.y + p->pad_y;
                    int wend = ox + p->size_x < p->in.x + p->pad_x ? ox + p->size_x : p->in.x + p->pad_x;
                    div = (uint32_t)((hend - oy) * (wend - ox)); if (!div) div = 1;
                } else div = (uint32_t)(p->size_x * p->size_y);
                const int64_t oi = tidx(&p->out, b, f, y, x);
                if (int_in) {
                    if (p->mode == CLDNN_B200_POOL_AVG) {
                        if (p->div_mode == CLDNN_B200_DIV_FIXED) ri = (int32_t)roundf((float)ri / (int)div);   /* :124 */
                        else ri = (int32_t)roundf((float)ri / (float)div);                                     /* :122 */
                    }
                    /* TO_OUTPUT_TYPE = convert_char / convert_uchar (wraps), then ACTIVATION in the 8-bit type */
                    if (p->out.dtype == CLDNN_B200_U8) { uint8_t v = (uint8_t)ri; ((uint8_t*)out)[oi] = (uint8_t)act_int(p->act, v, p->act_m, p->act_n); }
                    else if (p->out.dtype == CLDNN_B200_I8) { int8_t v = (int8_t)ri; ((int8_t*)out)[oi] = (int8_t)act_int(p->act, v, p->act_m, p->act_n); }
                    else store_sat_int(out, p->out.dtype, oi, act_int(p->act, ri, p->act_m, p->act_n));
                } else {
                    if (p->mode == CLDNN_B200_POOL_AVG) rf = rf / (float)div;
                    store_sat_float(out, p->out.dtype, oi, act_float(p->act, rf, p->act_m, p->act_n));
                }
            }
    }
    (void)threads;
    return CLDNN_B200_SUCCESS;
}

/*
 * fully_connected.  KERNEL(fc), cl_kernels/fully_connected_gpu_bfyx_ref.cl:18-84.
 * Quantised: out = ACT(convert_char(round(((float)acc*q[o]*I_QF + bias[o]) * calib[o]|O_QF))).
 * The reference's (char) casts do not saturate and are undefined for values
 * outside [-128,127]; `out_of_range` counts such outputs (the stored value is
 * then the saturated one) so tests can require the count to be zero.
 */
int32_t oracle_fc(const cldnn_b200_fc_params* p, const cldnn_b200_args* a, int32_t threads, int64_t* out_of_range)
{
    int64_t oor = 0;
    const int64_t BO = (int64_t)p->out.b * p->out.f;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1) reduction(+:oor)
#endif
    for (int64_t bo = 0; bo < BO; ++bo) {
        const int b = (int)(bo / p->out.f), o = (int)(bo % p->out.f);
        int32_t acc_i = 0; double acc_d = 0.0; float acc_f = 0.0f;
        for (int f = 0; f < p->in.f; ++f)
            for (int y = 0; y < p->in.y; ++y)
                for (int x = 0; x < p->in.x; ++x) {
                    const int64_t ii = tidx(&p->in, b, f, y, x);
                    const int64_t wi = p->w_offset + o * p->w_po + f * p->w_pi + y * p->w_py + x * p->w_px;
                    if (p->quantization) acc_i += load_int(a->input0, p->in.dtype, ii) * load_int(a->weights, p->w_dtype, wi);
                    else if (p->in.dtype == CLDNN_B200_F32) acc_f += (float)load_elem(a->input0, p->in.dtype, ii) * (float)load_elem(a->weights, p->w_dtype, wi);
                    else acc_d += load_elem(a->input0, p->in.dtype, ii) * load_elem(a->weights, p->w_dtype, wi);
                }
        const int64_t oi = tidx(&p->out, b, o, 0, 0);
        if (p->quantization) {
            int32_t r = acc_i;
            if (p->bias_dtype != CLDNN_B200_NONE) {
                float t = (float)acc_i * a->weights_quantization_factors[o];
                t = t * p->i_qf;
                t = t + (float)load_elem(a->bias, p->bias_dtype, o);
                t = t * (p->calibration ? a->output_calibration_factors[o] : p->o_qf);
                t = roundf(t);
                if (t < -128.0f || t > 127.0f) ++oor;
                r = sat_from_float(t, -128, 127);
            } else {
                if (r < -128 || r > 127) ++oor;
                r = sat_from_int(r, -128, 127);
            }
            int8_t c = (int8_t)r;
            c = (int8_t)act_int(p->act, c, p->act_m, p->act_n);
            store_sat_int(a->output, p->out.dtype, oi, c);
        } else {
            float v = p->in.dtype == CLDNN_B200_F32 ? acc_f : (float)acc_d;
            if (p->bias_dtype != CLDNN_B200_NONE) v += (float)load_elem(a->bias, p->bias_dtype, o);
            store_sat_float(a->output, p->out.dtype, oi, act_float(p->act, v, p->act_m, p->act_n));
        }
    }
    if (out_of_range) *out_of_range = oor;
    (void)threads;
    return CLDNN_B200_SUCCESS;
}

/*
 * softmax.  KERNEL(softmax), cl_kernels/softmax_gpu_ref.cl:22-58: per set of
 * values -- max-subtract, exp, float denominator, divide.  The sets follow
 * `dimension` (actual_kernels/softmax/softmax_items_class_kernel_base.cpp:45-99: the
 * class axis is x, y or f, the other two axes and the batch enumerate the sets;
 * src/gpu/softmax_gpu.cpp:42-63: normalize_fyx flattens f, y, x into one class axis).  native_exp is implementation-defined on the
 * device, so parity is tolerance-based.
 */
static void softmax_coords(const cldnn_b200_softmax_params* p, int64_t set, int64_t i, int* b, int* f, int* y, int* x)
{
    const int F = p->in.f, Y = p->in.y, X = p->in.x;
    switch (p->dimension) {
    case CLDNN_B200_SOFTMAX_X:   *x = (int)i; *y = (int)(set % Y); *f = (int)((set / Y) % F); *b = (int)(set / ((int64_t)Y * F)); break;
    case CLDNN_B200_SOFTMAX_Y:   *y = (int)i; *x = (int)(set % X); *f = (int)((set / X) % F); *b = (int)(set / ((int64_t)X * F)); break;
    case CLDNN_B200_SOFTMAX_FYX: *x = (int)(i % X); *y = (int)((i / X) % Y); *f = (int)(i / ((int64_t)X * Y)); *b = (int)set; break;
    default:                     *f = (int)i; *x = (int)(set % X); *y = (int)((set / X) % Y); *b = (int)(set / ((int64_t)X * Y)); break;
    }
}

int32_t oracle_softmax(const cldnn_b200_softmax_params* p, const void* in, void* out)
{
    const int64_t all = (int64_t)p->in.b * p->in.f * p->in.y * p->in.x;
    int64_t len;
    switch (p->dimension) {
    case CLDNN_B200_SOFTMAX_F:   len = p->in.f; break;
    case CLDNN_B200_SOFTMAX_X:   len = p->in.x; break;
    case CLDNN_B200_SOFTMAX_Y:   len = p->in.y; break;
    case CLDNN_B200_SOFTMAX_FYX: len = (int64_t)p->in.f * p->in.y * p->in.x; break;
    default: return CLDNN_B200_INVALID_ARG;
    }
    if (len <= 0) return CLDNN_B200_SUCCESS;
    for (int64_t set = 0; set < all / len; ++set) {
        int b, f, y, x;
        float mx = -3.402823466e38f;
        for (int64_t i = 0; i < len; ++i) { softmax_coords(p, set, i, &b, &f, &y, &x); mx = fmaxf(mx, (float)load_elem(in, p->in.dtype, tidx(&p->in, b, f, y, x))); }
        float den = 0.0f;
        for (int64_t i = 0; i < len; ++i) { softmax_coords(p, set, i, &b, &f, &y, &x); den += expf((float)load_elem(in, p->in.dtype, tidx(&p->in, b, f, y, x)) - mx); }
        for (int64_t i = 0; i < len; ++i) {
            softmax_coords(p, set, i, &b, &f, &y, &x);
            float e = expf((float)load_elem(in, p->in.dtype, tidx(&p->in, b, f, y, x)) - mx);
            store_sat_float(out, p->out.dtype, tidx(&p->out, b, f, y, x), e / den);
        }
    }
    return CLDNN_B200_SUCCESS;
}

/*
 * eltwise.  KERNEL(eltwise), cl_kernels/generic_eltwise_ref.cl:198-330 with the
 * operation strings of actual_kernels/eltwise/eltwise_kernel_base.cpp:280-340.
 * Quantised (:311-326): int op on the 8-bit inputs, (int)round((float)res *
 * calibrations[f] | O_QF), convert_char_sat, then the activation on the 8-bit
 * value.  Otherwise the op and the activation run in the unit type.
 */
int32_t oracle_eltwise(const cldnn_b200_eltwise_params* p, const void* in0, const void* in1, const float* calib, void* out)
{
    for (int b = 0; b < p->out.b; ++b)
        for (int f = 0; f < p->out.f; ++f)
            for (int y = 0; y < p->out.y; ++y)
                for (int x = 0; x < p->out.x; ++x) {
                    const int64_t i0 = tidx(&p->in0, b % p->in0.b, f % p->in0.f, ((int64_t)y * p->stride_y0) % p->in0.y, ((int64_t)x * p->stride_x0) % p->in0.x);
                    const int64_t i1 = tidx(&p->in1, b % p->in1.b, f % p->in1.f, ((int64_t)y * p->stride_y1) % p->in1.y, ((int64_t)x * p->stride_x1) % p->in1.x);
                    const int64_t oi = tidx(&p->out, b, f, y, x);
                    if (p->quantization) {
                        int32_t a = load_int(in0, p->in0.dtype, i0), c = load_int(in1, p->in1.dtype, i1), r;
                        switch (p->mode) {
                        case CLDNN_B200_ELTW_SUB: r = a - c; break;
                        case CLDNN_B200_ELTW_MAX: r = a > c ? a : c; break;
                        case CLDNN_B200_ELTW_MIN: r = a < c ? a : c; break;
                        case CLDNN_B200_ELTW_PROD: r = a * c; break;
                        default: r = a + c; break;
                        }
                        r = (int32_t)roundf((float)r * (p->calibration ? calib[f] : p->o_qf));
                        int8_t q = (int8_t)sat_from_int(r, -128, 127);
                        store_sat_int(out, p->out.dtype, oi, act_int(p->act, q, p->act_m, p->act_n));
                        continue;
                    }
                    float a = (float)load_elem(in0, p->in0.dtype, i0), c = (float)load_elem(in1, p->in1.dtype, i1), r;
                    switch (p->mode) {
                    case CLDNN_B200_ELTW_SUB: r = a - c; break;
                    case CLDNN_B200_ELTW_MAX: r = fmaxf(a, c); break;
                    case CLDNN_B200_ELTW_MIN: r = fminf(a, c); break;
                    case CLDNN_B200_ELTW_PROD: r = a * c; break;
                    default: r = a + c; break;
                    }
                    if (is_fp(p->out.dtype)) store_sat_float(out, p->out.dtype, oi, act_float(p->act, r, p->act_m, p->act_n));
                    else store_sat_int(out, p->out.dtype, oi, act_int(p->act, (int32_t)r, p->act_m, p->act_n));
                }
    return CLDNN_B200_SUCCESS;
}

/*
 * reorder.  KERNEL(reorder_data), cl_kernels/reorder_data.cl:72-128: read in the
 * source layout, optionally subtract a per-feature mean, convert with
 * saturation for integer destinations, write in the destination layout.
 */
int32_t oracle_reorder(const cldnn_b200_reorder_params* p, const void* in, void* out)
{
    for (int b = 0; b < p->out.b; ++b)
        for (int f = 0; f < p->out.f; ++f)
            for (int y = 0; y < p->out.y; ++y)
                for (int x = 0; x < p->out.x; ++x) {
                    const int64_t oi = tidx(&p->out, b, f, y, x);
                    if (f >= p->in.f) { store_sat_int(out, p->out.dtype, oi, 0); continue; }   /* feature padding of the destination */
                    const int64_t ii = tidx(&p->in, b, f, y, x);
                    if (!is_fp(p->in.dtype) && !p->has_mean) { store_sat_int(out, p->out.dtype, oi, load_int(in, p->in.dtype, ii)); continue; }
                    float v = (float)load_elem(in, p->in.dtype, ii);
                    if (p->has_mean) v -= p->mean[f < 4 ? f : 3];
                    store_sat_float(out, p->out.dtype, oi, v);
                }
    return CLDNN_B200_SUCCESS;
}

/*
 * lrn across channels.  KERNEL(lrn_gpu_across_channel_ref),
 * cl_kernels/lrn_gpu_across_channel_ref.cl:26-66:
 * out = in * (k + alpha/size * sum_{window} in^2)^(-beta); native_powr on the
 * device, so parity is tolerance-based.
 */
int32_t oracle_lrn(const cldnn_b200_lrn_params* p, const void* in, void* out)
{
    const int pad = (p->size - 1) / 2;
    for (int b = 0; b < p->in.b; ++b)
        for (int f = 0; f < p->in.f; ++f)
            for (int y = 0; y < p->in.y; ++y)
                for (int x = 0; x < p->in.x; ++x) {
                    float acc = 0.0f;
                    for (int i = 0; i < p->size; ++i) {
                        int ff = f - pad + i; if (ff < 0 || ff >= p->in.f) continue;
                        float v = (float)load_elem(in, p->in.dtype, tidx(&p->in, b, ff, y, x));
                        acc = acc + v * v;
                    }
                    acc = acc * (p->alpha / (float)p->size) + p->k;
                    float v = (float)load_elem(in, p->in.dtype, tidx(&p->in, b, f, y, x));
                    store_sat_float(out, p->out.dtype, tidx(&p->out, b, f, y, x), v * powf(acc, -p->beta));
                }
    return CLDNN_B200_SUCCESS;
}

/* standalone activation, cl_kernels/activation_ref.cl */
int32_t oracle_activation(const cldnn_b200_activation_params* p, const void* in, void* out)
{
    for (int b = 0; b < p->in.b; ++b)
        for (int f = 0; f < p->in.f; ++f)
            for (int y = 0; y < p->in.y; ++y)
                for (int x = 0; x < p->in.x; ++x) {
                    const int64_t ii = tidx(&p->in, b, f, y, x), oi = tidx(&p->out, b, f, y, x);
                    if (is_fp(p->in.dtype)) store_sat_float(out, p->out.dtype, oi, act_float(p->act, (float)load_elem(in, p->in.dtype, ii), p->act_m, p->act_n));
                    else store_sat_int(out, p->out.dtype, oi, act_int(p->act, load_int(in, p->in.dtype, ii), p->act_m, p->act_n));
                }
    return CLDNN_B200_SUCCESS;
}

/* Output range of a sliding window: calc_sliding_window_output_range<all>
 * (convolution; src/include/sliding_window_utils.h:87-124) and
 * <exceed_once_data> (pooling; :126-230, src/pooling.cpp:91-92).
 * `offset` is the (non-positive for padding) input_offset. */
int32_t oracle_conv_out_size(int32_t in, int32_t k, int32_t offset, int32_t stride, int32_t dil)
{
    int32_t wes = (k - 1) * dil + 1;
    if (2 * offset + wes > in) return 0;
    return (in - 2 * offset - wes) / stride + 1;
}
int32_t oracle_pool_out_size(int32_t in, int32_t k, int32_t offset, int32_t stride)
{
    int32_t ext = k > stride ? k : stride;
    int32_t a = (2 * offset + ext <= in + stride - 1) ? (in - 2 * offset - ext + stride - 1) / stride + 1 : 1;
    int32_t b = (offset <= in - 1) ? (in - offset - 1) / stride + 1 : 1;
    return a < b ? a : b;
}

int32_t oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
