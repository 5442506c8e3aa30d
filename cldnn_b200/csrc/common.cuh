// Shared host/device helpers of the sm_100a engine: error plumbing, tensor
// indexing and the bit-exact convolution epilogue.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <string>
#include "../../include/cldnn_b200.h"

namespace b200 {

// ---- host error plumbing -----------------------------------------------------
void set_error(const std::string& msg);
int32_t fail(int32_t code, const std::string& msg);
int32_t cuda_fail(cudaError_t e, const char* what);
#define B200_CUDA(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) return ::b200::cuda_fail(_e, #expr); } while (0)

// ---- device helpers ------------------------------------------------------------
__host__ __device__ inline bool is_int8(int32_t dt) { return dt == CLDNN_B200_I8 || dt == CLDNN_B200_U8; }
__host__ __device__ inline bool is_fp(int32_t dt) { return dt == CLDNN_B200_F16 || dt == CLDNN_B200_F32; }
__host__ __device__ inline int dtype_bytes(int32_t dt) { return dt & 0x0f; }

__device__ __forceinline__ int64_t tidx(const cldnn_b200_tensor& t, int64_t b, int64_t f, int64_t y, int64_t x)
{
    return t.offset + x * t.px + y * t.py + f * t.pf + b * t.pb;
}

__device__ __forceinline__ float load_as_float(const void* p, int32_t dt, int64_t i)
{
    switch (dt) {
    case CLDNN_B200_I8:  return (float)((const int8_t*)p)[i];
    case CLDNN_B200_U8:  return (float)((const uint8_t*)p)[i];
    case CLDNN_B200_I32: return (float)((const int32_t*)p)[i];
    case CLDNN_B200_F16: return __half2float(((const __half*)p)[i]);
    default:             return ((const float*)p)[i];
    }
}
__device__ __forceinline__ int32_t load_as_int(const void* p, int32_t dt, int64_t i)
{
    switch (dt) {
    case CLDNN_B200_I8:  return ((const int8_t*)p)[i];
    case CLDNN_B200_U8:  return ((const uint8_t*)p)[i];
    case CLDNN_B200_I32: return ((const int32_t*)p)[i];
    default:             return (int32_t)load_as_float(p, dt, i);
    }
}

// OpenCL round(): to nearest, ties away from zero.  trunc + exact remainder test
// (x - trunc(x) is exact in binary32), so no double rounding.
__device__ __forceinline__ float round_half_away(float x)
{
    float r = truncf(x);
    float d = x - r;
    if (fabsf(d) >= 0.5f) r += copysignf(1.0f, x);
    return r;
}

// OpenCL convert_<t>_sat(float): NaN -> 0, clamp, truncate toward zero.
__device__ __forceinline__ int32_t sat_i32_from_float(float v, int32_t lo, int32_t hi)
{
    int32_t i = __float2int_rz(v);         // saturating, NaN -> 0
    return min(hi, max(lo, i));
}

__device__ __forceinline__ void store_sat_float(void* p, int32_t dt, int64_t i, float v)
{
    switch (dt) {
    case CLDNN_B200_I8:  ((int8_t*)p)[i]  = (int8_t)sat_i32_from_float(v, -128, 127); break;
    case CLDNN_B200_U8:  ((uint8_t*)p)[i] = (uint8_t)sat_i32_from_float(v, 0, 255); break;
    case CLDNN_B200_I32: ((int32_t*)p)[i] = __float2int_rz(v); break;
    case CLDNN_B200_F16: ((__half*)p)[i]  = __float2half_rn(v); break;
    default:             ((float*)p)[i]   = v; break;
    }
}
__device__ __forceinline__ void store_sat_int(void* p, int32_t dt, int64_t i, int32_t v)
{
    switch (dt) {
    case CLDNN_B200_I8:  ((int8_t*)p)[i]  = (int8_t)min(127, max(-128, v)); break;
    case CLDNN_B200_U8:  ((uint8_t*)p)[i] = (uint8_t)min(255, max(0, v)); break;
    case CLDNN_B200_I32: ((int32_t*)p)[i] = v; break;
    case CLDNN_B200_F16: ((__half*)p)[i]  = __float2half_rn((float)v); break;
    default:             ((float*)p)[i]   = (float)v; break;
    }
}

// ACTIVATION_TYPED(float, ..): kernel_selector/core/common/jitter.cpp:366-397.
// Every product and sum rounds separately (no fused multiply-add).
__device__ __forceinline__ float act_float(int32_t fn, float x, float m, float n)
{
    switch (fn) {
    case CLDNN_B200_ACT_NONE: return x;
    case CLDNN_B200_ACT_RELU: return fmaxf(0.0f, x);
    case CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE:
        if (isinf(m)) return x >= 0.0f ? x : -m;
        return __fadd_rn(fmaxf(x, 0.0f), __fmul_rn(m, fminf(x, 0.0f)));
    case CLDNN_B200_ACT_CLAMP: return fmaxf(m, fminf(n, x));
    case CLDNN_B200_ACT_LOGISTIC: return 1.0f / (1.0f + expf(-x));
    case CLDNN_B200_ACT_TANH: return tanhf(x);
    case CLDNN_B200_ACT_ABS: return fabsf(x);
    case CLDNN_B200_ACT_LINEAR: return __fadd_rn(__fmul_rn(m, x), n);
    case CLDNN_B200_ACT_SQUARE: return __fmul_rn(x, x);
    case CLDNN_B200_ACT_SQRT: return sqrtf(x);
    case CLDNN_B200_ACT_ELU: return __fadd_rn(fmaxf(x, 0.0f), __fmul_rn(m, expf(fminf(x, 0.0f)) - 1.0f));
    }
    return x;
}
__device__ __forceinline__ int32_t act_int(int32_t fn, int32_t x, float m, float n)
{
    switch (fn) {
    case CLDNN_B200_ACT_RELU: return max(x, 0);
    case CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE: return max(x, 0) + (int32_t)m * min(x, 0);
    case CLDNN_B200_ACT_CLAMP: return max((int32_t)m, (int32_t)fminf(n, (float)x));
    case CLDNN_B200_ACT_ABS: return abs(x);
    }
    return x;
}

// The launch constants the epilogue needs, copied out of cldnn_b200_conv_params.
struct EpiCfg {
    int32_t quant_path;          // QUANTIZATION_TERM || CALIBRATION_TERM || defined(O_QF)
    int32_t int_path;            // fused eltwise on 8-bit data without quantisation
    int32_t quantization, calibration;
    int32_t bias_dtype, dont_dequantize_bias;
    int32_t act, fused_eltw, has_non_conv_scale, eltw_act, eltw_calibration;
    int32_t out_dtype, out_is_fp, eltw_dtype;
    int32_t order;               // CLDNN_B200_EPILOGUE_*
    float i_qf, o_qf, act_m, act_n, non_conv_scale, eltw_m, eltw_n;
};

inline EpiCfg make_epi_cfg(const cldnn_b200_conv_params& p)
{
    EpiCfg e{};
    e.quant_path = (p.quantization || p.calibration || p.has_o_qf) ? 1 : 0;
    e.int_path = (!e.quant_path && p.fused_eltw && is_int8(p.in.dtype)) ? 1 : 0;
    e.quantization = p.quantization; e.calibration = p.calibration;
    e.bias_dtype = p.bias_dtype;
    e.dont_dequantize_bias = (p.quantization && p.bias_dtype == CLDNN_B200_F32) ? 1 : 0;
    e.act = p.act; e.fused_eltw = p.fused_eltw; e.has_non_conv_scale = p.has_non_conv_scale;
    e.eltw_act = p.eltw_act; e.eltw_calibration = p.eltw_calibration;
    e.out_dtype = p.out.dtype; e.out_is_fp = is_fp(p.out.dtype) ? 1 : 0;
    e.eltw_dtype = p.in_out_opt ? p.out.dtype : p.eltw.dtype;
    e.order = p.epilogue_order;
    e.i_qf = p.i_qf; e.o_qf = p.o_qf; e.act_m = p.act_m; e.act_n = p.act_n;
    e.non_conv_scale = p.non_conv_scale; e.eltw_m = p.eltw_m; e.eltw_n = p.eltw_n;
    return e;
}

// The MMAD / IMAD epilogue orders exist for quantised signed 8-bit outputs with a float bias; IMAD's fused form needs eltwise
// calibration factors, MMAD has no fused form; neither knows a non-convolution scale.
inline bool epilogue_order_ok(const cldnn_b200_conv_params& p)
{
    if (p.epilogue_order == CLDNN_B200_EPILOGUE_REF) return true;
    if (p.epilogue_order != CLDNN_B200_EPILOGUE_MMAD && p.epilogue_order != CLDNN_B200_EPILOGUE_IMAD) return false;
    if (!p.quantization || p.bias_dtype != CLDNN_B200_F32 || p.out.dtype != CLDNN_B200_I8) return false;      // the kernels' unit type is char
    if (p.fused_eltw && (p.epilogue_order == CLDNN_B200_EPILOGUE_MMAD || !p.eltw_calibration || p.has_non_conv_scale)) return false;
    if (p.fused_eltw && !is_int8(p.in_out_opt ? p.out.dtype : p.eltw.dtype)) return false;
    return true;
}

// A clamp that the unsigned saturating store performs anyway is dropped: with an 8-bit unsigned output, a uniform O_QF > 0,
// a lower bound <= 0 and an upper bound n with n * O_QF >= 255, clamp(v) * O_QF, rounded and saturated, equals v * O_QF
// rounded and saturated for every v (values above n land on 255 either way, values below 0 on 0).  ReLU6 in front of a
// requantisation by 255 / 6 is the common case.  Not applicable in front of a fused residual sum.
inline cldnn_b200_conv_params simplified_conv_params(const cldnn_b200_conv_params& p0)
{
    cldnn_b200_conv_params p = p0;
    if (p.epilogue_order == CLDNN_B200_EPILOGUE_REF && p.act == CLDNN_B200_ACT_CLAMP && !p.fused_eltw && p.out.dtype == CLDNN_B200_U8 && !p.calibration && p.has_o_qf && p.o_qf > 0.0f &&
        p.act_m <= 0.0f && p.act_n * p.o_qf >= 255.0f) {
        p.act = CLDNN_B200_ACT_NONE; p.act_m = 0.0f; p.act_n = 0.0f;
    }
    return p;
}

// Quantised epilogue in the reference's order
// (cl_kernels/fused_conv_eltwise_gpu_ref.cl:148-232): i32 bias -> dequantise
// ((float)acc * q[f]) * I_QF -> (+ f32 bias) -> activation -> * calib[f] | O_QF ->
// round -> [+ scaled residual -> activation -> * eltw_calib[f] -> round].
// `acc` already holds the i32 bias when the bias is integer.  Returns the float
// value to hand to the saturating store.
// The MMAD / IMAD orders (convolution_gpu_mmad.cl:106-132, fused_conv_eltwise_gpu_imad.cl:171-207): everything up to the
// first rounding in float, then the value lives in the 8-bit output type (low 8 bits of the rounded integer), where the
// activation is applied; IMAD adds the residual as integers and requantises the sum.
static __device__ __noinline__ float epi_quant_alt(const EpiCfg& c, int32_t acc, float q, float bias_f, float calib, float eltw_elem, float eltw_calib)
{
    float v = __int2float_rn(acc);
    v = __fmul_rn(__fmul_rn(v, q), c.i_qf);
    v = __fadd_rn(v, bias_f);
    v = round_half_away(__fmul_rn(v, c.calibration ? calib : c.o_qf));
    const int32_t r = __float2int_rz(v);
    int32_t a8 = c.out_dtype == CLDNN_B200_U8 ? (int32_t)(uint8_t)r : (int32_t)(int8_t)r;
    a8 = act_int(c.act, a8, c.act_m, c.act_n);
    if (c.order == CLDNN_B200_EPILOGUE_MMAD || !c.fused_eltw) return (float)a8;
    const float s = round_half_away(__fmul_rn((float)(a8 + (int32_t)eltw_elem), eltw_calib));
    const int32_t lo = c.out_dtype == CLDNN_B200_U8 ? 0 : -128, hi = c.out_dtype == CLDNN_B200_U8 ? 255 : 127;
    return (float)act_int(c.eltw_act, sat_i32_from_float(s, lo, hi), c.eltw_m, c.eltw_n);
}

__device__ __forceinline__ float epi_quant(const EpiCfg& c, int32_t acc, float q, float bias_f, float calib,
                                           float eltw_elem, float eltw_calib)
{
    if (c.order != CLDNN_B200_EPILOGUE_REF) return epi_quant_alt(c, acc, q, bias_f, calib, eltw_elem, eltw_calib);
    float v = __int2float_rn(acc);
    if (c.quantization) { v = __fmul_rn(v, q); v = __fmul_rn(v, c.i_qf); }
    if (c.dont_dequantize_bias) v = __fadd_rn(v, bias_f);
    v = act_float(c.act, v, c.act_m, c.act_n);
    v = __fmul_rn(v, c.calibration ? calib : c.o_qf);
    if (c.fused_eltw || !c.out_is_fp) v = round_half_away(v);
    if (!c.fused_eltw) return v;
    float e = eltw_elem;
    if (c.has_non_conv_scale) e = __fmul_rn(e, c.non_conv_scale);
    float s = __fadd_rn(v, e);
    s = act_float(c.eltw_act, s, c.eltw_m, c.eltw_n);
    if (c.eltw_calibration) s = __fmul_rn(s, eltw_calib);
    if (!c.out_is_fp) s = round_half_away(s);
    return s;
}

}  // namespace b200
