// conv_ref: the any-layout, any-type convolution / fused conv+eltwise kernel.
// One thread per output element, reference operation order
// (cl_kernels/fused_conv_eltwise_gpu_ref.cl:65-234).  It is the implementation
// the selector falls back to when no tensor-core kernel accepts the parameters
// (what ConvolutionKernel_Ref is to the reference's selector,
// actual_kernels/convolution/convolution_kernel_ref.cpp:22-63).
#include "engine.hpp"

namespace b200 {

struct ConvRefArgs {
    const void* in; const void* eltw; void* out; const void* w; const void* bias;
    const float* quant; const float* calib; const float* eltw_calib;
};

__global__ void __launch_bounds__(256)
conv_ref_kernel(const __grid_constant__ cldnn_b200_conv_params p, const __grid_constant__ EpiCfg c, ConvRefArgs a)
{
    const int64_t total = (int64_t)p.out.b * p.out.f * p.out.y * p.out.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        // x fastest, then y, then f, then b: neighbouring threads read neighbouring inputs
        int x = (int)(idx % p.out.x); int64_t t = idx / p.out.x;
        int y = (int)(t % p.out.y); t /= p.out.y;
        int f = (int)(t % p.out.f); int b = (int)(t / p.out.f);
        const int g = f / p.ofm;
        const int ix0 = x * p.stride_x - p.pad_x, iy0 = y * p.stride_y - p.pad_y;
        const int64_t wb = p.w_offset + (int64_t)f * p.w_po;
        const bool int_acc = c.quant_path || c.int_path;
        const bool in8 = is_int8(p.in.dtype);
        int32_t acc_i = 0; float acc_f = 0.f; int32_t acc8 = 0;
        for (int k = 0; k < p.ifm; ++k) {
            const int fin = g * p.ifm + k;
            for (int j = 0; j < p.kh; ++j) {
                const int iy = iy0 + j * p.dil_y; if (iy < 0 || iy >= p.in.y) continue;
                for (int i = 0; i < p.kw; ++i) {
                    const int ix = ix0 + i * p.dil_x; if (ix < 0 || ix >= p.in.x) continue;
                    const int64_t ii = tidx(p.in, b, fin, iy, ix);
                    const int64_t wi = wb + k * p.w_pi + j * p.w_py + i * p.w_px;
                    if (int_acc) acc_i += load_as_int(a.in, p.in.dtype, ii) * load_as_int(a.w, p.w_dtype, wi);
                    else if (in8) {
                        int32_t s = acc8 + load_as_int(a.in, p.in.dtype, ii) * load_as_int(a.w, p.w_dtype, wi);
                        acc8 = p.in.dtype == CLDNN_B200_U8 ? (int32_t)(uint8_t)s : (int32_t)(int8_t)s;   // 8-bit accumulator wraps
                    } else acc_f = __fadd_rn(acc_f, __fmul_rn(load_as_float(a.in, p.in.dtype, ii), load_as_float(a.w, p.w_dtype, wi)));
                }
            }
        }
        const int64_t dst = tidx(p.out, b, f, y, x);
        const void* esrc = p.in_out_opt ? (const void*)a.out : a.eltw;
        const int64_t ei = !p.fused_eltw ? 0 : (p.in_out_opt ? dst : tidx(p.eltw, b, f, (int64_t)y * p.eltw_stride_y, (int64_t)x * p.eltw_stride_x));
        if (c.quant_path) {
            if (p.bias_dtype != CLDNN_B200_NONE && !c.dont_dequantize_bias) acc_i += load_as_int(a.bias, p.bias_dtype, f);
            float v = epi_quant(c, acc_i, p.quantization ? a.quant[f] : 1.f,
                                c.dont_dequantize_bias ? ((const float*)a.bias)[f] : 0.f,
                                p.calibration ? a.calib[f] : 1.f,
                                p.fused_eltw ? load_as_float(esrc, c.eltw_dtype, ei) : 0.f,
                                p.eltw_calibration ? a.eltw_calib[f] : 1.f);
            store_sat_float(a.out, p.out.dtype, dst, v);
        } else if (c.int_path) {
            if (p.bias_dtype != CLDNN_B200_NONE) acc_i += load_as_int(a.bias, p.bias_dtype, f);
            int32_t v = act_int(p.act, acc_i, p.act_m, p.act_n);
            int32_t s;
            if (p.has_non_conv_scale) s = (int32_t)__fadd_rn((float)v, __fmul_rn(load_as_float(esrc, c.eltw_dtype, ei), p.non_conv_scale));
            else s = v + load_as_int(esrc, c.eltw_dtype, ei);
            s = act_int(p.eltw_act, s, p.eltw_m, p.eltw_n);
            if (p.eltw_calibration) {
                float tq = __fmul_rn((float)s, a.eltw_calib[f]);
                if (c.out_is_fp) { store_sat_float(a.out, p.out.dtype, dst, tq); continue; }
                s = (int32_t)round_half_away(tq);
            }
            store_sat_int(a.out, p.out.dtype, dst, s);
        } else if (in8) {
            int32_t v = acc8;
            if (p.bias_dtype != CLDNN_B200_NONE) {
                int32_t s = v + load_as_int(a.bias, p.bias_dtype, f);
                v = p.in.dtype == CLDNN_B200_U8 ? (int32_t)(uint8_t)s : (int32_t)(int8_t)s;
            }
            store_sat_int(a.out, p.out.dtype, dst, act_int(p.act, v, p.act_m, p.act_n));
        } else {
            float v = acc_f;
            if (p.bias_dtype != CLDNN_B200_NONE) v = __fadd_rn(v, load_as_float(a.bias, p.bias_dtype, f));
            v = act_float(p.act, v, p.act_m, p.act_n);
            if (p.fused_eltw) {
                float e = load_as_float(esrc, c.eltw_dtype, ei);
                if (p.has_non_conv_scale) e = __fmul_rn(e, p.non_conv_scale);
                float s = act_float(p.eltw_act, __fadd_rn(v, e), p.eltw_m, p.eltw_n);
                if (p.eltw_calibration) s = __fmul_rn(s, a.eltw_calib[f]);
                if (!c.out_is_fp) s = round_half_away(s);
                v = s;
            }
            store_sat_float(a.out, p.out.dtype, dst, v);
        }
    }
}

static bool conv_ref_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_conv_params*)vp;
    if (p.groups < 1 || p.ofm < 1 || p.ifm < 1 || p.kh < 1 || p.kw < 1) return false;
    if (p.stride_x < 1 || p.stride_y < 1 || p.dil_x < 1 || p.dil_y < 1) return false;
    if (p.out.f != p.ofm * p.groups) return false;
    if (!epilogue_order_ok(p)) return false;
    return true;
}
static int conv_ref_tune_count(const void*) { return 1; }

static int32_t conv_ref_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* args, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params p = *(const cldnn_b200_conv_params*)vp;
    if (!args->input0 || !args->output || !args->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_ref: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !args->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_ref: bias_dtype set but no bias pointer");
    if (p.quantization && !args->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_ref: quantization set but no factors");
    if (p.calibration && !args->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_ref: calibration set but no factors");
    if (p.fused_eltw && !p.in_out_opt && !args->input1) return fail(CLDNN_B200_INVALID_ARG, "conv_ref: fused eltwise needs a second input");
    if (p.eltw_calibration && !args->eltw_output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_ref: eltwise calibration set but no factors");
    const EpiCfg c = make_epi_cfg(p);
    ConvRefArgs a{args->input0, args->input1, args->output, args->weights, args->bias,
                  args->weights_quantization_factors, args->output_calibration_factors, args->eltw_output_calibration_factors};
    const int64_t total = (int64_t)p.out.b * p.out.f * p.out.y * p.out.x;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const int grid = (int)blocks;
    out->fn = [p, c, a, grid](cudaStream_t s) { conv_ref_kernel<<<grid, 256, 0, s>>>(p, c, a); return cudaGetLastError(); };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

const KernelDef kdef_conv_ref = {"conv_ref", sizeof(cldnn_b200_conv_params), conv_ref_supports, conv_ref_tune_count, nullptr, conv_ref_prepare};

}  // namespace b200
