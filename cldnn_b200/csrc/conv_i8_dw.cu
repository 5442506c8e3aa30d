// conv_i8_dw: 8-bit depthwise convolution (groups == features, one filter per
// feature), the MobileNet building block.  A depthwise filter has no reduction
// over features, so there is nothing for the tensor cores: the kernel is
// bandwidth-bound CUDA-core code over the feature-innermost (byxf) layout --
// each thread owns 4 consecutive features of one output pixel, reads one 32-bit
// word per filter tap (a warp reads 128 contiguous bytes), takes the filter
// taps from a shared-memory copy laid out [tap][feature], accumulates in s32 and
// runs the quantised epilogue of fused_conv_eltwise_gpu_ref.cl:148-194 (integer
// bias, per-feature dequantisation, activation -- ReLU6 is CLAMP(0, 6) --
// calibration / O_QF, round, saturate).  It stands where the reference uses
// cl_kernels/convolution_gpu_byxf_af32_depthwise.cl.
#include "engine.hpp"

namespace b200 {

namespace {

struct DwArgs { const uint8_t* in; const int8_t* w; const void* bias; const float* quant; const float* calib; uint8_t* out; };

template <bool kUnsignedIn>
__global__ void __launch_bounds__(256)
conv_i8_dw_kernel(const __grid_constant__ cldnn_b200_conv_params p, const __grid_constant__ EpiCfg c, DwArgs a)
{
    extern __shared__ int8_t s_w[];                                  // [kh*kw][C]
    const int C = p.out.f, taps = p.kh * p.kw;
    for (int i = threadIdx.x; i < taps * C; i += blockDim.x) {
        const int f = i % C, t = i / C; const int j = t / p.kw, s = t - j * p.kw;
        s_w[i] = a.w[p.w_offset + (int64_t)f * p.w_po + j * p.w_py + s * p.w_px];
    }
    __syncthreads();
    const int c4n = C / 4;
    const int64_t total = (int64_t)p.out.b * p.out.y * p.out.x * c4n;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int c4 = (int)(idx % c4n); int64_t t = idx / c4n;
        const int x = (int)(t % p.out.x); t /= p.out.x;
        const int y = (int)(t % p.out.y); const int b = (int)(t / p.out.y);
        const int f0 = c4 * 4;
        const int ix0 = x * p.stride_x - p.pad_x, iy0 = y * p.stride_y - p.pad_y;
        int32_t acc[4] = {0, 0, 0, 0};
        const uint8_t* src = a.in + p.in.offset + (int64_t)b * p.in.pb + f0;
        for (int j = 0; j < p.kh; ++j) {
            const int iy = iy0 + j * p.dil_y; if (iy < 0 || iy >= p.in.y) continue;
            for (int s = 0; s < p.kw; ++s) {
                const int ix = ix0 + s * p.dil_x; if (ix < 0 || ix >= p.in.x) continue;
                const uint32_t xv = __ldg(reinterpret_cast<const uint32_t*>(src + (int64_t)iy * p.in.py + (int64_t)ix * p.in.px));
                const uint32_t wv = *reinterpret_cast<const uint32_t*>(s_w + (j * p.kw + s) * C + f0);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int32_t xe = kUnsignedIn ? (int32_t)((xv >> (8 * e)) & 0xffu) : (int32_t)(int8_t)(xv >> (8 * e));
                    acc[e] += xe * (int32_t)(int8_t)(wv >> (8 * e));
                }
            }
        }
        uint32_t ow = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int f = f0 + e;
            int32_t v_i = acc[e];
            if (p.bias_dtype != CLDNN_B200_NONE && !c.dont_dequantize_bias) v_i += load_as_int(a.bias, p.bias_dtype, f);
            const float v = epi_quant(c, v_i, p.quantization ? a.quant[f] : 1.f, c.dont_dequantize_bias ? ((const float*)a.bias)[f] : 0.f,
                                      p.calibration ? a.calib[f] : 1.f, 0.f, 1.f);
            const int32_t r = __float2int_rz(v);
            const int32_t sat = p.out.dtype == CLDNN_B200_U8 ? min(255, max(0, r)) : min(127, max(-128, r));
            ow |= ((uint32_t)sat & 0xffu) << (8 * e);
        }
        *reinterpret_cast<uint32_t*>(a.out + p.out.offset + (int64_t)b * p.out.pb + (int64_t)y * p.out.py + (int64_t)x * p.out.px + f0) = ow;
    }
}

bool dw_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (!is_int8(p.in.dtype) || p.w_dtype != CLDNN_B200_I8 || !is_int8(p.out.dtype)) return no("8-bit activations, weights and output only");
    if (p.groups < 2 || p.ofm != 1 || p.ifm != 1 || p.in.f != p.groups || p.out.f != p.groups) return no("depthwise only: one input and one output feature per group");
    if (p.fused_eltw) return no("no fused eltwise");
    if (!(p.quantization || p.calibration || p.has_o_qf)) return no("quantised epilogue only");
    if (p.in.pf != 1 || p.out.pf != 1 || p.in.f % 4) return no("byxf layout, features a multiple of 4");
    const int64_t al[] = {p.in.px, p.in.py, p.in.pb, p.in.offset, p.out.px, p.out.py, p.out.pb, p.out.offset};
    for (int64_t v : al) if (v % 4) return no("pitches must be 4-byte aligned");
    if (p.kh < 1 || p.kw < 1 || p.stride_x < 1 || p.stride_y < 1 || p.dil_x < 1 || p.dil_y < 1) return no("filter geometry");
    if ((int64_t)p.kh * p.kw * p.groups > 48 * 1024) return no("filters must fit in 48 KiB of shared memory");
    if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_I32 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    const int P_ = (p.in.y + 2 * p.pad_y - ((p.kh - 1) * p.dil_y + 1)) / p.stride_y + 1;
    const int Q_ = (p.in.x + 2 * p.pad_x - ((p.kw - 1) * p.dil_x + 1)) / p.stride_x + 1;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");
    return true;
}
bool dw_supports(const void* vp) { return dw_plan(*(const cldnn_b200_conv_params*)vp, nullptr); }
int dw_tune_count(const void*) { return 1; }

int32_t dw_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params p = *(const cldnn_b200_conv_params*)vp;
    std::string why;
    if (!dw_plan(p, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_dw: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: bias_dtype set but no bias pointer");
    if (p.quantization && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: quantization set but no factors");
    if (p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: calibration set but no factors");
    if (((uintptr_t)a->input0 | (uintptr_t)a->output) & 3) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: buffers must be 4-byte aligned");
    const EpiCfg c = make_epi_cfg(p);
    DwArgs d{(const uint8_t*)a->input0, (const int8_t*)a->weights, a->bias, a->weights_quantization_factors, a->output_calibration_factors, (uint8_t*)a->output};
    const int64_t items = (int64_t)p.out.b * p.out.y * p.out.x * (p.out.f / 4);
    int64_t blocks = (items + 255) / 256; const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 8;
    if (blocks > cap) blocks = cap; if (blocks < 1) blocks = 1;
    const int grid = (int)blocks; const size_t smem = (size_t)p.kh * p.kw * p.groups;
    const bool uns = p.in.dtype == CLDNN_B200_U8;
    out->fn = [p, c, d, grid, smem, uns](cudaStream_t s) {
        if (uns) conv_i8_dw_kernel<true><<<grid, 256, smem, s>>>(p, c, d);
        else conv_i8_dw_kernel<false><<<grid, 256, smem, s>>>(p, c, d);
        return cudaGetLastError();
    };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

}  // namespace

const KernelDef kdef_conv_i8_dw = {"conv_i8_dw", sizeof(cldnn_b200_conv_params), dw_supports, dw_tune_count, nullptr, dw_prepare};

}  // namespace b200
