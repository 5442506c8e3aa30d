// conv_i8_dw: 8-bit depthwise convolution (groups == features, one filter per
// feature), the MobileNet building block.  A depthwise filter has no reduction
// over features, so there is nothing for the tensor cores: the kernel is CUDA-core
// code over the feature-innermost (byxf) layout, bounded by instruction issue
// (one multiply-add per tap and output) and then by HBM.
//
// Main kernel (features a multiple of 16): a thread owns 16 consecutive features
// of two horizontally adjacent output pixels.  Per filter tap it reads one 128-bit
// word per pixel (a warp reads contiguous memory) and runs one dp4a per feature:
// the filter tap of feature e is kept in shared memory as a word that holds the
// weight in byte lane e % 4 and zeros elsewhere, so dp4a(input word, that word, acc)
// is exactly acc += x[e] * w[e] -- one instruction instead of two byte extractions
// and a multiply-add.  The weight words are loaded once per tap for both pixels.
// Epilogue: the quantised epilogue of fused_conv_eltwise_gpu_ref.cl:148-194 (integer
// bias, per-feature dequantisation, activation -- ReLU6 is CLAMP(0, 6) -- calibration /
// O_QF, round, saturate); the common configuration (per-feature scale, optional
// uniform O_QF, NONE / ReLU or a clamp the saturation subsumes) takes the
// conversion-free form of conv_epilogue.cuh, exact while |value| < 2^22, which a
// per-CTA scan of the constants checks.  A 4-features-per-thread kernel covers other
// feature counts.  It stands where the reference uses
// cl_kernels/convolution_gpu_byxf_af32_depthwise.cl.
#include "engine.hpp"
#include "conv_epilogue.cuh"

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

// ---- 16 features x 2 pixels per thread ------------------------------------------------
struct Dw16Args {
    const uint8_t* in; const void* bias; const float* quant; const float* calib; uint8_t* out;
    const uint32_t* wmask;          // [tap][feature]: the weight in byte lane (feature % 4) of a zero word
    int32_t q2, c16n, lean, mul_oqf; // pixel pairs per row, 16-feature groups, conversion-free epilogue allowed, uniform O_QF present
    float acc_bound;                // taps * max|activation| * 128
    uint32_t items;
    // column-walk kernel: every item is a strip of `strip_rows` output rows of one pixel pair and 4 features
    int32_t strips, strip_rows; uint32_t col_items;
    const uint32_t* wide_flag;      // column-walk kernel: non-zero when some feature's values may leave the range the conversion-free epilogue is exact in
};

__global__ void dw_pack_weights(const int8_t* __restrict__ w, int64_t po, int64_t py, int64_t px, int64_t off, int C, int kh, int kw, uint32_t* __restrict__ dst)
{
    const int total = kh * kw * C;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int f = i % C, t = i / C; const int j = t / kw, s = t - j * kw;
        dst[i] = ((uint32_t)(uint8_t)w[off + (int64_t)f * po + j * py + s * px]) << (8 * (f & 3));
    }
}

// Whether any feature's dequantised values could reach 2^22 (where the conversion-free epilogue stops being exact): evaluated
// once when the launch is prepared, so that the column-walk kernel needs no pass over the per-feature constants per CTA.
__global__ void dw_wide_flag(const void* __restrict__ bias, int bias_dtype, int use_bias, const float* __restrict__ quant, int quantization,
                             float acc_bound, float oqf_abs, int C, uint32_t* __restrict__ flag)
{
    for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < C; f += gridDim.x * blockDim.x) {
        const int32_t bi = use_bias ? load_as_int(bias, bias_dtype, f) : 0;
        const float q = quantization ? quant[f] : 1.0f;
        if (!(__fmul_rn(__fmul_rn(__fadd_rn(acc_bound, fabsf((float)bi)), fabsf(q)), oqf_abs) < 4.0e6f)) atomicOr(flag, 1u);
    }
}

template <bool kUnsignedIn>
__device__ __forceinline__ int32_t dp4a_in(uint32_t x, uint32_t w, int32_t c)
{
    int32_t d;
    if (kUnsignedIn) asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(c));
    else asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(c));
    return d;
}

// Four features of one pixel: accumulators -> requantised output word.  mode 0..2: conversion-free u8 / s8 / s8 after
// ReLU (fast_quad), 3: every other configuration through the general epilogue.
template <int kMode, bool kOqf>
__device__ __forceinline__ uint32_t dw_epi_word_t(const cldnn_b200_conv_params& p, const EpiCfg& c, const Dw16Args& a,
                                                  const int32_t (&a4)[4], const int4 b4, const float4 q4, int f);

__device__ __forceinline__ uint32_t dw_epi_word(int mode, const cldnn_b200_conv_params& p, const EpiCfg& c, const Dw16Args& a,
                                                const int32_t (&a4)[4], const int4 b4, const float4 q4, int f)
{
    if (mode == 0) return a.mul_oqf ? fast_quad<0, true>(a4, b4, q4, c.o_qf) : fast_quad<0, false>(a4, b4, q4, 1.0f);
    if (mode == 1) return a.mul_oqf ? fast_quad<1, true>(a4, b4, q4, c.o_qf) : fast_quad<1, false>(a4, b4, q4, 1.0f);
    if (mode == 2) return fast_quad<2, false>(a4, b4, q4, 1.0f);
    uint32_t word = 0;
    const int32_t bb[4] = {b4.x, b4.y, b4.z, b4.w}; const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float v = epi_quant(c, a4[e] + bb[e], qq[e], c.dont_dequantize_bias ? ((const float*)a.bias)[f + e] : 0.f,
                                  p.calibration ? a.calib[f + e] : 1.f, 0.f, 1.f);
        const int32_t r = __float2int_rz(v);
        const int32_t sat = p.out.dtype == CLDNN_B200_U8 ? min(255, max(0, r)) : min(127, max(-128, r));
        word |= ((uint32_t)sat & 0xffu) << (8 * e);
    }
    return word;
}

template <int kMode, bool kOqf>
__device__ __forceinline__ uint32_t dw_epi_word_t(const cldnn_b200_conv_params& p, const EpiCfg& c, const Dw16Args& a,
                                                  const int32_t (&a4)[4], const int4 b4, const float4 q4, int f)
{
    if (kMode < 3) return fast_quad<kMode, kOqf>(a4, b4, q4, kOqf ? c.o_qf : 1.0f);
    return dw_epi_word(3, p, c, a, a4, b4, q4, f);
}

template <bool kUnsignedIn>
__global__ void __launch_bounds__(256)
conv_i8_dw16_kernel(const __grid_constant__ cldnn_b200_conv_params p, const __grid_constant__ EpiCfg c, const __grid_constant__ Dw16Args a)
{
    extern __shared__ uint4 s_dw[];
    const int C = p.out.f, taps = p.kh * p.kw;
    uint4* s_w = s_dw;                                               // [tap][k][C / 16]: the 4 weight words of features 16 g + 4 k .. + 3 (threads of a warp differ in g: consecutive 16-byte reads)
    int32_t* s_bias = reinterpret_cast<int32_t*>(s_dw + taps * (C / 4));
    float* s_quant = reinterpret_cast<float*>(s_bias + C);
    __shared__ uint32_t s_wide;
    if (threadIdx.x == 0) s_wide = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < taps * (C / 4); i += blockDim.x) {
        const int tap = i / (C / 4), r = i - tap * (C / 4);          // global order [tap][g][k]
        s_w[(tap * 4 + (r & 3)) * a.c16n + (r >> 2)] = __ldg(reinterpret_cast<const uint4*>(a.wmask) + i);
    }
    bool wide = false;
    for (int f = threadIdx.x; f < C; f += blockDim.x) {
        const int32_t bi = (p.bias_dtype != CLDNN_B200_NONE && !c.dont_dequantize_bias) ? load_as_int(a.bias, p.bias_dtype, f) : 0;
        const float q = p.quantization ? a.quant[f] : 1.0f;
        s_bias[f] = bi; s_quant[f] = q;
        wide = wide || !(__fmul_rn(__fmul_rn(__fadd_rn(a.acc_bound, fabsf((float)bi)), fabsf(q)), a.mul_oqf ? fabsf(c.o_qf) : 1.0f) < 4.0e6f);
    }
    if (wide) atomicOr(&s_wide, 1u);
    __syncthreads();
    // 0..2: conversion-free u8 / s8 / s8 after ReLU, 3: general
    const int mode = (a.lean && !s_wide) ? (p.out.dtype == CLDNN_B200_U8 ? 0 : (c.act == CLDNN_B200_ACT_RELU ? 2 : 1)) : 3;
    const int c4n = C / 4;

    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < a.items; idx += gridDim.x * blockDim.x) {
        const uint32_t g = idx % (uint32_t)a.c16n; uint32_t t = idx / (uint32_t)a.c16n;
        const uint32_t xq = t % (uint32_t)a.q2; t /= (uint32_t)a.q2;
        const uint32_t y = t % (uint32_t)p.out.y; const uint32_t b = t / (uint32_t)p.out.y;
        const int f0 = (int)g * 16, x0 = (int)xq * 2;
        const bool second = x0 + 1 < p.out.x;
        const int iy0 = (int)y * p.stride_y - p.pad_y, ix0 = x0 * p.stride_x - p.pad_x, ix1 = ix0 + p.stride_x;
        int32_t acc0[16], acc1[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) { acc0[e] = 0; acc1[e] = 0; }
        const uint8_t* src = a.in + p.in.offset + (int64_t)b * p.in.pb + f0;
        for (int j = 0; j < p.kh; ++j) {
            const int iy = iy0 + j * p.dil_y; if (iy < 0 || iy >= p.in.y) continue;
            const uint8_t* rowp = src + (int64_t)iy * p.in.py;
            if (p.kw == 3) {
                // three-tap rows (the MobileNet case): the six loads of the row are issued before any arithmetic, so their
                // latency is paid once per filter row instead of once per tap
                uint4 xa3[3], xb3[3];
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    const int xa = ix0 + s * p.dil_x, xb = ix1 + s * p.dil_x;
                    xa3[s] = (xa >= 0 && xa < p.in.x) ? __ldg(reinterpret_cast<const uint4*>(rowp + (int64_t)xa * p.in.px)) : make_uint4(0, 0, 0, 0);
                    xb3[s] = (second && xb >= 0 && xb < p.in.x) ? __ldg(reinterpret_cast<const uint4*>(rowp + (int64_t)xb * p.in.px)) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    const uint32_t xw_a[4] = {xa3[s].x, xa3[s].y, xa3[s].z, xa3[s].w}, xw_b[4] = {xb3[s].x, xb3[s].y, xb3[s].z, xb3[s].w};
                    const uint4* wt = s_w + (j * 3 + s) * c4n + g;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint4 wm = wt[k * a.c16n];
                        acc0[4 * k + 0] = dp4a_in<kUnsignedIn>(xw_a[k], wm.x, acc0[4 * k + 0]); acc1[4 * k + 0] = dp4a_in<kUnsignedIn>(xw_b[k], wm.x, acc1[4 * k + 0]);
                        acc0[4 * k + 1] = dp4a_in<kUnsignedIn>(xw_a[k], wm.y, acc0[4 * k + 1]); acc1[4 * k + 1] = dp4a_in<kUnsignedIn>(xw_b[k], wm.y, acc1[4 * k + 1]);
                        acc0[4 * k + 2] = dp4a_in<kUnsignedIn>(xw_a[k], wm.z, acc0[4 * k + 2]); acc1[4 * k + 2] = dp4a_in<kUnsignedIn>(xw_b[k], wm.z, acc1[4 * k + 2]);
                        acc0[4 * k + 3] = dp4a_in<kUnsignedIn>(xw_a[k], wm.w, acc0[4 * k + 3]); acc1[4 * k + 3] = dp4a_in<kUnsignedIn>(xw_b[k], wm.w, acc1[4 * k + 3]);
                    }
                }
                continue;
            }
            for (int s = 0; s < p.kw; ++s) {
                const int xa = ix0 + s * p.dil_x, xb = ix1 + s * p.dil_x;
                const bool va = xa >= 0 && xa < p.in.x, vb = second && xb >= 0 && xb < p.in.x;
                if (!va && !vb) continue;
                uint4 x_a = make_uint4(0, 0, 0, 0), x_b = make_uint4(0, 0, 0, 0);
                if (va) x_a = __ldg(reinterpret_cast<const uint4*>(rowp + (int64_t)xa * p.in.px));
                if (vb) x_b = __ldg(reinterpret_cast<const uint4*>(rowp + (int64_t)xb * p.in.px));
                const uint32_t xw_a[4] = {x_a.x, x_a.y, x_a.z, x_a.w}, xw_b[4] = {x_b.x, x_b.y, x_b.z, x_b.w};
                const uint4* wt = s_w + (j * p.kw + s) * c4n + g;
#pragma unroll
                for (int k = 0; k < 4; ++k) {                          // 4 words of 4 features
                    const uint4 wm = wt[k * a.c16n];
                    acc0[4 * k + 0] = dp4a_in<kUnsignedIn>(xw_a[k], wm.x, acc0[4 * k + 0]); acc1[4 * k + 0] = dp4a_in<kUnsignedIn>(xw_b[k], wm.x, acc1[4 * k + 0]);
                    acc0[4 * k + 1] = dp4a_in<kUnsignedIn>(xw_a[k], wm.y, acc0[4 * k + 1]); acc1[4 * k + 1] = dp4a_in<kUnsignedIn>(xw_b[k], wm.y, acc1[4 * k + 1]);
                    acc0[4 * k + 2] = dp4a_in<kUnsignedIn>(xw_a[k], wm.z, acc0[4 * k + 2]); acc1[4 * k + 2] = dp4a_in<kUnsignedIn>(xw_b[k], wm.z, acc1[4 * k + 2]);
                    acc0[4 * k + 3] = dp4a_in<kUnsignedIn>(xw_a[k], wm.w, acc0[4 * k + 3]); acc1[4 * k + 3] = dp4a_in<kUnsignedIn>(xw_b[k], wm.w, acc1[4 * k + 3]);
                }
            }
        }
        uint8_t* dst = a.out + p.out.offset + (int64_t)b * p.out.pb + (int64_t)y * p.out.py + (int64_t)x0 * p.out.px + f0;
#pragma unroll
        for (int px = 0; px < 2; ++px) {
            if (px == 1 && !second) break;
            const int32_t (&acc)[16] = px ? acc1 : acc0;
            uint32_t ow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int32_t a4[4] = {acc[4 * k], acc[4 * k + 1], acc[4 * k + 2], acc[4 * k + 3]};
                const int4 b4 = *reinterpret_cast<const int4*>(s_bias + f0 + 4 * k);
                const float4 q4 = *reinterpret_cast<const float4*>(s_quant + f0 + 4 * k);
                ow[k] = dw_epi_word(mode, p, c, a, a4, b4, q4, f0 + 4 * k);
            }
            *reinterpret_cast<uint4*>(dst + (int64_t)px * p.out.px) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
}

// Item loop of the column-walk kernel below for one epilogue variant (kMode as in dw_epi_word, kOqf: uniform O_QF).
template <bool kUnsignedIn, int kStride, int kMode, bool kOqf>
__device__ __forceinline__ void dwcol_items(const cldnn_b200_conv_params& p, const EpiCfg& c, const Dw16Args& a)
{
    // The weight words, bias and scale of a thread's 4 features come straight from global memory (a warp reads 512
    // consecutive bytes per tap; the few KB involved stay in L1 / L2): a CTA that first stages all features' constants in
    // shared memory spends, on the small maps of a network's last stages, more time and L2 traffic on that than on its items.
    const uint4* g_w = reinterpret_cast<const uint4*>(a.wmask);
    const bool use_bias = p.bias_dtype != CLDNN_B200_NONE && !c.dont_dequantize_bias;
    constexpr int kCols = kStride + 3;
    const int c4n = p.out.f / 4;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < a.col_items; idx += gridDim.x * blockDim.x) {
        const uint32_t c4 = idx % (uint32_t)c4n; uint32_t t = idx / (uint32_t)c4n;
        const uint32_t xq = t % (uint32_t)a.q2; t /= (uint32_t)a.q2;
        const uint32_t strip = t % (uint32_t)a.strips; const uint32_t b = t / (uint32_t)a.strips;
        const int f0 = (int)c4 * 4, x0 = (int)xq * 2;
        const bool second = x0 + 1 < p.out.x;
        uint32_t w[9][4];
#pragma unroll
        for (int tap = 0; tap < 9; ++tap) {
            const uint4 wm = __ldg(g_w + tap * c4n + (int)c4);
            w[tap][0] = wm.x; w[tap][1] = wm.y; w[tap][2] = wm.z; w[tap][3] = wm.w;
        }
        // stride 1: the four columns under the pixel pair are transposed into one word per feature (4 consecutive pixels
        // of a row), so one dp4a takes a whole filter row: per feature and filter row the three weights in bytes 0..2
        // for the left pixel and in bytes 1..3 for the right one
        uint32_t wa[3][4], wb[3][4];
        if (kStride == 1) {
#pragma unroll
            for (int j = 0; j < 3; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t t0 = (w[j * 3 + 0][e] >> (8 * e)) & 0xffu, t1 = (w[j * 3 + 1][e] >> (8 * e)) & 0xffu, t2 = (w[j * 3 + 2][e] >> (8 * e)) & 0xffu;
                    wa[j][e] = t0 | (t1 << 8) | (t2 << 16); wb[j][e] = wa[j][e] << 8;
                }
        }
        int4 b4 = make_int4(0, 0, 0, 0);
        if (use_bias) {
            if (p.bias_dtype == CLDNN_B200_I32) b4 = __ldg(reinterpret_cast<const int4*>(a.bias) + c4);
            else b4 = make_int4(load_as_int(a.bias, p.bias_dtype, f0), load_as_int(a.bias, p.bias_dtype, f0 + 1), load_as_int(a.bias, p.bias_dtype, f0 + 2), load_as_int(a.bias, p.bias_dtype, f0 + 3));
        }
        const float4 q4 = p.quantization ? __ldg(reinterpret_cast<const float4*>(a.quant) + c4) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        // the kCols input columns under the pixel pair: byte offsets inside a row, -1 for a column outside the input
        const int ix0 = x0 * kStride - p.pad_x;
        int co[kCols];
#pragma unroll
        for (int s = 0; s < kCols; ++s) co[s] = (ix0 + s >= 0 && ix0 + s < p.in.x) ? (ix0 + s) * (int)p.in.px : -1;
        const uint8_t* src = a.in + p.in.offset + (int64_t)b * p.in.pb + f0;
        auto load_row = [&](int iy, uint32_t (&row)[kCols]) {
            const bool in_y = iy >= 0 && iy < p.in.y;
            const uint8_t* rowp = src + (int64_t)iy * p.in.py;
#pragma unroll
            for (int s = 0; s < kCols; ++s) row[s] = (in_y && co[s] >= 0) ? __ldg(reinterpret_cast<const uint32_t*>(rowp + co[s])) : 0u;
        };
        // stride 1, 4 x 4 byte transpose of a loaded row: (column, feature) -> (feature, column); done when the row enters
        // the window, not when it is loaded, so that the loads stay ahead of their first use
        auto transpose = [&](uint32_t (&row)[kCols]) {
            if (kStride == 1) {
                const uint32_t ta = __byte_perm(row[0], row[1], 0x5140), tb = __byte_perm(row[0], row[1], 0x7362);
                const uint32_t tc = __byte_perm(row[2], row[3], 0x5140), td = __byte_perm(row[2], row[3], 0x7362);
                row[0] = __byte_perm(ta, tc, 0x5410); row[1] = __byte_perm(ta, tc, 0x7632);
                row[2] = __byte_perm(tb, td, 0x5410); row[3] = __byte_perm(tb, td, 0x7632);
            }
        };
        const int y0 = (int)strip * a.strip_rows, y1 = min(p.out.y, y0 + a.strip_rows);
        int iy = y0 * kStride - p.pad_y;
        uint32_t win[3][kCols];
        load_row(iy, win[0]); load_row(iy + 1, win[1]); load_row(iy + 2, win[2]);
        // two output rows of loads in flight: `ahead` holds the new rows of the next output row, loaded one iteration earlier
        uint32_t ahead[kStride][kCols];
#pragma unroll
        for (int r = 0; r < kStride; ++r) {
            if (y0 + 1 < y1) load_row(iy + 3 + r, ahead[r]);
            else {
#pragma unroll
                for (int s = 0; s < kCols; ++s) ahead[r][s] = 0u;
            }
        }
        transpose(win[0]); transpose(win[1]); transpose(win[2]);
        uint8_t* dst = a.out + p.out.offset + (int64_t)b * p.out.pb + (int64_t)y0 * p.out.py + (int64_t)x0 * p.out.px + f0;
        for (int y = y0; y < y1; ++y, iy += kStride, dst += p.out.py) {
            uint32_t nxt[kStride][kCols];
            if (y + 2 < y1) {
#pragma unroll
                for (int r = 0; r < kStride; ++r) load_row(iy + 3 + kStride + r, nxt[r]);
            } else {
#pragma unroll
                for (int r = 0; r < kStride; ++r)
#pragma unroll
                    for (int s = 0; s < kCols; ++s) nxt[r][s] = 0u;
            }
            int32_t acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
            if (kStride == 1) {
#pragma unroll
                for (int j = 0; j < 3; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc0[e] = dp4a_in<kUnsignedIn>(win[j][e], wa[j][e], acc0[e]);
                        acc1[e] = dp4a_in<kUnsignedIn>(win[j][e], wb[j][e], acc1[e]);
                    }
            } else {
#pragma unroll
                for (int j = 0; j < 3; ++j)
#pragma unroll
                    for (int s = 0; s < 3; ++s)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc0[e] = dp4a_in<kUnsignedIn>(win[j][s], w[j * 3 + s][e], acc0[e]);
                            acc1[e] = dp4a_in<kUnsignedIn>(win[j][s + kStride], w[j * 3 + s][e], acc1[e]);
                        }
            }
            *reinterpret_cast<uint32_t*>(dst) = dw_epi_word_t<kMode, kOqf>(p, c, a, acc0, b4, q4, f0);
            if (second) *reinterpret_cast<uint32_t*>(dst + p.out.px) = dw_epi_word_t<kMode, kOqf>(p, c, a, acc1, b4, q4, f0);
            if (kStride == 1) transpose(ahead[0]);
#pragma unroll
            for (int s = 0; s < kCols; ++s) {
                if (kStride == 1) { win[0][s] = win[1][s]; win[1][s] = win[2][s]; win[2][s] = ahead[0][s]; }
                else { win[0][s] = win[2][s]; win[1][s] = ahead[0][s]; win[2][s] = ahead[kStride - 1][s]; }
#pragma unroll
                for (int r = 0; r < kStride; ++r) ahead[r][s] = nxt[r][s];
            }
        }
    }
}

// ---- 3x3 filters: 4 features x 2 pixels per thread, walking down a strip of output rows ----------
// The weight words of the thread's 4 features (stride 2: nine masked words per feature, one dp4a per multiply-add;
// stride 1: the input words transposed to 4 pixels of one feature, one dp4a per filter row), their bias and scale stay
// in registers for the whole strip, and so do the three input rows under the current output row (kStride + 3 columns of one word each):
// per output row a thread loads only the kStride new rows, one row ahead of their use.  No shared-memory traffic in
// the loop; a warp reads and writes 128 consecutive bytes of a pixel.
template <bool kUnsignedIn, int kStride>
__global__ void __launch_bounds__(256, kStride == 1 ? 3 : 2)
conv_i8_dwcol_kernel(const __grid_constant__ cldnn_b200_conv_params p, const __grid_constant__ EpiCfg c, const __grid_constant__ Dw16Args a)
{
    // the epilogue variant is uniform over the launch: chosen once, so that the row loop is straight-line code
    const bool wide = __ldg(a.wide_flag) != 0u;
    const int mode = (a.lean && !wide) ? (p.out.dtype == CLDNN_B200_U8 ? 0 : (c.act == CLDNN_B200_ACT_RELU ? 2 : 1)) : 3;
    if (mode == 0) { if (a.mul_oqf) dwcol_items<kUnsignedIn, kStride, 0, true>(p, c, a); else dwcol_items<kUnsignedIn, kStride, 0, false>(p, c, a); }
    else if (mode == 1) { if (a.mul_oqf) dwcol_items<kUnsignedIn, kStride, 1, true>(p, c, a); else dwcol_items<kUnsignedIn, kStride, 1, false>(p, c, a); }
    else if (mode == 2) dwcol_items<kUnsignedIn, kStride, 2, false>(p, c, a);
    else dwcol_items<kUnsignedIn, kStride, 3, false>(p, c, a);
}

bool dw_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (p.epilogue_order != CLDNN_B200_EPILOGUE_REF) return no("reference epilogue order only");
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

// the 16-feature kernel: 16-byte aligned rows of features, its weight words and constants within shared memory
bool dw16_ok(const cldnn_b200_conv_params& p)
{
    if (p.groups % 16) return false;
    const int64_t al[] = {p.in.px, p.in.py, p.in.pb, p.in.offset, p.out.px, p.out.py, p.out.pb, p.out.offset};
    for (int64_t v : al) if (v % 16) return false;
    if ((int64_t)p.kh * p.kw * p.groups * 4 + (int64_t)p.groups * 8 > 96 * 1024) return false;
    const int64_t items = (int64_t)p.out.b * p.out.y * ((p.out.x + 1) / 2) * (p.groups / 16);
    return items > 0 && items < 0x7fffffffLL;
}
// the column-walk kernel: 3x3 filters without dilation, stride 1 or 2 in both directions
bool dwcol_ok(const cldnn_b200_conv_params& p)
{
    return dw16_ok(p) && p.kh == 3 && p.kw == 3 && p.dil_x == 1 && p.dil_y == 1 && p.stride_x == p.stride_y && (p.stride_x == 1 || p.stride_x == 2) &&
           (int64_t)p.in.x * p.in.px < 0x7fffffffLL;
}
// tune 0: the column-walk kernel where it applies, 1: the 16-feature kernel
// 0 = automatic (the column-walk kernel where it applies, the 16-feature kernel otherwise), 1 = the 16-feature kernel,
// 2 = the column-walk kernel by name: the tuner times the indices from 1 up, index 0 being the untuned default everywhere.
int dw_tune_count(const void* vp) { return dwcol_ok(simplified_conv_params(*(const cldnn_b200_conv_params*)vp)) ? 3 : 1; }
size_t dw_scratch(const void* vp)
{
    const auto& p = *(const cldnn_b200_conv_params*)vp;
    return dw16_ok(p) ? (size_t)p.kh * p.kw * p.groups * 4 + 16 : 0;     // the weight words, then the range flag of the column-walk kernel
}

int32_t dw_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params p = simplified_conv_params(*(const cldnn_b200_conv_params*)vp);
    std::string why;
    if (!dw_plan(p, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_dw: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: bias_dtype set but no bias pointer");
    if (p.quantization && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: quantization set but no factors");
    if (p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: calibration set but no factors");
    if (((uintptr_t)a->input0 | (uintptr_t)a->output) & 3) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_dw: buffers must be 4-byte aligned");
    const EpiCfg c = make_epi_cfg(p);
    const bool uns_in = p.in.dtype == CLDNN_B200_U8;
    if (dw16_ok(p) && a->scratch && a->scratch_bytes >= dw_scratch(&p) && !(((uintptr_t)a->input0 | (uintptr_t)a->output | (uintptr_t)a->scratch) & 15)) {
        Dw16Args d{};
        d.in = (const uint8_t*)a->input0; d.bias = a->bias; d.quant = a->weights_quantization_factors; d.calib = a->output_calibration_factors;
        d.out = (uint8_t*)a->output; d.wmask = (const uint32_t*)a->scratch;
        d.q2 = (p.out.x + 1) / 2; d.c16n = p.groups / 16;
        d.mul_oqf = (p.calibration || p.o_qf != 1.0f) ? 1 : 0;
        const bool oqf_ok = !d.mul_oqf || (!p.calibration && p.o_qf > 0.0f && (p.out.dtype == CLDNN_B200_U8 || p.act != CLDNN_B200_ACT_RELU));
        d.lean = (p.quantization && p.i_qf == 1.0f && oqf_ok && !c.dont_dequantize_bias && (p.act == CLDNN_B200_ACT_NONE || p.act == CLDNN_B200_ACT_RELU) &&
                  (p.bias_dtype == CLDNN_B200_NONE || p.bias_dtype == CLDNN_B200_I32)) ? 1 : 0;
        d.acc_bound = (float)(p.kh * p.kw) * (uns_in ? 255.0f : 128.0f) * 128.0f;
        d.items = (uint32_t)((int64_t)p.out.b * p.out.y * d.q2 * d.c16n);
        // the weight words once, on the context's stream, before anything that is prepared here can run
        const int taps_c = p.kh * p.kw * p.groups;
        dw_pack_weights<<<(taps_c + 255) / 256, 256, 0, ctx->stream>>>((const int8_t*)a->weights, p.w_po, p.w_py, p.w_px, p.w_offset, p.groups, p.kh, p.kw, (uint32_t*)a->scratch);
        B200_CUDA(cudaGetLastError());
        uint32_t* flag = reinterpret_cast<uint32_t*>((char*)a->scratch + (size_t)taps_c * 4);
        B200_CUDA(cudaMemsetAsync(flag, 0, 16, ctx->stream));
        dw_wide_flag<<<(p.groups + 255) / 256, 256, 0, ctx->stream>>>(a->bias, p.bias_dtype, (p.bias_dtype != CLDNN_B200_NONE && !c.dont_dequantize_bias) ? 1 : 0,
                                                                   a->weights_quantization_factors, p.quantization, d.acc_bound,
                                                                   d.mul_oqf ? fabsf(p.o_qf) : 1.0f, p.groups, flag);
        B200_CUDA(cudaGetLastError());
        d.wide_flag = flag;
        const size_t smem = (size_t)taps_c * 4 + (size_t)p.groups * 8;
        if (smem > 48 * 1024) {
            // the limit is shared by every prepared launch of the function on this device: it only ever grows
            B200_CUDA(raise_smem_limit((const void*)conv_i8_dw16_kernel<true>, ctx->device, smem));
            B200_CUDA(raise_smem_limit((const void*)conv_i8_dw16_kernel<false>, ctx->device, smem));
        }
        if (dwcol_ok(p) && p.tune != 1) {
            // strips of 14 output rows, shorter while the items would not fill the device
            const int64_t per_row_strip = (int64_t)p.out.b * d.q2 * (p.groups / 4);
            int rows = p.out.y < 14 ? p.out.y : 14;
            while (rows > 4 && per_row_strip * ((p.out.y + rows - 1) / rows) < (int64_t)ctx->prop.multiProcessorCount * 1024) rows = (rows + 1) / 2;
            d.strip_rows = rows; d.strips = (p.out.y + rows - 1) / rows;
            const int64_t col_items = per_row_strip * d.strips;
            if (col_items < 0x7fffffffLL) {
                d.col_items = (uint32_t)col_items;
                int64_t cblocks = (col_items + 255) / 256; const int64_t ccap = (int64_t)ctx->prop.multiProcessorCount * 8;
                if (cblocks > ccap) cblocks = ccap;
                const int cgrid = (int)cblocks; const int stride = p.stride_x;
                out->fn = [p, c, d, cgrid, uns_in, stride](cudaStream_t s) {
                    if (uns_in) { if (stride == 1) conv_i8_dwcol_kernel<true, 1><<<cgrid, 256, 0, s>>>(p, c, d); else conv_i8_dwcol_kernel<true, 2><<<cgrid, 256, 0, s>>>(p, c, d); }
                    else { if (stride == 1) conv_i8_dwcol_kernel<false, 1><<<cgrid, 256, 0, s>>>(p, c, d); else conv_i8_dwcol_kernel<false, 2><<<cgrid, 256, 0, s>>>(p, c, d); }
                    return cudaGetLastError();
                };
                out->launches = 1;
                return CLDNN_B200_SUCCESS;
            }
        }
        int64_t blocks = ((int64_t)d.items + 255) / 256; const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 8;
        if (blocks > cap) blocks = cap;
        const int grid = (int)blocks;
        out->fn = [p, c, d, grid, smem, uns_in](cudaStream_t s) {
            if (uns_in) conv_i8_dw16_kernel<true><<<grid, 256, smem, s>>>(p, c, d);
            else conv_i8_dw16_kernel<false><<<grid, 256, smem, s>>>(p, c, d);
            return cudaGetLastError();
        };
        out->launches = 1;
        return CLDNN_B200_SUCCESS;
    }
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

const KernelDef kdef_conv_i8_dw = {"conv_i8_dw", sizeof(cldnn_b200_conv_params), dw_supports, dw_tune_count, dw_scratch, dw_prepare};

}  // namespace b200
