// The unrolled fast epilogue shared by the tensor-core convolution kernels:
// 32 s32 accumulators of one pixel -> requantised bytes.  The kernel's parameter
// block must provide `epi` (EpiCfg), `mul_iqf`, `mul_oqf`; its shared-memory
// block `bias_i`, `bias_f`, `quant`, `calib`, `ecal` as [buffers][features].
#pragma once
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200 {

using namespace ptx;

// The activations that are cheap enough to inline 32 times in the unrolled epilogue.
__host__ __device__ inline bool act_is_simple(int32_t fn, float m)
{
    return fn == CLDNN_B200_ACT_NONE || fn == CLDNN_B200_ACT_RELU || fn == CLDNN_B200_ACT_CLAMP ||
           (fn == CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE && m == m && m - m == 0.0f);
}
__device__ __forceinline__ float act_simple(int32_t fn, float x, float m, float n)
{
    if (fn == CLDNN_B200_ACT_RELU) return fmaxf(0.0f, x);
    if (fn == CLDNN_B200_ACT_NONE) return x;
    if (fn == CLDNN_B200_ACT_CLAMP) return fmaxf(m, fminf(n, x));
    return __fadd_rn(fmaxf(x, 0.0f), __fmul_rn(m, fminf(x, 0.0f)));
}

// round(x) with ties away from zero, returned still as a float whose fraction is
// not yet dropped: adding +-0.5 with round-toward-zero can never carry the sum
// across the next integer, so truncating afterwards gives exactly round().
__device__ __forceinline__ float half_away_pre(float x) { return __fadd_rz(x, copysignf(0.5f, x)); }

// 32 features of one pixel: s32 accumulators -> requantised bytes in eight words.
// Quantised path, 8-bit output, simple activations; same operation order as
// epi_quant().  `e` holds the 32 residual bytes when kFused.
template <bool kFused, bool kLean, class ParamsT, class AuxT>
__device__ __forceinline__ void epi_chunk_fast(const ParamsT& P, const AuxT* aux, int acc, int c0, const uint32_t (&r)[32],
                                               uint4 e0, uint4 e1, uint4& o0, uint4& o1)
{
    const EpiCfg& c = P.epi;
    const bool out_u8 = c.out_dtype == CLDNN_B200_U8;
    uint32_t ew[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
    float e_bias = 8388608.0f;
    if (kFused && c.eltw_dtype != CLDNN_B200_U8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) ew[i] ^= 0x80808080u;          // s8 + 128 as an unsigned byte
        e_bias = 8388736.0f;
    }
    uint32_t ow[8];
    if (kLean) {
        // The common network configuration, with every uniform decision hoisted out of
        // the unrolled body: per-channel quantisation, optionally a uniform O_QF (I_QF = 1,
        // integer or no bias), activations NONE or ReLU, plain residual sum.  ~8 instructions per
        // feature; max(v, -inf) stands for "no activation".
        const float lo1 = c.act == CLDNN_B200_ACT_RELU ? 0.0f : __int_as_float(0xff800000);
        const float lo2 = c.eltw_act == CLDNN_B200_ACT_RELU ? 0.0f : __int_as_float(0xff800000);
        const bool oq = P.mul_oqf != 0;                             // uniform O_QF (no per-feature calibration on this path)
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const int cj = c0 + 4 * g;
            const int4 bi = *reinterpret_cast<const int4*>(&aux->bias_i[acc][cj]);
            const float4 q = *reinterpret_cast<const float4*>(&aux->quant[acc][cj]);
            const int32_t b4[4] = {bi.x, bi.y, bi.z, bi.w};
            const float q4[4] = {q.x, q.y, q.z, q.w};
            int32_t o4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = fmaxf(__fmul_rn(__int2float_rn((int32_t)r[4 * g + i] + b4[i]), q4[i]), lo1);
                if (oq) v = __fmul_rn(v, c.o_qf);
                v = half_away_pre(v);
                if (kFused) {
                    const float e = __fadd_rn(__uint_as_float(__byte_perm(ew[g], 0x4B000000u, 0x7450u + i)), -e_bias);
                    v = half_away_pre(fmaxf(__fadd_rn(truncf(v), e), lo2));
                }
                o4[i] = __float2int_rz(v);
            }
            ow[g] = out_u8 ? pack_sat_u8(o4[1], o4[0], pack_sat_u8(o4[3], o4[2], 0u))
                           : pack_sat_s8(o4[1], o4[0], pack_sat_s8(o4[3], o4[2], 0u));
        }
        o0 = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        o1 = make_uint4(ow[4], ow[5], ow[6], ow[7]);
        return;
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int cj = c0 + 4 * g;
        const int4 bi = *reinterpret_cast<const int4*>(&aux->bias_i[acc][cj]);
        const int32_t b4[4] = {bi.x, bi.y, bi.z, bi.w};
        float q4[4] = {1.f, 1.f, 1.f, 1.f}, bf4[4] = {0.f, 0.f, 0.f, 0.f}, cal4[4], ec4[4] = {1.f, 1.f, 1.f, 1.f};
        if (c.quantization) { const float4 t = *reinterpret_cast<const float4*>(&aux->quant[acc][cj]); q4[0] = t.x; q4[1] = t.y; q4[2] = t.z; q4[3] = t.w; }
        if (c.dont_dequantize_bias) { const float4 t = *reinterpret_cast<const float4*>(&aux->bias_f[acc][cj]); bf4[0] = t.x; bf4[1] = t.y; bf4[2] = t.z; bf4[3] = t.w; }
        if (c.calibration) { const float4 t = *reinterpret_cast<const float4*>(&aux->calib[acc][cj]); cal4[0] = t.x; cal4[1] = t.y; cal4[2] = t.z; cal4[3] = t.w; }
        else { cal4[0] = cal4[1] = cal4[2] = cal4[3] = c.o_qf; }
        if (kFused && c.eltw_calibration) { const float4 t = *reinterpret_cast<const float4*>(&aux->ecal[acc][cj]); ec4[0] = t.x; ec4[1] = t.y; ec4[2] = t.z; ec4[3] = t.w; }
        int32_t o4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v = __int2float_rn((int32_t)r[4 * g + i] + b4[i]);
            if (c.quantization) { v = __fmul_rn(v, q4[i]); if (P.mul_iqf) v = __fmul_rn(v, c.i_qf); }
            if (c.dont_dequantize_bias) v = __fadd_rn(v, bf4[i]);
            v = act_simple(c.act, v, c.act_m, c.act_n);
            if (P.mul_oqf) v = __fmul_rn(v, cal4[i]);
            v = half_away_pre(v);
            if (kFused) {
                v = truncf(v);
                // byte -> float without a conversion instruction: 2^23 + byte, minus 2^23
                float e = __fadd_rn(__uint_as_float(__byte_perm(ew[g], 0x4B000000u, 0x7450u + i)), -e_bias);
                if (c.has_non_conv_scale) e = __fmul_rn(e, c.non_conv_scale);
                v = act_simple(c.eltw_act, __fadd_rn(v, e), c.eltw_m, c.eltw_n);
                if (c.eltw_calibration) v = __fmul_rn(v, ec4[i]);
                v = half_away_pre(v);
            }
            o4[i] = __float2int_rz(v);
        }
        ow[g] = out_u8 ? pack_sat_u8(o4[1], o4[0], pack_sat_u8(o4[3], o4[2], 0u))
                       : pack_sat_s8(o4[1], o4[0], pack_sat_s8(o4[3], o4[2], 0u));
    }
    o0 = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    o1 = make_uint4(ow[4], ow[5], ow[6], ow[7]);
}

// c + byte `sel` of the unsigned bytes in `a` (sel = 1 << 8*i picks byte i)
__device__ __forceinline__ int32_t dp4a_u8(uint32_t a, int32_t sel, int32_t c)
{
    int32_t d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(sel), "r"(c)); return d;
}

// bytes above 127 become 127 (a ReLU'd value saturated to u8, re-saturated to s8)
__device__ __forceinline__ uint32_t clamp_bytes_127(uint32_t w)
{
    const uint32_t m = w & 0x80808080u;
    return (w | (m - (m >> 7))) & 0x7f7f7f7fu;
}

constexpr float kMagic = 8388608.0f;             // 2^23: x + 2^23 toward zero leaves floor(x) in the mantissa for 0 <= x < 2^23
constexpr int32_t kMagicBits = 0x4B000000;

// Four features: s32 accumulators (+ integer bias) -> requantised bytes in one word, by the conversion-free steps of
// fast_chunk32 below (same requirement |v| < 2^22, same kOut / kOqf meaning; no residual).
template <int kOut, bool kOqf>
__device__ __forceinline__ uint32_t fast_quad(const int32_t (&acc)[4], const int4 bias, const float4 quant, float oqf)
{
    const int32_t b4[4] = {bias.x, bias.y, bias.z, bias.w};
    const float q4[4] = {quant.x, quant.y, quant.z, quant.w};
    int32_t o4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float v = __fmul_rn(__int2float_rn(acc[i] + b4[i]), q4[i]);
        if (kOqf) v = __fmul_rn(v, oqf);
        if (kOut != 1) o4[i] = __float_as_int(__fadd_rz(__fadd_rz(v, 0.5f), kMagic)) - kMagicBits;
        else {
            const int32_t wb = __float_as_int(__fadd_rz(__fadd_rz(fabsf(v), 0.5f), kMagic));
            o4[i] = v < 0.0f ? kMagicBits - wb : wb - kMagicBits;
        }
    }
    if (kOut == 1) return pack_sat_s8(o4[1], o4[0], pack_sat_s8(o4[3], o4[2], 0u));
    const uint32_t w = pack_sat_u8(o4[1], o4[0], pack_sat_u8(o4[3], o4[2], 0u));
    return kOut == 2 ? clamp_bytes_127(w) : w;
}

// 32 features of one pixel.  Requires |v| < 2^22 for every dequantised value v
// (guaranteed per feature tile by the caller), which makes every step exact
// without a float->int conversion instruction:
//   round-half-away(v) = sign(v) * floor(|v| + 0.5), floor taken by the 2^23 trick
//   with round-toward-zero additions (x + 0.5 toward zero never reaches the next integer).
// kOut: 0 = u8 output (its saturation covers a preceding ReLU), 1 = s8 output,
// 2 = s8 output after a ReLU.  kRelu1: ReLU between the convolution and the residual sum.
// e_xor / k_pos / k_neg: the residual word is made unsigned by e_xor (0 or 0x80808080),
// k_pos = 2^23 bits (+128 for a signed residual), k_neg = 2^23 bits (-128 for a signed residual).
// kOqf: the dequantised value is multiplied by the uniform `oqf` (O_QF) before rounding.
template <bool kFused, bool kRelu1, int kOut, bool kOqf = false>
__device__ __forceinline__ void fast_chunk32(const uint32_t (&r)[32], const int32_t* bias, const float* quant,
                                             uint4* p0, uint4* p1, uint32_t e_xor, int32_t k_pos, int32_t k_neg, float oqf = 1.0f)
{
    uint32_t ew[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (kFused) {
        const uint4 e0 = *p0, e1 = *p1;
        ew[0] = e0.x ^ e_xor; ew[1] = e0.y ^ e_xor; ew[2] = e0.z ^ e_xor; ew[3] = e0.w ^ e_xor;
        ew[4] = e1.x ^ e_xor; ew[5] = e1.y ^ e_xor; ew[6] = e1.z ^ e_xor; ew[7] = e1.w ^ e_xor;
    }
    uint32_t ow[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int4 bi = reinterpret_cast<const int4*>(bias)[g];
        const float4 q = reinterpret_cast<const float4*>(quant)[g];
        const int32_t b4[4] = {bi.x, bi.y, bi.z, bi.w};
        const float q4[4] = {q.x, q.y, q.z, q.w};
        int32_t o4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v = __fmul_rn(__int2float_rn((int32_t)r[4 * g + i] + b4[i]), q4[i]);
            if (kOqf) v = __fmul_rn(v, oqf);                           // (a ReLU in front of a positive O_QF commutes with it)
            int32_t o;
            if (!kFused && kOut != 1) {
                // negative values end at 0 either way (unsigned saturation), so no sign handling
                o = __float_as_int(__fadd_rz(__fadd_rz(v, 0.5f), kMagic)) - kMagicBits;
            } else if (kFused && kRelu1) {
                o = __float_as_int(__fadd_rz(__fadd_rz(v, 0.5f), kMagic)) - k_pos;
                if (v < 0.0f) o = kMagicBits - k_pos;                 // ReLU: the convolution contributes 0
            } else {
                const int32_t wb = __float_as_int(__fadd_rz(__fadd_rz(fabsf(v), 0.5f), kMagic));
                o = wb - (kFused ? k_pos : kMagicBits);
                if (v < 0.0f) o = (kFused ? k_neg : kMagicBits) - wb;
            }
            if (kFused) o = dp4a_u8(ew[g], 1 << (8 * i), o);
            o4[i] = o;
        }
        if (kOut == 1) ow[g] = pack_sat_s8(o4[1], o4[0], pack_sat_s8(o4[3], o4[2], 0u));
        else {
            ow[g] = pack_sat_u8(o4[1], o4[0], pack_sat_u8(o4[3], o4[2], 0u));
            if (kOut == 2) ow[g] = clamp_bytes_127(ow[g]);
        }
    }
    *p0 = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    *p1 = make_uint4(ow[4], ow[5], ow[6], ow[7]);
}

}  // namespace b200
