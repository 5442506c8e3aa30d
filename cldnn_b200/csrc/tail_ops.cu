// The bandwidth-bound tail of the convolution path: pooling, fully_connected
// (reference order), softmax, eltwise, reorder, lrn and standalone activation.
// The *_ref kernels take any layout through pitches; pooling_i8_byxf is the
// feature-innermost fast path with 16-byte accesses per lane.
#include <cuda_fp16.h>
#include "engine.hpp"

namespace b200 {

static inline int grid_for(int64_t total, int threads, const cldnn_b200_ctx_impl* ctx)
{
    int64_t blocks = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)ctx->prop.multiProcessorCount * 16;
    if (blocks > cap) blocks = cap;
    return blocks < 1 ? 1 : (int)blocks;
}

// ---------------------------------------------------------------------------------
// pooling, any layout.  int8: cl_kernels/pooling_gpu_int8_ref.cl:35-131;
// float: cl_kernels/pooling_gpu_ref.cl:36-201.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pool_divisor(const cldnn_b200_pool_params& p, int ox, int oy, uint32_t n)
{
    if (p.div_mode == CLDNN_B200_DIV_DYNAMIC) return n ? n : 1u;
    if (p.div_mode == CLDNN_B200_DIV_DYNAMIC_WITH_PADDING) {
        const int hend = min(oy + p.size_y, p.in.y + p.pad_y), wend = min(ox + p.size_x, p.in.x + p.pad_x);
        const uint32_t d = (uint32_t)((hend - oy) * (wend - ox));
        return d ? d : 1u;
    }
    return (uint32_t)(p.size_x * p.size_y);
}

// element index -> coordinates, x innermost (planar layouts) or f innermost (byxf)
__device__ __forceinline__ void decode_bfyx(int64_t idx, int F, int Y, int X, bool f_inner, int& b, int& f, int& y, int& x)
{
    if (f_inner) { f = (int)(idx % F); int64_t t = idx / F; x = (int)(t % X); t /= X; y = (int)(t % Y); b = (int)(t / Y); }
    else { x = (int)(idx % X); int64_t t = idx / X; y = (int)(t % Y); t /= Y; f = (int)(t % F); b = (int)(t / F); }
}

__global__ void __launch_bounds__(256)
pooling_ref_kernel(const __grid_constant__ cldnn_b200_pool_params p, const void* in, void* out)
{
    const int64_t total = (int64_t)p.out.b * p.out.f * p.out.y * p.out.x;
    const bool int_in = is_int8(p.in.dtype);
    const bool f_inner = p.in.pf == 1 && p.out.pf == 1;             // consecutive threads follow the innermost dimension of the layout
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int b, f, y, x;
        decode_bfyx(idx, p.out.f, p.out.y, p.out.x, f_inner, b, f, y, x);
        const int ox = x * p.stride_x - p.pad_x, oy = y * p.stride_y - p.pad_y;
        if (ox + p.size_x < 0 || ox >= p.in.x || oy + p.size_y < 0 || oy >= p.in.y) continue;
        int32_t ri = p.mode == CLDNN_B200_POOL_MAX ? -128 : 0;
        float rf = p.mode == CLDNN_B200_POOL_MAX ? (p.in.dtype == CLDNN_B200_F16 ? -65504.0f : -3.402823466e38f) : 0.0f;
        uint32_t n = 0;
        for (int j = 0; j < p.size_y; ++j) {
            const int iy = oy + j; if (iy < 0 || iy >= p.in.y) continue;
            for (int i = 0; i < p.size_x; ++i) {
                const int ix = ox + i; if (ix < 0 || ix >= p.in.x) continue;
                const int64_t ii = tidx(p.in, b, f, iy, ix);
                if (int_in) { const int32_t v = load_as_int(in, p.in.dtype, ii); ri = p.mode == CLDNN_B200_POOL_MAX ? max(ri, v) : ri + v; }
                else { const float v = load_as_float(in, p.in.dtype, ii); rf = p.mode == CLDNN_B200_POOL_MAX ? fmaxf(rf, v) : __fadd_rn(rf, v); }
                ++n;
            }
        }
        const uint32_t div = pool_divisor(p, ox, oy, n);
        const int64_t oi = tidx(p.out, b, f, y, x);
        if (int_in) {
            if (p.mode == CLDNN_B200_POOL_AVG) ri = (int32_t)round_half_away(__fdiv_rn((float)ri, (float)div));
            if (p.out.dtype == CLDNN_B200_U8) ((uint8_t*)out)[oi] = (uint8_t)act_int(p.act, (int32_t)(uint8_t)ri, p.act_m, p.act_n);
            else if (p.out.dtype == CLDNN_B200_I8) ((int8_t*)out)[oi] = (int8_t)act_int(p.act, (int32_t)(int8_t)ri, p.act_m, p.act_n);
            else store_sat_int(out, p.out.dtype, oi, act_int(p.act, ri, p.act_m, p.act_n));
        } else {
            if (p.mode == CLDNN_B200_POOL_AVG) rf = __fdiv_rn(rf, (float)div);
            store_sat_float(out, p.out.dtype, oi, act_float(p.act, rf, p.act_m, p.act_n));
        }
    }
}

static bool pooling_ref_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_pool_params*)vp;
    return p.size_x >= 1 && p.size_y >= 1 && p.stride_x >= 1 && p.stride_y >= 1 && p.in.f == p.out.f && p.in.b == p.out.b;
}
static int one_tune(const void*) { return 1; }

static int32_t pooling_ref_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_pool_params p = *(const cldnn_b200_pool_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "pooling_ref: input and output are required");
    const void* in = a->input0; void* o = a->output;
    const int grid = grid_for((int64_t)p.out.b * p.out.f * p.out.y * p.out.x, 256, ctx);
    out->fn = [p, in, o, grid](cudaStream_t s) { pooling_ref_kernel<<<grid, 256, 0, s>>>(p, in, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_pooling_ref = {"pooling_ref", sizeof(cldnn_b200_pool_params), pooling_ref_supports, one_tune, nullptr, pooling_ref_prepare};

// ---------------------------------------------------------------------------------
// pooling, 8-bit, feature-innermost (byxf) fast path: each thread owns 16
// consecutive features of one output pixel and moves them with one 128-bit
// load per window tap and one 128-bit store.  Same arithmetic as
// pooling_gpu_int8_ref.cl.
// ---------------------------------------------------------------------------------
template <bool kUnsigned>
__device__ __forceinline__ void unpack16(const uint4& v, int32_t (&e)[16])
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t byte = (w[i >> 2] >> ((i & 3) * 8)) & 0xffu;
        e[i] = kUnsigned ? (int32_t)byte : (int32_t)(int8_t)byte;
    }
}

// Item walk of the grid-stride loops over (batch, y, x, feature vector): the first item and the stride are
// decomposed once, every later item follows by digit-wise addition with carries (a division by a run-time
// divisor costs more instructions than the pooling of one item).
struct ItemWalk {
    int f, x, y, b, sf, sx, sy, sb, nf, nx, ny;
    __device__ __forceinline__ void init(uint32_t first, uint32_t stride, int fv, int X, int Y)
    {
        nf = fv; nx = X; ny = Y;
        f = (int)(first % (uint32_t)fv); uint32_t t = first / (uint32_t)fv;
        x = (int)(t % (uint32_t)X); t /= (uint32_t)X; y = (int)(t % (uint32_t)Y); b = (int)(t / (uint32_t)Y);
        sf = (int)(stride % (uint32_t)fv); t = stride / (uint32_t)fv;
        sx = (int)(t % (uint32_t)X); t /= (uint32_t)X; sy = (int)(t % (uint32_t)Y); sb = (int)(t / (uint32_t)Y);
    }
    __device__ __forceinline__ void next()
    {
        f += sf; int c = f >= nf ? 1 : 0; f -= c ? nf : 0;
        x += sx + c; c = x >= nx ? 1 : 0; x -= c ? nx : 0;
        y += sy + c; c = y >= ny ? 1 : 0; y -= c ? ny : 0;
        b += sb + c;
    }
};

// Running maximum of four packed bytes kept as two words of 16-bit lanes, for the three-input 16-bit-pair maximum of
// the hardware: the odd bytes are compared through the raw word (the upper byte of a lane decides, the lower byte is
// ignored at the end), the even bytes are moved into the upper bytes of the lanes first.
template <bool kUnsigned>
struct ByteMax {
    uint32_t odd = kUnsigned ? 0u : 0x80008000u, even = kUnsigned ? 0u : 0x80008000u;
    static __device__ __forceinline__ uint32_t up(uint32_t w) { return __byte_perm(w, 0u, 0x2404); }    // bytes 0, 2 -> bytes 1, 3
    static __device__ __forceinline__ uint32_t max3(uint32_t a, uint32_t b, uint32_t c) { return kUnsigned ? __vimax3_u16x2(a, b, c) : __vimax3_s16x2(a, b, c); }
    __device__ __forceinline__ void add3(uint32_t a, uint32_t b, uint32_t c)
    {
        odd = max3(odd, max3(a, b, c), odd);
        even = max3(even, max3(up(a), up(b), up(c)), even);
    }
    // relu: signed bytes, negative maxima become 0
    __device__ __forceinline__ uint32_t result(bool relu) const
    {
        uint32_t o = odd, e = even;
        if (!kUnsigned && relu) { o = __vimax3_s16x2_relu(o, o, o); e = __vimax3_s16x2_relu(e, e, e); }
        return __byte_perm(o, e, 0x3715);                                                              // e.b1, o.b1, e.b3, o.b3
    }
};

template <bool kUnsignedIn>
__global__ void __launch_bounds__(256)
pooling_i8_byxf_kernel(const __grid_constant__ cldnn_b200_pool_params p, const uint8_t* __restrict__ in, uint8_t* __restrict__ out)
{
    const int fv = p.in.f / 16;
    const int64_t total = (int64_t)p.out.b * p.out.y * p.out.x * fv;
    const bool fast_max = p.mode == CLDNN_B200_POOL_MAX && (p.act == CLDNN_B200_ACT_NONE || p.act == CLDNN_B200_ACT_RELU);
    // (32-bit index arithmetic: a 64-bit division costs more instructions than the pooling itself; the host admits < 2^31 items)
    ItemWalk it; it.init(blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x, fv, p.out.x, p.out.y);
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < (uint32_t)total; idx += gridDim.x * blockDim.x, it.next()) {
        const int f16 = it.f, x = it.x, y = it.y, b = it.b;
        const int ox = x * p.stride_x - p.pad_x, oy = y * p.stride_y - p.pad_y;
        if (ox + p.size_x < 0 || ox >= p.in.x || oy + p.size_y < 0 || oy >= p.in.y) continue;
        if (fast_max) {
            // maximum of the valid taps on packed bytes, no unpacking to 32 bits: the stored bits are the bits of the
            // largest input (the conversion to the output type wraps), ReLU on a signed output is one more max
            const int j0 = max(0, -oy), j1 = min(p.size_y, p.in.y - oy), i0 = max(0, -ox), i1 = min(p.size_x, p.in.x - ox);
            const uint8_t* src = in + tidx(p.in, b, f16 * 16, oy, ox);
            ByteMax<kUnsignedIn> bm[4];
            if (p.size_x == 3 && p.size_y == 3 && j0 < j1 && i0 < i1) {
                // 3x3 window: taps outside the input are replaced by the nearest valid tap (a repeated element does not
                // change a maximum), so the nine loads carry no branches and are all in flight together
                uint4 v[9];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int64_t ro = (int64_t)min(max(j, j0), j1 - 1) * p.in.py;
#pragma unroll
                    for (int i = 0; i < 3; ++i)
                        v[j * 3 + i] = __ldg((const uint4*)(src + ro + (int64_t)min(max(i, i0), i1 - 1) * p.in.px));
                }
#pragma unroll
                for (int k = 0; k < 9; k += 3) {
                    bm[0].add3(v[k].x, v[k + 1].x, v[k + 2].x); bm[1].add3(v[k].y, v[k + 1].y, v[k + 2].y);
                    bm[2].add3(v[k].z, v[k + 1].z, v[k + 2].z); bm[3].add3(v[k].w, v[k + 1].w, v[k + 2].w);
                }
            } else
            for (int j = j0; j < j1; ++j) {
#pragma unroll 3
                for (int i = i0; i < i1; ++i) {
                    const uint4 v = __ldg((const uint4*)(src + (int64_t)j * p.in.py + (int64_t)i * p.in.px));
                    bm[0].add3(v.x, v.x, v.x); bm[1].add3(v.y, v.y, v.y); bm[2].add3(v.z, v.z, v.z); bm[3].add3(v.w, v.w, v.w);
                }
            }
            const bool relu = p.act == CLDNN_B200_ACT_RELU && p.out.dtype == CLDNN_B200_I8;
            const uint4 m = make_uint4(bm[0].result(relu), bm[1].result(relu), bm[2].result(relu), bm[3].result(relu));
            *(uint4*)(out + tidx(p.out, b, f16 * 16, y, x)) = m;
            continue;
        }
        int32_t r[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = p.mode == CLDNN_B200_POOL_MAX ? -128 : 0;
        uint32_t n = 0;
        const int taps = p.size_x * p.size_y;
        if (p.mode == CLDNN_B200_POOL_AVG && ox >= 0 && oy >= 0 && ox + p.size_x <= p.in.x && oy + p.size_y <= p.in.y && taps <= 256) {
            // whole window inside the input: sums of at most 256 bytes fit 16-bit lanes, so two masks and two additions
            // take a word of four bytes (signed bytes are summed as byte + 128 and the 128s taken out at the end);
            // eight taps are loaded per batch so that a long window (a global average) is not one load latency per tap
            const uint8_t* src = in + tidx(p.in, b, f16 * 16, oy, ox);
            uint32_t a[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
            int ti = 0, tj = 0;
            for (int t0 = 0; t0 < taps; t0 += 8) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    v[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (t0 + u < taps) {
                        v[u] = __ldg((const uint4*)(src + (int64_t)tj * p.in.py + (int64_t)ti * p.in.px));
                        if (!kUnsignedIn) { v[u].x ^= 0x80808080u; v[u].y ^= 0x80808080u; v[u].z ^= 0x80808080u; v[u].w ^= 0x80808080u; }
                    }
                    if (++ti == p.size_x) { ti = 0; ++tj; }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) { a[2 * k] += w[k] & 0x00ff00ffu; a[2 * k + 1] += (w[k] >> 8) & 0x00ff00ffu; }
                }
            }
            n = (uint32_t)taps;
            const int32_t off = kUnsignedIn ? 0 : 128 * taps;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                r[4 * k + 0] = (int32_t)(a[2 * k] & 0xffffu) - off;     r[4 * k + 1] = (int32_t)(a[2 * k + 1] & 0xffffu) - off;
                r[4 * k + 2] = (int32_t)(a[2 * k] >> 16) - off;         r[4 * k + 3] = (int32_t)(a[2 * k + 1] >> 16) - off;
            }
        } else
        for (int j = 0; j < p.size_y; ++j) {
            const int iy = oy + j; if (iy < 0 || iy >= p.in.y) continue;
            for (int i = 0; i < p.size_x; ++i) {
                const int ix = ox + i; if (ix < 0 || ix >= p.in.x) continue;
                const uint4 v = __ldg((const uint4*)(in + tidx(p.in, b, f16 * 16, iy, ix)));
                int32_t e[16]; unpack16<kUnsignedIn>(v, e);
#pragma unroll
                for (int k = 0; k < 16; ++k) r[k] = p.mode == CLDNN_B200_POOL_MAX ? max(r[k], e[k]) : r[k] + e[k];
                ++n;
            }
        }
        const float div = (float)pool_divisor(p, ox, oy, n);
        uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            int32_t v = r[k];
            if (p.mode == CLDNN_B200_POOL_AVG) v = (int32_t)round_half_away(__fdiv_rn((float)v, div));
            // convert_char / convert_uchar wrap, then the activation runs on the 8-bit value
            v = p.out.dtype == CLDNN_B200_U8 ? (int32_t)(uint8_t)v : (int32_t)(int8_t)v;
            v = act_int(p.act, v, p.act_m, p.act_n);
            w[k >> 2] |= ((uint32_t)v & 0xffu) << ((k & 3) * 8);
        }
        *(uint4*)(out + tidx(p.out, b, f16 * 16, y, x)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

static bool pooling_i8_byxf_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_pool_params*)vp;
    if (!pooling_ref_supports(vp)) return false;
    if (!is_int8(p.in.dtype) || !is_int8(p.out.dtype)) return false;
    if (p.in.pf != 1 || p.out.pf != 1 || p.in.f % 16) return false;
    const int64_t pitches[] = {p.in.px, p.in.py, p.in.pb, p.in.offset, p.out.px, p.out.py, p.out.pb, p.out.offset};
    for (int64_t v : pitches) if (v % 16) return false;
    if ((int64_t)p.out.b * p.out.y * p.out.x * (p.in.f / 16) >= 0x7fffffffLL) return false;      // 32-bit item index
    return true;
}

static int32_t pooling_i8_byxf_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_pool_params p = *(const cldnn_b200_pool_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "pooling_i8_byxf: input and output are required");
    if (((uintptr_t)a->input0 | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "pooling_i8_byxf: buffers must be 16-byte aligned");
    const uint8_t* in = (const uint8_t*)a->input0; uint8_t* o = (uint8_t*)a->output;
    const int grid = grid_for((int64_t)p.out.b * p.out.y * p.out.x * (p.in.f / 16), 256, ctx);
    const bool uns = p.in.dtype == CLDNN_B200_U8;
    out->fn = [p, in, o, grid, uns](cudaStream_t s) {
        if (uns) pooling_i8_byxf_kernel<true><<<grid, 256, 0, s>>>(p, in, o);
        else pooling_i8_byxf_kernel<false><<<grid, 256, 0, s>>>(p, in, o);
        return cudaGetLastError();
    };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_pooling_i8_byxf = {"pooling_i8_byxf", sizeof(cldnn_b200_pool_params), pooling_i8_byxf_supports, one_tune, nullptr, pooling_i8_byxf_prepare};

// ---------------------------------------------------------------------------------
// pooling, fp16, feature-innermost (byxf): each thread owns 8 consecutive features of one
// output pixel, one 128-bit load per window tap and one 128-bit store; the maximum on
// packed halves, the average accumulated in fp32.  Same arithmetic as pooling_gpu_ref.cl
// (its half accumulator for the average is replaced by a float one: tolerance parity).
// ---------------------------------------------------------------------------------
template <int S>
__device__ __forceinline__ void pool_max_clamped(const __half* src, int64_t px, int64_t py, int i0, int i1, int j0, int j1, __half2 (&m)[4])
{
    uint4 v[S * S];
#pragma unroll
    for (int j = 0; j < S; ++j) {
        const int64_t ro = (int64_t)min(max(j, j0), j1 - 1) * py;
#pragma unroll
        for (int i = 0; i < S; ++i)
            v[j * S + i] = __ldg(reinterpret_cast<const uint4*>(src + ro + (int64_t)min(max(i, i0), i1 - 1) * px));
    }
#pragma unroll
    for (int t = 0; t < S * S; ++t) {
        const __half2* h = reinterpret_cast<const __half2*>(&v[t]);
#pragma unroll
        for (int k = 0; k < 4; ++k) m[k] = __hmax2(m[k], h[k]);
    }
}

__global__ void __launch_bounds__(256)
pooling_f16_byxf_kernel(const __grid_constant__ cldnn_b200_pool_params p, const __half* __restrict__ in, __half* __restrict__ out)
{
    const int fv = p.in.f / 8;
    const int64_t total = (int64_t)p.out.b * p.out.y * p.out.x * fv;
    const bool is_max = p.mode == CLDNN_B200_POOL_MAX;
    ItemWalk it; it.init(blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x, fv, p.out.x, p.out.y);
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < (uint32_t)total; idx += gridDim.x * blockDim.x, it.next()) {   // < 2^31 items (host check)
        const int f8 = it.f, x = it.x, y = it.y, b = it.b;
        const int ox = x * p.stride_x - p.pad_x, oy = y * p.stride_y - p.pad_y;
        if (ox + p.size_x < 0 || ox >= p.in.x || oy + p.size_y < 0 || oy >= p.in.y) continue;
        const int j0 = max(0, -oy), j1 = min(p.size_y, p.in.y - oy), i0 = max(0, -ox), i1 = min(p.size_x, p.in.x - ox);
        const __half* src = in + tidx(p.in, b, f8 * 8, oy, ox);
        const __half2 lowest = __half2half2(__ushort_as_half((unsigned short)0xfbffu));      // -65504, the reference's HALF_MIN start value
        __half2 m[4] = {lowest, lowest, lowest, lowest};
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint32_t n = 0;
        const bool sq3 = p.size_x == 3 && p.size_y == 3, sq2 = p.size_x == 2 && p.size_y == 2;
        if (is_max && (sq3 || sq2) && j0 < j1 && i0 < i1) {
            // small square window: taps outside the input are replaced by the nearest valid tap (a repeated element
            // does not change a maximum), so the loads carry no branches and are all in flight together
            if (sq3) pool_max_clamped<3>(src, p.in.px, p.in.py, i0, i1, j0, j1, m);
            else pool_max_clamped<2>(src, p.in.px, p.in.py, i0, i1, j0, j1, m);
        } else
        for (int j = j0; j < j1; ++j) {
            for (int i = i0; i < i1; ++i) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)j * p.in.py + (int64_t)i * p.in.px));
                const __half2* h = reinterpret_cast<const __half2*>(&v);
                if (is_max) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) m[k] = __hmax2(m[k], h[k]);
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); acc[2 * k] += f.x; acc[2 * k + 1] += f.y; }
                }
                ++n;
            }
        }
        if (is_max && (p.act == CLDNN_B200_ACT_NONE || p.act == CLDNN_B200_ACT_RELU)) {
            // the maximum is one of the inputs: stored as it is (ReLU: one more packed maximum), no trip through fp32
            if (p.act == CLDNN_B200_ACT_RELU) {
                const __half2 zero = __float2half2_rn(0.0f);
#pragma unroll
                for (int k = 0; k < 4; ++k) m[k] = __hmax2(m[k], zero);
            }
            *reinterpret_cast<uint4*>(out + tidx(p.out, b, f8 * 8, y, x)) = *reinterpret_cast<const uint4*>(m);
            continue;
        }
        float r[8];
        if (is_max) {
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(m[k]); r[2 * k] = f.x; r[2 * k + 1] = f.y; }
        } else {
            const float div = (float)pool_divisor(p, ox, oy, n);
#pragma unroll
            for (int k = 0; k < 8; ++k) r[k] = __fdiv_rn(acc[k], div);
        }
        __half2 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            o[k] = __floats2half2_rn(act_float(p.act, r[2 * k], p.act_m, p.act_n), act_float(p.act, r[2 * k + 1], p.act_m, p.act_n));
        *reinterpret_cast<uint4*>(out + tidx(p.out, b, f8 * 8, y, x)) = *reinterpret_cast<const uint4*>(o);
    }
}

static bool pooling_f16_byxf_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_pool_params*)vp;
    if (!pooling_ref_supports(vp)) return false;
    if (p.in.dtype != CLDNN_B200_F16 || p.out.dtype != CLDNN_B200_F16) return false;
    if (p.in.pf != 1 || p.out.pf != 1 || p.in.f % 8) return false;
    const int64_t pitches[] = {p.in.px, p.in.py, p.in.pb, p.in.offset, p.out.px, p.out.py, p.out.pb, p.out.offset};
    for (int64_t v : pitches) if (v % 8) return false;
    if ((int64_t)p.out.b * p.out.y * p.out.x * (p.in.f / 8) >= 0x7fffffffLL) return false;       // 32-bit item index
    return true;
}

static int32_t pooling_f16_byxf_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_pool_params p = *(const cldnn_b200_pool_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "pooling_f16_byxf: input and output are required");
    if (((uintptr_t)a->input0 | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "pooling_f16_byxf: buffers must be 16-byte aligned");
    const __half* in = (const __half*)a->input0; __half* o = (__half*)a->output;
    const int grid = grid_for((int64_t)p.out.b * p.out.y * p.out.x * (p.in.f / 8), 256, ctx);
    out->fn = [p, in, o, grid](cudaStream_t s) { pooling_f16_byxf_kernel<<<grid, 256, 0, s>>>(p, in, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_pooling_f16_byxf = {"pooling_f16_byxf", sizeof(cldnn_b200_pool_params), pooling_f16_byxf_supports, one_tune, nullptr, pooling_f16_byxf_prepare};

// ---------------------------------------------------------------------------------
// fully_connected in the reference's order (cl_kernels/fully_connected_gpu_bfyx_ref.cl:18-84):
// one warp per output, lanes stride the reduction, shuffle-reduce (integer sums
// are order-independent; float sums are tolerance-checked).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
fc_ref_kernel(const __grid_constant__ cldnn_b200_fc_params p, const void* in, const void* w, const void* bias,
              const float* quant, const float* calib, void* out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t total = (int64_t)p.out.b * p.out.f;
    const int K = p.in.f * p.in.y * p.in.x;
    for (int64_t bo = warp; bo < total; bo += nwarps) {
        const int b = (int)(bo / p.out.f), o = (int)(bo % p.out.f);
        int32_t acc_i = 0; float acc_f = 0.f;
        for (int k = lane; k < K; k += 32) {
            const int x = k % p.in.x, y = (k / p.in.x) % p.in.y, f = k / (p.in.x * p.in.y);
            const int64_t ii = tidx(p.in, b, f, y, x);
            const int64_t wi = p.w_offset + (int64_t)o * p.w_po + (int64_t)f * p.w_pi + (int64_t)y * p.w_py + (int64_t)x * p.w_px;
            if (p.quantization) acc_i += load_as_int(in, p.in.dtype, ii) * load_as_int(w, p.w_dtype, wi);
            else acc_f += load_as_float(in, p.in.dtype, ii) * load_as_float(w, p.w_dtype, wi);
        }
#pragma unroll
        for (int s = 16; s; s >>= 1) { acc_i += __shfl_xor_sync(0xffffffffu, acc_i, s); acc_f += __shfl_xor_sync(0xffffffffu, acc_f, s); }
        if (lane) continue;
        const int64_t oi = tidx(p.out, b, o, 0, 0);
        if (p.quantization) {
            int32_t r = acc_i;
            if (p.bias_dtype != CLDNN_B200_NONE) {
                float t = __fmul_rn(__fmul_rn((float)acc_i, quant[o]), p.i_qf);
                t = __fadd_rn(t, load_as_float(bias, p.bias_dtype, o));
                t = __fmul_rn(t, p.calibration ? calib[o] : p.o_qf);
                r = sat_i32_from_float(round_half_away(t), -128, 127);
            } else r = min(127, max(-128, r));
            store_sat_int(out, p.out.dtype, oi, act_int(p.act, r, p.act_m, p.act_n));
        } else {
            float v = acc_f;
            if (p.bias_dtype != CLDNN_B200_NONE) v += load_as_float(bias, p.bias_dtype, o);
            store_sat_float(out, p.out.dtype, oi, act_float(p.act, v, p.act_m, p.act_n));
        }
    }
}
static bool fc_ref_supports(const void* vp) { const auto& p = *(const cldnn_b200_fc_params*)vp; return p.in.b == p.out.b && p.out.f >= 1; }
static int32_t fc_ref_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_fc_params p = *(const cldnn_b200_fc_params*)vp;
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "fc_ref: input, output and weights are required");
    if (p.quantization && p.bias_dtype != CLDNN_B200_NONE && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "fc_ref: quantization factors missing");
    if (p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "fc_ref: calibration factors missing");
    const void* in = a->input0; const void* w = a->weights; const void* bias = a->bias; void* o = a->output;
    const float* q = a->weights_quantization_factors; const float* c = a->output_calibration_factors;
    const int grid = grid_for((int64_t)p.out.b * p.out.f * 32, 256, ctx);
    out->fn = [=](cudaStream_t s) { fc_ref_kernel<<<grid, 256, 0, s>>>(p, in, w, bias, q, c, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_fc_ref = {"fc_ref", sizeof(cldnn_b200_fc_params), fc_ref_supports, one_tune, nullptr, fc_ref_prepare};

// ---------------------------------------------------------------------------------
// softmax over features (cl_kernels/softmax_gpu_ref.cl:22-58): one warp per
// (b, y, x) row; max, sum and normalise with warp shuffles, float accumulation.
// ---------------------------------------------------------------------------------
// set index + position inside the set -> coordinates, by the scope of normalisation (api/C/softmax.h:34-40)
__device__ __forceinline__ void softmax_coords(const cldnn_b200_softmax_params& p, int64_t set, int i, int& b, int& f, int& y, int& x)
{
    const int F = p.in.f, Y = p.in.y, X = p.in.x;
    switch (p.dimension) {
    case CLDNN_B200_SOFTMAX_X:   x = i; y = (int)(set % Y); f = (int)((set / Y) % F); b = (int)(set / ((int64_t)Y * F)); break;
    case CLDNN_B200_SOFTMAX_Y:   y = i; x = (int)(set % X); f = (int)((set / X) % F); b = (int)(set / ((int64_t)X * F)); break;
    case CLDNN_B200_SOFTMAX_FYX: x = i % X; y = (i / X) % Y; f = i / (X * Y); b = (int)set; break;
    default:                     f = i; x = (int)(set % X); y = (int)((set / X) % Y); b = (int)(set / ((int64_t)X * Y)); break;
    }
}
__host__ __device__ inline int64_t softmax_len(const cldnn_b200_softmax_params& p)
{
    switch (p.dimension) {
    case CLDNN_B200_SOFTMAX_X: return p.in.x;
    case CLDNN_B200_SOFTMAX_Y: return p.in.y;
    case CLDNN_B200_SOFTMAX_FYX: return (int64_t)p.in.f * p.in.y * p.in.x;
    default: return p.in.f;
    }
}

__global__ void __launch_bounds__(256)
softmax_kernel(const __grid_constant__ cldnn_b200_softmax_params p, const void* in, void* out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int len = (int)softmax_len(p);
    const int64_t sets = len > 0 ? ((int64_t)p.in.b * p.in.f * p.in.y * p.in.x) / len : 0;
    for (int64_t r = warp; r < sets; r += nwarps) {
        int b, f, y, x;
        float mx = -3.402823466e38f;
        for (int i = lane; i < len; i += 32) { softmax_coords(p, r, i, b, f, y, x); mx = fmaxf(mx, load_as_float(in, p.in.dtype, tidx(p.in, b, f, y, x))); }
#pragma unroll
        for (int s = 16; s; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        float den = 0.f;
        for (int i = lane; i < len; i += 32) { softmax_coords(p, r, i, b, f, y, x); den += expf(load_as_float(in, p.in.dtype, tidx(p.in, b, f, y, x)) - mx); }
#pragma unroll
        for (int s = 16; s; s >>= 1) den += __shfl_xor_sync(0xffffffffu, den, s);
        for (int i = lane; i < len; i += 32) {
            softmax_coords(p, r, i, b, f, y, x);
            const float e = expf(load_as_float(in, p.in.dtype, tidx(p.in, b, f, y, x)) - mx);
            store_sat_float(out, p.out.dtype, tidx(p.out, b, f, y, x), __fdiv_rn(e, den));
        }
    }
}
// One block per row for long rows (classification heads): every thread keeps its elements in registers, two block
// reductions (max, sum) through shared memory, one pass over memory in, one out.
constexpr int kSoftmaxPerThread = 8;
__global__ void __launch_bounds__(256)
softmax_row_kernel(const __grid_constant__ cldnn_b200_softmax_params p, const void* in, void* out)
{
    __shared__ float red[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t rows = (int64_t)p.in.b * p.in.y * p.in.x;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int x = (int)(r % p.in.x), y = (int)((r / p.in.x) % p.in.y), b = (int)(r / ((int64_t)p.in.x * p.in.y));
        float v[kSoftmaxPerThread];
        float mx = -3.402823466e38f;
#pragma unroll
        for (int i = 0; i < kSoftmaxPerThread; ++i) {
            const int f = threadIdx.x + i * 256;
            v[i] = f < p.in.f ? load_as_float(in, p.in.dtype, tidx(p.in, b, f, y, x)) : -3.402823466e38f;
            mx = fmaxf(mx, v[i]);
        }
#pragma unroll
        for (int s = 16; s; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        mx = red[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
        __syncthreads();
        float den = 0.f;
#pragma unroll
        for (int i = 0; i < kSoftmaxPerThread; ++i) {
            const int f = threadIdx.x + i * 256;
            v[i] = f < p.in.f ? expf(v[i] - mx) : 0.f;
        }
        // the reference adds the exponentials of one row in feature order on one work-item; a tree sum differs from it in
        // the last bits only, inside the tolerance softmax is compared with
#pragma unroll
        for (int i = 0; i < kSoftmaxPerThread; ++i) den += v[i];
#pragma unroll
        for (int s = 16; s; s >>= 1) den += __shfl_xor_sync(0xffffffffu, den, s);
        if (lane == 0) red[warp] = den;
        __syncthreads();
        den = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) den += red[w];
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kSoftmaxPerThread; ++i) {
            const int f = threadIdx.x + i * 256;
            if (f < p.in.f) store_sat_float(out, p.out.dtype, tidx(p.out, b, f, y, x), __fdiv_rn(v[i], den));
        }
    }
}
static bool softmax_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_softmax_params*)vp;
    return is_fp(p.in.dtype) && is_fp(p.out.dtype) && p.in.f == p.out.f && p.in.x == p.out.x && p.in.y == p.out.y && p.in.b == p.out.b &&
           p.dimension >= CLDNN_B200_SOFTMAX_F && p.dimension <= CLDNN_B200_SOFTMAX_FYX && softmax_len(p) < 0x7fffffffLL;
}
static int32_t softmax_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_softmax_params p = *(const cldnn_b200_softmax_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "softmax: input and output are required");
    const void* in = a->input0; void* o = a->output;
    const int64_t len = softmax_len(p);
    const int64_t sets = len > 0 ? ((int64_t)p.in.b * p.in.f * p.in.y * p.in.x) / len : 0;
    const int grid = grid_for(sets * 32, 256, ctx);
    // the block-per-row kernel normalises over f; over a 1x1 map the whole-image scope is the same thing
    const bool over_f = p.dimension == CLDNN_B200_SOFTMAX_F || (p.dimension == CLDNN_B200_SOFTMAX_FYX && p.in.x == 1 && p.in.y == 1);
    const int64_t rows = (int64_t)p.in.b * p.in.y * p.in.x;
    const bool by_row = over_f && p.in.f >= 256 && p.in.f <= 256 * kSoftmaxPerThread && rows <= (int64_t)ctx->prop.multiProcessorCount * 32;
    const int row_grid = (int)(rows < 1 ? 1 : rows);
    out->fn = [=](cudaStream_t s) {
        if (by_row) softmax_row_kernel<<<row_grid, 256, 0, s>>>(p, in, o);
        else softmax_kernel<<<grid, 256, 0, s>>>(p, in, o);
        return cudaGetLastError();
    };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_softmax = {"softmax", sizeof(cldnn_b200_softmax_params), softmax_supports, one_tune, nullptr, softmax_prepare};

// ---------------------------------------------------------------------------------
// eltwise (cl_kernels/generic_eltwise_ref.cl:198-330)
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
eltwise_ref_kernel(const __grid_constant__ cldnn_b200_eltwise_params p, const void* in0, const void* in1, const float* calib, void* out)
{
    const int64_t total = (int64_t)p.out.b * p.out.f * p.out.y * p.out.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        // iterate in the output's memory order of its innermost axis
        int b, f, y, x;
        if (p.out.pf == 1) { f = (int)(idx % p.out.f); int64_t t = idx / p.out.f; x = (int)(t % p.out.x); t /= p.out.x; y = (int)(t % p.out.y); b = (int)(t / p.out.y); }
        else { x = (int)(idx % p.out.x); int64_t t = idx / p.out.x; y = (int)(t % p.out.y); t /= p.out.y; f = (int)(t % p.out.f); b = (int)(t / p.out.f); }
        const int64_t i0 = tidx(p.in0, b % p.in0.b, f % p.in0.f, ((int64_t)y * p.stride_y0) % p.in0.y, ((int64_t)x * p.stride_x0) % p.in0.x);
        const int64_t i1 = tidx(p.in1, b % p.in1.b, f % p.in1.f, ((int64_t)y * p.stride_y1) % p.in1.y, ((int64_t)x * p.stride_x1) % p.in1.x);
        const int64_t oi = tidx(p.out, b, f, y, x);
        if (p.quantization) {
            const int32_t a = load_as_int(in0, p.in0.dtype, i0), c = load_as_int(in1, p.in1.dtype, i1);
            int32_t r;
            switch (p.mode) {
            case CLDNN_B200_ELTW_SUB: r = a - c; break;
            case CLDNN_B200_ELTW_MAX: r = max(a, c); break;
            case CLDNN_B200_ELTW_MIN: r = min(a, c); break;
            case CLDNN_B200_ELTW_PROD: r = a * c; break;
            default: r = a + c; break;
            }
            r = sat_i32_from_float(round_half_away(__fmul_rn((float)r, p.calibration ? calib[f] : p.o_qf)), -128, 127);
            store_sat_int(out, p.out.dtype, oi, act_int(p.act, r, p.act_m, p.act_n));
            continue;
        }
        const float a = load_as_float(in0, p.in0.dtype, i0), c = load_as_float(in1, p.in1.dtype, i1);
        float r;
        switch (p.mode) {
        case CLDNN_B200_ELTW_SUB: r = __fsub_rn(a, c); break;
        case CLDNN_B200_ELTW_MAX: r = fmaxf(a, c); break;
        case CLDNN_B200_ELTW_MIN: r = fminf(a, c); break;
        case CLDNN_B200_ELTW_PROD: r = __fmul_rn(a, c); break;
        default: r = __fadd_rn(a, c); break;
        }
        if (is_fp(p.out.dtype)) store_sat_float(out, p.out.dtype, oi, act_float(p.act, r, p.act_m, p.act_n));
        else store_sat_int(out, p.out.dtype, oi, act_int(p.act, (int32_t)r, p.act_m, p.act_n));
    }
}
static bool eltwise_supports(const void* vp) { const auto& p = *(const cldnn_b200_eltwise_params*)vp; return p.stride_x0 >= 1 && p.stride_y0 >= 1 && p.stride_x1 >= 1 && p.stride_y1 >= 1; }
static int32_t eltwise_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_eltwise_params p = *(const cldnn_b200_eltwise_params*)vp;
    if (!a->input0 || !a->input1 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "eltwise_ref: two inputs and an output are required");
    if (p.quantization && p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "eltwise_ref: calibration factors missing");
    const void* i0 = a->input0; const void* i1 = a->input1; void* o = a->output; const float* c = a->output_calibration_factors;
    const int grid = grid_for((int64_t)p.out.b * p.out.f * p.out.y * p.out.x, 256, ctx);
    out->fn = [=](cudaStream_t s) { eltwise_ref_kernel<<<grid, 256, 0, s>>>(p, i0, i1, c, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_eltwise_ref = {"eltwise_ref", sizeof(cldnn_b200_eltwise_params), eltwise_supports, one_tune, nullptr, eltwise_prepare};

// ---------------------------------------------------------------------------------
// eltwise over equal dense layouts, 16 bytes per thread (the role of eltwise_simple_vload8.cl among the reference's kernels):
// both inputs and the output have the same sizes, pitches and element size, so the tensors are walked as flat arrays.
// 8-bit: the requantising form of generic_eltwise_ref.cl (integer operation, * O_QF or calibrations[f], round, saturate to
// char, activation, saturating store); fp16: the floating form.  Activations none / ReLU; features innermost when the
// factors are per feature.  Same results as eltwise_ref, element for element.
// ---------------------------------------------------------------------------------
template <bool kHalf>
__global__ void __launch_bounds__(256)
eltwise_vec_kernel(const __grid_constant__ cldnn_b200_eltwise_params p, const uint4* __restrict__ in0, const uint4* __restrict__ in1,
                   const float* __restrict__ calib, uint4* __restrict__ out, int64_t vectors, int32_t stored_f)
{
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vectors; v += (int64_t)gridDim.x * blockDim.x) {
        const uint4 a = in0[v], c = in1[v];
        uint4 r;
        if (kHalf) {
            const __half2* ah = reinterpret_cast<const __half2*>(&a); const __half2* ch = reinterpret_cast<const __half2*>(&c);
            __half2* rh = reinterpret_cast<__half2*>(&r);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 x = __half22float2(ah[i]), y = __half22float2(ch[i]);
                float2 z;
                switch (p.mode) {
                case CLDNN_B200_ELTW_SUB: z = make_float2(__fsub_rn(x.x, y.x), __fsub_rn(x.y, y.y)); break;
                case CLDNN_B200_ELTW_MAX: z = make_float2(fmaxf(x.x, y.x), fmaxf(x.y, y.y)); break;
                case CLDNN_B200_ELTW_MIN: z = make_float2(fminf(x.x, y.x), fminf(x.y, y.y)); break;
                case CLDNN_B200_ELTW_PROD: z = make_float2(__fmul_rn(x.x, y.x), __fmul_rn(x.y, y.y)); break;
                default: z = make_float2(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y)); break;
                }
                if (p.act == CLDNN_B200_ACT_RELU) { z.x = fmaxf(0.0f, z.x); z.y = fmaxf(0.0f, z.y); }
                rh[i] = __floats2half2_rn(z.x, z.y);
            }
        } else {
            const uint8_t* ab = reinterpret_cast<const uint8_t*>(&a); const uint8_t* cb = reinterpret_cast<const uint8_t*>(&c);
            uint8_t* rb = reinterpret_cast<uint8_t*>(&r);
            const int f0 = p.calibration ? (int)((v * 16) % stored_f) : 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int32_t x = p.in0.dtype == CLDNN_B200_U8 ? (int32_t)ab[i] : (int32_t)(int8_t)ab[i];
                const int32_t y = p.in1.dtype == CLDNN_B200_U8 ? (int32_t)cb[i] : (int32_t)(int8_t)cb[i];
                int32_t z;
                switch (p.mode) {
                case CLDNN_B200_ELTW_SUB: z = x - y; break;
                case CLDNN_B200_ELTW_MAX: z = max(x, y); break;
                case CLDNN_B200_ELTW_MIN: z = min(x, y); break;
                case CLDNN_B200_ELTW_PROD: z = x * y; break;
                default: z = x + y; break;
                }
                // a feature lane beyond the tensor's feature count (padding of the layout) has no factor: it stays what the operation gives on zeros
                const float factor = p.calibration ? (f0 + i < p.out.f ? calib[f0 + i] : 1.0f) : p.o_qf;
                z = sat_i32_from_float(round_half_away(__fmul_rn((float)z, factor)), -128, 127);
                if (p.act == CLDNN_B200_ACT_RELU) z = max(z, 0);
                rb[i] = p.out.dtype == CLDNN_B200_U8 ? (uint8_t)max(z, 0) : (uint8_t)(int8_t)z;
            }
        }
        out[v] = r;
    }
}
static bool same_dense(const cldnn_b200_tensor& a, const cldnn_b200_tensor& b)
{
    return a.b == b.b && a.f == b.f && a.y == b.y && a.x == b.x && a.pb == b.pb && a.pf == b.pf && a.py == b.py && a.px == b.px && a.offset == 0 && b.offset == 0;
}
// bytes of the tensor when it is one dense block (no padding between rows, images): 0 otherwise
static int64_t dense_elems(const cldnn_b200_tensor& t)
{
    if (t.pf == 1) return (t.py == t.px * t.x && t.pb == t.py * t.y && t.px >= t.f) ? t.pb * t.b : 0;        // byxf, features possibly padded
    if (t.px == 1) return (t.py == t.x && t.pf == t.py * t.y && t.pb == t.pf * t.f) ? t.pb * t.b : 0;          // bfyx
    return 0;
}
static bool eltwise_vec_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_eltwise_params*)vp;
    if (p.stride_x0 != 1 || p.stride_y0 != 1 || p.stride_x1 != 1 || p.stride_y1 != 1) return false;
    if (!same_dense(p.in0, p.out) || !same_dense(p.in1, p.out)) return false;
    if (p.act != CLDNN_B200_ACT_NONE && p.act != CLDNN_B200_ACT_RELU) return false;
    const bool half = p.in0.dtype == CLDNN_B200_F16 && p.in1.dtype == CLDNN_B200_F16 && p.out.dtype == CLDNN_B200_F16 && !p.quantization;
    const bool bytes = is_int8(p.in0.dtype) && is_int8(p.in1.dtype) && is_int8(p.out.dtype) && p.quantization;
    if (!half && !bytes) return false;
    const int64_t n = dense_elems(p.out);
    if (n <= 0 || (n * (half ? 2 : 1)) % 16) return false;
    if (bytes && p.calibration && (p.out.pf != 1 || p.out.px % 16)) return false;          // per-feature factors: 16 consecutive features per vector
    return true;
}
static int32_t eltwise_vec_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_eltwise_params p = *(const cldnn_b200_eltwise_params*)vp;
    if (!eltwise_vec_supports(vp)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "eltwise_byxf: equal dense layouts, strides 1, 8-bit requantising or fp16 form, NONE / ReLU only");
    if (!a->input0 || !a->input1 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "eltwise_byxf: two inputs and an output are required");
    if (p.quantization && p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "eltwise_byxf: calibration factors missing");
    if (((uintptr_t)a->input0 | (uintptr_t)a->input1 | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "eltwise_byxf: buffers must be 16-byte aligned");
    const bool half = p.in0.dtype == CLDNN_B200_F16;
    const int64_t vectors = dense_elems(p.out) * (half ? 2 : 1) / 16;
    const uint4* i0 = (const uint4*)a->input0; const uint4* i1 = (const uint4*)a->input1; uint4* o = (uint4*)a->output; const float* c = a->output_calibration_factors;
    const int32_t sf = (int32_t)(p.out.pf == 1 ? p.out.px : 1);
    const int grid = grid_for(vectors, 256, ctx);
    if (half) out->fn = [=](cudaStream_t s) { eltwise_vec_kernel<true><<<grid, 256, 0, s>>>(p, i0, i1, c, o, vectors, sf); return cudaGetLastError(); };
    else out->fn = [=](cudaStream_t s) { eltwise_vec_kernel<false><<<grid, 256, 0, s>>>(p, i0, i1, c, o, vectors, sf); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_eltwise_byxf = {"eltwise_byxf", sizeof(cldnn_b200_eltwise_params), eltwise_vec_supports, one_tune, nullptr, eltwise_vec_prepare};

// ---------------------------------------------------------------------------------
// reorder (cl_kernels/reorder_data.cl:72-128).  Threads walk the destination in
// its own memory order so writes coalesce; a destination feature beyond the
// source's feature count is written as zero (feature padding of the new layout).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
reorder_ref_kernel(const __grid_constant__ cldnn_b200_reorder_params p, const void* in, void* out)
{
    const int64_t total = (int64_t)p.out.b * p.out.f * p.out.y * p.out.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int b, f, y, x;
        if (p.out.pf == 1) { f = (int)(idx % p.out.f); int64_t t = idx / p.out.f; x = (int)(t % p.out.x); t /= p.out.x; y = (int)(t % p.out.y); b = (int)(t / p.out.y); }
        else if (p.out.pb == 1) { b = (int)(idx % p.out.b); int64_t t = idx / p.out.b; f = (int)(t % p.out.f); t /= p.out.f; x = (int)(t % p.out.x); y = (int)(t / p.out.x); }
        else { x = (int)(idx % p.out.x); int64_t t = idx / p.out.x; y = (int)(t % p.out.y); t /= p.out.y; f = (int)(t % p.out.f); b = (int)(t / p.out.f); }
        const int64_t oi = tidx(p.out, b, f, y, x);
        if (f >= p.in.f) { store_sat_int(out, p.out.dtype, oi, 0); continue; }
        const int64_t ii = tidx(p.in, b, f, y, x);
        if (!is_fp(p.in.dtype) && !p.has_mean) { store_sat_int(out, p.out.dtype, oi, load_as_int(in, p.in.dtype, ii)); continue; }
        float v = load_as_float(in, p.in.dtype, ii);
        if (p.has_mean) v = __fsub_rn(v, p.mean[f < 4 ? f : 3]);
        store_sat_float(out, p.out.dtype, oi, v);
    }
}
static bool reorder_supports(const void* vp) { const auto& p = *(const cldnn_b200_reorder_params*)vp; return p.in.b == p.out.b && p.in.y == p.out.y && p.in.x == p.out.x && p.out.f >= p.in.f; }
static int32_t reorder_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_reorder_params p = *(const cldnn_b200_reorder_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "reorder_ref: input and output are required");
    const void* in = a->input0; void* o = a->output;
    const int grid = grid_for((int64_t)p.out.b * p.out.f * p.out.y * p.out.x, 256, ctx);
    out->fn = [=](cudaStream_t s) { reorder_ref_kernel<<<grid, 256, 0, s>>>(p, in, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_reorder_ref = {"reorder_ref", sizeof(cldnn_b200_reorder_params), reorder_supports, one_tune, nullptr, reorder_prepare};

// ---------------------------------------------------------------------------------
// lrn across channels (cl_kernels/lrn_gpu_across_channel_ref.cl:26-66)
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
lrn_ref_kernel(const __grid_constant__ cldnn_b200_lrn_params p, const void* in, void* out)
{
    const int64_t total = (int64_t)p.in.b * p.in.f * p.in.y * p.in.x;
    const int pad = (p.size - 1) / 2;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int b, f, y, x;
        decode_bfyx(idx, p.in.f, p.in.y, p.in.x, p.in.pf == 1 && p.out.pf == 1, b, f, y, x);
        float acc = 0.f;
        for (int i = 0; i < p.size; ++i) {
            const int ff = f - pad + i; if (ff < 0 || ff >= p.in.f) continue;
            const float v = load_as_float(in, p.in.dtype, tidx(p.in, b, ff, y, x));
            acc = __fadd_rn(acc, __fmul_rn(v, v));
        }
        acc = __fadd_rn(__fmul_rn(acc, __fdiv_rn(p.alpha, (float)p.size)), p.k);
        const float v = load_as_float(in, p.in.dtype, tidx(p.in, b, f, y, x));
        store_sat_float(out, p.out.dtype, tidx(p.out, b, f, y, x), v * powf(acc, -p.beta));
    }
}
// The same for fp16 in the feature-innermost (byxf) layout, window 5: a thread owns 8 consecutive features of one pixel,
// reads them with one 128-bit load and the two neighbours on either side with one 32-bit load each, keeps the squares
// in fp32 and writes 8 halves; x^-beta = exp2(-beta * log2(x)) on the special-function unit (the reference's
// native_powr is as loosely specified).
__global__ void __launch_bounds__(256)
lrn_f16_byxf_kernel(const __grid_constant__ cldnn_b200_lrn_params p, const __half* __restrict__ in, __half* __restrict__ out)
{
    const int fv = p.in.f / 8;
    const int64_t total = (int64_t)p.in.b * p.in.y * p.in.x * fv;
    const float scale = __fdiv_rn(p.alpha, (float)p.size);
    ItemWalk it; it.init(blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x, fv, p.in.x, p.in.y);
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < (uint32_t)total; idx += gridDim.x * blockDim.x, it.next()) {   // < 2^31 items (host check)
        const int f8 = it.f, x = it.x, y = it.y, b = it.b;
        const int f0 = f8 * 8;
        const __half* src = in + tidx(p.in, b, f0, y, x);
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
        float val[12];                                               // features f0 - 2 .. f0 + 9
        {
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); val[2 + 2 * k] = f.x; val[3 + 2 * k] = f.y; }
            float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
            if (f0 >= 2) lo = __half22float2(__ldg(reinterpret_cast<const __half2*>(src - 2)));
            if (f0 + 8 < p.in.f) hi = __half22float2(__ldg(reinterpret_cast<const __half2*>(src + 8)));
            if (f0 + 9 >= p.in.f) hi.y = 0.f;
            val[0] = lo.x; val[1] = lo.y; val[10] = hi.x; val[11] = hi.y;
        }
        float sq[12];
#pragma unroll
        for (int k = 0; k < 12; ++k) sq[k] = val[k] * val[k];
        __half2 o[4];
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
            const float a0 = fmaf(sq[k] + sq[k + 1] + sq[k + 2] + sq[k + 3] + sq[k + 4], scale, p.k);
            const float a1 = fmaf(sq[k + 1] + sq[k + 2] + sq[k + 3] + sq[k + 4] + sq[k + 5], scale, p.k);
            o[k >> 1] = __floats2half2_rn(val[k + 2] * exp2f(-p.beta * __log2f(a0)), val[k + 3] * exp2f(-p.beta * __log2f(a1)));
        }
        *reinterpret_cast<uint4*>(out + tidx(p.out, b, f0, y, x)) = *reinterpret_cast<const uint4*>(o);
    }
}
static bool lrn_f16_byxf_supports(const void* vp)
{
    const auto& p = *(const cldnn_b200_lrn_params*)vp;
    if (p.size != 5 || p.in.dtype != CLDNN_B200_F16 || p.out.dtype != CLDNN_B200_F16) return false;
    if (p.in.pf != 1 || p.out.pf != 1 || p.in.f % 8) return false;
    const int64_t pitches[] = {p.in.px, p.in.py, p.in.pb, p.in.offset, p.out.px, p.out.py, p.out.pb, p.out.offset};
    for (int64_t v : pitches) if (v % 8) return false;
    if ((int64_t)p.in.b * p.in.y * p.in.x * (p.in.f / 8) >= 0x7fffffffLL) return false;         // 32-bit item index
    return true;
}
static int32_t lrn_f16_byxf_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_lrn_params p = *(const cldnn_b200_lrn_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "lrn_f16_byxf: input and output are required");
    if (((uintptr_t)a->input0 | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "lrn_f16_byxf: buffers must be 16-byte aligned");
    const __half* in = (const __half*)a->input0; __half* o = (__half*)a->output;
    const int grid = grid_for((int64_t)p.in.b * p.in.y * p.in.x * (p.in.f / 8), 256, ctx);
    out->fn = [p, in, o, grid](cudaStream_t s) { lrn_f16_byxf_kernel<<<grid, 256, 0, s>>>(p, in, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}

static bool lrn_supports(const void* vp) { const auto& p = *(const cldnn_b200_lrn_params*)vp; return p.size >= 1 && is_fp(p.in.dtype); }
static int32_t lrn_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_lrn_params p = *(const cldnn_b200_lrn_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "lrn_ref: input and output are required");
    const void* in = a->input0; void* o = a->output;
    const int grid = grid_for((int64_t)p.in.b * p.in.f * p.in.y * p.in.x, 256, ctx);
    out->fn = [=](cudaStream_t s) { lrn_ref_kernel<<<grid, 256, 0, s>>>(p, in, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_lrn_ref = {"lrn_ref", sizeof(cldnn_b200_lrn_params), lrn_supports, one_tune, nullptr, lrn_prepare};
const KernelDef kdef_lrn_f16_byxf = {"lrn_f16_byxf", sizeof(cldnn_b200_lrn_params), lrn_f16_byxf_supports, one_tune, nullptr, lrn_f16_byxf_prepare};

// ---------------------------------------------------------------------------------
// standalone activation (cl_kernels/activation_ref.cl)
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
activation_ref_kernel(const __grid_constant__ cldnn_b200_activation_params p, const void* in, void* out)
{
    const int64_t total = (int64_t)p.in.b * p.in.f * p.in.y * p.in.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int x = (int)(idx % p.in.x); int64_t t = idx / p.in.x;
        int y = (int)(t % p.in.y); t /= p.in.y;
        int f = (int)(t % p.in.f); int b = (int)(t / p.in.f);
        const int64_t ii = tidx(p.in, b, f, y, x), oi = tidx(p.out, b, f, y, x);
        if (is_fp(p.in.dtype)) store_sat_float(out, p.out.dtype, oi, act_float(p.act, load_as_float(in, p.in.dtype, ii), p.act_m, p.act_n));
        else store_sat_int(out, p.out.dtype, oi, act_int(p.act, load_as_int(in, p.in.dtype, ii), p.act_m, p.act_n));
    }
}
static bool activation_supports(const void*) { return true; }
static int32_t activation_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_activation_params p = *(const cldnn_b200_activation_params*)vp;
    if (!a->input0 || !a->output) return fail(CLDNN_B200_INVALID_ARG, "activation_ref: input and output are required");
    const void* in = a->input0; void* o = a->output;
    const int grid = grid_for((int64_t)p.in.b * p.in.f * p.in.y * p.in.x, 256, ctx);
    out->fn = [=](cudaStream_t s) { activation_ref_kernel<<<grid, 256, 0, s>>>(p, in, o); return cudaGetLastError(); };
    return CLDNN_B200_SUCCESS;
}
const KernelDef kdef_activation_ref = {"activation_ref", sizeof(cldnn_b200_activation_params), activation_supports, one_tune, nullptr, activation_prepare};

}  // namespace b200
