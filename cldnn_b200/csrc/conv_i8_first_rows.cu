// First layer, row form: the first convolution of an image network (few planar input features; written for the 8-bit case:
// stride 2, 64 or 32 output features) as a GEMM whose rows are OUTPUT ROWS and whose operand is the raw image, so that no thread
// ever assembles an im2col operand:
//
//   D[y, (i, f)] = sum over (ky, c)  A_(ky,c)[y, 0..31] . T_(ky,c)[(i, f), 0..31]
//
// for the output columns x = XB j + i of one "x-block" j (XB = 256 / features: four columns of 64 features, eight of 32).
// A_(ky,c)[y, :] are 32 consecutive bytes of input row 2y + ky - pad_y of feature c, starting at a 16-byte aligned column
// u(j).  The input rows a tile touches come in once per tile, as two TMA boxes of 32 bytes x rows x C features: the
// even-indexed rows and the odd-indexed ones (every second row through the row pitch; zero fill outside the image = the
// padding); filter row ky then reads its parity's plane from row floor((ky - pad_y) / 2) on, by a descriptor start address
// shifted by whole rows.  T_(ky,c) is the filter row (ky, c) laid out as a banded (Toeplitz) matrix:
// T[(i, f), k] = w[f][c][ky][k - off - 2i].  The window of 32 columns holds the 2 (XB - 1) + kw the outputs of a block need
// at offset `off`, which depends only on the parity of j (13 and 5 for a 7-wide filter with padding 3 and XB = 4): two
// variants of T, and a CTA works on x-blocks of one parity only, so it keeps one variant resident in shared memory
// (C * kh * 8 KB; 168 KB for 7x7x3).
// The tensor core multiplies several times the taps that exist (a 32-column window per filter row: 4.6 x for 7 taps); in
// exchange the per-tile work of the general first-layer kernel's four builder warps disappears, and what remains per tile
// of 128 rows x XB columns is C * kh MMAs (M 128, N 256, K 32), two TMA copies and the requantising epilogue.
//
// The same kernel serves fp16 images (kind::f16, fp32 accumulators, bias + activation + one rounding to half): a window is then
// 16 columns, and with a vertical stride of 1 there is one plane of all rows instead of two parity planes (VGG's 3x3 first
// layer).  What fits is decided on the host (first_rows_plan): stride 1 or 2, the window of a block within 32 bytes, x-blocks
// stepping by whole 16-byte units, the banded matrices and two stages of rows within shared memory.
//
// Roles: warp 0 issues the copies, warp 1 the MMAs, warps 4.. are two epilogue groups taking tiles in turn (one accumulator of
// 256 columns each) or four (the two groups of an accumulator share its tiles by column halves).  The operation order of the
// 8-bit epilogue is the reference's (kernel_selector/core/cl_kernels/fused_conv_eltwise_gpu_ref.cl:65-234); it is the
// conversion-free form of conv_epilogue.cuh, with the float-domain form per value where a feature's range demands it.
#include <cuda.h>
#include <cuda_fp16.h>
#include <mutex>
#include <string>
#include "engine.hpp"
#include "sm100_ptx.cuh"
#include "conv_epilogue.cuh"
#include "conv_i8_first_rows.hpp"

namespace b200 {

using namespace ptx;

constexpr int rows_threads(int groups) { return 128 + 128 * groups; }
constexpr int kRMaxStages = 4;
constexpr int kRCols = 256;                     // accumulator columns of a tile: XB output columns x features
constexpr int kROfm = 64;                       // at most; 32 features make x-blocks of eight output columns
constexpr uint32_t kErrRows = 0x58u;

struct RowsParams {
    alignas(64) CUtensorMap tmA[2];             // input rows of even / odd index
    alignas(64) CUtensorMap tmB;                // banded filter rows, both variants
    int32_t N, C, P, Q, kh, ofm;
    int32_t ofm_shift, xb;                      // log2(ofm); output columns of an x-block = 256 / ofm
    int32_t planes, ustep;                      // row planes per stage (= vertical stride); window step between x-blocks of one parity
    int32_t act, bias_dtype; float act_m, act_n;   // fp16 path
    int32_t tiles_y, jcount[2], total[2];       // x-blocks of even / odd index per row of tiles, tiles per variant
    int32_t u0[2];                              // window start of the first x-block of each parity
    int32_t row_q[16], row_r[16];               // filter row ky reads input rows 2 (y + row_q) + row_r
    int32_t stages, a_plane_bytes, a_stage_bytes, b_bytes;  // one (row parity, feature) plane of a stage, 2 C of them, the filter image
    int32_t st32;                                       // output rows are 32-byte aligned: one 32-byte store per 32 features
    uint32_t idesc;
    int64_t out_px, out_py, out_pb, out_off;
    int32_t mul_oqf, mode;                      // mode: 0 u8, 1 s8, 2 s8 after ReLU; +4 with a uniform O_QF
    int32_t pad_bytes;                          // behind the last stage: what the last plane's 128-row reads may touch
    int32_t m_lo;                               // first row of a plane relative to the tile's first output row
    int32_t groups;                             // epilogue warp groups: 2 (a tile each) or 4 (half the columns of a tile each)
    float acc_bound;
    uint8_t* out; const void* bias; const float* quant;
    uint32_t* status;
    EpiCfg epi;
};

struct RowsAux {
    uint64_t full[kRMaxStages], empty[kRMaxStages], tmem_full[2], tmem_empty[2], b_full, drain;
    uint32_t tmem_base, abort, wide;
    alignas(16) int32_t bias_i[kROfm];
    alignas(16) float quant[kROfm];
    alignas(16) float bias_f[kROfm];            // fp16 path
};

// filter [ofm][C][kh][kw] (any pitches) -> [variant][ky * C + c][n = i * ofm + f][k = 0 .. 32 bytes of elements], zero outside the
// band; `s` = horizontal stride
template <typename T>
__global__ void rows_pack_weights(const T* __restrict__ w, int64_t po, int64_t pi, int64_t py, int64_t px, int64_t off,
                                  int C, int kh, int kw, int ofm, int s, int off0, int off1, T* __restrict__ dst)
{
    constexpr int KW = 32 / (int)sizeof(T);                          // window in elements
    const int chunks = C * kh;
    const int total = 2 * chunks * kRCols * KW;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int k = idx % KW; int r = idx / KW;
        const int n = r % kRCols; r /= kRCols;
        const int g = r % chunks; const int v = r / chunks;
        const int ky = g / C, c = g - ky * C;
        const int i = n / ofm, f = n - i * ofm;
        const int kx = k - (v ? off1 : off0) - s * i;
        T val = T(0);
        if (kx >= 0 && kx < kw) val = w[off + f * po + c * pi + ky * py + kx * px];
        dst[idx] = val;
    }
}

struct RowsTile { int n, ty, j, jv; };
__device__ __forceinline__ RowsTile rows_tile(const RowsParams& P, int v, int t)
{
    RowsTile r;
    r.jv = t % P.jcount[v]; const int rest = t / P.jcount[v];
    r.ty = rest % P.tiles_y; r.n = rest / P.tiles_y;
    r.j = 2 * r.jv + v;
    return r;
}

// 32 accumulator columns of one row, float-domain form (features whose values may leave the exact range of the other)
__device__ __noinline__ void rows_chunk_wide(const EpiCfg& c, const RowsAux* aux, const uint32_t (&r)[32], int f0, uint8_t* dst)
{
    alignas(16) uint8_t b[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float v = epi_quant(c, (int32_t)r[j] + aux->bias_i[f0 + j], aux->quant[f0 + j], 0.0f, 1.0f, 0.0f, 1.0f);
        const int32_t i = __float2int_rz(v);
        b[j] = c.out_dtype == CLDNN_B200_U8 ? (uint8_t)min(255, max(0, i)) : (uint8_t)(int8_t)min(127, max(-128, i));
    }
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(b)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(b)[1];
}

// 32 output bytes of one pixel: one 32-byte store (a whole sector) where the address allows it
__device__ __forceinline__ void rows_store32(uint8_t* p, const uint4& a, const uint4& b, bool st32)
{
    if (st32) asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" :: "l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
    else { reinterpret_cast<uint4*>(p)[0] = a; reinterpret_cast<uint4*>(p)[1] = b; }
}

template <int kMode, bool kOqf>
__device__ __forceinline__ void rows_epi_tile(const RowsParams& P, const RowsAux* aux, uint32_t t_row, uint8_t* out_row, bool row_ok, int x_left,
                                              uint32_t tmem_empty_bar, int lane)
{
    const float oqf = P.epi.o_qf;
    const bool st32 = P.st32 != 0;
    uint32_t ra[32], rb[32];
    tmem_ld_32x32(t_row, ra);
#pragma unroll 1
    for (int c0 = 0; c0 < kRCols; c0 += 64) {
        // two chunks of 32 columns: the two halves of one pixel's 64 features, or two pixels of 32 features
        const int ia = c0 >> P.ofm_shift, ib = (c0 + 32) >> P.ofm_shift;
        const int fa = c0 & (P.ofm - 1), fb = (c0 + 32) & (P.ofm - 1);
        tmem_ld_wait();
        tmem_ld_32x32(t_row + (uint32_t)(c0 + 32), rb);
        if (row_ok && ia < x_left) { uint4 o0, o1; fast_chunk32<false, false, kMode, kOqf>(ra, &aux->bias_i[fa], &aux->quant[fa], &o0, &o1, 0u, kMagicBits, kMagicBits, oqf); rows_store32(out_row + (int64_t)ia * P.out_px + fa, o0, o1, st32); }
        tmem_ld_wait();
        if (c0 + 64 < kRCols) tmem_ld_32x32(t_row + (uint32_t)(c0 + 64), ra);
        else { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        if (row_ok && ib < x_left) { uint4 o0, o1; fast_chunk32<false, false, kMode, kOqf>(rb, &aux->bias_i[fb], &aux->quant[fb], &o0, &o1, 0u, kMagicBits, kMagicBits, oqf); rows_store32(out_row + (int64_t)ib * P.out_px + fb, o0, o1, st32); }
    }
}

// the same over columns [c_lo, c_lo + 128) with one register array (four epilogue groups: 96 registers per thread)
template <int kMode, bool kOqf>
__device__ __forceinline__ void rows_epi_half(const RowsParams& P, const RowsAux* aux, uint32_t t_row, uint8_t* out_row, bool row_ok, int x_left,
                                              uint32_t tmem_empty_bar, int lane, int c_lo)
{
    const float oqf = P.epi.o_qf;
    const bool st32 = P.st32 != 0;
#pragma unroll 1
    for (int c0 = c_lo; c0 < c_lo + 128; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + (uint32_t)c0, r);
        tmem_ld_wait();
        if (c0 + 32 >= c_lo + 128) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        const int i = c0 >> P.ofm_shift, f0 = c0 & (P.ofm - 1);
        if (row_ok && i < x_left) {
            uint4 o0, o1;
            fast_chunk32<false, false, kMode, kOqf>(r, &aux->bias_i[f0], &aux->quant[f0], &o0, &o1, 0u, kMagicBits, kMagicBits, oqf);
            rows_store32(out_row + (int64_t)i * P.out_px + f0, o0, o1, st32);
        }
    }
}

__device__ __noinline__ float rows_act_other(int32_t fn, float x, float m, float n) { return act_float(fn, x, m, n); }
__device__ __forceinline__ float rows_act(int32_t fn, float x, float m, float n)
{
    if (fn == CLDNN_B200_ACT_NONE) return x;
    if (fn == CLDNN_B200_ACT_RELU) return fmaxf(0.0f, x);
    return rows_act_other(fn, x, m, n);
}

// fp16: fp32 accumulators + bias -> activation -> one rounding to half; 32 columns = 64 output bytes per trip
__device__ __forceinline__ void rows_epi_f16(const RowsParams& P, const RowsAux* aux, uint32_t t_row, uint8_t* out_row, bool row_ok, int x_left,
                                             uint32_t tmem_empty_bar, int lane, int c_lo, int c_hi)
{
    const bool st32 = P.st32 != 0;
#pragma unroll 1
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + (uint32_t)c0, r);
        tmem_ld_wait();
        if (c0 + 32 >= c_hi) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        const int i = c0 >> P.ofm_shift, f0 = c0 & (P.ofm - 1);
        if (row_ok && i < x_left) {
            uint4 o[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float4 b0 = *reinterpret_cast<const float4*>(&aux->bias_f[f0 + 8 * w]), b1 = *reinterpret_cast<const float4*>(&aux->bias_f[f0 + 8 * w + 4]);
                const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                uint32_t ow[4];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float v0 = rows_act(P.act, __uint_as_float(r[8 * w + 2 * h]) + bb[2 * h], P.act_m, P.act_n);
                    const float v1 = rows_act(P.act, __uint_as_float(r[8 * w + 2 * h + 1]) + bb[2 * h + 1], P.act_m, P.act_n);
                    const __half2 hv = __floats2half2_rn(v0, v1);
                    ow[h] = *reinterpret_cast<const uint32_t*>(&hv);
                }
                o[w] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
            uint8_t* dst = out_row + (int64_t)i * P.out_px + 2 * f0;
            rows_store32(dst, o[0], o[1], st32);
            rows_store32(dst + 32, o[2], o[3], st32);
        }
    }
}

__device__ __noinline__ void rows_epi_tile_wide(const RowsParams& P, const RowsAux* aux, uint32_t t_row, uint8_t* out_row, bool row_ok, int x_left,
                                                uint32_t tmem_empty_bar, int lane, int c_lo, int c_hi)
{
#pragma unroll 1
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + (uint32_t)c0, r);
        tmem_ld_wait();
        if (c0 + 32 >= c_hi) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        const int i = c0 >> P.ofm_shift, f0 = c0 & (P.ofm - 1);
        if (row_ok && i < x_left) rows_chunk_wide(P.epi, aux, r, f0, out_row + (int64_t)i * P.out_px + f0);
    }
}

template <int G, bool kHalf>
__global__ void __launch_bounds__(rows_threads(G), 1)
conv_i8_first_rows_kernel(const __grid_constant__ RowsParams P)
{
    constexpr int kRThreads = 128 + 128 * G;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t b_base = base;
    const uint32_t a_base = base + (uint32_t)P.b_bytes;
    RowsAux* aux = reinterpret_cast<RowsAux*>(smem + P.b_bytes + P.stages * P.a_stage_bytes + P.pad_bytes);
    volatile uint32_t* s_abort = &aux->abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const EpiCfg& c = P.epi;
    const int v = (int)(blockIdx.x & 1u);                            // parity of the x-blocks this CTA works on
    const int ctas_v = ((int)gridDim.x + 1 - v) >> 1, bv = (int)(blockIdx.x >> 1);
    const int my_tiles = P.total[v] > bv ? (P.total[v] - bv + ctas_v - 1) / ctas_v : 0;
    const int chunks = P.C * P.kh;

    if (tid == 0) {
        for (int s = 0; s < P.stages; ++s) { mbar_init(smem_u32(&aux->full[s]), 1); mbar_init(smem_u32(&aux->empty[s]), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&aux->tmem_full[a]), 1); mbar_init(smem_u32(&aux->tmem_empty[a]), 2 * G); }
        mbar_init(smem_u32(&aux->b_full), 1); mbar_init(smem_u32(&aux->drain), 1);
        aux->abort = 0u; aux->wide = 0u;
        mbar_fence_init();
        prefetch_tensormap(&P.tmA[0]); prefetch_tensormap(&P.tmA[1]); prefetch_tensormap(&P.tmB);
    }
    if (warp == 1) { tmem_alloc(smem_u32(&aux->tmem_base), 512u); tmem_relinquish(); }
    __syncthreads();
    for (int j = tid; j < P.ofm; j += kRThreads) {
        if (kHalf) { aux->bias_f[j] = P.bias_dtype != CLDNN_B200_NONE ? load_as_float(P.bias, P.bias_dtype, j) : 0.0f; continue; }
        const int32_t bi = c.bias_dtype != CLDNN_B200_NONE ? ((const int32_t*)P.bias)[j] : 0;
        const float q = P.quant[j];
        aux->bias_i[j] = bi; aux->quant[j] = q;
        // the conversion-free epilogue is exact while every dequantised value stays below 2^22
        if (!(__fmul_rn(__fmul_rn(__fadd_rn(P.acc_bound, fabsf((float)bi)), fabsf(q)), P.mul_oqf ? fabsf(c.o_qf) : 1.0f) < 4.0e6f)) atomicOr(&aux->wide, 1u);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        const bool leader = elect_one();
        if (leader && my_tiles > 0) {
            // the banded filter rows of this CTA's parity, once
            const uint32_t bf = smem_u32(&aux->b_full);
            mbar_expect_tx(bf, (uint32_t)P.b_bytes);
            for (int g = 0; g < chunks; ++g) tma_load_2d(b_base + (uint32_t)g * (uint32_t)(kRCols * 32), &P.tmB, bf, 0, (v * chunks + g) * kRCols);
        }
        int stage = 0; uint32_t phase = 0; int64_t issued = 0; bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            const RowsTile t = rows_tile(P, v, bv + it * ctas_v);
            const int u = P.u0[v] + P.ustep * t.jv, y0 = t.ty * 128;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1u, s_abort, P.status, kErrRows + 1u))) { ok = false; break; }
            if (leader) {
                // the tile's input rows, once: with a vertical stride of two the even-indexed ones and the odd-indexed ones as
                // two boxes of C planes each
                const uint32_t full = smem_u32(&aux->full[stage]);
                const uint32_t dst = a_base + (uint32_t)(stage * P.a_stage_bytes);
                mbar_expect_tx(full, (uint32_t)P.a_stage_bytes);
                tma_load_4d(dst, &P.tmA[0], full, u, y0 + P.m_lo, 0, t.n);
                if (P.planes == 2) tma_load_4d(dst + (uint32_t)(P.C * P.a_plane_bytes), &P.tmA[1], full, u, y0 + P.m_lo, 0, t.n);
            }
            ++issued;
            if (++stage == P.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) {
            // unwind: let the copies already in flight land before the CTA's shared memory goes away
            int st = stage; uint32_t ph = phase;
            const int pending = issued < P.stages ? (int)issued : P.stages;
            for (int i = 0; i < pending; ++i) {
                if (--st < 0) { st = P.stages - 1; ph ^= 1u; }
                const uint64_t t0 = globaltimer();
                while (!mbar_try_wait(smem_u32(&aux->full[st]), ph) && globaltimer() - t0 < 100000000ull) { }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        const bool leader = elect_one();
        int stage = 0; uint32_t phase = 0; bool ok = true;
        if (my_tiles > 0) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->b_full), 0u, s_abort, P.status, kErrRows + 2u));
        for (int it = 0; it < my_tiles && ok; ++it) {
            const int acc = it & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->tmem_empty[acc]), (((uint32_t)(it >> 1) & 1u)) ^ 1u, s_abort, P.status, kErrRows + 3u))) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kRCols);
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->full[stage]), phase, s_abort, P.status, kErrRows + 4u))) { ok = false; break; }
            tc_fence_after();
            if (leader) {
                // filter row ky of feature ch reads plane (row parity, ch) from row row_q - m_lo on: a descriptor start address
                // shifted by whole rows inside the swizzle pattern reads what TMA wrote (the swizzle is a function of the address)
                const uint32_t a_stage = a_base + (uint32_t)(stage * P.a_stage_bytes);
                uint32_t accf = 0u, b_addr = b_base;
                for (int ky = 0; ky < P.kh; ++ky) {
                    uint32_t a_addr = a_stage + (uint32_t)(P.row_r[ky] * P.C * P.a_plane_bytes) + (uint32_t)((P.row_q[ky] - P.m_lo) * 32);
                    for (int ch = 0; ch < P.C; ++ch, a_addr += (uint32_t)P.a_plane_bytes, b_addr += (uint32_t)(kRCols * 32)) {
                        if (kHalf) mma_f16_ss(d_tmem, make_smem_desc(a_addr, 256u, 6u), make_smem_desc(b_addr, 256u, 6u), P.idesc, accf);
                        else mma_i8_ss(d_tmem, make_smem_desc(a_addr, 256u, 6u), make_smem_desc(b_addr, 256u, 6u), P.idesc, accf);
                        accf = 1u;
                    }
                }
                tc_commit(smem_u32(&aux->empty[stage]));
            }
            if (++stage == P.stages) { stage = 0; phase ^= 1u; }
            if (ok && leader) tc_commit(smem_u32(&aux->tmem_full[acc]));
        }
        // drain: every issued MMA must have retired before tensor memory is released
        if (leader) tc_commit(smem_u32(&aux->drain));
        const uint64_t t0 = globaltimer();
        while (!mbar_try_wait(smem_u32(&aux->drain), 0u)) {
            if (globaltimer() - t0 > kWaitLimitNs) { atomicCAS(P.status, 0u, kErrRows + 5u); break; }
        }
    } else if (warp >= 4) {
        // ------------------------------ epilogue ----------------------------------
        // two groups: a tile each in turn; four: the two of an accumulator share its tiles by column halves
        const int ew = warp - 4, quad = ew & 3, group = (ew >> 2) & 1, half = ew >> 3;
        const int row = quad * 32 + lane;
        const bool wide = aux->wide != 0u;
        const int c_lo = G == 4 ? 128 * half : 0, c_hi = G == 4 ? c_lo + 128 : kRCols;
        for (int it = group; it < my_tiles; it += 2) {
            const int acc = it & 1;                                  // = group
            const RowsTile t = rows_tile(P, v, bv + it * ctas_v);
            const int y = t.ty * 128 + row, x0 = P.xb * t.j;
            const bool row_ok = y < P.P;
            const int x_left = P.Q - x0;
            uint8_t* out_row = P.out + P.out_off + (int64_t)t.n * P.out_pb + (int64_t)y * P.out_py + (int64_t)x0 * P.out_px;
            if (!mbar_wait(smem_u32(&aux->tmem_full[acc]), (uint32_t)(it >> 1) & 1u, s_abort, P.status, kErrRows)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kRCols);
            const uint32_t te = smem_u32(&aux->tmem_empty[acc]);
            if (kHalf) rows_epi_f16(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo, c_hi);
            else if (wide) rows_epi_tile_wide(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo, c_hi);
            else if (G == 4) switch (P.mode) {
                case 0: rows_epi_half<0, false>(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo); break;
                case 1: rows_epi_half<1, false>(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo); break;
                case 2: rows_epi_half<2, false>(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo); break;
                case 4: rows_epi_half<0, true>(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo); break;
                default: rows_epi_half<1, true>(P, aux, t_row, out_row, row_ok, x_left, te, lane, c_lo); break;
            }
            else switch (P.mode) {
                case 0: rows_epi_tile<0, false>(P, aux, t_row, out_row, row_ok, x_left, te, lane); break;
                case 1: rows_epi_tile<1, false>(P, aux, t_row, out_row, row_ok, x_left, te, lane); break;
                case 2: rows_epi_tile<2, false>(P, aux, t_row, out_row, row_ok, x_left, te, lane); break;
                case 4: rows_epi_tile<0, true>(P, aux, t_row, out_row, row_ok, x_left, te, lane); break;
                default: rows_epi_tile<1, true>(P, aux, t_row, out_row, row_ok, x_left, te, lane); break;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512u); }
}

// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn r_encode_tiled = nullptr;
static bool rows_load_entry_point()
{
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr; cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            r_encode_tiled = (EncodeTiledFn)fn;
        (void)cudaGetLastError();
    });
    return r_encode_tiled != nullptr;
}

static inline int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }

// everything the shapes decide: element size, x-block, windows of the two parities, row planes, shared-memory sizes
struct RowsGeom {
    int es, xb, kwin, align;                      // bytes per element; output columns per x-block; window and TMA alignment in elements
    int u0[2], off[2], ustep;                     // window start of the first x-block of each parity, first tap's place in it, step
    int planes, m_lo, plane_rows, pad_bytes;      // row planes (vertical stride), first plane row of a tile, rows per plane
    size_t b_bytes, stage_bytes;
};
static RowsGeom rows_geom(const cldnn_b200_conv_params& p)
{
    RowsGeom g;
    g.es = p.in.dtype == CLDNN_B200_F16 ? 2 : 1;
    g.xb = kRCols / (p.ofm > 0 ? p.ofm : 64); g.kwin = 32 / g.es; g.align = 16 / g.es;
    const int s = p.stride_x;
    for (int v = 0; v < 2; ++v) {
        const int col0 = s * g.xb * v - p.pad_x;                     // first input column of x-block v
        g.u0[v] = floor_div(col0, g.align) * g.align; g.off[v] = col0 - g.u0[v];
    }
    g.ustep = 2 * s * g.xb;
    g.planes = p.stride_y;
    g.m_lo = floor_div(-p.pad_y, p.stride_y);
    const int q_max = floor_div(p.kh - 1 - p.pad_y, p.stride_y);
    const int rows_in_tile = p.out.y <= 128 ? p.out.y : 128;
    g.plane_rows = (rows_in_tile + q_max - g.m_lo + 7) / 8 * 8;
    const int surplus = q_max - g.m_lo + 128 - g.plane_rows;
    g.pad_bytes = surplus > 0 ? (surplus * 32 + 255) / 256 * 256 : 0;
    g.b_bytes = (size_t)p.ifm * p.kh * kRCols * 32;
    g.stage_bytes = (size_t)g.planes * p.ifm * g.plane_rows * 32;
    return g;
}
constexpr size_t kRowsSmemLimit = 227 * 1024;          // opt-in shared memory per CTA on sm_100

bool first_rows_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    const bool half = p.in.dtype == CLDNN_B200_F16;
    if (half) {
        if (p.w_dtype != CLDNN_B200_F16 || p.out.dtype != CLDNN_B200_F16) return no("fp16 weights and output with fp16 input");
        if (p.quantization || p.calibration || p.has_o_qf) return no("no quantisation on the fp16 path");
        if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_F16 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    } else if (!is_int8(p.in.dtype) || p.w_dtype != CLDNN_B200_I8 || !is_int8(p.out.dtype)) return no("fp16, or 8-bit activations, weights and output");
    if (p.groups != 1 || p.fused_eltw) return no("plain convolution only");
    if (p.epilogue_order != CLDNN_B200_EPILOGUE_REF) return no("reference epilogue order only");
    const int es = half ? 2 : 1;
    if (p.in.px != 1 || (p.in.py * es) % 16 || (p.in.pf * es) % 16 || (p.in.pb * es) % 16 || (p.in.offset * es) % 16) return no("row form: planar input with 16-byte aligned pitches");
    if (p.out.pf != 1) return no("output must be byxf");
    if ((p.out.px * es) % 16 || (p.out.py * es) % 16 || (p.out.pb * es) % 16 || (p.out.offset * es) % 16) return no("output pitches must be 16-byte aligned");
    if (p.stride_x != p.stride_y || (p.stride_x != 1 && p.stride_x != 2) || p.dil_x != 1 || p.dil_y != 1) return no("row form: stride 1 or 2, no dilation");
    if ((p.ofm != 64 && p.ofm != 32) || p.out.f != p.ofm || p.in.f != p.ifm) return no("row form: 32 or 64 output features");
    if (p.kh < 1 || p.kh > 16 || p.kw < 1 || p.ifm < 1 || p.ifm * p.kh > 24) return no("row form: C * kh up to 24");
    if (p.pad_x < 0 || p.pad_y < 0) return no("row form: non-negative padding");
    const RowsGeom g = rows_geom(p);
    if (g.ustep % g.align) return no("row form: x-blocks do not step by whole 16-byte units");
    if (p.in.x < g.kwin || p.in.y < p.stride_y) return no("row form: image narrower than a window");
    for (int v = 0; v < 2; ++v) if (g.off[v] + p.stride_x * (g.xb - 1) + p.kw - 1 > g.kwin - 1) return no("row form: the filter window exceeds 32 bytes of columns");
    if (!half) {
        if (!p.quantization || p.i_qf != 1.0f) return no("row form: per-feature quantisation factors, no input factor");
        const bool mul_oqf = p.calibration || p.o_qf != 1.0f;
        if (mul_oqf && !(!p.calibration && p.o_qf > 0.0f && (p.out.dtype == CLDNN_B200_U8 || p.act != CLDNN_B200_ACT_RELU))) return no("row form: output factor not in the conversion-free set");
        if (p.act != CLDNN_B200_ACT_NONE && p.act != CLDNN_B200_ACT_RELU) return no("row form: activation none or ReLU");
        if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_I32) return no("row form: 32-bit integer bias");
        if (make_epi_cfg(p).dont_dequantize_bias) return no("row form: bias in the accumulator's scale");
    }
    const int P_ = (p.in.y + 2 * p.pad_y - p.kh) / p.stride_y + 1, Q_ = (p.in.x + 2 * p.pad_x - p.kw) / p.stride_x + 1;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");
    if (g.plane_rows > 256) return no("row form: filter too tall");
    if (1024 + g.b_bytes + 2 * g.stage_bytes + g.pad_bytes + sizeof(RowsAux) > kRowsSmemLimit) return no("row form: filter image and two stages of rows exceed shared memory");
    return true;
}

size_t first_rows_scratch(const cldnn_b200_conv_params& p) { return (size_t)2 * p.ifm * p.kh * kRCols * 32; }

int32_t first_rows_prepare(cldnn_b200_ctx_impl* ctx, const cldnn_b200_conv_params& p_in, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out, int groups)
{
    const bool half = p_in.in.dtype == CLDNN_B200_F16;
    const cldnn_b200_conv_params p = half ? p_in : simplified_conv_params(p_in);
    std::string why;
    if (!first_rows_plan(p, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "first layer: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "first layer: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "first layer: bias_dtype set but no bias pointer");
    if (!half && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "first layer: quantization set but no factors");
    const size_t need = first_rows_scratch(p);
    if (!a->scratch || a->scratch_bytes < need) return fail(CLDNN_B200_INVALID_ARG, "first layer: needs " + std::to_string(need) + " bytes of scratch for the packed weights");
    if (((uintptr_t)a->scratch | (uintptr_t)a->output | (uintptr_t)a->input0) & 15) return fail(CLDNN_B200_INVALID_ARG, "first layer: input, scratch and output must be 16-byte aligned");
    if (!rows_load_entry_point()) return fail(CLDNN_B200_ERROR, "first layer: cuTensorMapEncodeTiled is not available");

    const RowsGeom g = rows_geom(p);
    const int es = g.es;
    RowsParams P{};
    P.N = p.in.b; P.C = p.ifm; P.P = p.out.y; P.Q = p.out.x; P.kh = p.kh; P.ofm = p.ofm;
    P.tiles_y = (P.P + 127) / 128;
    P.xb = g.xb; P.ofm_shift = p.ofm == 64 ? 6 : 5;
    const int tiles_x = (P.Q + P.xb - 1) / P.xb;
    P.jcount[0] = (tiles_x + 1) / 2; P.jcount[1] = tiles_x / 2;
    for (int v = 0; v < 2; ++v) { P.u0[v] = g.u0[v]; P.total[v] = P.N * P.tiles_y * P.jcount[v]; }
    P.ustep = g.ustep; P.planes = g.planes;
    for (int ky = 0; ky < p.kh; ++ky) { const int t = ky - p.pad_y; P.row_q[ky] = floor_div(t, p.stride_y); P.row_r[ky] = t - P.row_q[ky] * p.stride_y; }
    // A plane holds the input rows of one parity (one plane of all rows with stride 1) that the tile's output rows touch, in whole
    // 8-row groups.  The MMA reads 128 rows from its start row whatever the plane holds: the surplus are the next plane's bytes
    // (or the pad behind the last stage) and feed accumulator rows that nothing reads.
    const int plane_rows = g.plane_rows;
    P.m_lo = g.m_lo;
    P.a_plane_bytes = plane_rows * 32; P.a_stage_bytes = (int32_t)g.stage_bytes; P.b_bytes = (int32_t)g.b_bytes;
    const size_t max_smem = (size_t)ctx->prop.sharedMemPerBlockOptin;
    if (max_smem < 1024 + g.b_bytes + 2 * g.stage_bytes + g.pad_bytes + sizeof(RowsAux)) return fail(CLDNN_B200_OUT_OF_RESOURCES, "first layer: not enough shared memory for the row form");
    P.stages = (int)std::min<size_t>(kRMaxStages, (max_smem - 1024 - g.pad_bytes - g.b_bytes - sizeof(RowsAux)) / g.stage_bytes);
    P.pad_bytes = g.pad_bytes;
    const size_t smem = 1024 + g.b_bytes + (size_t)P.stages * g.stage_bytes + g.pad_bytes + sizeof(RowsAux);
    if (half) P.idesc = (1u << 4) | ((uint32_t)(kRCols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);          // f16 x f16 -> f32
    else P.idesc = (2u << 4) | ((p.in.dtype == CLDNN_B200_U8 ? 0u : 1u) << 7) | (1u << 10) | ((uint32_t)(kRCols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    P.out_px = p.out.px * es; P.out_py = p.out.py * es; P.out_pb = p.out.pb * es; P.out_off = p.out.offset * es;      // bytes
    P.epi = make_epi_cfg(p);
    P.mul_oqf = (!half && (p.calibration || p.o_qf != 1.0f)) ? 1 : 0;
    P.mode = (p.out.dtype == CLDNN_B200_U8 ? 0 : (p.act == CLDNN_B200_ACT_RELU ? 2 : 1)) + (P.mul_oqf ? 4 : 0);
    P.acc_bound = (float)p.ifm * (float)p.kh * (float)p.kw * (p.in.dtype == CLDNN_B200_U8 ? 255.0f : 128.0f) * 128.0f;
    P.act = p.act; P.act_m = p.act_m; P.act_n = p.act_n; P.bias_dtype = p.bias_dtype;
    P.st32 = (((uintptr_t)a->output + (uintptr_t)P.out_off) % 32 == 0 && P.out_px % 32 == 0 && P.out_py % 32 == 0 && P.out_pb % 32 == 0) ? 1 : 0;
    P.out = (uint8_t*)a->output; P.bias = a->bias; P.quant = a->weights_quantization_factors;
    P.status = ctx->d_status;
    P.groups = groups == 4 ? 4 : 2;

    const CUtensorMapDataType dt = half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    for (int r = 0; r < g.planes; ++r) {
        const int rows_r = (p.in.y - r + g.planes - 1) / g.planes;
        cuuint64_t dims[4] = {(cuuint64_t)p.in.x, (cuuint64_t)rows_r, (cuuint64_t)p.ifm, (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)(g.planes * p.in.py * es), (cuuint64_t)(p.in.pf * es), (cuuint64_t)(p.in.pb * es)};
        cuuint32_t box[4] = {(cuuint32_t)g.kwin, (cuuint32_t)plane_rows, (cuuint32_t)p.ifm, 1u};
        cuuint32_t est[4] = {1, 1, 1, 1};
        void* ptr = (char*)const_cast<void*>(a->input0) + (p.in.offset + (int64_t)r * p.in.py) * es;
        const CUresult cr = r_encode_tiled(&P.tmA[r], dt, 4, ptr, dims, strides, box, est, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                           CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_ERROR, "first layer: tensor map of the input rows refused (" + std::to_string((int)cr) + ")");
    }
    if (g.planes == 1) P.tmA[1] = P.tmA[0];
    {
        cuuint64_t dims[2] = {(cuuint64_t)g.kwin, (cuuint64_t)(2 * p.ifm * p.kh * kRCols)};
        cuuint64_t strides[1] = {32u};
        cuuint32_t box[2] = {(cuuint32_t)g.kwin, (cuuint32_t)kRCols};
        cuuint32_t est[2] = {1, 1};
        const CUresult cr = r_encode_tiled(&P.tmB, dt, 2, a->scratch, dims, strides, box, est, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                           CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_ERROR, "first layer: tensor map of the filter rows refused (" + std::to_string((int)cr) + ")");
    }
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_rows_kernel<2, false>, ctx->device, smem));
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_rows_kernel<4, false>, ctx->device, smem));
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_rows_kernel<2, true>, ctx->device, smem));
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_rows_kernel<4, true>, ctx->device, smem));
    int grid = ctx->prop.multiProcessorCount & ~1;
    if (grid < 2) grid = 2;
    const int most = std::max(P.total[0], P.total[1]);
    if (grid > 2 * most) grid = 2 * most;

    // pack the filter once, on the context's stream, before anything that is prepared here can run
    const int pack_total = 2 * p.ifm * p.kh * kRCols * g.kwin;
    if (half) rows_pack_weights<__half><<<(pack_total + 255) / 256, 256, 0, ctx->stream>>>((const __half*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset,
                                                                                          p.ifm, p.kh, p.kw, p.ofm, p.stride_x, g.off[0], g.off[1], (__half*)a->scratch);
    else rows_pack_weights<int8_t><<<(pack_total + 255) / 256, 256, 0, ctx->stream>>>((const int8_t*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset,
                                                                                      p.ifm, p.kh, p.kw, p.ofm, p.stride_x, g.off[0], g.off[1], (int8_t*)a->scratch);
    B200_CUDA(cudaGetLastError());
    out->fn = [P, grid, smem, half](cudaStream_t s) {
        if (half) {
            if (P.groups == 4) conv_i8_first_rows_kernel<4, true><<<grid, rows_threads(4), smem, s>>>(P);
            else conv_i8_first_rows_kernel<2, true><<<grid, rows_threads(2), smem, s>>>(P);
        } else {
            if (P.groups == 4) conv_i8_first_rows_kernel<4, false><<<grid, rows_threads(4), smem, s>>>(P);
            else conv_i8_first_rows_kernel<2, false><<<grid, rows_threads(2), smem, s>>>(P);
        }
        return cudaGetLastError();
    };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

}  // namespace b200
