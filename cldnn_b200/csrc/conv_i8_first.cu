// conv_i8_first: the first convolution of an 8-bit network -- few input
// features (3 for images), planar bfyx input as the caller provides it, large
// strided filter (7x7 / 2 for ResNet, 11x11 would need kw <= 8) -- computed on
// the tensor cores without any reordered or padded copy of the input in HBM.
// It replaces the reference's special first-layer kernels
// (cl_kernels/convolution_gpu_byxf_fs_bs_yx_bsv4_fsv32.cl,
// convolution_gpu_byx8_f4__fs_bs_yx_bsv4_fsv32.cl) and the input reorder in
// front of them; the operation order is that of fused_conv_eltwise_gpu_ref.cl.
//
// Each CTA owns tiles of 8 x 16 output pixels.  Per tile the threads copy the
// small input patch (C x (7*sy+kh) x (15*sx+8) bytes) into shared memory, build
// the 128 x K im2col operand from it in the tensor core's K-major core-matrix
// layout -- K ordered (feature, filter row, 8 taps), so every 8-byte group is
// one shifted read of a patch row -- then one thread issues K/32 tcgen05.mma
// into tensor memory and all warps run the requantising epilogue, writing byxf
// (features innermost) for the next layer.  Weights are packed once, at
// prepare time, into the matching shared-memory image (scratch buffer).
// Several CTAs share an SM, so the phases of different tiles overlap.
#include <cuda.h>
#include <mutex>
#include <string>
#include "engine.hpp"
#include "sm100_ptx.cuh"
#include "conv_epilogue.cuh"
#include "conv_i8_first_rows.hpp"

namespace b200 {

using namespace ptx;

constexpr int kFThreads = 288;
constexpr int kTileH = 8, kTileW = 16;          // 128 output pixels = 128 TMEM lanes
constexpr int kFMaxOfm = 256;
constexpr int kFMaxK = 256;
constexpr uint32_t kErrFirst = 0x50u;

struct FirstParams {
    int32_t N, C, H, W, P, Q, ofm, kh, kw, sx, sy, pad_x, pad_y;
    int64_t in_pb, in_pf, in_py, in_off;
    int32_t groups;                  // C*kh filter rows of 8 taps
    int32_t Kp;                      // padded K in bytes (multiple of 32)
    int32_t patch_h, patch_wp;       // patch rows per feature, row pitch in bytes (multiple of 4)
    int32_t tiles_x, tiles_y, total_tiles;
    uint32_t idesc, tmem_cols, sbo;
    int64_t out_px, out_py, out_pb, out_off;
    int32_t mul_iqf, mul_oqf, lean;
    float acc_bound;                 // C * kh * kw * max|activation| * 128
    int32_t ctas_per_sm;
    const uint8_t* in; uint8_t* out; const uint8_t* wpacked; const void* bias; const float* quant; const float* calib;
    uint32_t* status;
    EpiCfg epi;
};

struct FirstAux {
    uint64_t a_full[2], a_empty[2], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t wide;                   // a feature's values may leave the range the conversion-free epilogue is exact in
    uint16_t goff[64];               // per (feature, filter row) group: word offset of that row in the patch
    alignas(16) int32_t bias_i[1][kFMaxOfm];
    alignas(16) float bias_f[1][kFMaxOfm];
    alignas(16) float quant[1][kFMaxOfm];
    alignas(16) float calib[1][kFMaxOfm];
    alignas(16) float ecal[1][kFMaxOfm];
};

// K-major operand without swizzle: 8 x 16-byte core matrices, `lbo` bytes apart along K, `sbo` bytes apart along M/N
__device__ __forceinline__ uint64_t make_desc_interleaved(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// weights [ofm][C][kh][kw] (any pitches) -> shared-memory image: element (n, k) at (n/8)*sbo + (k/16)*128 + (n%8)*16 + k%16,
// k = ((c*kh + r)*8 + s); taps s >= kw and k beyond the last group are zero
__global__ void first_pack_weights(const int8_t* __restrict__ w, int64_t po, int64_t pi, int64_t py, int64_t px, int64_t off,
                                   int ofm, int C, int kh, int kw, int Kp, uint8_t* __restrict__ dst)
{
    const int total = ofm * Kp;
    const int sbo = (Kp / 16) * 128;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int n = i / Kp, k = i - n * Kp;
        const int g = k >> 3, s = k & 7;
        int8_t v = 0;
        if (g < C * kh && s < kw) { const int c = g / kh, r = g - c * kh; v = w[off + n * po + c * pi + r * py + s * px]; }
        dst[(n >> 3) * sbo + (k >> 4) * 128 + (n & 7) * 16 + (k & 15)] = (uint8_t)v;
    }
}

// ---- pipeline roles ------------------------------------------------------------------
// warps 0..3 build the im2col operand (two operand buffers), warps 4..7 run the epilogue
// (two accumulator buffers in tensor memory), warp 8 issues the MMAs.  The phases of
// consecutive tiles overlap: while the tensor core works on tile t the builders already
// assemble tile t+1 (with tile t+2's patch words in flight from global memory in their
// registers) and the epilogue warps requantise tile t-1.
constexpr int kBuilders = 128;
constexpr int kMaxPre = 9;                         // patch words a builder thread keeps in flight

// one aligned 4-byte word of the input patch, zero outside the image (the reference skips those taps).
// `rel` = offset of the word from the patch origin in the image, `pk` = patch row | (byte column << 8): both fixed per thread.
__device__ __forceinline__ uint32_t patch_word(const FirstParams& P, const uint8_t* origin, int32_t rel, int32_t pk, int y0, int xa)
{
    if (pk < 0) return 0u;                                                    // no such word in the patch
    const int iy = y0 + (pk & 0xff), ix = xa + (pk >> 8);
    if (iy < 0 || iy >= P.H || ix + 3 < 0 || ix >= P.W) return 0u;
    const uint8_t* src = origin + rel;
    if (ix >= 0 && ix + 3 < P.W && (reinterpret_cast<uintptr_t>(src) & 3u) == 0u) return __ldg(reinterpret_cast<const uint32_t*>(src));
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) { const int x = ix + b; if (x >= 0 && x < P.W) word |= (uint32_t)__ldg(src + b) << (8 * b); }
    return word;
}

__device__ __forceinline__ void tile_origin(const FirstParams& P, int tile, int& tx, int& ty, int& n, int& x0, int& y0, int& xa)
{
    tx = tile % P.tiles_x; const int t2 = tile / P.tiles_x;
    ty = t2 % P.tiles_y; n = t2 / P.tiles_y;
    x0 = tx * kTileW * P.sx - P.pad_x; y0 = ty * kTileH * P.sy - P.pad_y;
    xa = (x0 >= 0 ? x0 : x0 - 3) / 4 * 4;          // 4-byte aligned patch origin (floor)
}

// epilogue of one 32-row quadrant: kMode 0..2 = the conversion-free variants (u8 / s8 / s8 after ReLU), 3 = general
template <int kMode, bool kOqf = false>
__device__ __forceinline__ void first_epi_tile(const FirstParams& P, const FirstAux* aux, uint32_t t_row, uint8_t* out_row, bool valid,
                                               uint32_t tmem_empty_bar, int lane)
{
    const float oqf = P.epi.o_qf;
    uint32_t ra[32], rb[32];
    tmem_ld_32x32(t_row, ra);
#pragma unroll 1
    for (int c0 = 0; c0 < P.ofm; c0 += 64) {
        const bool second = c0 + 32 < P.ofm;
        tmem_ld_wait();
        if (second) tmem_ld_32x32(t_row + (uint32_t)(c0 + 32), rb);
        else { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        if (valid) {
            uint4* op = reinterpret_cast<uint4*>(out_row + c0);
            if (kMode < 3) fast_chunk32<false, false, kMode < 3 ? kMode : 0, kOqf>(ra, &aux->bias_i[0][c0], &aux->quant[0][c0], op, op + 1, 0u, kMagicBits, kMagicBits, oqf);
            else { uint4 o0, o1; epi_chunk_fast<false, false>(P, aux, 0, c0, ra, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1); op[0] = o0; op[1] = o1; }
        }
        if (!second) break;
        tmem_ld_wait();
        if (c0 + 64 < P.ofm) tmem_ld_32x32(t_row + (uint32_t)(c0 + 64), ra);
        else { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        if (valid) {
            uint4* op = reinterpret_cast<uint4*>(out_row + c0 + 32);
            if (kMode < 3) fast_chunk32<false, false, kMode < 3 ? kMode : 0, kOqf>(rb, &aux->bias_i[0][c0 + 32], &aux->quant[0][c0 + 32], op, op + 1, 0u, kMagicBits, kMagicBits, oqf);
            else { uint4 o0, o1; epi_chunk_fast<false, false>(P, aux, 0, c0 + 32, rb, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1); op[0] = o0; op[1] = o1; }
        }
    }
}

// the same with one register array (load, wait, convert): for launches that keep two CTAs per SM
template <int kMode, bool kOqf = false>
__device__ __forceinline__ void first_epi_tile_single(const FirstParams& P, const FirstAux* aux, uint32_t t_row, uint8_t* out_row, bool valid,
                                                      uint32_t tmem_empty_bar, int lane)
{
    const float oqf = P.epi.o_qf;
#pragma unroll 1
    for (int c0 = 0; c0 < P.ofm; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + (uint32_t)c0, r);
        tmem_ld_wait();
        if (c0 + 32 >= P.ofm) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(tmem_empty_bar); }
        if (valid) {
            uint4* op = reinterpret_cast<uint4*>(out_row + c0);
            fast_chunk32<false, false, kMode, kOqf>(r, &aux->bias_i[0][c0], &aux->quant[0][c0], op, op + 1, 0u, kMagicBits, kMagicBits, oqf);
        }
    }
}

// the general (not conversion-free) epilogue, out of line: it is the rare path and must not cost the common one registers
__device__ __noinline__ void first_epi_tile_general(const FirstParams& P, const FirstAux* aux, uint32_t t_row, uint8_t* out_row, bool valid,
                                                    uint32_t tmem_empty_bar, int lane)
{
    first_epi_tile<3>(P, aux, t_row, out_row, valid, tmem_empty_bar, lane);
}

template <int kCtas>
__global__ void __launch_bounds__(kFThreads, kCtas)
conv_i8_first_kernel(const __grid_constant__ FirstParams P)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 127u) & ~127u;
    uint8_t* smem = smem_raw + (base - raw);
    const int a_bytes = 128 * P.Kp, b_bytes = P.ofm * P.Kp;
    const int patch_bytes = P.C * P.patch_h * P.patch_wp;
    uint8_t* sA = smem; uint8_t* sB = smem + 2 * a_bytes; uint8_t* sPatch = sB + b_bytes;
    FirstAux* aux = reinterpret_cast<FirstAux*>(sPatch + ((patch_bytes + 15) & ~15));
    volatile uint32_t* s_abort = &aux->abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const EpiCfg& c = P.epi;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&aux->a_full[i]), 1); mbar_init(smem_u32(&aux->a_empty[i]), 1);
            mbar_init(smem_u32(&aux->tmem_full[i]), 1); mbar_init(smem_u32(&aux->tmem_empty[i]), 4);
        }
        aux->abort = 0u; aux->wide = 0u;
        mbar_fence_init();
    }
    if (warp == 8) { tmem_alloc(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish(); }
    __syncthreads();
    // weights image and per-feature constants: once per CTA
    for (int i = tid; i < b_bytes / 16; i += kFThreads) reinterpret_cast<uint4*>(sB)[i] = __ldg(reinterpret_cast<const uint4*>(P.wpacked) + i);
    for (int j = tid; j < P.ofm; j += kFThreads) {
        int32_t bi = 0; float bf = 0.f;
        if (c.bias_dtype != CLDNN_B200_NONE) { if (c.bias_dtype == CLDNN_B200_F32) bf = ((const float*)P.bias)[j]; else bi = load_as_int(P.bias, c.bias_dtype, j); }
        const float q = c.quantization ? P.quant[j] : 1.f;
        aux->bias_i[0][j] = bi; aux->bias_f[0][j] = bf;
        aux->quant[0][j] = q;
        aux->calib[0][j] = c.calibration ? P.calib[j] : 1.f;
        aux->ecal[0][j] = 1.f;
        // the conversion-free epilogue is exact while every dequantised value stays below 2^22
        if (!(__fmul_rn(__fmul_rn(__fadd_rn(P.acc_bound, fabsf((float)bi)), fabsf(q)), P.mul_oqf ? fabsf(c.o_qf) : 1.0f) < 4.0e6f)) atomicOr(&aux->wide, 1u);
    }
    for (int g = tid; g < P.groups && g < 64; g += kFThreads) { const int ch = g / P.kh, r = g - ch * P.kh; aux->goff[g] = (uint16_t)((ch * P.patch_h + r) * (P.patch_wp >> 2)); }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    const uint32_t sbo = P.sbo;
    const int my_tiles = (P.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp < 4) {
        // ------------------------------ builders ----------------------------------
        const int words_per_row = P.patch_wp >> 2;
        const int patch_words = P.C * P.patch_h * words_per_row;
        // what does not depend on the tile is computed once: where each of this thread's patch words lies relative to
        // the patch origin, and (in shared memory, by group) where each filter row starts in the patch
        int32_t rel[kMaxPre], pk[kMaxPre];
#pragma unroll
        for (int j = 0; j < kMaxPre; ++j) {
            const int i = tid + j * kBuilders;
            const int wq = i % words_per_row; const int r2 = i / words_per_row;
            const int pr = r2 % P.patch_h, ch = r2 / P.patch_h;
            rel[j] = (int32_t)(ch * P.in_pf + pr * P.in_py + wq * 4);
            pk[j] = i < patch_words ? (pr | ((wq * 4) << 8)) : -1;
        }
        const int m = tid;                                      // output pixel of the tile this thread assembles
        const int py_ = m / kTileW, px_ = m - py_ * kTileW;
        const int chunks = P.Kp >> 4;
        const uint32_t* prow = reinterpret_cast<const uint32_t*>(sPatch) + py_ * P.sy * words_per_row;
        // patch words of tile `it` of this CTA into a register set (nothing when the CTA has no such tile)
        auto fetch = [&](int it, uint32_t (&regs)[kMaxPre]) {
            if (it >= my_tiles) return;
            int tx, ty, n, x0, y0, xa;
            tile_origin(P, blockIdx.x + it * gridDim.x, tx, ty, n, x0, y0, xa);
            const uint8_t* origin = P.in + P.in_off + (int64_t)n * P.in_pb + (int64_t)y0 * P.in_py + xa;
#pragma unroll
            for (int j = 0; j < kMaxPre; ++j) regs[j] = patch_word(P, origin, rel[j], pk[j], y0, xa);
        };
        // one tile: registers -> patch in shared memory, refill the registers with the tile two ahead (those loads stay
        // in flight across this and the next tile), assemble the operand
        auto step = [&](int it, uint32_t (&regs)[kMaxPre]) -> bool {
            const int buf = it & 1;
#pragma unroll
            for (int j = 0; j < kMaxPre; ++j) if (pk[j] >= 0) reinterpret_cast<uint32_t*>(sPatch)[tid + j * kBuilders] = regs[j];
            named_bar_sync(1, kBuilders);
            fetch(it + 2, regs);
            int tx, ty, n, x0, y0, xa;
            tile_origin(P, blockIdx.x + it * gridDim.x, tx, ty, n, x0, y0, xa);
            const int colb = (x0 - xa) + px_ * P.sx;
            if (!mbar_wait(smem_u32(&aux->a_empty[buf]), (((uint32_t)(it >> 1) & 1u)) ^ 1u, s_abort, P.status, kErrFirst + 1u)) return false;
            // im2col row of pixel m: every 8-byte group is one shifted read of a patch row
            const uint32_t* pw = prow + (colb >> 2); const uint32_t sh = (uint32_t)(colb & 3) * 8u;
            uint8_t* dstrow = sA + buf * a_bytes + (m >> 3) * sbo + (m & 7) * 16;
            for (int kc = 0; kc < chunks; ++kc) {
                uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int g = kc * 2 + q;
                    if (g < P.groups) {
                        const uint32_t* rowp = pw + aux->goff[g];
                        const uint32_t w0 = rowp[0], w1 = rowp[1], w2 = rowp[2];
                        v[2 * q] = __funnelshift_r(w0, w1, sh); v[2 * q + 1] = __funnelshift_r(w1, w2, sh);
                    }
                }
                *reinterpret_cast<uint4*>(dstrow + kc * 128) = make_uint4(v[0], v[1], v[2], v[3]);
            }
            fence_async_smem();
            named_bar_sync(1, kBuilders);                       // operand complete, patch buffer free for the next tile
            if (tid == 0) mbar_arrive(smem_u32(&aux->a_full[buf]));
            return true;
        };
        uint32_t pre0[kMaxPre], pre1[kMaxPre];
#pragma unroll
        for (int j = 0; j < kMaxPre; ++j) { pre0[j] = 0u; pre1[j] = 0u; }
        fetch(0, pre0); fetch(1, pre1);
        for (int it = 0; it < my_tiles; it += 2) {
            if (!step(it, pre0)) break;
            if (it + 1 < my_tiles && !step(it + 1, pre1)) break;
        }
    } else if (warp == 8) {
        // ------------------------------ MMA issuer --------------------------------
        // the whole warp runs the loop, one elected lane issues (loop state stays on the uniform datapath)
        {
            const bool leader = elect_one();
            const int kk = P.Kp >> 5;
            const uint64_t bdesc = make_desc_interleaved(smem_u32(sB), 128u, sbo);
            for (int it = 0; it < my_tiles; ++it) {
                const int buf = it & 1; const uint32_t par = (uint32_t)(it >> 1) & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->tmem_empty[buf]), par ^ 1u, s_abort, P.status, kErrFirst + 2u))) break;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->a_full[buf]), par, s_abort, P.status, kErrFirst + 3u))) break;
                tc_fence_after();
                const uint64_t adesc = make_desc_interleaved(smem_u32(sA + buf * a_bytes), 128u, sbo);
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P.ofm);
                if (leader) {
                    for (int k = 0; k < kk; ++k)                // one instruction consumes two core matrices along K: 2 * 128 bytes
                        mma_i8_ss(d_tmem, adesc + (uint64_t)(k * 16), bdesc + (uint64_t)(k * 16), P.idesc, k ? 1u : 0u);
                    tc_commit(smem_u32(&aux->a_empty[buf]));
                    tc_commit(smem_u32(&aux->tmem_full[buf]));
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quad = warp & 3;                              // warps 4..7 -> TMEM lanes 32*quad ..
        const int row = quad * 32 + lane;
        const int py_ = row / kTileW, px_ = row - py_ * kTileW;
        // modes 0..2: conversion-free (u8 / s8 / s8 after ReLU), +4: with a uniform O_QF (modes 0 and 1 only), 3: general
        const int mode = (P.lean && !aux->wide) ? ((c.out_dtype == CLDNN_B200_U8 ? 0 : (c.act == CLDNN_B200_ACT_RELU ? 2 : 1)) + (P.mul_oqf ? 4 : 0)) : 3;
        for (int it = 0; it < my_tiles; ++it) {
            const int buf = it & 1;
            int tx, ty, n, x0, y0, xa;
            tile_origin(P, blockIdx.x + it * gridDim.x, tx, ty, n, x0, y0, xa);
            const int oy = ty * kTileH + py_, ox = tx * kTileW + px_;
            const bool valid = oy < P.P && ox < P.Q;
            uint8_t* out_row = P.out + P.out_off + (int64_t)n * P.out_pb + (int64_t)oy * P.out_py + (int64_t)ox * P.out_px;
            if (!mbar_wait(smem_u32(&aux->tmem_full[buf]), (uint32_t)(it >> 1) & 1u, s_abort, P.status, kErrFirst)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * P.ofm);
            const uint32_t te = smem_u32(&aux->tmem_empty[buf]);
            if (kCtas == 1) {
                switch (mode) {
                    case 0: first_epi_tile<0>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 1: first_epi_tile<1>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 2: first_epi_tile<2>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 4: first_epi_tile_single<0, true>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 5: first_epi_tile_single<1, true>(P, aux, t_row, out_row, valid, te, lane); break;
                    default: first_epi_tile_general(P, aux, t_row, out_row, valid, te, lane); break;
                }
            } else {
                switch (mode) {
                    case 0: first_epi_tile_single<0>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 1: first_epi_tile_single<1>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 2: first_epi_tile_single<2>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 4: first_epi_tile_single<0, true>(P, aux, t_row, out_row, valid, te, lane); break;
                    case 5: first_epi_tile_single<1, true>(P, aux, t_row, out_row, valid, te, lane); break;
                    default: first_epi_tile_general(P, aux, t_row, out_row, valid, te, lane); break;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem_base, P.tmem_cols); }
}

// ------------------------------------------------------------------------------------
static bool first_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (!is_int8(p.in.dtype) || p.w_dtype != CLDNN_B200_I8) return no("8-bit activations and weights only");
    if (p.groups != 1 || p.fused_eltw) return no("plain convolution only");
    if (p.epilogue_order != CLDNN_B200_EPILOGUE_REF) return no("reference epilogue order only");
    if (p.in.px != 1) return no("input must be planar (bfyx)");
    if (p.out.pf != 1 || !is_int8(p.out.dtype)) return no("output must be 8-bit byxf");
    if (p.kw > 8 || p.kh < 1 || p.kw < 1) return no("filter width up to 8");
    if (p.dil_x != 1 || p.dil_y != 1) return no("no dilation");
    if (p.ifm < 1 || (int64_t)p.ifm * p.kh * 8 > kFMaxK) return no("C*kh*8 must not exceed 256");
    if (p.ofm % 32 || p.ofm > kFMaxOfm || p.out.f != p.ofm || p.in.f != p.ifm) return no("output features: multiple of 32, at most 256");
    if (p.out.px % 16 || p.out.py % 16 || p.out.pb % 16 || p.out.offset % 16) return no("output pitches must be 16-byte aligned");
    if (p.stride_x < 1 || p.stride_y < 1 || p.stride_x > 4 || p.stride_y > 4) return no("stride 1..4");
    const bool quant_path = p.quantization || p.calibration || p.has_o_qf;
    if (!quant_path) return no("quantised epilogue only");
    if (!act_is_simple(p.act, p.act_m)) return no("activation not in the fast set");
    if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_I32 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    const int P_ = (p.in.y + 2 * p.pad_y - p.kh) / p.stride_y + 1, Q_ = (p.in.x + 2 * p.pad_x - p.kw) / p.stride_x + 1;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");
    const int patch_h = (kTileH - 1) * p.stride_y + p.kh, patch_wp = ((kTileW - 1) * p.stride_x + 8 + 3 + 4 + 3) / 4 * 4;
    if (p.ifm * patch_h * patch_wp / 4 > 128 * 9) return no("the input patch of one tile is too large");
    return true;
}
constexpr int kTuneRows = 4;
static bool first_supports(const void* vp)
{
    const cldnn_b200_conv_params& p = *(const cldnn_b200_conv_params*)vp;
    if (p.tune >= kTuneRows) return first_rows_plan(simplified_conv_params(p), nullptr);
    return first_plan(p, nullptr);
}
// tune 0 / 2: as many CTAs per SM as fit (at most two), 1: one CTA per SM with the double-buffered epilogue,
// 3: up to three CTAs per SM (72 registers per thread: more warps against the latency of the patch loads),
// 4, 5: the row form (conv_i8_first_rows.cu: output rows as GEMM rows, the raw image rows as the TMA-loaded operand) with two / four
// epilogue warp groups
static int first_tune_count(const void*) { return 6; }
static int first_kp(const cldnn_b200_conv_params& p) { return (p.ifm * p.kh * 8 + 31) / 32 * 32; }
static size_t first_scratch(const void* vp)
{
    const auto& p = *(const cldnn_b200_conv_params*)vp;
    if (p.tune >= kTuneRows) return first_rows_scratch(p);
    return (size_t)p.ofm * first_kp(p);
}

// Validates the arguments and fills the launch constants; `wpacked` is where the packed weights will live.
static int32_t first_setup(cldnn_b200_ctx_impl* ctx, const cldnn_b200_conv_params& p_in, const cldnn_b200_args* a, void* wpacked, size_t wpacked_bytes,
                           FirstParams& P, int& grid, size_t& smem)
{
    const cldnn_b200_conv_params p = simplified_conv_params(p_in);
    std::string why;
    if (!first_plan(p, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_first: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_first: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_first: bias_dtype set but no bias pointer");
    if (p.quantization && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_first: quantization set but no factors");
    if (p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_first: calibration set but no factors");
    const size_t need = first_scratch(&p);
    if (!wpacked || wpacked_bytes < need) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_first: needs " + std::to_string(need) + " bytes of scratch for the packed weights");
    if (((uintptr_t)wpacked | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_first: scratch and output must be 16-byte aligned");

    P = FirstParams{};
    P.N = p.in.b; P.C = p.ifm; P.H = p.in.y; P.W = p.in.x; P.P = p.out.y; P.Q = p.out.x; P.ofm = p.ofm;
    P.kh = p.kh; P.kw = p.kw; P.sx = p.stride_x; P.sy = p.stride_y; P.pad_x = p.pad_x; P.pad_y = p.pad_y;
    P.in_pb = p.in.pb; P.in_pf = p.in.pf; P.in_py = p.in.py; P.in_off = p.in.offset;
    P.groups = p.ifm * p.kh; P.Kp = first_kp(p);
    P.patch_h = (kTileH - 1) * p.stride_y + p.kh;
    P.patch_wp = ((kTileW - 1) * p.stride_x + 8 + 3 + 4 + 3) / 4 * 4;      // window + alignment slack + one spare word for the shifted read
    P.tiles_x = (P.Q + kTileW - 1) / kTileW; P.tiles_y = (P.P + kTileH - 1) / kTileH; P.total_tiles = P.N * P.tiles_x * P.tiles_y;
    const uint32_t a_fmt = p.in.dtype == CLDNN_B200_U8 ? 0u : 1u;
    P.idesc = (2u << 4) | (a_fmt << 7) | (1u << 10) | ((uint32_t)(p.ofm >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    uint32_t cols = 32; while (cols < (uint32_t)(2 * p.ofm)) cols <<= 1;   // two accumulator buffers
    P.tmem_cols = cols;
    P.acc_bound = (float)p.ifm * (float)p.kh * (float)p.kw * (p.in.dtype == CLDNN_B200_U8 ? 255.0f : 128.0f) * 128.0f;
    P.sbo = (uint32_t)(P.Kp / 16) * 128u;
    P.out_px = p.out.px; P.out_py = p.out.py; P.out_pb = p.out.pb; P.out_off = p.out.offset;
    P.epi = make_epi_cfg(p);
    P.mul_iqf = p.i_qf != 1.0f ? 1 : 0; P.mul_oqf = (p.calibration || p.o_qf != 1.0f) ? 1 : 0;
    // a uniform positive O_QF is part of the conversion-free epilogue in front of an unsigned or a plain signed saturation
    const bool oqf_ok = !P.mul_oqf || (!p.calibration && p.o_qf > 0.0f && (p.out.dtype == CLDNN_B200_U8 || p.act != CLDNN_B200_ACT_RELU));
    P.lean = (p.quantization && !P.mul_iqf && oqf_ok && !P.epi.dont_dequantize_bias &&
              (p.act == CLDNN_B200_ACT_NONE || p.act == CLDNN_B200_ACT_RELU)) ? 1 : 0;
    P.in = (const uint8_t*)a->input0; P.out = (uint8_t*)a->output; P.wpacked = (const uint8_t*)wpacked;
    P.bias = a->bias; P.quant = a->weights_quantization_factors; P.calib = a->output_calibration_factors;
    P.status = ctx->d_status;

    const int patch_bytes = P.C * P.patch_h * P.patch_wp;
    if (patch_bytes / 4 > kBuilders * kMaxPre) return fail(CLDNN_B200_UNSUPPORTED_SIZE, "conv_i8_first: the input patch of one tile is too large");
    smem = 128 + (size_t)2 * 128 * P.Kp + (size_t)P.ofm * P.Kp + ((patch_bytes + 15) & ~15) + sizeof(FirstAux);
    if (smem > (size_t)ctx->prop.sharedMemPerBlockOptin) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_i8_first: not enough shared memory");
    // the limit is shared by every prepared launch of the function on this device: it only ever grows
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_kernel<1>, ctx->device, smem));
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_kernel<2>, ctx->device, smem));
    B200_CUDA(raise_smem_limit((const void*)conv_i8_first_kernel<3>, ctx->device, smem));
    // CTAs per SM: bounded by shared memory and by tensor memory (512 columns per SM)
    int per_sm = (int)(ctx->prop.sharedMemPerMultiprocessor / (smem + 1024));
    per_sm = std::min(per_sm, std::min(p.tune == 3 ? 3 : 2, (int)(512 / P.tmem_cols)));
    if (per_sm < 1) per_sm = 1;
    if (p.tune == 1) per_sm = 1;
    P.ctas_per_sm = per_sm;
    grid = ctx->prop.multiProcessorCount * per_sm;
    if (grid > P.total_tiles) grid = P.total_tiles;
    return CLDNN_B200_SUCCESS;
}

static cudaError_t first_launch(const FirstParams& P, int grid, size_t smem, cudaStream_t s)
{
    if (P.ctas_per_sm >= 3) conv_i8_first_kernel<3><<<grid, kFThreads, smem, s>>>(P);
    else if (P.ctas_per_sm == 2) conv_i8_first_kernel<2><<<grid, kFThreads, smem, s>>>(P);
    else conv_i8_first_kernel<1><<<grid, kFThreads, smem, s>>>(P);
    return cudaGetLastError();
}

static cudaError_t first_pack(const cldnn_b200_conv_params& p, const cldnn_b200_args* a, const FirstParams& P, void* wpacked, cudaStream_t stream)
{
    first_pack_weights<<<(p.ofm * P.Kp + 255) / 256, 256, 0, stream>>>((const int8_t*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset,
                                                                        p.ofm, p.ifm, p.kh, p.kw, P.Kp, (uint8_t*)wpacked);
    return cudaGetLastError();
}

static int32_t first_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params& p = *(const cldnn_b200_conv_params*)vp;
    if (p.tune >= kTuneRows) return first_rows_prepare(ctx, p, a, out, p.tune == kTuneRows + 1 ? 4 : 2);
    FirstParams P; int grid = 0; size_t smem = 0;
    const int32_t st = first_setup(ctx, p, a, a->scratch, a->scratch_bytes, P, grid, smem);
    if (st != CLDNN_B200_SUCCESS) return st;
    // pack the weights once, on the context's stream, before anything that is prepared here can run
    B200_CUDA(first_pack(p, a, P, a->scratch, ctx->stream));
    out->fn = [P, grid, smem](cudaStream_t s) { return first_launch(P, grid, smem, s); };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

const KernelDef kdef_conv_i8_first = {"conv_i8_first", sizeof(cldnn_b200_conv_params), first_supports, first_tune_count, first_scratch, first_prepare};

// ------------------------------------------------------------------------------------
// Allocation-free variant.  The packed-weights workspace that conv_i8_first normally
// receives from its caller lives here in a fixed array inside the library image, so a
// caller that owns no device allocator can still run the first-layer convolution.
// 32 KiB holds, for example, 128 output features x 256 bytes of padded K (ResNet's 7x7x3 -> 64
// first layer needs 12 KiB); larger weight images are refused.  Every GPU that loads the
// library carries the array until exit.
// ------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = 32 * 1024;
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
static void* g_noalloc_ptr[kNoAllocMaxDevices];      // device address of the array, per device ordinal
static std::mutex g_noalloc_mutex;

// Resolves the array's device address for the context's device.  In host code the
// symbol name is only a stand-in; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static int32_t noalloc_scratch_address(cldnn_b200_ctx_impl* ctx, void** out)
{
    if (ctx->device < 0 || ctx->device >= kNoAllocMaxDevices) return fail(CLDNN_B200_INVALID_ARG, "conv_first_noalloc: device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[ctx->device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(conv_first_noalloc scratch)");
        if (!p) return fail(CLDNN_B200_DEVICE_ERROR, "conv_first_noalloc: the built-in scratch has no device address");
        g_noalloc_ptr[ctx->device] = p;
    }
    *out = g_noalloc_ptr[ctx->device];
    return CLDNN_B200_SUCCESS;
}

}  // namespace b200

extern "C" int32_t cldnn_b200_conv_first_noalloc(cldnn_b200_ctx ctx, const cldnn_b200_conv_params* params, const cldnn_b200_args* args)
{
    using namespace b200;
    if (!ctx || !params || !args) return fail(CLDNN_B200_INVALID_ARG, "conv_first_noalloc: null argument");
    {
        // shapes the kernel cannot run are refused first, with the same code conv_i8_first gives them; only then the size
        // of the packed weights (64-bit: the counts come from the caller) is held against the built-in array
        const cldnn_b200_conv_params sp = simplified_conv_params(*params);
        std::string why;
        if (!first_plan(sp, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_first_noalloc: " + why);
        const uint64_t kp = ((uint64_t)sp.ifm * (uint64_t)sp.kh * 8u + 31u) / 32u * 32u;
        const uint64_t need = (uint64_t)sp.ofm * kp;
        if (need > kNoAllocScratchBytes)
            return fail(CLDNN_B200_UNSUPPORTED_SIZE, "conv_first_noalloc: the packed weights need " + std::to_string(need) + " bytes, the built-in scratch holds " +
                                                     std::to_string(kNoAllocScratchBytes) + "; use conv_i8_first with caller-provided scratch");
    }
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); prev = -1; }
    if (prev != ctx->device) B200_CUDA(cudaSetDevice(ctx->device));
    struct Restore { int prev, cur; ~Restore() { if (prev >= 0 && prev != cur) (void)cudaSetDevice(prev); } } restore{prev, ctx->device};

    void* scratch = nullptr;
    int32_t st = noalloc_scratch_address(ctx, &scratch);
    if (st != CLDNN_B200_SUCCESS) return st;
    FirstParams P; int grid = 0; size_t smem = 0;
    st = first_setup(ctx, *params, args, scratch, kNoAllocScratchBytes, P, grid, smem);   // validates everything else, refuses what the kernel cannot do
    if (st != CLDNN_B200_SUCCESS) return st;
    // The array still holds whatever the previous call packed.  The packing kernel rewrites every byte of the image
    // this call reads (zero taps and zero K padding included), so nothing stale can leak into the result.
    B200_CUDA(first_pack(*params, args, P, scratch, ctx->stream));
    B200_CUDA(first_launch(P, grid, smem, ctx->stream));
    ctx->launches += 2;
    return CLDNN_B200_SUCCESS;
}
