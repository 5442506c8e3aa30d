// conv_f16_tc: fp16 convolution (fp16 activations x fp16 weights, fp32
// accumulation in tensor memory) as an implicit GEMM on the sm_100a tensor
// cores -- the B200 replacement for the reference's fp16 kernel family
// (cl_kernels/convolution_gpu_bfyx_os_iyx_osv16.cl, convolution_gpu_bfyx_f16*.cl,
// convolution_gpu_yxfb_yxio_b16_fp16.cl, the 1x1 and gemm-like variants), with
// bias, activation and the optional fused residual sum of
// fused_conv_eltwise_gpu_ref.cl:195-232 in the epilogue.
//
// Same structure as the 8-bit kernels: M = N*P*Q output pixels (128 per tile =
// TMEM lanes), N = output features, K = kh*kw*C; activations byxf with the
// stored feature count a multiple of 16, never materialised as im2col: one TMA
// copy per (filter tap, channel chunk) in flat 2-D, TMA-im2col or tiled 4-D
// addressing; weights oyxi.  One persistent CTA per SM: warp 0 loads operands,
// warp 1 issues tcgen05.mma kind::f16 (16 channels per instruction), warp 2
// issues the TMA stores, warp 3 loads the residual tile, warps 4..11 (two
// groups taking alternate tiles) run the epilogue:
// tcgen05.ld -> + bias -> activation -> [+ residual -> activation] -> fp16 ->
// swizzled shared-memory tile -> TMA store.
// The reference accumulates fp16 convolutions in half precision with
// device-defined rounding of mad(); parity is therefore a tolerance (1e-2
// relative), and fp32 accumulation is the accurate side of it.
#include <cuda.h>
#include <cuda_fp16.h>
#include <mutex>
#include <string>
#include "engine.hpp"
#include "sm100_ptx.cuh"

namespace b200 {

using namespace ptx;

namespace f16tc {

constexpr int kBM = 128;
constexpr int kThreads = 384;
constexpr int kEpiWarp0 = 4;
constexpr int kGroups = 2;
constexpr int kMaxStages = 8;
constexpr int kMaxBufs = 4;
constexpr int kMaxBN = 256;
constexpr uint32_t kErr = 0x60u;
// A_PATCH: stride-1 filters whose weights fit in shared memory beside the ring.  The weights of every tap stay resident; per
// channel chunk and filter COLUMN one patch of (bh + kh - 1) x bw input pixels is loaded, and the kh taps of that column read it
// from row r * bw on (128 rows each: the tile's bw x bh pixels under filter row r) -- a third of the activation bytes of one
// load per tap, and no weight traffic per tile.  The deep-pipeline layers with 64 features are bound by what an SM can take
// in per clock, so bytes are what counts there.
enum AMode { A_FLAT = 0, A_IM2COL = 1, A_TILED = 2, A_PATCH = 3 };

struct alignas(64) Params {
    CUtensorMap tmA, tmB, tmO, tmE;
    int32_t a_mode;
    int32_t N, P, Q;
    int32_t kh, kw, stride_x, stride_y, pad_x, pad_y, dil_x, dil_y;
    int32_t bk, chunks, k_steps;             // bytes of K per stage (32 / 64 / 128 = 16 / 32 / 64 channels), chunks per tap, stages per tile
    int32_t bn, n_tiles, m_tiles, total_tiles;
    int64_t M_total;
    int32_t bw, bh, bb, tiles_w, tiles_h;
    int32_t stages, a_stage_bytes, b_stage_bytes, a_tx_bytes, b_tx_bytes, ring_bytes, stage_rows;
    uint32_t sbo, layout_type, idesc, tmem_cols;
    int32_t b_total_bytes, patch_alloc;      // patch mode: all taps' weights (resident), bytes reserved per patch
    int32_t batch_tiles;                     // batched GEMM view: tiles per batch, the weight 'tap' is the batch index (0 = plain convolution)
    int32_t ofm, fused, bias_dtype, act, eltw_act;
    float act_m, act_n, eltw_m, eltw_n;
    const void* bias;
    uint32_t* status;
};

struct Aux {
    uint64_t full[kMaxStages], empty[kMaxStages];
    uint64_t tmem_full[kMaxBufs], tmem_empty[kMaxBufs], res_full[kMaxBufs], stage_free[kMaxBufs], out_ready[kMaxBufs];
    uint64_t b_full;                         // patch mode: the resident weights have landed
    uint32_t tmem_base, abort;
    alignas(16) float bias[kGroups][kMaxBN];
};

__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout_type)
{
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | ((layout_type & 7u) << 29);
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3ffffu) >> 4) | (1u << 16); }
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi)
{
    uint64_t d; asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi)); return d;
}
template <int KK>
__device__ __forceinline__ void mma_chunk(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t acc_first)
{
#pragma unroll
    for (int k = 0; k < KK; ++k)
        mma_f16_ss(d_tmem, desc64(a_lo + 2u * k, hi), desc64(b_lo + 2u * k, hi), idesc, k ? 1u : acc_first);
}

// the activations outside NONE / ReLU stay out of line: the unrolled epilogue body would otherwise carry 64 copies
__device__ __noinline__ float act_other(int32_t fn, float x, float m, float n) { return act_float(fn, x, m, n); }
__device__ __forceinline__ float act_apply(int32_t fn, float x, float m, float n)
{
    if (fn == CLDNN_B200_ACT_NONE) return x;
    if (fn == CLDNN_B200_ACT_RELU) return fmaxf(0.0f, x);
    return act_other(fn, x, m, n);
}

// 32 features of one pixel: fp32 accumulators -> 32 halves (four 16-byte words)
template <bool kFused>
__device__ __forceinline__ void chunk32(const Params& P, const uint32_t (&r)[32], const float* bias, uint4* (&p)[4])
{
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        uint32_t ew[4] = {0, 0, 0, 0};
        if (kFused) { const uint4 e = *p[w]; ew[0] = e.x; ew[1] = e.y; ew[2] = e.z; ew[3] = e.w; }
        const float4 b0 = reinterpret_cast<const float4*>(bias)[2 * w], b1 = reinterpret_cast<const float4*>(bias)[2 * w + 1];
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint32_t ow[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float v0 = act_apply(P.act, __uint_as_float(r[8 * w + 2 * h]) + bb[2 * h], P.act_m, P.act_n);
            float v1 = act_apply(P.act, __uint_as_float(r[8 * w + 2 * h + 1]) + bb[2 * h + 1], P.act_m, P.act_n);
            if (kFused) {
                // the convolution's result is a half in the reference before the sum: round it there too
                const __half2 c = __floats2half2_rn(v0, v1);
                const float2 cf = __half22float2(c);
                const float2 e = __half22float2(*reinterpret_cast<const __half2*>(&ew[h]));
                v0 = act_apply(P.eltw_act, cf.x + e.x, P.eltw_m, P.eltw_n);
                v1 = act_apply(P.eltw_act, cf.y + e.y, P.eltw_m, P.eltw_n);
            }
            const __half2 o = __floats2half2_rn(v0, v1);
            ow[h] = *reinterpret_cast<const uint32_t*>(&o);
        }
        *p[w] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// staging tile: column blocks of 64 halves (128 bytes, 128B swizzle), 128 rows each
__device__ __forceinline__ void chunk_ptrs(uint8_t* stg, int row, uint32_t sw, int c0, uint4* (&p)[4])
{
    const int cb = c0 >> 6, o = (c0 & 63) * 2;                      // byte offset inside the 128-byte row
    uint8_t* rowp = stg + (size_t)cb * kBM * 128 + (size_t)row * 128;
#pragma unroll
    for (int w = 0; w < 4; ++w) p[w] = reinterpret_cast<uint4*>(rowp + ((((uint32_t)o >> 4) + (uint32_t)w) ^ sw) * 16u);
}

template <int BN, bool kFused>
__global__ void __launch_bounds__(kThreads, 1)
conv_f16_tc_kernel(const __grid_constant__ Params P)
{
    constexpr int NBUF = BN >= 256 ? 2 : 4;                          // fp32 accumulators: BN columns each, 512 in all
    // Staging goes by units of up to 128 features (32 KiB): a 256-feature tile is converted and stored in two halves through
    // the same two unit buffers, which leaves 64 KiB more of shared memory to the operand ring than whole-tile staging would
    // (the deep layers are bound by the bytes the ring keeps in flight, not by the epilogue).  Each epilogue group owns one unit
    // buffer and fills it for the halves of its tiles in turn (use n = (local tile / 2) * UNITS + half, barrier parity n & 1):
    // every use of a buffer waits for the use directly before it, by the same group, so a parity wait can never be two
    // phases ahead of its barrier.  The store and residual warps serve the units in the order
    // (tile i, half 0), (tile i + 1, half 0), (tile i, half 1), (tile i + 1, half 1), i even, which keeps each buffer's order.
    constexpr int NSTG = 2;                                          // unit buffers = epilogue groups
    constexpr int UNITS = BN > 128 ? BN / 128 : 1;                   // units per tile
    constexpr int UW = BN / UNITS;                                   // features per unit
    constexpr int COLB = UW / 64;                                    // 64-half column blocks per unit
    constexpr uint32_t kStagingBytes = (uint32_t)(kBM * UW * 2);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t a_base = base;
    const uint32_t b_base = base + (uint32_t)(P.stages * P.a_stage_bytes);
    uint8_t* staging = smem + (uint32_t)P.ring_bytes;
    Aux* aux = reinterpret_cast<Aux*>(smem + (uint32_t)P.ring_bytes + (uint32_t)NSTG * kStagingBytes);
    volatile uint32_t* s_abort = &aux->abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P.stages; ++s) { mbar_init(smem_u32(&aux->full[s]), 1); mbar_init(smem_u32(&aux->empty[s]), 1); }
        for (int a = 0; a < kMaxBufs; ++a) {
            mbar_init(smem_u32(&aux->tmem_full[a]), 1); mbar_init(smem_u32(&aux->tmem_empty[a]), 4);
            mbar_init(smem_u32(&aux->res_full[a]), 1); mbar_init(smem_u32(&aux->stage_free[a]), 1);
            mbar_init(smem_u32(&aux->out_ready[a]), 4);
        }
        mbar_init(smem_u32(&aux->b_full), 1);
        aux->abort = 0u;
        mbar_fence_init();
        prefetch_tensormap(&P.tmA); prefetch_tensormap(&P.tmB); prefetch_tensormap(&P.tmO);
        if (kFused) prefetch_tensormap(&P.tmE);
    }
    if (warp == 1) { tmem_alloc(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    const bool patch = P.a_mode == A_PATCH;
    const bool boxed = P.a_mode == A_TILED || patch;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        // The whole warp walks the tiles and waits on the barriers, one elected lane issues the copies: a warp-uniform loop
        // lets the compiler keep its state on the uniform datapath, which a loop inside a one-lane branch cannot use.
        {
            const bool leader = elect_one();
            int stage = 0; uint32_t phase = 0; int64_t issued = 0; bool ok = true;
            const int bke = P.bk >> 1;                               // channels per chunk
            if (patch && leader && blockIdx.x < (unsigned)P.total_tiles) {
                // every tap's weights, once per CTA (one feature tile in this mode)
                const uint32_t bf = smem_u32(&aux->b_full);
                mbar_expect_tx(bf, (uint32_t)P.b_total_bytes);
                uint32_t dst = b_base;
                for (int tp = 0; tp < P.kh * P.kw; ++tp)
                    for (int ch = 0; ch < P.chunks; ++ch, dst += (uint32_t)P.b_stage_bytes) tma_load_3d(dst, &P.tmB, bf, ch * bke, tp, 0);
            }
            for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x) {
                const int n_tile = tile / P.m_tiles, m_tile = tile - n_tile * P.m_tiles;
                int c_w = 0, c_h = 0, c_n = 0;
                if (P.a_mode == A_IM2COL) {
                    const int64_t m = (int64_t)m_tile * kBM; const int pq = P.P * P.Q;
                    const int n = (int)(m / pq); const int rr = (int)(m - (int64_t)n * pq); const int p = rr / P.Q, q = rr - p * P.Q;
                    c_w = q * P.stride_x - P.pad_x; c_h = p * P.stride_y - P.pad_y; c_n = n;
                } else if (boxed) {
                    const int tw = m_tile % P.tiles_w; const int t2 = m_tile / P.tiles_w;
                    c_w = tw * P.bw - P.pad_x; c_h = (t2 % P.tiles_h) * P.bh - P.pad_y; c_n = (t2 / P.tiles_h) * P.bb;
                }
                int tap = P.batch_tiles ? m_tile / P.batch_tiles : 0, cc = 0, r = 0, s = 0;
                for (int ks = 0; ks < P.k_steps; ++ks) {
                    if (!__all_sync(0xffffffffu, mbar_wait_lean(smem_u32(&aux->empty[stage]), phase ^ 1u, s_abort, P.status, kErr))) { ok = false; break; }
                    const uint32_t full = smem_u32(&aux->full[stage]);
                    const uint32_t a_dst = a_base + (uint32_t)(stage * P.a_stage_bytes);
                    const uint32_t b_dst = b_base + (uint32_t)(stage * P.b_stage_bytes);
                    const int c0 = cc * bke;
                    if (leader && patch) {
                        mbar_expect_tx(full, (uint32_t)P.a_tx_bytes);
                        for (int sc = 0; sc < P.kw; ++sc) tma_load_4d(a_dst + (uint32_t)(sc * P.patch_alloc), &P.tmA, full, c0, c_w + sc, c_h, c_n);
                    } else if (leader) {
                        mbar_expect_tx(full, (uint32_t)(P.a_tx_bytes + P.b_tx_bytes));
                        if (P.a_mode == A_FLAT) tma_load_2d(a_dst, &P.tmA, full, c0, m_tile * kBM);
                        else if (P.a_mode == A_IM2COL) tma_load_im2col_4d(a_dst, &P.tmA, full, c0, c_w, c_h, c_n, (uint16_t)(s * P.dil_x), (uint16_t)(r * P.dil_y));
                        else tma_load_4d(a_dst, &P.tmA, full, c0, c_w + s * P.dil_x, c_h + r * P.dil_y, c_n);
                        tma_load_3d(b_dst, &P.tmB, full, c0, tap, n_tile * BN);
                    }
                    ++issued;
                    if (++cc == P.chunks) { cc = 0; ++tap; if (++s == P.kw) { s = 0; ++r; } }
                    if (++stage == P.stages) { stage = 0; phase ^= 1u; }
                }
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
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        {
            const bool leader = elect_one();
            const uint32_t hi = desc_hi(P.sbo, P.layout_type);
            const uint32_t a_lo0 = desc_lo(a_base), b_lo0 = desc_lo(b_base);
            const uint32_t a_step = (uint32_t)P.a_stage_bytes >> 4, b_step = (uint32_t)P.b_stage_bytes >> 4;
            const uint32_t full0 = smem_u32(&aux->full[0]), empty0 = smem_u32(&aux->empty[0]);
            const int kk = P.bk >> 5, stages = P.stages, k_steps = P.k_steps;
            const uint32_t idesc = P.idesc;
            int stage = 0; uint32_t phase = 0; bool ok = true; int t = 0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            const uint32_t patch_step = (uint32_t)P.patch_alloc >> 4, row_step = (uint32_t)(P.bw * P.bk) >> 4;
            const uint32_t b_chunk = (uint32_t)P.b_stage_bytes >> 4;
            if (patch && blockIdx.x < (unsigned)P.total_tiles) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->b_full), 0u, s_abort, P.status, kErr + 7u));
            for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x, ++t) {
                const int acc = t % NBUF;
                if (!__all_sync(0xffffffffu, mbar_wait_lean(smem_u32(&aux->tmem_empty[acc]), (((uint32_t)(t / NBUF) & 1u)) ^ 1u, s_abort, P.status, kErr + 1u))) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                uint32_t accf = 0u;
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!__all_sync(0xffffffffu, mbar_wait_lean(full0 + 8u * (uint32_t)stage, phase, s_abort, P.status, kErr + 2u))) { ok = false; break; }
                    if (leader && patch) {
                        // channel chunk ks: per filter column sc one patch; its rows r * bw .. r * bw + 127 are the tile under filter row r
                        uint32_t af = accf;
                        for (int sc = 0; sc < P.kw; ++sc)
                            for (int r = 0; r < P.kh; ++r) {
                                const uint32_t al = a_lo + (uint32_t)sc * patch_step + (uint32_t)r * row_step;
                                const uint32_t bl = b_lo0 + (uint32_t)((r * P.kw + sc) * P.chunks + ks) * b_chunk;
                                if (kk == 4) mma_chunk<4>(d_tmem, al, bl, hi, idesc, af);
                                else if (kk == 2) mma_chunk<2>(d_tmem, al, bl, hi, idesc, af);
                                else mma_chunk<1>(d_tmem, al, bl, hi, idesc, af);
                                af = 1u;
                            }
                        tc_commit(empty0 + 8u * (uint32_t)stage);
                    } else if (leader) {
                        if (kk == 4) mma_chunk<4>(d_tmem, a_lo, b_lo, hi, idesc, accf);
                        else if (kk == 2) mma_chunk<2>(d_tmem, a_lo, b_lo, hi, idesc, accf);
                        else mma_chunk<1>(d_tmem, a_lo, b_lo, hi, idesc, accf);
                        tc_commit(empty0 + 8u * (uint32_t)stage);
                    }
                    accf = 1u;
                    if (++stage == stages) { stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0; }
                    else { a_lo += a_step; b_lo += b_step; }
                }
                if (ok && leader) tc_commit(smem_u32(&aux->tmem_full[acc]));
            }
        }
    } else if (warp == 2) {
        // ------------------------------ TMA store issuer --------------------------
        {
            const bool leader = elect_one();                           // issues, commits and waits for the stores: bulk groups are per thread
            bool alive = true;
            for (int i0 = 0; alive && (int64_t)blockIdx.x + (int64_t)i0 * gridDim.x < P.total_tiles; i0 += 2) {
                for (int h = 0; h < UNITS && alive; ++h) {
                    for (int g = 0; g < 2 && alive; ++g) {
                        const int64_t tile64 = (int64_t)blockIdx.x + (int64_t)(i0 + g) * gridDim.x;
                        if (tile64 >= P.total_tiles) break;
                        const int tile = (int)tile64;
                        const int n_tile = tile / P.m_tiles, m_tile = tile - n_tile * P.m_tiles;
                        const int n = (i0 >> 1) * UNITS + h;               // this buffer's use count
                        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->out_ready[g]), (uint32_t)n & 1u, s_abort, P.status, kErr + 3u))) { alive = false; break; }
                        if (!leader) continue;
                        int tw = 0, th = 0, tb = 0;
                        if (boxed) { tw = m_tile % P.tiles_w; const int t2 = m_tile / P.tiles_w; th = t2 % P.tiles_h; tb = t2 / P.tiles_h; }
#pragma unroll
                        for (int cb = 0; cb < COLB; ++cb) {
                            const int f0 = n_tile * BN + h * UW + cb * 64;
                            if (f0 >= P.ofm) break;
                            const uint32_t src = smem_u32(staging) + (uint32_t)g * kStagingBytes + (uint32_t)(cb * kBM * 128);
                            if (boxed) tma_store_4d(&P.tmO, src, f0, tw * P.bw, th * P.bh, tb * P.bb);
                            else tma_store_2d(&P.tmO, src, f0, m_tile * kBM);
                        }
                        bulk_commit();
                        bulk_wait_read0();
                        mbar_arrive(smem_u32(&aux->stage_free[g]));
                    }
                }
            }
        }
    } else if (warp == 3) {
        // ------------------------------ residual loader ---------------------------
        if (kFused) {
            const bool leader = elect_one();
            bool alive = true;
            for (int i0 = 0; alive && (int64_t)blockIdx.x + (int64_t)i0 * gridDim.x < P.total_tiles; i0 += 2) {
                for (int h = 0; h < UNITS && alive; ++h) {
                    for (int g = 0; g < 2 && alive; ++g) {
                        const int64_t tile64 = (int64_t)blockIdx.x + (int64_t)(i0 + g) * gridDim.x;
                        if (tile64 >= P.total_tiles) break;
                        const int tile = (int)tile64;
                        const int n_tile = tile / P.m_tiles, m_tile = tile - n_tile * P.m_tiles;
                        int o_w = 0, o_h = 0, c_n = 0;
                        if (boxed) { const int tw = m_tile % P.tiles_w; const int t2 = m_tile / P.tiles_w; o_w = tw * P.bw; o_h = (t2 % P.tiles_h) * P.bh; c_n = (t2 / P.tiles_h) * P.bb; }
                        const int n = (i0 >> 1) * UNITS + h;
                        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->stage_free[g]), ((uint32_t)n & 1u) ^ 1u, s_abort, P.status, kErr + 4u))) { alive = false; break; }
                        if (!leader) continue;
                        const uint32_t rf = smem_u32(&aux->res_full[g]);
                        int cbs = 0;
                        for (int cb = 0; cb < COLB; ++cb) if (n_tile * BN + h * UW + cb * 64 < P.ofm) ++cbs;
                        mbar_expect_tx(rf, (uint32_t)(P.stage_rows * 128 * cbs));
                        for (int cb = 0; cb < cbs; ++cb) {
                            const uint32_t dst = smem_u32(staging) + (uint32_t)g * kStagingBytes + (uint32_t)(cb * kBM * 128);
                            const int f0 = n_tile * BN + h * UW + cb * 64;
                            if (boxed) tma_load_4d(dst, &P.tmE, rf, f0, o_w, o_h, c_n);
                            else tma_load_2d(dst, &P.tmE, rf, f0, m_tile * kBM);
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int ew = warp - kEpiWarp0;
        const int quad = ew & 3, group = ew >> 2;
        const int row = quad * 32 + lane;
        const int gt = quad * 32 + lane;
        const uint32_t sw = (uint32_t)row & 7u;
        int cur_n_tile = -1; bool ok = true;
        int t = group;
        for (int tile = blockIdx.x + group * gridDim.x; tile < P.total_tiles && ok; tile += kGroups * gridDim.x, t += kGroups) {
            const int n_tile = tile / P.m_tiles;
            const int acc = t % NBUF;
            if (n_tile != cur_n_tile) {
                named_bar_sync(1 + group, 128);
                for (int j = gt; j < BN; j += 128) {
                    const int f = n_tile * BN + j;
                    float b = 0.0f;
                    if (f < P.ofm && P.bias_dtype != CLDNN_B200_NONE) b = load_as_float(P.bias, P.bias_dtype, f);
                    aux->bias[group][j] = b;
                }
                named_bar_sync(1 + group, 128);
                cur_n_tile = n_tile;
            }
            if (!mbar_wait(smem_u32(&aux->tmem_full[acc]), (uint32_t)(t / NBUF) & 1u, s_abort, P.status, kErr + 5u)) { ok = false; break; }
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
            const float* bias = aux->bias[group];
            for (int h = 0; h < UNITS && ok; ++h) {
                const int n = (t >> 1) * UNITS + h, sb = group;       // this group's buffer, its use count
                const bool got = kFused ? mbar_wait(smem_u32(&aux->res_full[sb]), (uint32_t)n & 1u, s_abort, P.status, kErr + 6u)
                                        : mbar_wait(smem_u32(&aux->stage_free[sb]), ((uint32_t)n & 1u) ^ 1u, s_abort, P.status, kErr + 6u);
                if (!got) { ok = false; break; }
                tc_fence_after();
                uint8_t* stg = staging + (size_t)sb * kStagingBytes;
#pragma unroll 1
                for (int c0 = h * UW; c0 < (h + 1) * UW; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
                    if (c0 + 32 >= BN) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(smem_u32(&aux->tmem_empty[acc])); }
                    if (n_tile * BN + c0 >= P.ofm) continue;
                    uint4* p[4];
                    chunk_ptrs(stg, row, sw, c0 - h * UW, p);
                    chunk32<kFused>(P, r, bias + c0, p);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->out_ready[sb]));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, P.tmem_cols); }
}

}  // namespace f16tc

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
using f16tc::Params;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn h_encode_tiled = nullptr;
static EncodeIm2colFn h_encode_im2col = nullptr;

static bool f16_driver_entry_points()
{
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr; cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            h_encode_tiled = (EncodeTiledFn)fn;
        fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            h_encode_im2col = (EncodeIm2colFn)fn;
        (void)cudaGetLastError();
    });
    return h_encode_tiled && h_encode_im2col;
}

struct F16Plan { int a_mode, bn, bk, bw, bh, bb; };
static const int kF16TuneBN[3] = {64, 128, 256};
// tune index -> (addressing mode, feature tile): 1 + mode * 3 + {64, 128, 256}; 0 = automatic
static int f16_tune_count(const void*) { return 1 + 4 * 3; }           // 1 + 3 * mode + feature tile; modes flat / im2col / tiled / patch
constexpr size_t kF16PatchWeightBytes = 80 * 1024;                  // largest weight tensor the patch mode keeps resident

static bool f16_dense(const cldnn_b200_tensor& t) { return t.py == t.px * t.x && t.pb == t.py * t.y; }

static void f16_choose_box(int Q, int Pn, int N, int& bw, int& bh, int& bb)
{
    double best = -1.0; bw = 1; bh = 1; bb = 1;
    for (int w = 1; w <= Q && w <= 128; ++w)
        for (int h = 1; h <= Pn && w * h <= 128; ++h) {
            int b = 128 / (w * h); if (b > N) b = N; if (b < 1) continue;
            const double tiles = (double)((Q + w - 1) / w) * ((Pn + h - 1) / h) * ((N + b - 1) / b);
            const double score = ((double)Q * Pn * N) / (tiles * 128.0) + 1e-4 * w + 1e-6 * h;
            if (score > best) { best = score; bw = w; bh = h; bb = b; }
        }
}

// patch mode: a tile of tw x th output pixels of one image (tw * th <= 128); fewest wasted tile rows first, then least traffic
static void f16_choose_patch(int Q, int Pn, int kh, int kw, int& tw, int& th)
{
    double best = -1.0; tw = 1; th = 1;
    for (int w = 1; w <= Q && w <= 128; ++w)
        for (int h = 1; h <= Pn && w * h <= 128; ++h) {
            if (h + kh - 1 > 256) continue;
            const double tiles = (double)((Q + w - 1) / w) * ((Pn + h - 1) / h);
            const double eff = ((double)Q * Pn) / (tiles * 128.0);
            const double traffic = tiles * kw * (h + kh - 1) * w / ((double)Q * Pn * kh * kw);   // relative to one load per tap
            const double score = eff - 0.25 * traffic;
            if (score > best) { best = score; tw = w; th = h; }
        }
}

static bool f16_plan(const cldnn_b200_conv_params& p, F16Plan& pl, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (p.in.dtype != CLDNN_B200_F16 || p.w_dtype != CLDNN_B200_F16 || p.out.dtype != CLDNN_B200_F16) return no("fp16 activations, weights and output only");
    if (p.groups != 1) return no("grouped convolution is handled by other kernels");
    if (p.quantization || p.calibration || p.has_o_qf) return no("no quantisation on the fp16 path");
    if (p.kh < 1 || p.kw < 1 || p.kh * p.kw > 255 || p.stride_x < 1 || p.stride_y < 1 || p.dil_x < 1 || p.dil_y < 1) return no("filter geometry");
    if (p.out.f != p.ofm || p.in.f != p.ifm) return no("feature counts");
    // pitches are in elements
    if (p.in.pf != 1 || p.in.px % 16 || p.in.py % 8 || p.in.pb % 8 || p.in.offset % 8 || p.in.px < p.in.f || p.in.py < p.in.px * p.in.x || p.in.pb < p.in.py * p.in.y)
        return no("input must be byxf with the stored feature count a multiple of 16");
    if (p.out.pf != 1 || p.out.px % 8 || p.out.py % 8 || p.out.pb % 8 || p.out.offset % 8) return no("output must be byxf with 16-byte aligned pitches");
    if (p.w_pi != 1 || p.w_px != p.in.px || p.w_py != p.w_px * p.kw || p.w_po % 8 || p.w_offset % 8) return no("weights must be oyxi with the input's stored feature count");
    if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_F16 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    if (p.fused_eltw) {
        const cldnn_b200_tensor& e = p.in_out_opt ? p.out : p.eltw;
        if (e.dtype != CLDNN_B200_F16 || e.pf != 1 || e.px % 8 || e.py % 8 || e.pb % 8 || e.offset % 8) return no("residual must be fp16 byxf with 16-byte aligned pitches");
        if (p.has_non_conv_scale || p.eltw_calibration) return no("no scales on the fp16 residual");
    }
    const int P_ = (p.in.y + 2 * p.pad_y - ((p.kh - 1) * p.dil_y + 1)) / p.stride_y + 1;
    const int Q_ = (p.in.x + 2 * p.pad_x - ((p.kw - 1) * p.dil_x + 1)) / p.stride_x + 1;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");

    const int cs = (int)p.in.px;                                    // stored channels
    pl.bk = cs % 64 == 0 ? 128 : (cs % 32 == 0 ? 64 : 32);          // bytes of K per stage
    const bool is_1x1_s1 = p.kh == 1 && p.kw == 1 && p.stride_x == 1 && p.stride_y == 1 && p.pad_x == 0 && p.pad_y == 0 && f16_dense(p.in);
    const bool pointwise = p.kh == 1 && p.kw == 1 && p.pad_x == 0 && p.pad_y == 0;
    const bool tiled_ok = (p.stride_x == 1 && p.stride_y == 1) || pointwise;
    const bool im2col_ok = p.pad_x <= 127 && p.pad_y <= 127 && (p.kw - 1) * p.dil_x <= 255 && (p.kh - 1) * p.dil_y <= 255 &&
                           p.stride_x <= 8 && p.stride_y <= 8 && (int64_t)p.in.b * p.in.pb * 2 >= 131072;
    int mode = -1, bn = 0;
    if (p.tune > 0) { mode = (p.tune - 1) / 3; bn = kF16TuneBN[(p.tune - 1) % 3]; }
    if (mode < 0) mode = is_1x1_s1 ? f16tc::A_FLAT : (im2col_ok ? f16tc::A_IM2COL : f16tc::A_TILED);
    if (mode == f16tc::A_FLAT && !is_1x1_s1) return no("flat addressing needs a dense 1x1 stride-1 convolution");
    if (mode == f16tc::A_TILED && !tiled_ok) return no("tiled addressing needs stride 1 or a pointwise filter");
    if (mode == f16tc::A_IM2COL && !im2col_ok) return no("im2col addressing limits exceeded (or tensor below 128 KiB)");
    if (bn == 0) bn = p.ofm > 128 ? 256 : (p.ofm > 64 ? 128 : 64);
    if (mode == f16tc::A_PATCH) {
        if (p.stride_x != 1 || p.stride_y != 1 || p.dil_x != 1 || p.dil_y != 1 || p.kh * p.kw == 1) return no("patch mode needs a stride-1 undilated filter larger than 1x1");
        if (p.ofm > bn) return no("patch mode keeps one feature tile's weights resident: output features within one tile");
        if ((size_t)p.kh * p.kw * cs * 2 * bn > kF16PatchWeightBytes) return no("patch mode keeps all weights in shared memory: at most 80 KiB");
    }
    pl.a_mode = mode; pl.bn = bn; pl.bw = pl.bh = pl.bb = 1;
    if (mode == f16tc::A_TILED) f16_choose_box(p.out.x, p.out.y, p.out.b, pl.bw, pl.bh, pl.bb);
    if (mode == f16tc::A_PATCH) f16_choose_patch(p.out.x, p.out.y, p.kh, p.kw, pl.bw, pl.bh);
    // TMA needs the flat output / residual views pixel-dense; the tiled and patch modes take pitches
    if (mode != f16tc::A_TILED && mode != f16tc::A_PATCH) {
        if (!f16_dense(p.out)) return no("flat and im2col addressing need a pixel-dense output");
        if (p.fused_eltw && !p.in_out_opt && (!f16_dense(p.eltw) || p.eltw_stride_x != 1 || p.eltw_stride_y != 1)) return no("flat and im2col addressing need a pixel-dense unstrided residual");
    }
    return true;
}
static bool f16_supports(const void* vp) { F16Plan pl; return f16_plan(*(const cldnn_b200_conv_params*)vp, pl, nullptr); }

static CUresult f16_pixel_map(CUtensorMap* tm, const F16Plan& pl, void* ptr, const cldnn_b200_tensor& t, int ofm, int sx, int sy)
{
    if (pl.a_mode == f16tc::A_TILED || pl.a_mode == f16tc::A_PATCH) {
        cuuint64_t dims[4] = {(cuuint64_t)ofm, (cuuint64_t)((t.x + sx - 1) / sx), (cuuint64_t)((t.y + sy - 1) / sy), (cuuint64_t)t.b};
        cuuint64_t strides[3] = {(cuuint64_t)(t.px * sx * 2), (cuuint64_t)(t.py * sy * 2), (cuuint64_t)(t.pb * 2)};
        cuuint32_t box[4] = {64, (cuuint32_t)pl.bw, (cuuint32_t)pl.bh, (cuuint32_t)pl.bb};
        cuuint32_t es[4] = {1, 1, 1, 1};
        return h_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    cuuint64_t dims[2] = {(cuuint64_t)ofm, (cuuint64_t)((int64_t)t.b * t.y * t.x)};
    cuuint64_t strides[1] = {(cuuint64_t)(t.px * 2)};
    cuuint32_t box[2] = {64, (cuuint32_t)f16tc::kBM};
    cuuint32_t es[2] = {1, 1};
    return h_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

template <int BN, bool kFused>
static cudaError_t f16_launch_inst(const Params& P, int grid, size_t smem, cudaStream_t s)
{
    f16tc::conv_f16_tc_kernel<BN, kFused><<<grid, f16tc::kThreads, smem, s>>>(P);
    return cudaGetLastError();
}
static cudaError_t f16_launch(const Params& P, int grid, size_t smem, cudaStream_t s)
{
    const bool f = P.fused != 0;
    switch (P.bn) {
    case 64:  return f ? f16_launch_inst<64, true>(P, grid, smem, s) : f16_launch_inst<64, false>(P, grid, smem, s);
    case 128: return f ? f16_launch_inst<128, true>(P, grid, smem, s) : f16_launch_inst<128, false>(P, grid, smem, s);
    default:  return f ? f16_launch_inst<256, true>(P, grid, smem, s) : f16_launch_inst<256, false>(P, grid, smem, s);
    }
}
// The dynamic shared-memory limit belongs to (function, device): it is raised to the device maximum every time a launch
// is prepared, with the context's device current, so that each GPU of a process gets it and nothing is kept in a
// process-wide flag.
static cudaError_t f16_configure(const Params& P, int max_smem)
{
    const bool f = P.fused != 0;
    const void* fn;
    switch (P.bn) {
    case 64:  fn = f ? (const void*)f16tc::conv_f16_tc_kernel<64, true> : (const void*)f16tc::conv_f16_tc_kernel<64, false>; break;
    case 128: fn = f ? (const void*)f16tc::conv_f16_tc_kernel<128, true> : (const void*)f16tc::conv_f16_tc_kernel<128, false>; break;
    default:  fn = f ? (const void*)f16tc::conv_f16_tc_kernel<256, true> : (const void*)f16tc::conv_f16_tc_kernel<256, false>; break;
    }
    return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

static int32_t f16_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params& p = *(const cldnn_b200_conv_params*)vp;
    F16Plan pl; std::string why;
    if (!f16_plan(p, pl, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_f16_tc: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_tc: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_tc: bias_dtype set but no bias pointer");
    if (p.fused_eltw && !p.in_out_opt && !a->input1) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_tc: fused eltwise needs a second input");
    if (((uintptr_t)a->input0 | (uintptr_t)a->weights | (uintptr_t)a->output | (uintptr_t)(p.fused_eltw && !p.in_out_opt ? a->input1 : nullptr)) & 15)
        return fail(CLDNN_B200_INVALID_ARG, "conv_f16_tc: buffers must be 16-byte aligned");
    if (!f16_driver_entry_points()) return fail(CLDNN_B200_DEVICE_ERROR, "conv_f16_tc: the CUDA driver does not export cuTensorMapEncodeTiled/Im2col");

    Params P{};
    P.a_mode = pl.a_mode;
    P.N = p.out.b; P.P = p.out.y; P.Q = p.out.x;
    P.kh = p.kh; P.kw = p.kw; P.stride_x = p.stride_x; P.stride_y = p.stride_y; P.pad_x = p.pad_x; P.pad_y = p.pad_y; P.dil_x = p.dil_x; P.dil_y = p.dil_y;
    const int cs = (int)p.in.px;
    const int bke = pl.bk / 2;
    P.bk = pl.bk; P.chunks = cs / bke; P.k_steps = p.kh * p.kw * P.chunks;
    P.bn = pl.bn; P.n_tiles = (p.ofm + pl.bn - 1) / pl.bn;
    P.M_total = (int64_t)P.N * P.P * P.Q;
    P.bw = pl.bw; P.bh = pl.bh; P.bb = pl.bb;
    const bool patch = pl.a_mode == f16tc::A_PATCH;
    const bool boxed = pl.a_mode == f16tc::A_TILED || patch;
    if (boxed) {
        P.tiles_w = (P.Q + pl.bw - 1) / pl.bw; P.tiles_h = (P.P + pl.bh - 1) / pl.bh;
        P.m_tiles = P.tiles_w * P.tiles_h * ((P.N + pl.bb - 1) / pl.bb);
    } else { P.tiles_w = P.tiles_h = 1; P.m_tiles = (int)((P.M_total + f16tc::kBM - 1) / f16tc::kBM); }
    P.total_tiles = P.m_tiles * P.n_tiles;
    P.stage_rows = boxed ? pl.bw * pl.bh * pl.bb : f16tc::kBM;
    P.a_stage_bytes = f16tc::kBM * pl.bk; P.b_stage_bytes = pl.bn * pl.bk;
    P.a_tx_bytes = P.stage_rows * pl.bk; P.b_tx_bytes = pl.bn * pl.bk;
    if (patch) {
        // a stage holds the kw patches of one channel chunk; the tensor core reads 128 rows from row r * bw, r < kh
        const int patch_rows = (pl.bh + p.kh - 1) * pl.bw, read_rows = (p.kh - 1) * pl.bw + f16tc::kBM;
        P.k_steps = P.chunks;
        P.patch_alloc = (((patch_rows > read_rows ? patch_rows : read_rows) * pl.bk) + 1023) / 1024 * 1024;
        P.a_tx_bytes = p.kw * patch_rows * pl.bk;
        P.a_stage_bytes = p.kw * P.patch_alloc;
        P.b_total_bytes = p.kh * p.kw * P.chunks * P.b_stage_bytes;
    }
    P.sbo = 8u * (uint32_t)pl.bk;
    P.layout_type = pl.bk == 128 ? 2u : (pl.bk == 64 ? 4u : 6u);
    // instruction descriptor: f32 accumulate, f16 x f16, both K-major, N, M
    P.idesc = (1u << 4) | ((uint32_t)(pl.bn >> 3) << 17) | ((uint32_t)(f16tc::kBM >> 4) << 24);
    const int nbuf = pl.bn >= 256 ? 2 : 4;
    P.tmem_cols = (uint32_t)(nbuf * pl.bn);
    P.ofm = p.ofm; P.fused = p.fused_eltw; P.bias_dtype = p.bias_dtype; P.act = p.act; P.eltw_act = p.eltw_act;
    P.act_m = p.act_m; P.act_n = p.act_n; P.eltw_m = p.eltw_m; P.eltw_n = p.eltw_n;
    P.bias = a->bias; P.status = ctx->d_status;

    const size_t max_smem = (size_t)ctx->prop.sharedMemPerBlockOptin;
    const size_t resident = patch ? (size_t)P.b_total_bytes : 0;
    const size_t stage_bytes = (size_t)P.a_stage_bytes + (patch ? 0 : P.b_stage_bytes);
    const size_t staging_total = (size_t)2 * f16tc::kBM * (pl.bn > 128 ? 128 : pl.bn) * 2;   // two unit buffers of up to 128 features
    const size_t aux_bytes = sizeof(f16tc::Aux);
    if (max_smem < 1024 + aux_bytes + staging_total + resident + 2 * stage_bytes) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_f16_tc: not enough shared memory");
    int stages = (int)((max_smem - 1024 - aux_bytes - staging_total - resident) / stage_bytes);
    if (stages > f16tc::kMaxStages) stages = f16tc::kMaxStages;
    P.stages = stages;
    P.ring_bytes = (int32_t)(stages * stage_bytes + resident);
    size_t smem_bytes = 1024 + (size_t)P.ring_bytes + staging_total + aux_bytes;
    const size_t one_cta_floor = max_smem / 2 + 1024;                // one CTA per SM, so tensor-memory allocation never waits
    if (smem_bytes < one_cta_floor) smem_bytes = one_cta_floor;

    const CUtensorMapSwizzle sw = pl.bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (pl.bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    void* in_ptr = (char*)const_cast<void*>(a->input0) + p.in.offset * 2;
    CUresult cr;
    if (pl.a_mode == f16tc::A_FLAT) {
        cuuint64_t dims[2] = {(cuuint64_t)cs, (cuuint64_t)P.M_total};
        cuuint64_t strides[1] = {(cuuint64_t)(p.in.px * 2)};
        cuuint32_t box[2] = {(cuuint32_t)bke, (cuuint32_t)f16tc::kBM};
        cuuint32_t es[2] = {1, 1};
        cr = h_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, in_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (pl.a_mode == f16tc::A_IM2COL) {
        cuuint64_t dims[4] = {(cuuint64_t)cs, (cuuint64_t)p.in.x, (cuuint64_t)p.in.y, (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)(p.in.px * 2), (cuuint64_t)(p.in.py * 2), (cuuint64_t)(p.in.pb * 2)};
        int lower[2] = {-p.pad_x, -p.pad_y};
        int upper[2] = {p.pad_x - (p.kw - 1) * p.dil_x, p.pad_y - (p.kh - 1) * p.dil_y};
        cuuint32_t es[4] = {1, (cuuint32_t)p.stride_x, (cuuint32_t)p.stride_y, 1};
        cr = h_encode_im2col(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, in_ptr, dims, strides, lower, upper, (cuuint32_t)bke, (cuuint32_t)f16tc::kBM, es,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (patch) {
        cuuint64_t dims[4] = {(cuuint64_t)cs, (cuuint64_t)p.in.x, (cuuint64_t)p.in.y, (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)(p.in.px * 2), (cuuint64_t)(p.in.py * 2), (cuuint64_t)(p.in.pb * 2)};
        cuuint32_t box[4] = {(cuuint32_t)bke, (cuuint32_t)pl.bw, (cuuint32_t)(pl.bh + p.kh - 1), 1};
        cuuint32_t es[4] = {1, 1, 1, 1};
        cr = h_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, in_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const int sx = p.stride_x, sy = p.stride_y;
        const bool strided_view = sx != 1 || sy != 1;
        cuuint64_t dims[4] = {(cuuint64_t)cs, (cuuint64_t)(strided_view ? P.Q : p.in.x), (cuuint64_t)(strided_view ? P.P : p.in.y), (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)(p.in.px * sx * 2), (cuuint64_t)(p.in.py * sy * 2), (cuuint64_t)(p.in.pb * 2)};
        cuuint32_t box[4] = {(cuuint32_t)bke, (cuuint32_t)pl.bw, (cuuint32_t)pl.bh, (cuuint32_t)pl.bb};
        cuuint32_t es[4] = {1, 1, 1, 1};
        cr = h_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, in_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "conv_f16_tc: activation tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");
    {
        cuuint64_t dims[3] = {(cuuint64_t)cs, (cuuint64_t)(p.kh * p.kw), (cuuint64_t)p.ofm};
        cuuint64_t strides[2] = {(cuuint64_t)(p.w_px * 2), (cuuint64_t)(p.w_po * 2)};
        cuuint32_t box[3] = {(cuuint32_t)bke, 1, (cuuint32_t)pl.bn};
        cuuint32_t es[3] = {1, 1, 1};
        void* w_ptr = (char*)const_cast<void*>(a->weights) + p.w_offset * 2;
        cr = h_encode_tiled(&P.tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, w_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "conv_f16_tc: weights tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");
    }
    cr = f16_pixel_map(&P.tmO, pl, (char*)a->output + p.out.offset * 2, p.out, p.ofm, 1, 1);
    if (cr == CUDA_SUCCESS && p.fused_eltw) {
        const cldnn_b200_tensor& et = p.in_out_opt ? p.out : p.eltw;
        const void* eptr = p.in_out_opt ? a->output : a->input1;
        cr = f16_pixel_map(&P.tmE, pl, (char*)const_cast<void*>(eptr) + et.offset * 2, et, p.ofm, p.in_out_opt ? 1 : p.eltw_stride_x, p.in_out_opt ? 1 : p.eltw_stride_y);
    }
    if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "conv_f16_tc: output tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");

    int grid = ctx->prop.multiProcessorCount;
    if (grid > P.total_tiles) grid = P.total_tiles;
    if (grid < 1) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_tc: empty output");
    const size_t smem = smem_bytes;
    B200_CUDA(f16_configure(P, (int)max_smem));
    out->fn = [P, grid, smem](cudaStream_t s) { return f16_launch(P, grid, smem, s); };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

// Batched GEMM on the same kernel: D[b] (rows x ofm) = A[b] (rows x cs) * B[b] (ofm x cs)^T for b < batches, all fp16 with fp32
// accumulation; rows per batch a multiple of 128, cs a multiple of 16, every pointer 16-byte aligned.  Used by the Winograd path.
int32_t f16_batched_gemm_prepare(cldnn_b200_ctx_impl* ctx, const void* A, const void* B, void* D, int batches, int rows, int cs, int ofm,
                                 std::function<cudaError_t(cudaStream_t)>& fn)
{
    if (rows % f16tc::kBM || cs % 16 || ofm % 8 || batches < 1) return fail(CLDNN_B200_INVALID_ARG, "f16 batched gemm: rows % 128, cs % 16, ofm % 8");
    if (!f16_driver_entry_points()) return fail(CLDNN_B200_DEVICE_ERROR, "conv_f16_tc: the CUDA driver does not export cuTensorMapEncodeTiled/Im2col");
    F16Plan pl{}; pl.a_mode = f16tc::A_FLAT; pl.bw = pl.bh = pl.bb = 1;
    pl.bn = ofm > 128 ? 256 : (ofm > 64 ? 128 : 64);
    pl.bk = cs % 64 == 0 ? 128 : (cs % 32 == 0 ? 64 : 32);
    Params P{};
    P.a_mode = f16tc::A_FLAT; P.N = 1; P.P = 1; P.Q = batches * rows;
    P.kh = P.kw = 1; P.stride_x = P.stride_y = P.dil_x = P.dil_y = 1;
    const int bke = pl.bk / 2;
    P.bk = pl.bk; P.chunks = cs / bke; P.k_steps = P.chunks;
    P.bn = pl.bn; P.n_tiles = (ofm + pl.bn - 1) / pl.bn;
    P.M_total = (int64_t)batches * rows;
    P.bw = P.bh = P.bb = 1; P.tiles_w = P.tiles_h = 1;
    P.m_tiles = (int)(P.M_total / f16tc::kBM); P.total_tiles = P.m_tiles * P.n_tiles;
    P.batch_tiles = rows / f16tc::kBM;
    P.stage_rows = f16tc::kBM;
    P.a_stage_bytes = f16tc::kBM * pl.bk; P.b_stage_bytes = pl.bn * pl.bk;
    P.a_tx_bytes = P.a_stage_bytes; P.b_tx_bytes = P.b_stage_bytes;
    P.sbo = 8u * (uint32_t)pl.bk;
    P.layout_type = pl.bk == 128 ? 2u : (pl.bk == 64 ? 4u : 6u);
    P.idesc = (1u << 4) | ((uint32_t)(pl.bn >> 3) << 17) | ((uint32_t)(f16tc::kBM >> 4) << 24);
    P.tmem_cols = (uint32_t)((pl.bn >= 256 ? 2 : 4) * pl.bn);
    P.ofm = ofm; P.bias_dtype = CLDNN_B200_NONE; P.act = CLDNN_B200_ACT_NONE; P.eltw_act = CLDNN_B200_ACT_NONE;
    P.status = ctx->d_status;
    const size_t max_smem = (size_t)ctx->prop.sharedMemPerBlockOptin;
    const size_t stage_bytes = (size_t)P.a_stage_bytes + P.b_stage_bytes;
    const size_t staging_total = (size_t)2 * f16tc::kBM * (pl.bn > 128 ? 128 : pl.bn) * 2;   // two unit buffers of up to 128 features
    const size_t aux_bytes = sizeof(f16tc::Aux);
    if (max_smem < 1024 + aux_bytes + staging_total + 2 * stage_bytes) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_f16_tc: not enough shared memory");
    int stages = (int)((max_smem - 1024 - aux_bytes - staging_total) / stage_bytes);
    if (stages > f16tc::kMaxStages) stages = f16tc::kMaxStages;
    P.stages = stages; P.ring_bytes = (int32_t)(stages * stage_bytes);
    size_t smem_bytes = 1024 + (size_t)P.ring_bytes + staging_total + aux_bytes;
    if (smem_bytes < max_smem / 2 + 1024) smem_bytes = max_smem / 2 + 1024;
    const CUtensorMapSwizzle sw = pl.bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (pl.bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult cr;
    {
        cuuint64_t dims[2] = {(cuuint64_t)cs, (cuuint64_t)P.M_total}; cuuint64_t strides[1] = {(cuuint64_t)cs * 2};
        cuuint32_t box[2] = {(cuuint32_t)bke, (cuuint32_t)f16tc::kBM}; cuuint32_t es[2] = {1, 1};
        cr = h_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(A), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (cr == CUDA_SUCCESS) {
        cuuint64_t dims[3] = {(cuuint64_t)cs, (cuuint64_t)batches, (cuuint64_t)ofm};
        cuuint64_t strides[2] = {(cuuint64_t)ofm * cs * 2, (cuuint64_t)cs * 2};
        cuuint32_t box[3] = {(cuuint32_t)bke, 1, (cuuint32_t)pl.bn}; cuuint32_t es[3] = {1, 1, 1};
        cr = h_encode_tiled(&P.tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(B), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (cr == CUDA_SUCCESS) {
        cuuint64_t dims[2] = {(cuuint64_t)ofm, (cuuint64_t)P.M_total}; cuuint64_t strides[1] = {(cuuint64_t)ofm * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)f16tc::kBM}; cuuint32_t es[2] = {1, 1};
        cr = h_encode_tiled(&P.tmO, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, D, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "f16 batched gemm: tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");
    int grid = ctx->prop.multiProcessorCount;
    if (grid > P.total_tiles) grid = P.total_tiles;
    const size_t smem = smem_bytes;
    B200_CUDA(f16_configure(P, (int)max_smem));
    fn = [P, grid, smem](cudaStream_t s) { return f16_launch(P, grid, smem, s); };
    return CLDNN_B200_SUCCESS;
}

const KernelDef kdef_conv_f16_tc = {"conv_f16_tc", sizeof(cldnn_b200_conv_params), f16_supports, f16_tune_count, nullptr, f16_prepare};

}  // namespace b200
