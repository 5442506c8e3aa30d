// conv_i8_tc: 8-bit convolution (u8/s8 activations x s8 weights -> s32) as an
// implicit GEMM on the sm_100a tensor cores, with the reference's requantising
// epilogue fused in.  It takes the place of the reference's MMAD / IMAD kernel
// family (cl_kernels/convolution_gpu_mmad*.cl, fused_conv_eltwise_gpu_imad.cl,
// convolution_gpu_mmad_32x32sg_128x128wg_slm_int8.cl) while keeping the
// operation order of the reference kernel fused_conv_eltwise_gpu_ref.cl:148-232.
//
// GEMM view:  M = N*P*Q output pixels, N = output features, K = kh*kw*C.
//   A (M x K): activations, byxf (feature innermost, C a multiple of 32), never
//              materialised: one TMA copy per (filter tap, channel chunk) brings
//              the 128 pixels of a tile straight into swizzled shared memory.
//              Three addressing modes: flat 2-D (1x1, stride 1), TMA im2col
//              (any filter / stride / padding / dilation, zero fill outside the
//              image = the reference's skipped taps), and a tiled 4-D box.
//   B (N x K): weights, oyxi (input features innermost), one TMA box per step.
//   D        : s32 accumulators in tensor memory, two buffers so the epilogue of
//              tile t overlaps the main loop of tile t+1.
// One persistent CTA per SM: warp 0 issues TMA loads (operands and, for the
// fused residual, the tile of the second input), warp 1 issues tcgen05.mma,
// warps 2..9 run the epilogue: tcgen05.ld -> bias / dequantise / activation /
// requantise / round / residual / saturate -> swizzled shared-memory tile ->
// one TMA store per 128-byte column block (fully coalesced HBM writes).
// Outputs that TMA cannot address (ragged pitches, float outputs, exotic
// activations) take a direct-store epilogue instead.
#include <cuda.h>
#include <mutex>
#include "conv_i8_tc.hpp"
#include "conv_epilogue.cuh"

namespace b200 {

struct TcSmemAux {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[kMaxBufs];
    uint64_t tmem_empty[kMaxBufs];
    uint64_t res_full[kMaxBufs];                // residual tile landed in staging buffer
    uint64_t stage_free[kMaxBufs];              // staging buffer read out by its TMA store
    uint64_t out_ready[kMaxBufs];               // staging buffer holds a finished output tile
    uint64_t drain;
    uint32_t tmem_base;
    uint32_t abort;
    alignas(16) int32_t bias_i[2][kMaxBN];
    alignas(16) float bias_f[2][kMaxBN];
    alignas(16) float quant[2][kMaxBN];
    alignas(16) float calib[2][kMaxBN];
    alignas(16) float ecal[2][kMaxBN];
};


__device__ __forceinline__ void tile_coords(const TcParams& P, int tile, int& m_tile, int& n_tile)
{
    // feature-tile major: a CTA's successive tiles mostly share their per-channel constants
    n_tile = tile / P.m_tiles; m_tile = tile - n_tile * P.m_tiles;
}

// pixel of row `row` of tile `m_tile`: returns false when the row is padding
__device__ __forceinline__ bool row_pixel(const TcParams& P, int m_tile, int row, int& n, int& p, int& q)
{
    if (P.a_mode == A_TILED) {
        const int tw = m_tile % P.tiles_w; const int t2 = m_tile / P.tiles_w;
        const int th = t2 % P.tiles_h; const int tb = t2 / P.tiles_h;
        const int rw = row % P.bw; const int r2 = row / P.bw;
        const int rh = r2 % P.bh; const int rb = r2 / P.bh;
        q = tw * P.bw + rw; p = th * P.bh + rh; n = tb * P.bb + rb;
        return rb < P.bb && q < P.Q && p < P.P && n < P.N;
    }
    const int64_t m = (int64_t)m_tile * kBM + row;
    const int pq = P.P * P.Q;
    n = (int)(m / pq); const int r = (int)(m - (int64_t)n * pq);
    p = r / P.Q; q = r - p * P.Q;
    return m < P.M_total;
}

// One output element, every epilogue variant.  Kept out of line: it is the rare path.
__device__ __noinline__ void epi_general_elem(const TcParams& P, const TcSmemAux* aux, int acc, int cj, int f, int32_t raw,
                                              int64_t o_pix, int64_t e_pix)
{
    const EpiCfg& c = P.epi;
    const int32_t a = raw + aux->bias_i[acc][cj];
    if (c.quant_path) {
        const float e = c.fused_eltw ? load_as_float(P.eltw, c.eltw_dtype, e_pix + f) : 0.f;
        const float v = epi_quant(c, a, aux->quant[acc][cj], aux->bias_f[acc][cj], aux->calib[acc][cj], e, aux->ecal[acc][cj]);
        store_sat_float(P.out, c.out_dtype, o_pix + f, v);
        return;
    }
    // 8-bit fused eltwise without quantisation: integer activation domain
    int32_t v = act_int(c.act, a, c.act_m, c.act_n), s;
    if (c.has_non_conv_scale) s = (int32_t)__fadd_rn((float)v, __fmul_rn(load_as_float(P.eltw, c.eltw_dtype, e_pix + f), c.non_conv_scale));
    else s = v + load_as_int(P.eltw, c.eltw_dtype, e_pix + f);
    s = act_int(c.eltw_act, s, c.eltw_m, c.eltw_n);
    if (c.eltw_calibration) {
        const float tq = __fmul_rn((float)s, aux->ecal[acc][cj]);
        if (c.out_is_fp) { store_sat_float(P.out, c.out_dtype, o_pix + f, tq); return; }
        s = (int32_t)round_half_away(tq);
    }
    store_sat_int(P.out, c.out_dtype, o_pix + f, s);
}

__global__ void __launch_bounds__(kThreads, 1)
conv_i8_tc_kernel(const __grid_constant__ TcParams P)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t a_base = base;
    const uint32_t b_base = base + (uint32_t)(P.stages * P.a_stage_bytes);
    const uint32_t ring_bytes = (uint32_t)(P.stages * (P.a_stage_bytes + P.b_stage_bytes));
    const uint32_t staging_bytes = P.staged ? (uint32_t)(kBM * P.bn) : 0u;           // per buffer, two buffers
    uint8_t* staging = smem + ring_bytes;
    TcSmemAux* aux = reinterpret_cast<TcSmemAux*>(smem + ring_bytes + (uint32_t)P.nbuf * staging_bytes);
    volatile uint32_t* s_abort = &aux->abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool fused_staged = P.staged && P.epi.fused_eltw;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P.stages; ++s) { mbar_init(smem_u32(&aux->full[s]), 1); mbar_init(smem_u32(&aux->empty[s]), 1); }
        for (int a = 0; a < kMaxBufs; ++a) {
            mbar_init(smem_u32(&aux->tmem_full[a]), 1); mbar_init(smem_u32(&aux->tmem_empty[a]), kEpiWarps);
            mbar_init(smem_u32(&aux->res_full[a]), 1); mbar_init(smem_u32(&aux->stage_free[a]), 1);
            mbar_init(smem_u32(&aux->out_ready[a]), kEpiWarps);
        }
        mbar_init(smem_u32(&aux->drain), 1);
        aux->abort = 0u;
        mbar_fence_init();
        prefetch_tensormap(&P.tmA); prefetch_tensormap(&P.tmB);
        if (P.staged) { prefetch_tensormap(&P.tmO); if (P.epi.fused_eltw) prefetch_tensormap(&P.tmE); }
    }
    if (warp == 1) { tmem_alloc(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        // The whole warp walks the tiles and waits on the barriers, one elected lane issues the copies: a warp-uniform loop
        // lets the compiler keep its state on the uniform datapath, which a loop inside a one-lane branch cannot use.
        {
            const bool leader = ptx::elect_one();
            int stage = 0; uint32_t phase = 0; int64_t issued = 0; bool ok = true; int t = 0;
            for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x, ++t) {
                int m_tile, n_tile; tile_coords(P, tile, m_tile, n_tile);
                // base coordinates of the tile's first pixel
                int c_w = 0, c_h = 0, c_n = 0, o_w = 0, o_h = 0;
                if (P.a_mode == A_IM2COL) {
                    int n, p, q; row_pixel(P, m_tile, 0, n, p, q);
                    c_w = q * P.stride_x - P.pad_x; c_h = p * P.stride_y - P.pad_y; c_n = n;
                } else if (P.a_mode == A_TILED) {
                    const int tw = m_tile % P.tiles_w; const int t2 = m_tile / P.tiles_w;
                    o_w = tw * P.bw; o_h = (t2 % P.tiles_h) * P.bh; c_n = (t2 / P.tiles_h) * P.bb;
                    c_w = o_w - P.pad_x; c_h = o_h - P.pad_y;
                }
                if (fused_staged) {
                    // second input of the fused eltwise: same pixels and features as the output tile
                    const int a = t % P.nbuf;
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->stage_free[a]), (((uint32_t)(t / P.nbuf) & 1u)) ^ 1u, s_abort, P.status, kErrProducer + 1u))) { ok = false; break; }
                    const uint32_t rf = smem_u32(&aux->res_full[a]);
                    if (leader) mbar_expect_tx(rf, (uint32_t)(P.stage_rows * P.cw * P.col_blocks));
                    for (int cb = 0; cb < P.col_blocks && leader; ++cb) {
                        const uint32_t dst = smem_u32(staging) + (uint32_t)a * staging_bytes + (uint32_t)(cb * kBM * P.cw);
                        const int f0 = n_tile * P.bn + cb * P.cw;
                        if (P.a_mode == A_TILED) tma_load_4d(dst, &P.tmE, rf, f0, o_w, o_h, c_n);
                        else tma_load_2d(dst, &P.tmE, rf, f0, m_tile * kBM);
                    }
                }
                int tap = 0, cc = 0, r = 0, s = 0;
                for (int ks = 0; ks < P.k_steps; ++ks) {
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1u, s_abort, P.status, kErrProducer))) { ok = false; break; }
                    const uint32_t full = smem_u32(&aux->full[stage]);
                    const uint32_t a_dst = a_base + (uint32_t)(stage * P.a_stage_bytes);
                    const uint32_t b_dst = b_base + (uint32_t)(stage * P.b_stage_bytes);
                    const int c0 = cc * P.bk;
                    if (leader) {
                        mbar_expect_tx(full, (uint32_t)(P.a_tx_bytes + P.b_tx_bytes));
                        if (P.a_mode == A_FLAT) tma_load_2d(a_dst, &P.tmA, full, c0, m_tile * kBM);
                        else if (P.a_mode == A_IM2COL) tma_load_im2col_4d(a_dst, &P.tmA, full, c0, c_w, c_h, c_n, (uint16_t)(s * P.dil_x), (uint16_t)(r * P.dil_y));
                        else tma_load_4d(a_dst, &P.tmA, full, c0, c_w + s * P.dil_x, c_h + r * P.dil_y, c_n);
                        tma_load_3d(b_dst, &P.tmB, full, c0, tap, n_tile * P.bn);
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
            const bool leader = ptx::elect_one();
            int stage = 0; uint32_t phase = 0; bool ok = true; int t = 0;
            for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x, ++t) {
                const int acc = t % P.nbuf;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->tmem_empty[acc]), (((uint32_t)(t / P.nbuf) & 1u)) ^ 1u, s_abort, P.status, kErrMma))) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * P.bn);
                for (int ks = 0; ks < P.k_steps; ++ks) {
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->full[stage]), phase, s_abort, P.status, kErrMma + 1u))) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = make_smem_desc(a_base + (uint32_t)(stage * P.a_stage_bytes), P.sbo, P.layout_type);
                    const uint64_t bdesc = make_smem_desc(b_base + (uint32_t)(stage * P.b_stage_bytes), P.sbo, P.layout_type);
                    const int kk = P.bk >> 5;                       // one instruction consumes K = 32 bytes
                    if (leader) {
                        for (int k = 0; k < kk; ++k)
                            mma_i8_ss(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), P.idesc, (ks | k) ? 1u : 0u);
                        tc_commit(smem_u32(&aux->empty[stage]));    // frees the stage once these MMAs have read it
                    }
                    if (++stage == P.stages) { stage = 0; phase ^= 1u; }
                }
                if (ok && leader) tc_commit(smem_u32(&aux->tmem_full[acc]));
            }
            // drain: every issued MMA must have retired before TMEM is released
            if (leader) tc_commit(smem_u32(&aux->drain));
            const uint64_t t0 = globaltimer();
            while (!mbar_try_wait(smem_u32(&aux->drain), 0u)) {
                if (globaltimer() - t0 > kWaitLimitNs) { atomicCAS(P.status, 0u, kErrDrain); break; }
            }
        }
    } else if (warp == kStoreWarp) {
        // ------------------------------ TMA store issuer --------------------------
        if (lane == 0 && P.staged) {
            int t = 0;
            for (int tile = blockIdx.x; tile < P.total_tiles; tile += gridDim.x, ++t) {
                int m_tile, n_tile; tile_coords(P, tile, m_tile, n_tile);
                const int a = t % P.nbuf;
                if (!mbar_wait(smem_u32(&aux->out_ready[a]), ((uint32_t)(t / P.nbuf) & 1u), s_abort, P.status, kErrEpilogue + 2u)) break;
                int tw = 0, th = 0, tb = 0;
                if (P.a_mode == A_TILED) { tw = m_tile % P.tiles_w; const int t2 = m_tile / P.tiles_w; th = t2 % P.tiles_h; tb = t2 / P.tiles_h; }
                const int n0 = n_tile * P.bn;
                for (int cb = 0; cb < P.col_blocks; ++cb) {
                    const int f0 = n0 + cb * P.cw;
                    if (f0 >= P.ofm) break;
                    const uint32_t src = smem_u32(staging) + (uint32_t)a * staging_bytes + (uint32_t)(cb * kBM * P.cw);
                    if (P.a_mode == A_TILED) tma_store_4d(&P.tmO, src, f0, tw * P.bw, th * P.bh, tb * P.bb);
                    else tma_store_2d(&P.tmO, src, f0, m_tile * kBM);
                }
                bulk_commit();
                bulk_wait_read0();                                  // the buffer may be refilled once TMA has read it
                mbar_arrive(smem_u32(&aux->stage_free[a]));
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        // Warps run independently: no block-wide synchronisation per tile, only the
        // mbarriers of the accumulator and staging buffers they touch.
        const int quad = warp & 3;                                  // TMEM lanes 32*quad .. 32*quad+31
        const int half = (warp - 2) >> 2;                           // two warps share a lane quadrant, alternate column chunks
        const int row = quad * 32 + lane;
        const int et = threadIdx.x - 64;                            // 0..255
        const EpiCfg& c = P.epi;
        const uint32_t sw = (uint32_t)((row >> P.sw_shift) & P.sw_mask);
        int t = 0; bool ok = true; int cur_n_tile = -1;
        for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x, ++t) {
            int m_tile, n_tile; tile_coords(P, tile, m_tile, n_tile);
            const int acc = t % P.nbuf;
            const int n0 = n_tile * P.bn;
            if (n_tile != cur_n_tile) {
                // per-channel constants of this feature range; every warp has left the previous range
                named_bar_sync(1, kEpiThreads);
                for (int j = et; j < P.bn; j += kEpiThreads) {
                    const int f = n0 + j; const bool v = f < P.ofm;
                    int32_t bi = 0; float bf = 0.f;
                    if (v && c.bias_dtype != CLDNN_B200_NONE) {
                        if (c.bias_dtype == CLDNN_B200_F32) bf = ((const float*)P.bias)[f];
                        else bi = load_as_int(P.bias, c.bias_dtype, f);
                    }
                    aux->bias_i[0][j] = bi; aux->bias_f[0][j] = bf;
                    aux->quant[0][j] = (v && c.quantization) ? P.quant[f] : 1.f;
                    aux->calib[0][j] = (v && c.calibration) ? P.calib[f] : 1.f;
                    aux->ecal[0][j] = (v && c.eltw_calibration) ? P.ecal[f] : 1.f;
                }
                named_bar_sync(1, kEpiThreads);
                cur_n_tile = n_tile;
            }
            if (!mbar_wait(smem_u32(&aux->tmem_full[acc]), ((uint32_t)(t / P.nbuf) & 1u), s_abort, P.status, kErrEpilogue)) { ok = false; break; }
            if (P.staged) {
                // the staging buffer is ours once its residual tile has landed (fused) or its previous store has read it out
                const bool got = fused_staged ? mbar_wait(smem_u32(&aux->res_full[acc]), ((uint32_t)(t / P.nbuf) & 1u), s_abort, P.status, kErrEpilogue + 1u)
                                              : mbar_wait(smem_u32(&aux->stage_free[acc]), (((uint32_t)(t / P.nbuf) & 1u)) ^ 1u, s_abort, P.status, kErrEpilogue + 1u);
                if (!got) { ok = false; break; }
            }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * P.bn);

            if (P.staged) {
                uint8_t* stg = staging + (size_t)acc * staging_bytes;
                for (int c0 = half * 32; c0 < P.bn; c0 += 64) {
                    if (n0 + c0 >= P.ofm) break;
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
                    const int cb = c0 / P.cw, o = c0 - cb * P.cw;
                    uint8_t* rowp = stg + (size_t)cb * kBM * P.cw + (size_t)row * P.cw;
                    uint4* p0 = reinterpret_cast<uint4*>(rowp + ((((uint32_t)o >> 4) ^ sw) << 4));
                    uint4* p1 = reinterpret_cast<uint4*>(rowp + (((((uint32_t)o >> 4) + 1u) ^ sw) << 4));
                    uint4 o0, o1;
                    if (P.lean) {
                        if (c.fused_eltw) epi_chunk_fast<true, true>(P, aux, 0, c0, r, *p0, *p1, o0, o1);
                        else epi_chunk_fast<false, true>(P, aux, 0, c0, r, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1);
                    } else {
                        if (c.fused_eltw) epi_chunk_fast<true, false>(P, aux, 0, c0, r, *p0, *p1, o0, o1);
                        else epi_chunk_fast<false, false>(P, aux, 0, c0, r, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1);
                    }
                    *p0 = o0; *p1 = o1;
                }
                tc_fence_before();
                fence_async_smem();
                __syncwarp();
                if (lane == 0) { mbar_arrive(smem_u32(&aux->tmem_empty[acc])); mbar_arrive(smem_u32(&aux->out_ready[acc])); }
            } else {
                int n, p, q; const bool valid = row_pixel(P, m_tile, row, n, p, q);
                const int64_t o_pix = P.out_off + (int64_t)n * P.out_pb + (int64_t)p * P.out_py + (int64_t)q * P.out_px;
                const int64_t e_pix = c.fused_eltw ? P.el_off + (int64_t)n * P.el_pb + (int64_t)p * P.el_sy * P.el_py + (int64_t)q * P.el_sx * P.el_px : 0;
                for (int c0 = half * 32; c0 < P.bn; c0 += 64) {
                    if (n0 + c0 >= P.ofm) break;
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + (uint32_t)c0, r);
                    tmem_ld_wait();
                    if (!valid) continue;
                    const int fbase = n0 + c0;
                    const bool full32 = fbase + 32 <= P.ofm;
                    if (P.fast_epi && full32 && ((o_pix + fbase) & 15) == 0 && (!c.fused_eltw || ((e_pix + fbase) & 15) == 0)) {
                        uint4* op = reinterpret_cast<uint4*>((uint8_t*)P.out + o_pix + fbase);
                        uint4 o0, o1;
                        if (c.fused_eltw) {
                            const uint4* ep = reinterpret_cast<const uint4*>((const uint8_t*)P.eltw + e_pix + fbase);
                            epi_chunk_fast<true, false>(P, aux, 0, c0, r, ep[0], ep[1], o0, o1);
                        } else epi_chunk_fast<false, false>(P, aux, 0, c0, r, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1);
                        op[0] = o0; op[1] = o1;
                    } else {
                        // general path: any output type, any activation, ragged feature tail, unaligned rows
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (fbase + j < P.ofm) epi_general_elem(P, aux, 0, c0 + j, fbase + j, (int32_t)r[j], o_pix, e_pix);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->tmem_empty[acc]));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, P.tmem_cols); }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;

static bool load_driver_entry_points()
{
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr; cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            g_encode_tiled = (EncodeTiledFn)fn;
        fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            g_encode_im2col = (EncodeIm2colFn)fn;
        (void)cudaGetLastError();
    });
    return g_encode_tiled && g_encode_im2col;
}

struct TcPlan { int a_mode; int bn; int bk; int bw, bh, bb; int epi_groups; int pair; };

// tune index -> (addressing mode, feature tile).  0 = automatic choice.
static const int kTuneBN[4] = {32, 64, 128, 256};
// Indices 13..24 repeat 1..12 on the general kernel where the specialised one (conv_i8_tc_fast.cu) would be used;
// 25..28 are the patch mode (resident weights, one activation patch per filter column) of the specialised kernel;
// 29..40 and 41..44 repeat 1..12 and 25..28 on the specialised kernel with four epilogue warp groups instead of two
// (16 epilogue warps per SM: for the layers whose time is the epilogue's instruction issue).
// 45..50: CTA pairs on the specialised kernel (two epilogue groups): 45 + 2 * mode + {128, 256}[i], mode flat / im2col / tiled
constexpr int kTuneFourGroups = 28;
constexpr int kTunePair = 44;
static int tc_tune_count(const void*) { return 1 + 2 * 3 * 4 + 4 + 3 * 4 + 4 + 6; }
constexpr size_t kPatchWeightBytes = 72 * 1024;       // largest weight tensor the patch mode keeps resident

static bool dense_byxf(const cldnn_b200_tensor& t)
{
    return t.pf == 1 && t.px % 16 == 0 && t.py % 16 == 0 && t.pb % 16 == 0 && t.offset % 16 == 0 && t.px >= t.f && t.py >= t.px * t.x && t.pb >= t.py * t.y;
}
static bool pixel_dense(const cldnn_b200_tensor& t) { return t.py == t.px * t.x && t.pb == t.py * t.y; }

// choose a box of bw x bh x bb <= 128 pixels that wastes the fewest tile rows
static void choose_box(int Q, int Pn, int N, int& bw, int& bh, int& bb)
{
    double best = -1.0; bw = 1; bh = 1; bb = 1;
    for (int w = 1; w <= Q && w <= 128; ++w) {
        for (int h = 1; h <= Pn && w * h <= 128; ++h) {
            int b = 128 / (w * h); if (b > N) b = N; if (b < 1) continue; if (b > 128) b = 128;
            const double tiles = (double)((Q + w - 1) / w) * ((Pn + h - 1) / h) * ((N + b - 1) / b);
            const double eff = ((double)Q * Pn * N) / (tiles * 128.0);
            // prefer long contiguous runs when the efficiency ties
            const double score = eff + 1e-4 * w + 1e-6 * h;
            if (score > best) { best = score; bw = w; bh = h; bb = b; }
        }
    }
}

// The epilogue configuration the specialised kernels cover: per-channel dequantisation only, NONE / ReLU,
// 8-bit output (and residual), integer or no bias.
static bool lean_params(const cldnn_b200_conv_params& p)
{
    auto none_or_relu = [](int32_t fn) { return fn == CLDNN_B200_ACT_NONE || fn == CLDNN_B200_ACT_RELU; };
    if (!p.quantization || p.i_qf != 1.0f || p.calibration || p.epilogue_order != CLDNN_B200_EPILOGUE_REF) return false;
    if (!is_int8(p.out.dtype) || !none_or_relu(p.act)) return false;
    if (p.o_qf != 1.0f) {
        // a uniform O_QF: positive, in front of an unsigned or a plain signed saturation, no ReLU in front of a residual sum
        const int32_t last = p.fused_eltw ? p.eltw_act : p.act;
        if (!(p.o_qf > 0.0f) || (p.fused_eltw && p.act == CLDNN_B200_ACT_RELU) || (p.out.dtype != CLDNN_B200_U8 && last == CLDNN_B200_ACT_RELU)) return false;
    }
    if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_I32) return false;
    if (p.fused_eltw) {
        const int32_t edt = p.in_out_opt ? p.out.dtype : p.eltw.dtype;
        if (!is_int8(edt) || p.has_non_conv_scale || p.eltw_calibration || !none_or_relu(p.eltw_act)) return false;
    }
    return true;
}

// patch mode: a tile of tw x th output pixels of one image (tw * th <= 128); per filter column one patch of
// (th + kh - 1) x tw input pixels serves the kh taps of that column.  Fewest wasted tile rows first, then least traffic.
static void choose_patch(int Q, int Pn, int kh, int kw, int& tw, int& th)
{
    double best = -1.0; tw = 1; th = 1;
    for (int w = 1; w <= Q && w <= 128; ++w) {
        for (int h = 1; h <= Pn && w * h <= 128; ++h) {
            if (h + kh - 1 > 256) continue;
            const double tiles = (double)((Q + w - 1) / w) * ((Pn + h - 1) / h);
            const double eff = ((double)Q * Pn) / (tiles * 128.0);
            const double traffic = tiles * kw * (h + kh - 1) * w / ((double)Q * Pn * kh * kw);   // relative to one load per tap
            const double score = eff - 0.25 * traffic;
            if (score > best) { best = score; tw = w; th = h; }
        }
    }
}

static bool tc_plan(const cldnn_b200_conv_params& p, TcPlan& pl, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (!is_int8(p.in.dtype)) return no("activations must be u8 or i8");
    if (p.w_dtype != CLDNN_B200_I8) return no("weights must be i8");
    if (p.groups != 1) return no("grouped convolution is handled by other kernels");
    if (!epilogue_order_ok(p)) return no("the MMAD / IMAD epilogue orders need quantisation, an f32 bias and an 8-bit output (IMAD fused: eltwise calibration)");
    if (p.kh < 1 || p.kw < 1 || p.kh * p.kw > 255) return no("filter size");
    if (p.stride_x < 1 || p.stride_y < 1 || p.dil_x < 1 || p.dil_y < 1) return no("stride/dilation");
    if (p.out.f != p.ofm || p.in.f != p.ifm) return no("feature counts");
    if (!dense_byxf(p.in)) return no("input must be byxf with 16-byte aligned pitches");
    if (p.in.px % 32) return no("stored input features must be a multiple of 32");
    if (p.out.pf != 1) return no("output must be byxf");
    if (!(is_int8(p.out.dtype) || p.out.dtype == CLDNN_B200_F32 || p.out.dtype == CLDNN_B200_F16 || p.out.dtype == CLDNN_B200_I32)) return no("output type");
    if (p.w_pi != 1 || p.w_px % 16 || p.w_po % 16 || p.w_offset % 16 || p.w_py != p.w_px * p.kw) return no("weights must be oyxi with 16-byte aligned pitches");
    if (p.w_px != p.in.px) return no("weights and input must store the same (padded) feature count");
    const bool quant_path = p.quantization || p.calibration || p.has_o_qf;
    if (!quant_path && !p.fused_eltw) return no("non-quantised 8-bit convolution accumulates in 8 bits; handled by conv_ref");
    if (p.fused_eltw && !p.in_out_opt && p.eltw.pf != 1) return no("residual must be byxf");
    if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_I32 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    if (!quant_path && p.bias_dtype == CLDNN_B200_F32) return no("float bias needs quantisation");
    // expected output size
    const int P_ = (p.in.y + 2 * p.pad_y - ((p.kh - 1) * p.dil_y + 1)) / p.stride_y + 1;
    const int Q_ = (p.in.x + 2 * p.pad_x - ((p.kw - 1) * p.dil_x + 1)) / p.stride_x + 1;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");
    if ((int64_t)p.out.b * p.out.y * p.out.x > (int64_t)1 << 31) return no("too many output pixels");

    const int cs = (int)p.in.px;                                    // stored channels = bytes of K per tap
    pl.bk = cs % 128 == 0 ? 128 : (cs % 64 == 0 ? 64 : 32);
    const bool is_1x1_s1 = p.kh == 1 && p.kw == 1 && p.stride_x == 1 && p.stride_y == 1 && p.pad_x == 0 && p.pad_y == 0 && pixel_dense(p.in);
    const bool pointwise = p.kh == 1 && p.kw == 1 && p.pad_x == 0 && p.pad_y == 0;
    const bool tiled_ok = (p.stride_x == 1 && p.stride_y == 1) || pointwise;
    const bool im2col_ok = p.pad_x <= 127 && p.pad_y <= 127 && (p.kw - 1) * p.dil_x <= 255 && (p.kh - 1) * p.dil_y <= 255 &&
                           p.stride_x <= 8 && p.stride_y <= 8 &&
                           (int64_t)p.in.b * p.in.pb >= 131072;     // small tensors take the tiled path
    int tune = p.tune;
    int mode = -1, bn = 0;
    pl.epi_groups = 2; pl.pair = 0;
    if (tune > kTunePair) {
        if (tune > kTunePair + 6) return no("unknown tuning index");
        if (!lean_params(p)) return no("CTA pairs exist on the specialised kernel only");
        pl.pair = 1;
        const int t6 = tune - kTunePair - 1;
        tune = 1 + 4 * (t6 / 2) + 2 + (t6 & 1);                   // the same addressing mode with a 128- or 256-feature tile
    }
    else if (tune > kTuneFourGroups) {
        pl.epi_groups = 4;
        tune -= kTuneFourGroups;                                   // 1..12 as they are, 13..16 are the patch modes 25..28
        if (tune > 12) tune += 12;
        if (!lean_params(p)) return no("four epilogue groups exist on the specialised kernel only");
    }
    // every ring a group waits on (accumulators, staging tiles) must hold a multiple of the group count: a group then meets
    // every phase of the barriers it waits on, which is what a parity wait needs.  256-feature tiles have two accumulators.
    auto groups_fit = [&](int fbn) { return pl.epi_groups == 2 || fbn == 64 || fbn == 128; };
    if (tune > 24) { mode = A_PATCH; bn = kTuneBN[(tune - 25) % 4]; }
    else {
        if (tune > 12) tune -= 12;
        if (tune > 0) { mode = (tune - 1) / 4; bn = kTuneBN[(tune - 1) % 4]; }
    }
    // patch mode: stride-1 undilated filters whose weights fit in shared memory, specialised epilogue configuration
    auto patch_why = [&](int fbn) -> const char* {
        if (p.stride_x != 1 || p.stride_y != 1 || p.dil_x != 1 || p.dil_y != 1 || p.kh * p.kw == 1) return "patch mode needs a stride-1 undilated filter larger than 1x1";
        if (fbn < 64 || p.ofm % fbn) return "patch mode needs output features in whole tiles of 64, 128 or 256";
        if ((size_t)p.kh * p.kw * cs * p.ofm > kPatchWeightBytes) return "patch mode keeps all weights in shared memory: at most 72 KiB";
        if (!lean_params(p)) return "patch mode exists for the specialised epilogue configuration only";
        const cldnn_b200_tensor& rt = p.in_out_opt ? p.out : p.eltw;
        if (p.out.px % 16 || p.out.py % 16 || p.out.pb % 16 || p.out.offset % 16) return "patch mode needs a 16-byte aligned output";
        if (p.fused_eltw && (rt.pf != 1 || rt.px % 16 || rt.py % 16 || rt.pb % 16 || rt.offset % 16)) return "patch mode needs a 16-byte aligned byxf residual";
        return nullptr;
    };
    if (mode < 0) {
        const int fbn = p.ofm % 256 == 0 ? 256 : (p.ofm % 128 == 0 ? 128 : 64);
        if (!patch_why(fbn)) { mode = A_PATCH; bn = fbn; }
        else mode = is_1x1_s1 ? A_FLAT : (im2col_ok ? A_IM2COL : A_TILED);
    }
    if (mode == A_FLAT && !is_1x1_s1) return no("flat addressing needs a dense 1x1 stride-1 convolution");
    if (mode == A_TILED && !tiled_ok) return no("tiled addressing needs stride 1 or a pointwise filter");
    if (mode == A_IM2COL && !im2col_ok) return no("im2col addressing limits exceeded (or tensor below 128 KiB)");
    if (bn == 0) bn = p.ofm > 128 ? 256 : (p.ofm > 64 ? 128 : (p.ofm > 32 ? 64 : 32));
    if (!groups_fit(bn)) return no("four epilogue groups need feature tiles of 64 or 128 (eight or four accumulators)");
    if (mode == A_PATCH) { if (const char* m = patch_why(bn)) return no(m); }
    if (pl.pair && (p.ofm % bn || (int64_t)p.out.b * p.out.y * p.out.x < 2 * kBM)) return no("CTA pairs need whole feature tiles and at least two pixel tiles");
    // 256-feature tiles with a fused residual: three 32 KiB staging tiles + three operand stages need 24 KiB stages;
    // worth it unless the reduction is long (>= 4 chunks of 128 channels), where fewer, larger stages win
    if (bn == 256 && p.fused_eltw && pl.bk == 128 && cs < 512 && lean_params(p)) pl.bk = 64;
    pl.a_mode = mode; pl.bn = bn;
    pl.bw = pl.bh = pl.bb = 1;
    if (mode == A_TILED) choose_box(p.out.x, p.out.y, p.out.b, pl.bw, pl.bh, pl.bb);
    if (mode == A_PATCH) choose_patch(p.out.x, p.out.y, p.kh, p.kw, pl.bw, pl.bh);
    return true;
}

static bool tc_supports(const void* vp)
{
    TcPlan pl; return tc_plan(simplified_conv_params(*(const cldnn_b200_conv_params*)vp), pl, nullptr);
}

// tensor map over the pixels x features of an 8-bit byxf tensor, boxed like the tile
static CUresult encode_pixel_map(CUtensorMap* tm, const TcPlan& pl, void* ptr, const cldnn_b200_tensor& t, int stride_x, int stride_y,
                                 int cw, CUtensorMapSwizzle sw)
{
    if (pl.a_mode == A_TILED || pl.a_mode == A_PATCH) {
        cuuint64_t dims[4] = {(cuuint64_t)t.f, (cuuint64_t)((t.x + stride_x - 1) / stride_x), (cuuint64_t)((t.y + stride_y - 1) / stride_y), (cuuint64_t)t.b};
        cuuint64_t strides[3] = {(cuuint64_t)(t.px * stride_x), (cuuint64_t)(t.py * stride_y), (cuuint64_t)t.pb};
        cuuint32_t box[4] = {(cuuint32_t)cw, (cuuint32_t)pl.bw, (cuuint32_t)pl.bh, (cuuint32_t)pl.bb};
        cuuint32_t es[4] = {1, 1, 1, 1};
        return g_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    cuuint64_t dims[2] = {(cuuint64_t)t.f, (cuuint64_t)((int64_t)t.b * t.y * t.x)};
    cuuint64_t strides[1] = {(cuuint64_t)t.px};
    cuuint32_t box[2] = {(cuuint32_t)cw, (cuuint32_t)kBM};
    cuuint32_t es[2] = {1, 1};
    return g_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

static int32_t tc_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params p = simplified_conv_params(*(const cldnn_b200_conv_params*)vp);
    TcPlan pl; std::string why;
    if (!tc_plan(p, pl, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_tc: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: bias_dtype set but no bias pointer");
    if (p.quantization && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: quantization set but no factors");
    if (p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: calibration set but no factors");
    if (p.fused_eltw && !p.in_out_opt && !a->input1) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: fused eltwise needs a second input");
    if (p.eltw_calibration && !a->eltw_output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: eltwise calibration set but no factors");
    if (((uintptr_t)a->input0 | (uintptr_t)a->weights) & 15) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: input and weights must be 16-byte aligned");
    if (!load_driver_entry_points()) return fail(CLDNN_B200_DEVICE_ERROR, "conv_i8_tc: the CUDA driver does not export cuTensorMapEncodeTiled/Im2col");

    TcParams P{};
    P.a_mode = pl.a_mode;
    P.N = p.out.b; P.P = p.out.y; P.Q = p.out.x;
    P.kh = p.kh; P.kw = p.kw; P.stride_x = p.stride_x; P.stride_y = p.stride_y; P.pad_x = p.pad_x; P.pad_y = p.pad_y; P.dil_x = p.dil_x; P.dil_y = p.dil_y;
    const int cs = (int)p.in.px;
    P.bk = pl.bk; P.chunks = cs / pl.bk; P.k_steps = p.kh * p.kw * P.chunks;
    P.bn = pl.bn; P.n_tiles = (p.ofm + pl.bn - 1) / pl.bn;
    P.M_total = (int64_t)P.N * P.P * P.Q;
    P.bw = pl.bw; P.bh = pl.bh; P.bb = pl.bb;
    const bool boxed = pl.a_mode == A_TILED || pl.a_mode == A_PATCH;
    if (boxed) {
        P.tiles_w = (P.Q + pl.bw - 1) / pl.bw; P.tiles_h = (P.P + pl.bh - 1) / pl.bh;
        P.m_tiles = P.tiles_w * P.tiles_h * ((P.N + pl.bb - 1) / pl.bb);
    } else {
        P.tiles_w = P.tiles_h = 1;
        P.m_tiles = (int)((P.M_total + kBM - 1) / kBM);
    }
    P.pair = pl.pair;
    // CTA pairs take pixel tiles two at a time: an odd count gets one phantom tile past the tensor (its loads read the
    // out-of-range fill, its stores are clipped away); each CTA loads half of the feature tile's weight rows
    if (pl.pair) P.m_tiles = (P.m_tiles + 1) & ~1;
    const int b_rows = pl.pair ? pl.bn / 2 : pl.bn;
    P.total_tiles = P.m_tiles * P.n_tiles;
    P.stage_rows = boxed ? pl.bw * pl.bh * pl.bb : kBM;
    P.a_stage_bytes = kBM * pl.bk; P.b_stage_bytes = b_rows * pl.bk;
    P.a_tx_bytes = P.stage_rows * pl.bk;
    P.b_tx_bytes = b_rows * pl.bk;
    if (pl.a_mode == A_PATCH) {
        // a stage holds the patch; the tensor core reads 128 rows from row r * bw, r < kh, so the stage spans that far
        const int patch_rows = (pl.bh + p.kh - 1) * pl.bw, read_rows = (p.kh - 1) * pl.bw + kBM;
        // one stage = the kw patches (one per filter column) of one channel chunk: one barrier round trip per chunk
        P.k_steps = P.chunks;
        P.patch_alloc = (((patch_rows > read_rows ? patch_rows : read_rows) * pl.bk) + 1023) / 1024 * 1024;
        P.a_tx_bytes = p.kw * patch_rows * pl.bk;
        P.a_stage_bytes = p.kw * P.patch_alloc;
        P.b_total_bytes = P.n_tiles * p.kh * p.kw * P.chunks * P.b_stage_bytes;
    }
    P.sbo = 8u * (uint32_t)pl.bk;
    P.layout_type = pl.bk == 128 ? 2u : (pl.bk == 64 ? 4u : 6u);
    const uint32_t a_fmt = p.in.dtype == CLDNN_B200_U8 ? 0u : 1u;     // operand signedness in the instruction descriptor
    P.idesc = (2u << 4) | (a_fmt << 7) | (1u << 10) | ((uint32_t)(pl.bn >> 3) << 17) | ((uint32_t)((pl.pair ? 2 * kBM : kBM) >> 4) << 24);
    P.nbuf = pl.bn >= 256 ? 2 : (pl.bn >= 128 ? 4 : 8);         // accumulator and staging buffers in flight: all of tensor memory
    P.tmem_cols = (uint32_t)(P.nbuf * pl.bn < 32 ? 32 : P.nbuf * pl.bn);
    P.ofm = p.ofm;
    P.out_px = p.out.px; P.out_py = p.out.py; P.out_pb = p.out.pb; P.out_off = p.out.offset;
    const cldnn_b200_tensor& et = p.in_out_opt ? p.out : p.eltw;
    const int esx = p.in_out_opt ? 1 : p.eltw_stride_x, esy = p.in_out_opt ? 1 : p.eltw_stride_y;
    if (p.fused_eltw) {
        P.el_px = et.px; P.el_py = et.py; P.el_pb = et.pb; P.el_off = et.offset;
        P.el_sx = esx; P.el_sy = esy;
    }
    P.out = a->output; P.eltw = p.in_out_opt ? a->output : a->input1; P.bias = a->bias;
    P.quant = a->weights_quantization_factors; P.calib = a->output_calibration_factors; P.ecal = a->eltw_output_calibration_factors;
    P.status = ctx->d_status;
    P.epi = make_epi_cfg(p);
    P.fast_epi = (p.epilogue_order == CLDNN_B200_EPILOGUE_REF && P.epi.quant_path && is_int8(p.out.dtype) && act_is_simple(p.act, p.act_m) &&
                  (!p.fused_eltw || (is_int8(P.epi.eltw_dtype) && act_is_simple(p.eltw_act, p.eltw_m)))) ? 1 : 0;
    P.mul_iqf = p.i_qf != 1.0f ? 1 : 0;
    P.mul_oqf = (p.calibration || p.o_qf != 1.0f) ? 1 : 0;
    auto none_or_relu = [](int32_t fn) { return fn == CLDNN_B200_ACT_NONE || fn == CLDNN_B200_ACT_RELU; };
    P.lean = (P.fast_epi && p.quantization && !P.mul_iqf && (!P.mul_oqf || !p.calibration) && !P.epi.dont_dequantize_bias && none_or_relu(p.act) &&
              (!p.fused_eltw || (!p.has_non_conv_scale && !p.eltw_calibration && none_or_relu(p.eltw_act)))) ? 1 : 0;

    // staged epilogue: the output (and residual) tile must be addressable by one TMA box per column block
    auto tma_ok = [&](const cldnn_b200_tensor& t, const void* ptr, int sx, int sy) {
        if (t.pf != 1 || t.px % 16 || t.py % 16 || t.pb % 16 || t.offset % 16 || ((uintptr_t)ptr & 15)) return false;
        if (boxed) return true;
        return sx == 1 && sy == 1 && pixel_dense(t);
    };
    P.staged = (P.fast_epi && tma_ok(p.out, a->output, 1, 1) && (!p.fused_eltw || tma_ok(et, P.eltw, esx, esy))) ? 1 : 0;
    if (p.fused_eltw && !p.in_out_opt && (et.b != p.out.b || (et.y + esy - 1) / esy < p.out.y || (et.x + esx - 1) / esx < p.out.x || et.f < p.ofm)) P.staged = 0;
    P.cw = pl.bn < 128 ? pl.bn : 128; P.col_blocks = pl.bn / P.cw;
    P.sw_shift = P.cw == 128 ? 0 : (P.cw == 64 ? 1 : 2);
    P.sw_mask = P.cw == 128 ? 7 : (P.cw == 64 ? 3 : 1);

    const bool out_u8 = p.out.dtype == CLDNN_B200_U8;
    const int out_kind = out_u8 ? 0 : ((p.fused_eltw ? p.eltw_act : p.act) == CLDNN_B200_ACT_RELU ? 2 : 1);
    P.fast_variant = (out_kind << 1) | ((p.fused_eltw && p.act == CLDNN_B200_ACT_RELU) ? 1 : 0) | (P.mul_oqf ? 8 : 0);
    P.acc_bound = (float)p.kh * (float)p.kw * (float)p.ifm * (p.in.dtype == CLDNN_B200_U8 ? 255.0f : 128.0f) * 128.0f;
    P.epi_groups = pl.epi_groups;
    const bool use_fast = (p.tune <= 12 || p.tune > 24) && tc_fast_eligible(P);
    if (pl.pair && !use_fast) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_tc: CTA pairs exist on the specialised kernel only");
    if (pl.epi_groups > 2 && !use_fast) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_tc: four epilogue groups exist on the specialised kernel only");

    const size_t aux_bytes = use_fast ? tc_fast_aux_bytes() : sizeof(TcSmemAux);
    const size_t max_smem = (size_t)ctx->prop.sharedMemPerBlockOptin;
    const bool patch = pl.a_mode == A_PATCH;
    if (patch && !use_fast) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_i8_tc: the patch mode exists for the specialised epilogue configuration only");
    // Small weight tensors stay resident outside the patch mode as well: re-fetching them per tile costs as many memory requests
    // as the activation tile (a weight box has one row per output feature however few bytes a row holds), which is what
    // bounds the pointwise layers with few features.
    constexpr size_t kResidentWeightBytes = 48 * 1024;
    const size_t b_all = (size_t)P.n_tiles * P.k_steps * P.b_stage_bytes;
    if (use_fast && !patch && !pl.pair && b_all <= kResidentWeightBytes && P.total_tiles >= 2 * ctx->prop.multiProcessorCount) {
        P.b_resident = 1; P.b_total_bytes = (int32_t)b_all;
    }
    const bool resb = patch || P.b_resident;
    const size_t stage_bytes = (size_t)P.a_stage_bytes + (resb ? 0 : P.b_stage_bytes);
    const size_t resident = resb ? (size_t)P.b_total_bytes : 0;
    size_t staging_total = P.staged ? (size_t)P.nbuf * kBM * pl.bn : 0;
    // the specialised kernel's fused path keeps more staging tiles than accumulators (residual loads run further ahead)
    // as long as three operand stages still fit beside them
    P.nstg = P.nbuf;
    if (use_fast && p.fused_eltw && pl.bn >= 256 &&
        max_smem >= 1024 + aux_bytes + (size_t)3 * kBM * pl.bn + resident + 3 * stage_bytes) {
        // 256-feature tiles have two accumulators; a third staging tile lets the residual load of tile t+2 start before
        // the store of tile t has drained (measured: 108 -> 97 us on the 64 -> 256 layer of ResNet-50's first stage)
        P.nstg = 3;
        staging_total = (size_t)P.nstg * kBM * pl.bn;
    }
    // Few, large operand stages (the patch mode's three patches per stage) leave the loads of a tile in flight for only one
    // tile's worth of tensor-core work; with fewer staging tiles than accumulators another stage fits, and the producer runs a
    // tile further ahead of the load latency.  Four staging tiles keep both group counts a divisor of the ring.
    if (use_fast && P.staged && P.nstg == P.nbuf && P.nbuf > 4) {
        auto stages_with = [&](size_t staging) { return max_smem > 1024 + aux_bytes + staging + resident ? (max_smem - 1024 - aux_bytes - staging - resident) / stage_bytes : 0; };
        const size_t fewer = (size_t)4 * kBM * pl.bn;
        if (stages_with(staging_total) < 4 && stages_with(fewer) > stages_with(staging_total)) { P.nstg = 4; staging_total = fewer; }
    }
    if (max_smem < 1024 + aux_bytes + staging_total + resident + 2 * stage_bytes) {
        if (patch) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_i8_tc: not enough shared memory for the patch mode");
        P.staged = 0; staging_total = 0;
    }
    if (max_smem < 1024 + aux_bytes + 2 * stage_bytes) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_i8_tc: not enough shared memory");
    int stages = (int)((max_smem - 1024 - aux_bytes - staging_total - resident) / stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    P.stages = stages;
    P.ring_bytes = (int32_t)((size_t)stages * stage_bytes + resident);
    size_t smem_bytes = 1024 + (size_t)P.ring_bytes + staging_total + aux_bytes;
    const size_t one_cta_floor = max_smem / 2 + 1024;                // keeps one CTA per SM, so TMEM allocation never waits
    if (smem_bytes < one_cta_floor) smem_bytes = one_cta_floor;
    if (smem_bytes > max_smem) smem_bytes = max_smem;

    const CUtensorMapSwizzle sw = pl.bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (pl.bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    void* in_ptr = (char*)const_cast<void*>(a->input0) + p.in.offset;
    CUresult cr;
    if (pl.a_mode == A_FLAT) {
        cuuint64_t dims[2] = {(cuuint64_t)cs, (cuuint64_t)P.M_total};
        cuuint64_t strides[1] = {(cuuint64_t)p.in.px};
        cuuint32_t box[2] = {(cuuint32_t)pl.bk, (cuuint32_t)kBM};
        cuuint32_t es[2] = {1, 1};
        cr = g_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, in_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (pl.a_mode == A_IM2COL) {
        cuuint64_t dims[4] = {(cuuint64_t)cs, (cuuint64_t)p.in.x, (cuuint64_t)p.in.y, (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)p.in.px, (cuuint64_t)p.in.py, (cuuint64_t)p.in.pb};
        int lower[2] = {-p.pad_x, -p.pad_y};
        int upper[2] = {p.pad_x - (p.kw - 1) * p.dil_x, p.pad_y - (p.kh - 1) * p.dil_y};
        // the box of base pixels must produce exactly Q x P positions per image
        const int q_tm = (p.in.x + upper[0] - lower[0] - 1) / p.stride_x + 1, p_tm = (p.in.y + upper[1] - lower[1] - 1) / p.stride_y + 1;
        if (q_tm != P.Q || p_tm != P.P) return fail(CLDNN_B200_UNSUPPORTED_SIZE, "conv_i8_tc: im2col traversal does not match the output size");
        cuuint32_t es[4] = {1, (cuuint32_t)p.stride_x, (cuuint32_t)p.stride_y, 1};
        cr = g_encode_im2col(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, in_ptr, dims, strides, lower, upper, (cuuint32_t)pl.bk, (cuuint32_t)kBM, es,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (pl.a_mode == A_PATCH) {
        cuuint64_t dims[4] = {(cuuint64_t)cs, (cuuint64_t)p.in.x, (cuuint64_t)p.in.y, (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)p.in.px, (cuuint64_t)p.in.py, (cuuint64_t)p.in.pb};
        cuuint32_t box[4] = {(cuuint32_t)pl.bk, (cuuint32_t)pl.bw, (cuuint32_t)(pl.bh + p.kh - 1), 1};
        cuuint32_t es[4] = {1, 1, 1, 1};
        cr = g_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, in_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        // tiled 4-D box; a pointwise strided convolution reads a strided view of the input
        const int sx = p.stride_x, sy = p.stride_y;
        const bool strided_view = sx != 1 || sy != 1;
        cuuint64_t dims[4] = {(cuuint64_t)cs, (cuuint64_t)(strided_view ? P.Q : p.in.x), (cuuint64_t)(strided_view ? P.P : p.in.y), (cuuint64_t)p.in.b};
        cuuint64_t strides[3] = {(cuuint64_t)(p.in.px * sx), (cuuint64_t)(p.in.py * sy), (cuuint64_t)p.in.pb};
        cuuint32_t box[4] = {(cuuint32_t)pl.bk, (cuuint32_t)pl.bw, (cuuint32_t)pl.bh, (cuuint32_t)pl.bb};
        cuuint32_t es[4] = {1, 1, 1, 1};
        cr = g_encode_tiled(&P.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, in_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "conv_i8_tc: activation tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");
    {
        cuuint64_t dims[3] = {(cuuint64_t)cs, (cuuint64_t)(p.kh * p.kw), (cuuint64_t)p.ofm};
        cuuint64_t strides[2] = {(cuuint64_t)p.w_px, (cuuint64_t)p.w_po};
        cuuint32_t box[3] = {(cuuint32_t)pl.bk, 1, (cuuint32_t)b_rows};
        cuuint32_t es[3] = {1, 1, 1};
        void* w_ptr = (char*)const_cast<void*>(a->weights) + p.w_offset;
        cr = g_encode_tiled(&P.tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w_ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "conv_i8_tc: weights tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");
    }
    if (P.staged) {
        const CUtensorMapSwizzle osw = P.cw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (P.cw == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
        cldnn_b200_tensor ot = p.out; ot.f = p.ofm;
        cr = encode_pixel_map(&P.tmO, pl, (char*)a->output + p.out.offset, ot, 1, 1, P.cw, osw);
        if (cr == CUDA_SUCCESS && p.fused_eltw) {
            cldnn_b200_tensor rt = et; rt.f = p.ofm;
            cr = encode_pixel_map(&P.tmE, pl, (char*)const_cast<void*>(P.eltw) + et.offset, rt, esx, esy, P.cw, osw);
        }
        if (cr != CUDA_SUCCESS) return fail(CLDNN_B200_DEVICE_ERROR, "conv_i8_tc: output tensor map rejected by the driver (CUresult " + std::to_string((int)cr) + ")");
    }

    B200_CUDA(cudaFuncSetAttribute(conv_i8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)max_smem));

    int grid = ctx->prop.multiProcessorCount;
    if (grid > P.total_tiles) grid = P.total_tiles;
    if (pl.pair) grid &= ~1;                                           // whole clusters of two (total_tiles is even)
    if (grid < 1) return fail(CLDNN_B200_INVALID_ARG, "conv_i8_tc: empty output");
    const size_t smem = smem_bytes;
    if (use_fast) {
        if (!P.staged) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_i8_tc: not enough shared memory for the staged epilogue");
        B200_CUDA(tc_fast_configure(P, (int)max_smem));
        out->fn = [P, grid, smem](cudaStream_t s) { return tc_fast_launch(P, grid, smem, s); };
    } else
        out->fn = [P, grid, smem](cudaStream_t s) { conv_i8_tc_kernel<<<grid, kThreads, smem, s>>>(P); return cudaGetLastError(); };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

const KernelDef kdef_conv_i8_tc = {"conv_i8_tc", sizeof(cldnn_b200_conv_params), tc_supports, tc_tune_count, nullptr, tc_prepare};

}  // namespace b200
