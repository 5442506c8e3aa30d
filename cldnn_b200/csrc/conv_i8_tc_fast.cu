// conv_i8_tc_fast: the tensor-core 8-bit convolution specialised for the
// configuration whole quantised networks run in: per-channel dequantisation
// only (I_QF = O_QF = 1, integer or no bias), activations NONE / ReLU, 8-bit
// output, optional fused residual sum with a plain 8-bit second input, output
// features a multiple of the feature tile.  Same main loop and the same
// operation order as conv_i8_tc (fused_conv_eltwise_gpu_ref.cl:148-232); what
// differs is the epilogue, which is where those layers spend their time:
//   * the feature tile is a template parameter, every loop bound is static;
//   * two groups of four epilogue warps take alternate tiles, each warp owns one
//     32-row quadrant of its tile for all feature columns and loads the next 32
//     accumulator columns from tensor memory while it converts the current ones;
//   * rounding without conversion instructions (float->int conversions run at a sixth of
//     the add rate here): round-half-away(v) = sign(v) * floor(|v| + 0.5), the floor taken
//     from the mantissa of (|v| + 0.5) + 2^23, both additions rounding toward zero.  After
//     that every value is an integer, so the residual sum (one dp4a that also picks the
//     byte out of the residual word), the second ReLU and the saturation run in integer
//     arithmetic: round(relu(round(v) + e)) == relu(int(round(v)) + e).  All of it is exact
//     while |v| < 2^22; a bound on |v| is evaluated per feature tile from the constants
//     ((K * 255 * 128 + |bias|) * |q|) and tiles that could exceed it run the float-domain
//     path of the general kernel, element by element;
//   * unsigned saturation stands in for a ReLU that precedes it;
//   * the single thread that issues tcgen05.mma has its descriptors precomputed: at small
//     feature tiles an MMA runs for 48-64 clocks and the issue loop is the critical path.
// Patch mode (small 3x3-like filters whose whole weight tensor fits in shared memory): the
// weights are loaded once per CTA and each filter column needs one activation patch of
// (tile rows + kh - 1) x tile width pixels; the kh taps of the column read that patch at
// row offsets through the operand descriptor's start address, instead of kh separate loads.
// The kernel is launched with programmatic stream serialisation: its prologue
// (barrier set-up, tensor-memory allocation, descriptor prefetch) overlaps the
// tail of the previous kernel in the stream; griddepcontrol.wait orders every
// global-memory access after that kernel's completion.
#include "conv_i8_tc.hpp"
#include "conv_epilogue.cuh"

namespace b200 {

constexpr int kFastEpiWarp0 = 4;            // warp 0 operand loads, 1 MMA issue, 2 TMA stores, 3 residual loads, 4.. epilogue
constexpr int kMaxGroups = 4;               // epilogue warp groups of four warps each: two or four per CTA (template parameter)
constexpr int fast_threads(int groups) { return 128 + 128 * groups; }
constexpr int kMaxStg = 8;                 // staging tiles

struct FastAux {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[kMaxBufs];
    uint64_t tmem_empty[kMaxBufs];
    uint64_t res_full[kMaxStg];
    uint64_t stage_free[kMaxStg];
    uint64_t out_ready[kMaxStg];
    uint64_t drain;
    uint64_t b_full;                       // patch mode: the resident weights have landed
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t wide[kMaxGroups][4];          // per epilogue warp: a feature of the current tile may leave the integer-safe range
    alignas(16) int32_t bias_i[kMaxGroups][kMaxBN];
    alignas(16) float quant[kMaxGroups][kMaxBN];
};

size_t tc_fast_aux_bytes() { return sizeof(FastAux); }


__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A K-major swizzled operand descriptor split in halves: the high word is constant per launch
// (8-row group stride, descriptor version, swizzle mode), the low word holds the start address.
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout_type)
{
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | ((layout_type & 7u) << 29);
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3ffffu) >> 4) | (1u << 16); }
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi)
{
    uint64_t d; asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi)); return d;
}
// KK tensor-core instructions over one channel chunk, 32 bytes of K each
template <int KK, bool kPair = false>
__device__ __forceinline__ void mma_chunk(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t acc_first)
{
#pragma unroll
    for (int k = 0; k < KK; ++k) {
        if (kPair) mma_i8_ss_pair(d_tmem, desc64(a_lo + 2u * k, hi), desc64(b_lo + 2u * k, hi), idesc, k ? 1u : acc_first);
        else mma_i8_ss(d_tmem, desc64(a_lo + 2u * k, hi), desc64(b_lo + 2u * k, hi), idesc, k ? 1u : acc_first);
    }
}

// Patch mode, one channel chunk: KH x KW filter taps straight-line (a loop over run-time filter sizes costs the issuing
// thread ~130 clocks per MMA in address arithmetic and branches, against the 48 an N = 64 instruction runs for).
template <int KH, int KW, int KK>
__device__ __forceinline__ void patch_issue(uint32_t d_tmem, uint32_t a_lo, uint32_t b_col, uint32_t patch_step, uint32_t b_tap_step,
                                            uint32_t row_step, uint32_t b_row_step, uint32_t hi, uint32_t idesc, uint32_t accf)
{
#pragma unroll
    for (int s = 0; s < KW; ++s)
#pragma unroll
        for (int r = 0; r < KH; ++r)
            mma_chunk<KK>(d_tmem, a_lo + (uint32_t)s * patch_step + (uint32_t)r * row_step, b_col + (uint32_t)s * b_tap_step + (uint32_t)r * b_row_step,
                          hi, idesc, (s | r) ? 1u : accf);
}

// The accumulator has been read out: tell the MMA issuer (in a CTA pair it sits in the CTA of rank 0, and `bar` is then
// that CTA's barrier as a cluster address).
__device__ __forceinline__ void release_acc(uint32_t bar, bool pair)
{
    if (pair) mbar_arrive_cluster(bar); else mbar_arrive(bar);
}

template <int BN>
__device__ __forceinline__ void fast_chunk_ptrs(uint8_t* stg, int row, uint32_t sw, int c0, uint4*& p0, uint4*& p1)
{
    constexpr int CW = BN < 128 ? BN : 128;
    const int cb = c0 / CW, o = c0 - cb * CW;
    uint8_t* rowp = stg + (size_t)cb * kBM * CW + (size_t)row * CW;
    p0 = reinterpret_cast<uint4*>(rowp + ((((uint32_t)o >> 4) ^ sw) << 4));
    p1 = reinterpret_cast<uint4*>(rowp + (((((uint32_t)o >> 4) + 1u) ^ sw) << 4));
}

// One 32-row quadrant of a tile, feature columns 0 .. c_hi - 1 (c_hi: BN, or for the last feature tile of a ragged feature
// count the real columns rounded up to the loop's granularity: the surplus columns inside that hold zero accumulators and
// neutral constants, the columns beyond it are not converted at all, and the store clips both).
template <int BN, bool kFused, bool kRelu1, int kOut, bool kOqf = false>
__device__ __forceinline__ void fast_tile(const FastAux* aux, int group, uint32_t t_row, uint8_t* stg, int row, uint32_t sw,
                                          uint32_t tmem_empty_bar, int lane, uint32_t e_xor, int32_t k_pos, int32_t k_neg, float oqf = 1.0f,
                                          bool pair = false, int c_hi = BN)
{
    const int32_t* bias = aux->bias_i[group];
    const float* quant = aux->quant[group];
    uint32_t ra[32], rb[32];
    tmem_ld_32x32(t_row, ra);
#pragma unroll 1
    for (int c0 = 0; c0 < c_hi; c0 += 64) {
        uint4 *p0, *p1;
        tmem_ld_wait();
        tmem_ld_32x32(t_row + (uint32_t)(c0 + 32), rb);             // in flight while `ra` is converted
        fast_chunk_ptrs<BN>(stg, row, sw, c0, p0, p1);
        fast_chunk32<kFused, kRelu1, kOut, kOqf>(ra, bias + c0, quant + c0, p0, p1, e_xor, k_pos, k_neg, oqf);
        tmem_ld_wait();
        if (c0 + 64 < c_hi) tmem_ld_32x32(t_row + (uint32_t)(c0 + 64), ra);
        else {
            // the accumulator has been read out: the MMA issuer may reuse it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) release_acc(tmem_empty_bar, pair);
        }
        fast_chunk_ptrs<BN>(stg, row, sw, c0 + 32, p0, p1);
        fast_chunk32<kFused, kRelu1, kOut, kOqf>(rb, bias + c0 + 32, quant + c0 + 32, p0, p1, e_xor, k_pos, k_neg, oqf);
    }
}

// The same quadrant with one register buffer: used by the four-group variant, where 16 epilogue warps per SM hide the
// latency of the tensor-memory load between them and the register budget is 102 per thread.
template <int BN, bool kFused, bool kRelu1, int kOut, bool kOqf = false>
__device__ __forceinline__ void fast_tile_single(const FastAux* aux, int group, uint32_t t_row, uint8_t* stg, int row, uint32_t sw,
                                                 uint32_t tmem_empty_bar, int lane, uint32_t e_xor, int32_t k_pos, int32_t k_neg, float oqf = 1.0f,
                                                 bool pair = false, int c_hi = BN)
{
    const int32_t* bias = aux->bias_i[group];
    const float* quant = aux->quant[group];
#pragma unroll 1
    for (int c0 = 0; c0 < c_hi; c0 += 32) {
        uint32_t r[32];
        uint4 *p0, *p1;
        tmem_ld_32x32(t_row + (uint32_t)c0, r);
        fast_chunk_ptrs<BN>(stg, row, sw, c0, p0, p1);
        tmem_ld_wait();
        if (c0 + 32 >= c_hi) {
            // the accumulator has been read out: the MMA issuer may reuse it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) release_acc(tmem_empty_bar, pair);
        }
        fast_chunk32<kFused, kRelu1, kOut, kOqf>(r, bias + c0, quant + c0, p0, p1, e_xor, k_pos, k_neg, oqf);
    }
}

// The variants with a uniform O_QF stay out of line, so that the common ones keep their registers and code layout.
template <int BN, bool kFused, int kOut, int G>
__device__ __noinline__ void fast_tile_oqf(const FastAux* aux, int group, uint32_t t_row, uint8_t* stg, int row, uint32_t sw,
                                           uint32_t tmem_empty_bar, int lane, uint32_t e_xor, int32_t k_pos, int32_t k_neg, float oqf, bool pair, int c_hi)
{
    if (G > 2) fast_tile_single<BN, kFused, false, kOut, true>(aux, group, t_row, stg, row, sw, tmem_empty_bar, lane, e_xor, k_pos, k_neg, oqf, pair, c_hi);
    else fast_tile<BN, kFused, false, kOut, true>(aux, group, t_row, stg, row, sw, tmem_empty_bar, lane, e_xor, k_pos, k_neg, oqf, pair, c_hi);
}
// two register buffers with two groups, one with four
template <int BN, bool kFused, bool kRelu1, int kOut, int G>
__device__ __forceinline__ void fast_tile_any(const FastAux* aux, int group, uint32_t t_row, uint8_t* stg, int row, uint32_t sw,
                                              uint32_t tmem_empty_bar, int lane, uint32_t e_xor, int32_t k_pos, int32_t k_neg, bool pair, int c_hi)
{
    if (G > 2) fast_tile_single<BN, kFused, kRelu1, kOut>(aux, group, t_row, stg, row, sw, tmem_empty_bar, lane, e_xor, k_pos, k_neg, 1.0f, pair, c_hi);
    else fast_tile<BN, kFused, kRelu1, kOut>(aux, group, t_row, stg, row, sw, tmem_empty_bar, lane, e_xor, k_pos, k_neg, 1.0f, pair, c_hi);
}

// The same tile in float arithmetic, element by element (fused residual only):
// taken when a feature's value range could leave the integer-safe range.
template <int BN>
__device__ __noinline__ void fast_tile_wide(const TcParams& P, const FastAux* aux, int group, uint32_t t_row, uint8_t* stg, int row,
                                            uint32_t sw, uint32_t tmem_empty_bar, int lane, bool pair)
{
    const EpiCfg& c = P.epi;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + (uint32_t)c0, r);
        tmem_ld_wait();
        uint4 *p0, *p1;
        fast_chunk_ptrs<BN>(stg, row, sw, c0, p0, p1);
        uint8_t* b0 = reinterpret_cast<uint8_t*>(p0);
        uint8_t* b1 = reinterpret_cast<uint8_t*>(p1);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            uint8_t* bp = (j < 16 ? b0 : b1) + (j & 15);
            const float e = c.eltw_dtype == CLDNN_B200_U8 ? (float)*bp : (float)*reinterpret_cast<int8_t*>(bp);
            const float v = epi_quant(c, (int32_t)r[j] + aux->bias_i[group][c0 + j], aux->quant[group][c0 + j], 0.0f, 1.0f, e, 1.0f);
            const int32_t i = __float2int_rz(v);
            *bp = c.out_dtype == CLDNN_B200_U8 ? (uint8_t)min(255, max(0, i)) : (uint8_t)(int8_t)min(127, max(-128, i));
        }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) release_acc(tmem_empty_bar, pair);
}

// The tiles a role visits: tile = first + i * step.  Integer division costs a single thread ~120 clocks, so the
// decomposition of the tile index (feature tile, pixel tile, and the pixel tile's box or first-pixel coordinates) is kept
// incrementally: mixed-radix digits advance by the digits of the step, and are recomputed only when the feature tile changes.
struct TileWalk {
    int tile, step, n_tile, m_tile;
    int d0, d1, d2;                 // boxed: box column, box row, box batch; im2col: q, p, n of the tile's first pixel
    int s0, s1, s2;                 // digits of the step
    int r0, r1;                     // radices
    int mode, m_tiles, total;
    __device__ __forceinline__ void digits(int m)
    {
        if (mode == A_IM2COL) { const int64_t px = (int64_t)m * kBM; d0 = (int)(px % r0); const int64_t t = px / r0; d1 = (int)(t % r1); d2 = (int)(t / r1); }
        else if (mode == A_TILED || mode == A_PATCH) { d0 = m % r0; const int t = m / r0; d1 = t % r1; d2 = t / r1; }
    }
    __device__ __forceinline__ void init(const TcParams& P, int first, int stp)
    {
        tile = first; step = stp; mode = P.a_mode; m_tiles = P.m_tiles; total = P.total_tiles;
        const bool im = mode == A_IM2COL;
        r0 = im ? P.Q : P.tiles_w; r1 = im ? P.P : P.tiles_h;
        if (r0 < 1) r0 = 1; if (r1 < 1) r1 = 1;
        const int64_t sm = im ? (int64_t)stp * kBM : (int64_t)stp;
        s0 = (int)(sm % r0); const int64_t t = sm / r0; s1 = (int)(t % r1); s2 = (int)(t / r1);
        n_tile = first / m_tiles; m_tile = first - n_tile * m_tiles;
        d0 = d1 = d2 = 0;
        if (first < total) digits(m_tile);
    }
    __device__ __forceinline__ bool valid() const { return tile < total; }
    __device__ __forceinline__ void next()
    {
        tile += step; m_tile += step;
        if (m_tile >= m_tiles) {
            while (m_tile >= m_tiles) { m_tile -= m_tiles; ++n_tile; }
            if (tile < total) digits(m_tile);
            return;
        }
        d0 += s0; if (d0 >= r0) { d0 -= r0; ++d1; }
        d1 += s1; if (d1 >= r1) { d1 -= r1; ++d2; }
        d2 += s2;
    }
};

// kPair: the CTAs of a cluster of two work on two vertically adjacent pixel tiles with one tensor-core instruction stream
// (tcgen05 cta_group::2, M = 256): each CTA loads its own 128 pixel rows and HALF of the feature tile's weight rows, so a
// stage costs an SM (128 + BN / 2) x BK bytes of L2 traffic instead of (128 + BN) x BK for the same tensor-core work.
template <int BN, bool kFused, int G, bool kPair = false>
__global__ void __launch_bounds__(fast_threads(G), 1)
conv_i8_tc_fast_kernel(const __grid_constant__ TcParams P)
{
    constexpr int kGroups = G;                                          // epilogue warp groups, taking tiles in turn
    constexpr int NBUF = BN >= 256 ? 2 : (BN >= 128 ? 4 : 8);         // all 512 columns of tensor memory
    constexpr int CW = BN < 128 ? BN : 128;
    constexpr int COLB = BN / CW;
    constexpr uint32_t kStagingBytes = (uint32_t)(kBM * BN);
    // staging tiles: with a fused residual they also receive the residual tile, whose load has HBM latency in front of the
    // epilogue; more of them than accumulators (the host decides how many fit) lets those loads run further ahead
    const int NSTG = P.nstg;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t a_base = base;
    const uint32_t b_base = base + (uint32_t)(P.stages * P.a_stage_bytes);
    const uint32_t ring_bytes = (uint32_t)P.ring_bytes;
    uint8_t* staging = smem + ring_bytes;
    FastAux* aux = reinterpret_cast<FastAux*>(smem + ring_bytes + (uint32_t)NSTG * kStagingBytes);
    volatile uint32_t* s_abort = &aux->abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = kPair ? cluster_ctarank() : 0u;              // 0 issues the tensor-core instructions of the pair

    if (threadIdx.x == 0) {
        for (int s = 0; s < P.stages; ++s) { mbar_init(smem_u32(&aux->full[s]), 1); mbar_init(smem_u32(&aux->empty[s]), 1); }
        // in a pair the accumulators of both CTAs are released to rank 0's barrier: four warps from each
        for (int a = 0; a < kMaxBufs; ++a) { mbar_init(smem_u32(&aux->tmem_full[a]), 1); mbar_init(smem_u32(&aux->tmem_empty[a]), kPair ? 8 : 4); }
        for (int a = 0; a < kMaxStg; ++a) {
            mbar_init(smem_u32(&aux->res_full[a]), 1); mbar_init(smem_u32(&aux->stage_free[a]), 1);
            mbar_init(smem_u32(&aux->out_ready[a]), 4);
        }
        mbar_init(smem_u32(&aux->drain), 1);
        mbar_init(smem_u32(&aux->b_full), 1);
        aux->abort = 0u;
        mbar_fence_init();
        prefetch_tensormap(&P.tmA); prefetch_tensormap(&P.tmB); prefetch_tensormap(&P.tmO);
        if (kFused) prefetch_tensormap(&P.tmE);
    }
    if (warp == 1) {
        if (kPair) { tmem_alloc_pair(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish_pair(); }
        else { tmem_alloc(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish(); }
    }
    tc_fence_before();
    if (kPair) cluster_sync_all();                     // the peer's barriers exist before anything arrives on them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    griddep_launch_dependents();
    // Each role waits for the previous kernel of the stream itself, right before it first touches memory that kernel wrote or
    // read (activations, residual, output).  The weights are constants of the network: the producer starts their resident
    // copy before it waits, so that copy runs under the previous kernel's tail.  The MMA issuers touch no global memory.

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        const bool patch = P.a_mode == A_PATCH;
        // The whole warp walks the tiles and waits on the barriers; one elected lane issues the copies.  With the loop
        // warp-uniform the compiler keeps the loop state and the copies' operands on the uniform datapath, which a loop
        // inside a one-lane branch cannot use: the role's instruction count per stage is what bounds small-tile layers.
        {
            const bool leader = ptx::elect_one();
            // Weights that are small enough stay resident in the other modes too (P.b_resident): a layer with few input and
            // output features would otherwise fetch the same few KB again for every tile -- as many requests as the
            // activation tile itself costs, for nothing.
            const bool resb = patch || P.b_resident != 0;
            if (leader && resb && blockIdx.x < (unsigned)P.total_tiles) {
                // every filter tap (and channel chunk) of every feature tile, once per CTA
                const uint32_t bf = smem_u32(&aux->b_full);
                mbar_expect_tx(bf, (uint32_t)P.b_total_bytes);
                uint32_t dst = b_base;
                for (int nt = 0; nt < P.n_tiles; ++nt)
                    for (int tp = 0; tp < P.kh * P.kw; ++tp)
                        for (int ch = 0; ch < P.chunks; ++ch, dst += (uint32_t)P.b_stage_bytes)
                            tma_load_3d(dst, &P.tmB, bf, ch * P.bk, tp, nt * BN);
            }
            griddep_wait();
            int stage = 0; uint32_t phase = 0; int64_t issued = 0; bool ok = true;
            const int stages = P.stages, k_steps = P.k_steps, chunks = P.chunks, bk = P.bk, kw = P.kw;
            const uint32_t tx = (uint32_t)(resb ? P.a_tx_bytes : P.a_tx_bytes + P.b_tx_bytes);
            const uint32_t a_stage = (uint32_t)P.a_stage_bytes, b_stage = (uint32_t)P.b_stage_bytes;
            const uint32_t full0 = smem_u32(&aux->full[0]), empty0 = smem_u32(&aux->empty[0]);
            TileWalk w; w.init(P, blockIdx.x, gridDim.x);
            // Everything the loop needs sits in registers: this thread's scalar instructions are on the critical path of
            // the layers whose stages hold little tensor-core work.
            const int mode = P.a_mode, dil_x = P.dil_x, dil_y = P.dil_y, patch_alloc = P.patch_alloc;
            for (; w.valid() && ok; w.next()) {
                int c_w = 0, c_h = 0, c_n = 0;
                if (mode == A_IM2COL) { c_w = w.d0 * P.stride_x - P.pad_x; c_h = w.d1 * P.stride_y - P.pad_y; c_n = w.d2; }
                else if (mode == A_TILED || patch) { c_w = w.d0 * P.bw - P.pad_x; c_h = w.d1 * P.bh - P.pad_y; c_n = w.d2 * P.bb; }
                const int m0 = w.m_tile * kBM, n0 = w.n_tile * BN;
                int tap = 0, cc = 0, off_w = 0, off_h = 0, sx = 0;
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!__all_sync(0xffffffffu, mbar_wait_lean(empty0 + 8u * (uint32_t)stage, phase ^ 1u, s_abort, P.status, kErrProducer))) { ok = false; break; }
                    const uint32_t full = full0 + 8u * (uint32_t)stage;
                    const uint32_t dst = a_base + (uint32_t)stage * a_stage;
                    const int c0 = cc * bk;
                    if (leader && kPair) {
                        // both CTAs' copies report to rank 0's barrier, which expects the bytes of both
                        const uint32_t full_r0 = mapa_rank(full, 0u);
                        if (rank == 0u) mbar_expect_tx(full, 2u * tx);
                        tma_load_3d_pair(b_base + (uint32_t)stage * b_stage, &P.tmB, full_r0, c0, tap, n0 + (int)rank * (BN / 2));
                        if (mode == A_FLAT) tma_load_2d_pair(dst, &P.tmA, full_r0, c0, m0);
                        else if (mode == A_IM2COL) tma_load_im2col_4d_pair(dst, &P.tmA, full_r0, c0, c_w, c_h, c_n, (uint16_t)off_w, (uint16_t)off_h);
                        else tma_load_4d_pair(dst, &P.tmA, full_r0, c0, c_w + off_w, c_h + off_h, c_n);
                    } else if (leader) {
                        mbar_expect_tx(full, tx);
                        if (!resb) tma_load_3d(b_base + (uint32_t)stage * b_stage, &P.tmB, full, c0, tap, n0);
                        if (patch) {                                                            // one patch per filter column
                            for (int s = 0; s < kw; ++s) tma_load_4d(dst + (uint32_t)(s * patch_alloc), &P.tmA, full, c0, c_w + s, c_h, c_n);
                        }
                        else if (mode == A_FLAT) tma_load_2d(dst, &P.tmA, full, c0, m0);
                        else if (mode == A_IM2COL) tma_load_im2col_4d(dst, &P.tmA, full, c0, c_w, c_h, c_n, (uint16_t)off_w, (uint16_t)off_h);
                        else tma_load_4d(dst, &P.tmA, full, c0, c_w + off_w, c_h + off_h, c_n);
                    }
                    ++issued;
                    if (++cc == chunks) { cc = 0; ++tap; off_w += dil_x; if (++sx == kw) { sx = 0; off_w = 0; off_h += dil_y; } }
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // unwind: let the copies already in flight land before the CTA's shared memory goes away
                int st = stage; uint32_t ph = phase;
                const int pending = issued < stages ? (int)issued : stages;
                for (int i = 0; i < pending; ++i) {
                    if (--st < 0) { st = stages - 1; ph ^= 1u; }
                    const uint64_t t0 = globaltimer();
                    while (!mbar_try_wait(full0 + 8u * (uint32_t)st, ph) && globaltimer() - t0 < 100000000ull) { }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        // One elected lane feeds the tensor core while the whole warp runs the loop (see the producer); everything that can be
        // precomputed is precomputed, because at small feature tiles an MMA runs for only 48-64 clocks and a dependent
        // scalar instruction costs ~4.
        // In a pair only the CTA of rank 0 issues; its instructions and commits act on both CTAs.
        if (!kPair || rank == 0u) {
            const bool leader = ptx::elect_one();
            const uint32_t hi = desc_hi(P.sbo, P.layout_type);
            const uint32_t a_lo0 = desc_lo(a_base), b_lo0 = desc_lo(b_base);
            const uint32_t a_step = (uint32_t)P.a_stage_bytes >> 4, b_step = (uint32_t)P.b_stage_bytes >> 4;
            const uint32_t full0 = smem_u32(&aux->full[0]), empty0 = smem_u32(&aux->empty[0]);
            const int kk = P.bk >> 5, stages = P.stages, k_steps = P.k_steps;
            const uint32_t idesc = P.idesc;
            const bool patch = P.a_mode == A_PATCH;
            const uint32_t row_step = (uint32_t)(P.bw * P.bk) >> 4;                    // patch mode: one filter row further down the patch
            const uint32_t b_row_step = (uint32_t)(P.kw * P.chunks) * b_step;          //             the weights of the next filter row
            const int kh = P.kh, kw_ = P.kw;
            const uint32_t patch_step = (uint32_t)P.patch_alloc >> 4;                  //             the next filter column's patch
            const uint32_t b_tap_step = (uint32_t)P.chunks * b_step;                   //             the weights of the next filter column
            const int patch_kind = (kh == 3 && kw_ == 3) ? (kk == 2 ? 1 : (kk == 4 ? 2 : 0)) : 0;   // 3x3 filters are issued straight-line
            int stage = 0; uint32_t phase = 0; bool ok = true; int t = 0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            const bool resb = !patch && P.b_resident != 0;                           // resident weights outside the patch mode
            if ((patch || resb) && blockIdx.x < (unsigned)P.total_tiles) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->b_full), 0u, s_abort, P.status, kErrMma + 2u));
            TileWalk walk; walk.init(P, blockIdx.x, gridDim.x);
            for (; walk.valid() && ok; walk.next(), ++t) {
                const int acc = t % NBUF;
                if (!__all_sync(0xffffffffu, mbar_wait_lean(smem_u32(&aux->tmem_empty[acc]), (((uint32_t)(t / NBUF) & 1u)) ^ 1u, s_abort, P.status, kErrMma))) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                uint32_t accf = 0u;
                uint32_t b_col = 0u;                                                   // patch mode: weights of (filter column, channel chunk)
                if (patch) b_col = b_lo0 + (uint32_t)(walk.n_tile * kh) * b_row_step;
                uint32_t b_res = b_lo0 + (uint32_t)(walk.n_tile * k_steps) * b_step;  // resident weights: step ks of this feature tile
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!__all_sync(0xffffffffu, mbar_wait_lean(full0 + 8u * (uint32_t)stage, phase, s_abort, P.status, kErrMma + 1u))) { ok = false; break; }
                    if (!patch) {
                        const uint32_t b_cur = resb ? b_res : b_lo;
                        if (kk == 4) { if (leader) mma_chunk<4, kPair>(d_tmem, a_lo, b_cur, hi, idesc, accf); }
                        else if (kk == 2) { if (leader) mma_chunk<2, kPair>(d_tmem, a_lo, b_cur, hi, idesc, accf); }
                        else { if (leader) mma_chunk<1, kPair>(d_tmem, a_lo, b_cur, hi, idesc, accf); }
                        accf = 1u; b_res += b_step;
                    } else {
                        if (patch_kind == 1) { if (leader) patch_issue<3, 3, 2>(d_tmem, a_lo, b_col, patch_step, b_tap_step, row_step, b_row_step, hi, idesc, accf); }
                        else if (patch_kind == 2) { if (leader) patch_issue<3, 3, 4>(d_tmem, a_lo, b_col, patch_step, b_tap_step, row_step, b_row_step, hi, idesc, accf); }
                        else {
                            // per filter column s one patch; rows r*bw .. r*bw+127 of it are the tile's 128 pixels under filter row r
                            uint32_t as = a_lo, bs = b_col;
                            for (int s = 0; s < kw_; ++s, as += patch_step, bs += b_tap_step) {
                                uint32_t ar = as, br = bs;
                                for (int r = 0; r < kh; ++r, ar += row_step, br += b_row_step) {
                                    if (kk == 4) { if (leader) mma_chunk<4>(d_tmem, ar, br, hi, idesc, accf); }
                                    else if (kk == 2) { if (leader) mma_chunk<2>(d_tmem, ar, br, hi, idesc, accf); }
                                    else { if (leader) mma_chunk<1>(d_tmem, ar, br, hi, idesc, accf); }
                                    accf = 1u;
                                }
                            }
                        }
                        accf = 1u;
                        b_col += b_step;                                                     // next channel chunk
                    }
                    if (leader) { if (kPair) tc_commit_pair(empty0 + 8u * (uint32_t)stage); else tc_commit(empty0 + 8u * (uint32_t)stage); }                           // frees the stage once these MMAs have read it
                    if (++stage == stages) { stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0; }
                    else { a_lo += a_step; b_lo += b_step; }
                }
                if (ok && leader) { if (kPair) tc_commit_pair(smem_u32(&aux->tmem_full[acc])); else tc_commit(smem_u32(&aux->tmem_full[acc])); }
            }
            // drain: every issued MMA must have retired before TMEM is released
            if (leader) tc_commit(smem_u32(&aux->drain));
            const uint64_t t0 = globaltimer();
            while (!mbar_try_wait(smem_u32(&aux->drain), 0u)) {
                if (globaltimer() - t0 > kWaitLimitNs) { atomicCAS(P.status, 0u, kErrDrain); break; }
            }
        }
    } else if (warp == 2) {
        // ------------------------------ TMA store issuer --------------------------
        {
            const bool leader = ptx::elect_one();                    // issues, commits and waits for the stores: bulk groups are per thread
            griddep_wait();
            int t = 0;
            TileWalk walk; walk.init(P, blockIdx.x, gridDim.x);
            if (P.a_mode == A_IM2COL) walk.mode = A_FLAT;            // the output of an im2col tile is addressed by its first pixel index
            for (; walk.valid(); walk.next(), ++t) {
                const int n_tile = walk.n_tile, m_tile = walk.m_tile;
                const int a = t % NSTG;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->out_ready[a]), ((uint32_t)(t / NSTG) & 1u), s_abort, P.status, kErrEpilogue + 2u))) break;
                if (!leader) continue;
                const bool boxed = P.a_mode == A_TILED || P.a_mode == A_PATCH;
                const int tw = walk.d0, th = walk.d1, tb = walk.d2;
#pragma unroll
                for (int cb = 0; cb < COLB; ++cb) {
                    const int f0 = n_tile * BN + cb * CW;
                    if (f0 >= P.ofm) break;                         // ragged feature count: nothing of the tensor in this block
                    const uint32_t src = smem_u32(staging) + (uint32_t)a * kStagingBytes + (uint32_t)(cb * kBM * CW);
                    if (boxed) tma_store_4d(&P.tmO, src, f0, tw * P.bw, th * P.bh, tb * P.bb);
                    else tma_store_2d(&P.tmO, src, f0, m_tile * kBM);
                }
                bulk_commit();
                bulk_wait_read0();                                  // the buffer may be refilled once TMA has read it
                mbar_arrive(smem_u32(&aux->stage_free[a]));
            }
        }
    } else if (warp == 3) {
        // ------------------------------ residual loader ---------------------------
        // Second input of the fused sum: same pixels and features as the output tile, brought into the
        // staging buffer the epilogue will overwrite.  Its own warp, so that waiting for a staging buffer
        // never holds back the operand loads of later tiles.
        if (kFused) {
            const bool leader = ptx::elect_one();
            griddep_wait();
            int t = 0;
            TileWalk walk; walk.init(P, blockIdx.x, gridDim.x);
            if (P.a_mode == A_IM2COL) walk.mode = A_FLAT;
            for (; walk.valid(); walk.next(), ++t) {
                const int n_tile = walk.n_tile, m_tile = walk.m_tile;
                const bool boxed = P.a_mode == A_TILED || P.a_mode == A_PATCH;
                const int o_w = walk.d0 * P.bw, o_h = walk.d1 * P.bh, c_n = walk.d2 * P.bb;
                const int a = t % NSTG;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->stage_free[a]), (((uint32_t)(t / NSTG) & 1u)) ^ 1u, s_abort, P.status, kErrProducer + 1u))) break;
                if (!leader) continue;
                const uint32_t rf = smem_u32(&aux->res_full[a]);
                int cbs = 0;                                        // column blocks that hold features of the tensor
#pragma unroll
                for (int cb = 0; cb < COLB; ++cb) if (n_tile * BN + cb * CW < P.ofm) ++cbs;
                mbar_expect_tx(rf, (uint32_t)(P.stage_rows * CW * cbs));
#pragma unroll
                for (int cb = 0; cb < COLB; ++cb) {
                    const uint32_t dst = smem_u32(staging) + (uint32_t)a * kStagingBytes + (uint32_t)(cb * kBM * CW);
                    const int f0 = n_tile * BN + cb * CW;
                    if (f0 >= P.ofm) break;
                    if (boxed) tma_load_4d(dst, &P.tmE, rf, f0, o_w, o_h, c_n);
                    else tma_load_2d(dst, &P.tmE, rf, f0, m_tile * kBM);
                }
            }
        }
    } else if (warp >= kFastEpiWarp0) {
        // ------------------------------ epilogue ----------------------------------
        griddep_wait();                                             // (it reads only constants from global memory, and the status word)
        const int ew = warp - kFastEpiWarp0;
        const int quad = ew & 3;                                    // TMEM lanes 32*quad .. 32*quad+31 (warp index mod 4)
        const int group = ew >> 2;
        const int row = quad * 32 + lane;
        const int gt = (ew & 3) * 32 + lane;                        // thread index within the group
        const uint32_t sw = CW == 128 ? ((uint32_t)row & 7u) : (((uint32_t)row >> 1) & 3u);
        const EpiCfg& c = P.epi;
        // a signed residual is read as unsigned bytes + 128 and the 128 taken back out of the constants
        const bool res_s8 = kFused && c.eltw_dtype != CLDNN_B200_U8;
        const uint32_t e_xor = res_s8 ? 0x80808080u : 0u;
        const int32_t k_pos = kMagicBits + (res_s8 ? 128 : 0), k_neg = kMagicBits - (res_s8 ? 128 : 0);
        const int variant = P.fast_variant & 7;
        const bool with_oqf = (P.fast_variant & 8) != 0;            // uniform O_QF after the dequantisation
        const float oqf = c.o_qf, oqf_abs = with_oqf ? fabsf(c.o_qf) : 1.0f;
        int cur_n_tile = -1; bool ok = true; bool wide = false;
        int t = group;
        TileWalk walk; walk.init(P, blockIdx.x + group * gridDim.x, kGroups * gridDim.x);
        walk.mode = A_FLAT;                                         // only the feature tile is needed here
        for (; walk.valid() && ok; walk.next(), t += kGroups) {
            const int n_tile = walk.n_tile;
            const int acc = t % NBUF;
            const uint32_t par = (uint32_t)(t / NBUF) & 1u;
            if (n_tile != cur_n_tile) {
                named_bar_sync(1 + group, 128);                     // every warp of the group has left the previous feature range
                bool w = false;
                for (int j = gt; j < BN; j += 128) {
                    const int f = n_tile * BN + j;
                    // columns past the last feature (ragged count): zero accumulators (their weight rows are out of the
                    // tensor map's range), neutral constants, and the store clips them
                    const bool real = f < P.ofm;
                    const int32_t bi = (real && c.bias_dtype != CLDNN_B200_NONE) ? ((const int32_t*)P.bias)[f] : 0;
                    const float q = real ? P.quant[f] : 1.0f;
                    aux->bias_i[group][j] = bi; aux->quant[group][j] = q;
                    // (columns past the last feature hold zero accumulators: they cannot leave the range, whatever O_QF is)
                    w = w || (real && !(__fmul_rn(__fmul_rn(__fadd_rn(P.acc_bound, fabsf((float)bi)), fabsf(q)), oqf_abs) < 4.0e6f));
                }
                w = __any_sync(0xffffffffu, w);
                if (lane == 0) aux->wide[group][quad] = w ? 1u : 0u;
                named_bar_sync(1 + group, 128);
                wide = (aux->wide[group][0] | aux->wide[group][1] | aux->wide[group][2] | aux->wide[group][3]) != 0u;
                cur_n_tile = n_tile;
            }
            if (!mbar_wait(smem_u32(&aux->tmem_full[acc]), par, s_abort, P.status, kErrEpilogue)) { ok = false; break; }
            // the staging buffer is ours once its residual tile has landed (fused) or its previous store has been read out
            const int sb = t % NSTG; const uint32_t spar = (uint32_t)(t / NSTG) & 1u;
            const bool got = kFused ? mbar_wait(smem_u32(&aux->res_full[sb]), spar, s_abort, P.status, kErrEpilogue + 1u)
                                    : mbar_wait(smem_u32(&aux->stage_free[sb]), spar ^ 1u, s_abort, P.status, kErrEpilogue + 1u);
            if (!got) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
            uint8_t* stg = staging + (size_t)sb * kStagingBytes;
            const uint32_t te = kPair ? mapa_rank(smem_u32(&aux->tmem_empty[acc]), 0u) : smem_u32(&aux->tmem_empty[acc]);
            // columns to convert: all of the tile, or the real ones of a ragged last feature tile in whole loop trips
            const int real_cols = P.ofm - n_tile * BN;
            const int c_hi = real_cols >= BN ? BN : ((real_cols + (G > 2 ? 31 : 63)) & ~(G > 2 ? 31 : 63));
            if (wide) fast_tile_wide<BN>(P, aux, group, t_row, stg, row, sw, te, lane, kPair);
            else if (with_oqf) {
                // u8 or plain s8 output, no ReLU between convolution and residual sum (the host admits nothing else here)
                if (kFused) {
                    if ((variant >> 1) == 0) fast_tile_oqf<BN, true, 0, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, oqf, kPair, c_hi);
                    else fast_tile_oqf<BN, true, 1, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, oqf, kPair, c_hi);
                } else {
                    if ((variant >> 1) == 0) fast_tile_oqf<BN, false, 0, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, oqf, kPair, c_hi);
                    else fast_tile_oqf<BN, false, 1, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, oqf, kPair, c_hi);
                }
            }
            else if (kFused) {
                switch (variant) {
                    case 0: fast_tile_any<BN, true, false, 0, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    case 1: fast_tile_any<BN, true, true, 0, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    case 2: fast_tile_any<BN, true, false, 1, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    case 3: fast_tile_any<BN, true, true, 1, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    case 4: fast_tile_any<BN, true, false, 2, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    default: fast_tile_any<BN, true, true, 2, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                }
            } else {
                switch (variant >> 1) {
                    case 0: fast_tile_any<BN, false, false, 0, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    case 1: fast_tile_any<BN, false, false, 1, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                    default: fast_tile_any<BN, false, false, 2, G>(aux, group, t_row, stg, row, sw, te, lane, e_xor, k_pos, k_neg, kPair, c_hi); break;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->out_ready[sb]));
        }
    }

    tc_fence_before();
    // a pair leaves together: rank 0's tensor-core instructions read the peer's shared memory and the peer arrives on rank 0's barriers
    if (kPair) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) { tc_fence_after(); if (kPair) tmem_dealloc_pair(tmem_base, P.tmem_cols); else tmem_dealloc(tmem_base, P.tmem_cols); }
}


// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
bool tc_fast_eligible(const TcParams& P)
{
    if (!P.lean || !P.staged) return false;
    if (P.bn != 64 && P.bn != 128 && P.bn != 256) return false;
    if (P.pair && (P.bn < 128 || P.a_mode == A_PATCH || P.epi_groups != 2)) return false;
    // a uniform O_QF: positive, and only in front of an unsigned or plain signed saturation
    if (P.mul_oqf) {
        if (P.epi.calibration || !(P.epi.o_qf > 0.0f)) return false;
        if ((P.fast_variant & 1) || ((P.fast_variant >> 1) & 3) == 2) return false;
    }
    if (P.epi.bias_dtype != CLDNN_B200_NONE && P.epi.bias_dtype != CLDNN_B200_I32) return false;
    return true;
}

static const void* fast_kernel_pair(const TcParams& P)
{
    const bool f = P.epi.fused_eltw != 0;
    if (P.bn == 128) return f ? (const void*)conv_i8_tc_fast_kernel<128, true, 2, true> : (const void*)conv_i8_tc_fast_kernel<128, false, 2, true>;
    return f ? (const void*)conv_i8_tc_fast_kernel<256, true, 2, true> : (const void*)conv_i8_tc_fast_kernel<256, false, 2, true>;
}
template <int G>
static const void* fast_kernel_of_g(const TcParams& P)
{
    const bool f = P.epi.fused_eltw != 0;
    switch (P.bn) {
    case 64:  return f ? (const void*)conv_i8_tc_fast_kernel<64, true, G> : (const void*)conv_i8_tc_fast_kernel<64, false, G>;
    case 128: return f ? (const void*)conv_i8_tc_fast_kernel<128, true, G> : (const void*)conv_i8_tc_fast_kernel<128, false, G>;
    default:  return f ? (const void*)conv_i8_tc_fast_kernel<256, true, G> : (const void*)conv_i8_tc_fast_kernel<256, false, G>;
    }
}
static const void* fast_kernel_of(const TcParams& P)
{
    if (P.pair) return fast_kernel_pair(P);
    return P.epi_groups > 2 ? fast_kernel_of_g<4>(P) : fast_kernel_of_g<2>(P);
}

cudaError_t tc_fast_configure(const TcParams& P, int max_smem)
{
    return cudaFuncSetAttribute(fast_kernel_of(P), cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

cudaError_t tc_fast_launch(const TcParams& P, int grid, size_t smem_bytes, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3((unsigned)fast_threads(P.epi_groups > 2 ? 4 : 2)); cfg.dynamicSmemBytes = smem_bytes; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (P.pair) {                                                       // clusters of two CTAs (the grid is even)
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    void* args[1] = {const_cast<TcParams*>(&P)};
    return cudaLaunchKernelExC(&cfg, fast_kernel_of(P), args);
}

}  // namespace b200
