// conv_first_tc: the first convolution of a network in its general form -- few
// input features (3 for images), any filter size / stride / dilation (VGG's
// 3x3, AlexNet's 11x11 stride 4), fp16 or 8-bit -- on the tensor cores, read
// straight from the caller's input layout (planar bfyx as images arrive, or any
// other pitches) with no padded or reordered copy of the input in HBM.  With 3
// input features the generic tensor-core kernels would pad every filter tap to
// 16 / 32 features and multiply mostly zeros; here only the filter rows are
// padded, to 8 bytes.  It stands where the reference uses its first-layer kernels
// (cl_kernels/convolution_gpu_bfyx_os_iyx_osv16.cl for fp16 images,
// convolution_gpu_byxf_fs_bs_yx_bsv4_fsv32.cl for 8-bit ones) behind a reorder.
//
// M = N*P*Q output pixels, 128 consecutive ones per tile (= TMEM lanes).  K is
// ordered (feature, filter row, filter column) with every filter row padded to
// whole 8-byte quanta (4 halves / 8 bytes; the padding taps carry zero
// weights), so each quantum of a pixel's im2col row is one run of consecutive
// input elements.
//   warps 0..15  gather, in four groups of four warps; a group builds every
//                fourth operand stage on its own (thread = pixel): it issues the
//                aligned 64-bit loads around the runs of four 16-byte cores (two
//                words per run, which starts at any element; only words that
//                hold a tap inside the image are read), then funnel-shifts them
//                into place and clears padding and border taps.  Four stages are
//                under construction at once, which hides the load latency.
//                Dilated or non-contiguous inputs go element by element.  Stages
//                hold 8 cores in the K-major no-swizzle core-matrix layout.
//   warps 16..19 epilogue (fp16: bias + activation; 8-bit: the quantised
//                epilogue of fused_conv_eltwise_gpu_ref.cl:148-198), writing byxf
//                for the next layer.
//   warp 20      issues tcgen05.mma (kind::f16 / kind::i8) against the resident
//                weight image; up to four accumulator buffers in tensor memory.
// Every barrier wait is bounded and reports through the device status word.
#include <cuda.h>
#include <cuda_fp16.h>
#include <string>
#include "engine.hpp"
#include "sm100_ptx.cuh"
#include "conv_epilogue.cuh"
#include "conv_i8_first_rows.hpp"

namespace b200 {

using namespace ptx;

namespace firsttc {

constexpr int kBuildWarps = 16, kEpiWarps = 4;          // gather warps: four groups of four, one operand stage per group
constexpr int kBuilders = kBuildWarps * 32;
constexpr int kMmaWarp = kBuildWarps + kEpiWarps;
constexpr int kThreads = (kBuildWarps + kEpiWarps + 1) * 32;
constexpr int kStages = 4;
constexpr int kAccBufs = 4;                       // most accumulator buffers in tensor memory (ofm columns each)
constexpr int kStageBytes = 128 * 128;            // 128 pixels x 8 cores x 16 bytes
constexpr int kMaxCores = 256;                    // table entries: 16-byte cores of the padded K
constexpr int kMaxOfm = 256;
constexpr uint32_t kErr = 0x70u;

struct Params {
    int32_t N, H, W, Pn, Q, ofm, runs, cores, chunks; // runs = C*kh*(quanta per filter row): 8-byte quanta that hold taps; cores = 16-byte groups of the padded K (even); chunks = ceil(cores / 8)
    int32_t run_len, fast_ok;                        // elements of one padded filter row; 1: contiguous undilated rows (the shifted-word gather applies)
    int32_t sx, sy, pad_x, pad_y, ext_x, ext_y, dil_x; // ext = (kw-1)*dil_x, (kh-1)*dil_y
    int32_t total_tiles;
    int64_t M_total;
    int64_t in_pb, in_py, in_px, in_off;             // elements
    int64_t out_px, out_py, out_pb, out_off;         // elements
    uint32_t idesc, tmem_cols, sbo_b;
    int32_t bias_dtype, act; float act_m, act_n;     // fp16 epilogue
    int32_t nacc;                                    // accumulator buffers in tensor memory: up to kAccBufs of ofm columns each
    int32_t mul_iqf, mul_oqf, lean;                  // 8-bit epilogue (lean: per-feature scale, optional uniform O_QF, NONE / ReLU, integer bias)
    const void* in; void* out; const uint8_t* wpacked; const int4* table; const void* bias; const float* quant; const float* calib;
    uint32_t* status;
    EpiCfg epi;
};


struct Aux {
    uint64_t a_full[kStages], a_empty[kStages], tmem_full[kAccBufs], tmem_empty[kAccBufs];
    uint32_t tmem_base, abort;
    alignas(16) int32_t bias_i[1][kMaxOfm];
    alignas(16) float bias_f[1][kMaxOfm];
    alignas(16) float quant[1][kMaxOfm];
    alignas(16) float calib[1][kMaxOfm];
    alignas(16) float ecal[1][kMaxOfm];
};

// K-major operand without swizzle: 8 x 16-byte core matrices, `lbo` bytes apart along K, `sbo` bytes apart along M/N
__device__ __forceinline__ uint64_t desc_interleaved(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// weights [ofm][C][kh][kw] (any pitches) -> shared-memory image: element (n, k), k = ((c*kh + r)*qpr + j)*QE + e for tap
// s = j*QE + e of filter row (c, r) (qpr quanta of QE = 8 / sizeof(T) taps per row), at
// (n/8)*sbo + (k/EPC)*128 + (n%8)*16 + (k%EPC)*sizeof(T); zero for s >= kw and beyond the last row.  And the gather table,
// one entry per quantum: (offset of its first tap from the window origin in elements, row shift | column shift << 12 |
// taps in the quantum << 24, byte masks of its two 32-bit words that keep the filter row's taps).
template <typename T>
__global__ void first_tc_pack(const T* __restrict__ w, int64_t po, int64_t pi, int64_t py, int64_t px, int64_t off,
                              int ofm, int C, int kh, int kw, int cores, T* __restrict__ dst,
                              int4* __restrict__ table, int64_t in_pf, int64_t in_py, int64_t in_px, int dil_x, int dil_y)
{
    constexpr int EPC = 16 / (int)sizeof(T), QE = EPC / 2;
    const int qpr = (kw + QE - 1) / QE, quanta = C * kh * qpr, Kp = cores * EPC;
    const int sbo = cores * 128 / (int)sizeof(T);                       // in elements
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ofm * Kp; i += gridDim.x * blockDim.x) {
        const int n = i / Kp, k = i - n * Kp;
        const int g = k / QE, e = k - g * QE;
        T v = T(0);
        if (g < quanta) {
            const int j = g % qpr, t = g / qpr; const int r = t % kh, c = t / kh; const int s_ = j * QE + e;
            if (s_ < kw) v = w[off + n * po + c * pi + r * py + s_ * px];
        }
        dst[(n >> 3) * sbo + (k / EPC) * (128 / (int)sizeof(T)) + (n & 7) * EPC + (k % EPC)] = v;
    }
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < 2 * cores; g += gridDim.x * blockDim.x) {
        int4 ent = make_int4(0, 0, 0, 0);
        if (g < quanta) {
            const int j = g % qpr, t = g / qpr; const int r = t % kh, c = t / kh; const int s0 = j * QE;
            const int nv = min(QE, kw - s0), nb = nv * (int)sizeof(T);    // taps / bytes of the quantum that belong to the filter row
            ent.x = (int)(c * in_pf + (int64_t)r * dil_y * in_py + (int64_t)s0 * dil_x * in_px);
            ent.y = (r * dil_y) | ((s0 * dil_x) << 12) | (nv << 24);
            ent.z = (int)(nb >= 4 ? 0xffffffffu : ((1u << (8 * nb)) - 1u));                        // byte masks of the two words
            ent.w = (int)(nb >= 8 ? 0xffffffffu : (nb <= 4 ? 0u : ((1u << (8 * (nb - 4))) - 1u)));
        }
        table[g] = ent;
    }
}

// (image, row, column) of one output pixel, advanced by a fixed number of pixels per tile without divisions
struct PixelWalk {
    int n, p, q, dn, dp, dq, Pn, Q;
    __device__ __forceinline__ void init(uint32_t first, uint32_t step, int Pn_, int Q_)
    {
        Pn = Pn_; Q = Q_;
        q = (int)(first % (uint32_t)Q); uint32_t t = first / (uint32_t)Q; p = (int)(t % (uint32_t)Pn); n = (int)(t / (uint32_t)Pn);
        dq = (int)(step % (uint32_t)Q); t = step / (uint32_t)Q; dp = (int)(t % (uint32_t)Pn); dn = (int)(t / (uint32_t)Pn);
    }
    __device__ __forceinline__ void next()
    {
        q += dq; if (q >= Q) { q -= Q; ++p; }
        p += dp; if (p >= Pn) { p -= Pn; ++n; }
        n += dn;
    }
};

__device__ __forceinline__ uint32_t load_elem(const __half* p) { return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p)); }
__device__ __forceinline__ uint32_t load_elem(const uint8_t* p) { return (uint32_t)__ldg(p); }

__device__ __noinline__ float act_other(int32_t fn, float x, float m, float n) { return act_float(fn, x, m, n); }
__device__ __forceinline__ float act_apply(int32_t fn, float x, float m, float n)
{
    if (fn == CLDNN_B200_ACT_NONE) return x;
    if (fn == CLDNN_B200_ACT_RELU) return fmaxf(0.0f, x);
    return act_other(fn, x, m, n);
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
conv_first_tc_kernel(const __grid_constant__ Params P)
{
    constexpr bool kHalf = sizeof(T) == 2;
    constexpr int EPC = 16 / (int)sizeof(T);                          // elements per 16-byte core row
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 127u) & ~127u;
    uint8_t* smem = smem_raw + (base - raw);
    const int b_bytes = P.ofm * P.cores * 16;
    uint8_t* sA = smem; uint8_t* sB = sA + kStages * kStageBytes;
    int4* sTab = reinterpret_cast<int4*>(sB + b_bytes);
    Aux* aux = reinterpret_cast<Aux*>(reinterpret_cast<uint8_t*>(sTab) + (size_t)P.cores * 2 * sizeof(int4));
    volatile uint32_t* s_abort = &aux->abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const EpiCfg& c = P.epi;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(smem_u32(&aux->a_full[i]), kBuildWarps / kStages); mbar_init(smem_u32(&aux->a_empty[i]), 1); }
        for (int i = 0; i < kAccBufs; ++i) { mbar_init(smem_u32(&aux->tmem_full[i]), 1); mbar_init(smem_u32(&aux->tmem_empty[i]), kEpiWarps); }
        aux->abort = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp) { tmem_alloc(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish(); }
    // weights image, gather table and per-feature constants: once per CTA
    for (int i = tid; i < b_bytes / 16; i += kThreads) reinterpret_cast<uint4*>(sB)[i] = __ldg(reinterpret_cast<const uint4*>(P.wpacked) + i);
    for (int i = tid; i < P.cores * 2; i += kThreads) sTab[i] = __ldg(P.table + i);
    for (int j = tid; j < P.ofm; j += kThreads) {
        int32_t bi = 0; float bf = 0.f;
        if (kHalf) { if (P.bias_dtype != CLDNN_B200_NONE) bf = load_as_float(P.bias, P.bias_dtype, j); }
        else if (c.bias_dtype != CLDNN_B200_NONE) { if (c.bias_dtype == CLDNN_B200_F32) bf = ((const float*)P.bias)[j]; else bi = load_as_int(P.bias, c.bias_dtype, j); }
        aux->bias_i[0][j] = bi; aux->bias_f[0][j] = bf;
        aux->quant[0][j] = (!kHalf && c.quantization) ? P.quant[j] : 1.f;
        aux->calib[0][j] = (!kHalf && c.calibration) ? P.calib[j] : 1.f;
        aux->ecal[0][j] = 1.f;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    const int my_tiles = (P.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp < kBuildWarps) {
        // ------------------------------ gather ------------------------------------
        // Four groups of four warps; group g assembles every fourth operand stage (stage buffer g) on its own, all 128
        // pixels of it, so four stages are under construction at once and each barrier round trip pays for a whole stage.
        const int m = tid & 127, group = tid >> 7;
        const T* in = reinterpret_cast<const T*>(P.in) + P.in_off;
        uint8_t* dst = sA + group * kStageBytes + (m >> 3) * 1024 + (m & 7) * 16;
        uint32_t phase = 0; bool ok = true;
        PixelWalk px; px.init(blockIdx.x * 128u + (uint32_t)m, gridDim.x * 128u, P.Pn, P.Q);      // the host admits fewer than 2^31 pixels
        int it = 0, ch = group;                                 // this group's next stage: chunk `ch` of the CTA's tile `it`
        while (ch >= P.chunks) { ch -= P.chunks; ++it; px.next(); }
        while (it < my_tiles && ok) {
            const bool valid = px.n < P.N;
            const int y0 = px.p * P.sy - P.pad_y, x0 = px.q * P.sx - P.pad_x;
            const T* src = in + (int64_t)px.n * P.in_pb + (int64_t)y0 * P.in_py + (int64_t)x0 * P.in_px;   // dereferenced only at taps inside the image
            // one lane per warp polls the barrier, and one arrives for the warp: 128 threads on one shared-memory word serialise
            if (lane == 0) ok = mbar_wait(smem_u32(&aux->a_empty[group]), phase ^ 1u, s_abort, P.status, kErr + 1u);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            if (!ok) break;
            const int ncore = min(8, P.cores - ch * 8);
            if (P.fast_ok) {
                // Every quantum is one run of QE consecutive input elements starting anywhere: the two aligned 8-byte words
                // around it, shifted into place.  Elements [lo, hi) of the run are taps inside the image; only words holding
                // one of them are read (an aligned word that holds a valid byte lies in the same page: the read cannot
                // fault), everything else becomes zero (padding taps have zero weights, but 0 * Inf is not 0).  The loads
                // of four cores are issued before the first of them is used.
                // every tap of the pixel's window inside the image: no bounds to check, only the filter rows' padding taps to clear
                const bool inside = valid && y0 >= 0 && y0 + P.ext_y < P.H && x0 >= 0 && x0 + P.ext_x < P.W;
#pragma unroll 1
                for (int jb = 0; jb < ncore; jb += 4) {
                    uint2 w[8][2]; int meta[8];                              // per quantum: two aligned 8-byte words; byte offset | lo << 8 | hi << 16
                    if (inside) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int j = jb + (u >> 1);
                            w[u][0] = w[u][1] = make_uint2(0u, 0u); meta[u] = 0;
                            if (j < ncore) {
                                const int2 t = *reinterpret_cast<const int2*>(&sTab[(ch * 8 + j) * 2 + (u & 1)]);
                                const int nb = (t.y >> 24) * (int)sizeof(T);
                                if (nb) {
                                    const uintptr_t addr = reinterpret_cast<uintptr_t>(src + t.x);
                                    const uint2* wp = reinterpret_cast<const uint2*>(addr & ~(uintptr_t)7);
                                    const int o = (int)(addr & 7u);
                                    w[u][0] = __ldg(wp);
                                    if (o + nb > 8) w[u][1] = __ldg(wp + 1);       // the word holds a tap of the row: inside the tensor
                                    meta[u] = o;
                                }
                            }
                        }
#pragma unroll
                        for (int c4 = 0; c4 < 4; ++c4) {
                            const int j = jb + c4;
                            if (j >= ncore) break;
                            uint32_t d[4];
#pragma unroll
                            for (int h2 = 0; h2 < 2; ++h2) {
                                const int u = 2 * c4 + h2;
                                const int o = meta[u];
                                const uint32_t sh = (uint32_t)(o & 3) * 8u;
                                const int2 mk = *reinterpret_cast<const int2*>(&sTab[(ch * 8 + j) * 2 + h2].z);
                                const uint32_t x0w = (o & 4) ? w[u][0].y : w[u][0].x, x1w = (o & 4) ? w[u][1].x : w[u][0].y, x2w = (o & 4) ? w[u][1].y : w[u][1].x;
                                d[2 * h2] = __funnelshift_r(x0w, x1w, sh) & (uint32_t)mk.x;
                                d[2 * h2 + 1] = __funnelshift_r(x1w, x2w, sh) & (uint32_t)mk.y;
                            }
                            *reinterpret_cast<uint4*>(dst + j * 128) = make_uint4(d[0], d[1], d[2], d[3]);
                        }
                        continue;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int j = jb + (u >> 1);
                        w[u][0] = w[u][1] = make_uint2(0u, 0u); meta[u] = 0;
                        if (j < ncore) {
                            const int4 t = sTab[(ch * 8 + j) * 2 + (u & 1)];
                            const int nv = t.y >> 24, iy = y0 + (t.y & 0xfff), ix0 = x0 + ((t.y >> 12) & 0xfff);
                            const int lo = max(0, -ix0), hi = (valid && iy >= 0 && iy < P.H) ? min(nv, P.W - ix0) : 0;
                            if (hi > lo) {
                                const uintptr_t addr = reinterpret_cast<uintptr_t>(src + t.x);
                                const uint2* wp = reinterpret_cast<const uint2*>(addr & ~(uintptr_t)7);
                                const int o = (int)(addr & 7u);
                                const int b0 = o + lo * (int)sizeof(T), b1 = o + hi * (int)sizeof(T);   // valid bytes, from the first word
                                if (b0 < 8) w[u][0] = __ldg(wp);
                                if (b1 > 8) w[u][1] = __ldg(wp + 1);
                                meta[u] = o | (lo << 8) | (hi << 16);
                            }
                        }
                    }
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        const int j = jb + c4;
                        if (j >= ncore) break;
                        uint32_t d[4];
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2) {
                            const int u = 2 * c4 + h2;
                            const int o = meta[u] & 0xff;
                            const uint32_t sh = (uint32_t)(o & 3) * 8u;
                            const int v0 = ((meta[u] >> 8) & 0xff) * (int)sizeof(T), v1 = (meta[u] >> 16) * (int)sizeof(T);   // valid bytes of the quantum
                            // the run starts in the first or the second 32-bit half of the first word
                            const uint32_t x0w = (o & 4) ? w[u][0].y : w[u][0].x, x1w = (o & 4) ? w[u][1].x : w[u][0].y, x2w = (o & 4) ? w[u][1].y : w[u][1].x;
                            uint32_t q0 = __funnelshift_r(x0w, x1w, sh), q1 = __funnelshift_r(x1w, x2w, sh);
                            if (v0 != 0 || v1 != 8) {
                                const int a1 = min(v1, 4), c0 = max(v0 - 4, 0), c1 = v1 - 4;
                                q0 = (a1 > v0) ? (q0 & ((a1 >= 4 ? 0xffffffffu : ((1u << (8 * a1)) - 1u)) & ~((1u << (8 * min(v0, 3))) - 1u))) : 0u;
                                q1 = (c1 > c0) ? (q1 & ((c1 >= 4 ? 0xffffffffu : ((1u << (8 * c1)) - 1u)) & ~((1u << (8 * c0)) - 1u))) : 0u;
                            }
                            d[2 * h2] = q0; d[2 * h2 + 1] = q1;
                        }
                        *reinterpret_cast<uint4*>(dst + j * 128) = make_uint4(d[0], d[1], d[2], d[3]);
                    }
                }
            } else {
                for (int j = 0; j < ncore; ++j) {
                    uint32_t e[EPC];
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int4 t = sTab[(ch * 8 + j) * 2 + h2];
                        const int nv = t.y >> 24, iy = y0 + (t.y & 0xfff), ix0 = x0 + ((t.y >> 12) & 0xfff);
                        const int64_t step = (int64_t)P.dil_x * P.in_px;
#pragma unroll
                        for (int i = 0; i < EPC / 2; ++i) {
                            const int ix = ix0 + i * P.dil_x;
                            const bool in_image = valid && i < nv && iy >= 0 && iy < P.H && ix >= 0 && ix < P.W;
                            e[h2 * (EPC / 2) + i] = in_image ? load_elem(src + t.x + i * step) : 0u;
                        }
                    }
                    uint4 v;
                    if (kHalf) {
                        v = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
                    } else {
                        uint32_t wv[4];
#pragma unroll
                        for (int g = 0; g < 4; ++g) wv[g] = e[(4 * g) % EPC] | (e[(4 * g + 1) % EPC] << 8) | (e[(4 * g + 2) % EPC] << 16) | (e[(4 * g + 3) % EPC] << 24);
                        v = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    }
                    *reinterpret_cast<uint4*>(dst + j * 128) = v;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->a_full[group]));
            phase ^= 1u;
            ch += kStages;
            while (ch >= P.chunks) { ch -= P.chunks; ++it; px.next(); }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer --------------------------------
        // the whole warp runs the loop, one elected lane issues (loop state stays on the uniform datapath)
        {
            const bool leader = elect_one();
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int it = 0; it < my_tiles && ok; ++it) {
                const int buf = it % P.nacc; const uint32_t par = (uint32_t)(it / P.nacc) & 1u;
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->tmem_empty[buf]), par ^ 1u, s_abort, P.status, kErr + 2u))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P.ofm);
                for (int ch = 0; ch < P.chunks; ++ch) {
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&aux->a_full[stage]), phase, s_abort, P.status, kErr + 3u))) { ok = false; break; }
                    tc_fence_after();
                    const int nm = min(8, P.cores - ch * 8) >> 1;           // one instruction consumes two cores along K
                    const uint64_t adesc = desc_interleaved(smem_u32(sA + stage * kStageBytes), 128u, 1024u);
                    const uint64_t bdesc = desc_interleaved(smem_u32(sB + ch * 8 * 128), 128u, P.sbo_b);
                    if (leader) {
                        for (int i = 0; i < nm; ++i) {
                            if (kHalf) mma_f16_ss(d_tmem, adesc + (uint64_t)(i * 16), bdesc + (uint64_t)(i * 16), P.idesc, (ch | i) ? 1u : 0u);
                            else mma_i8_ss(d_tmem, adesc + (uint64_t)(i * 16), bdesc + (uint64_t)(i * 16), P.idesc, (ch | i) ? 1u : 0u);
                        }
                        tc_commit(smem_u32(&aux->a_empty[stage]));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok && leader) tc_commit(smem_u32(&aux->tmem_full[buf]));
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quad = warp & 3;                              // warps 16..19 -> TMEM lanes 32*quad ..
        const int row = quad * 32 + lane;
        PixelWalk px; px.init(blockIdx.x * 128u + (uint32_t)row, gridDim.x * 128u, P.Pn, P.Q);
        for (int it = 0; it < my_tiles; ++it, px.next()) {
            const int buf = it % P.nacc;
            const bool valid = px.n < P.N;
            const int n = px.n, p = px.p, q = px.q;
            T* out_row = reinterpret_cast<T*>(P.out) + P.out_off + (int64_t)n * P.out_pb + (int64_t)p * P.out_py + (int64_t)q * P.out_px;
            if (!mbar_wait(smem_u32(&aux->tmem_full[buf]), (uint32_t)(it / P.nacc) & 1u, s_abort, P.status, kErr)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * P.ofm);
#pragma unroll 1
            for (int c0 = 0; c0 < P.ofm; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_row + (uint32_t)c0, r);
                tmem_ld_wait();
                if (c0 + 32 >= P.ofm) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(smem_u32(&aux->tmem_empty[buf])); }
                if (!valid) continue;
                if (kHalf) {
                    uint4* op = reinterpret_cast<uint4*>(out_row + c0);
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float4 b0 = *reinterpret_cast<const float4*>(&aux->bias_f[0][c0 + 8 * w]), b1 = *reinterpret_cast<const float4*>(&aux->bias_f[0][c0 + 8 * w + 4]);
                        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                        uint32_t ow[4];
#pragma unroll
                        for (int h = 0; h < 4; ++h) {
                            const float v0 = act_apply(P.act, __uint_as_float(r[8 * w + 2 * h]) + bb[2 * h], P.act_m, P.act_n);
                            const float v1 = act_apply(P.act, __uint_as_float(r[8 * w + 2 * h + 1]) + bb[2 * h + 1], P.act_m, P.act_n);
                            const __half2 o = __floats2half2_rn(v0, v1);
                            ow[h] = *reinterpret_cast<const uint32_t*>(&o);
                        }
                        op[w] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                } else {
                    uint4 o0, o1;
                    if (P.lean) epi_chunk_fast<false, true>(P, aux, 0, c0, r, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1);
                    else epi_chunk_fast<false, false>(P, aux, 0, c0, r, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), o0, o1);
                    uint4* op = reinterpret_cast<uint4*>(out_row + c0);
                    op[0] = o0; op[1] = o1;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) { tc_fence_after(); tmem_dealloc(tmem_base, P.tmem_cols); }
}

}  // namespace firsttc

// ------------------------------------------------------------------------------------
using firsttc::Params;

static int ftc_esize(const cldnn_b200_conv_params& p) { return p.in.dtype == CLDNN_B200_F16 ? 2 : 1; }
static int ftc_qpr(const cldnn_b200_conv_params& p) { const int qe = 8 / ftc_esize(p); return (p.kw + qe - 1) / qe; }   // 8-byte quanta per filter row
static int ftc_cores(const cldnn_b200_conv_params& p)
{
    const int cores = (p.ifm * p.kh * ftc_qpr(p) + 1) / 2;             // two quanta per 16-byte core
    return (cores + 1) / 2 * 2;                                        // one instruction consumes two cores
}
static size_t ftc_smem(const cldnn_b200_conv_params& p)
{
    const int cores = ftc_cores(p);
    return 128 + (size_t)firsttc::kStages * firsttc::kStageBytes + (size_t)p.ofm * cores * 16 + (size_t)cores * 2 * sizeof(int4) + sizeof(firsttc::Aux);
}

static bool ftc_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (p.epilogue_order != CLDNN_B200_EPILOGUE_REF) return no("reference epilogue order only");
    const bool half = p.in.dtype == CLDNN_B200_F16;
    if (half) {
        if (p.w_dtype != CLDNN_B200_F16 || p.out.dtype != CLDNN_B200_F16) return no("fp16 weights and output with fp16 input");
        if (p.quantization || p.calibration || p.has_o_qf) return no("no quantisation on the fp16 path");
        if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_F16 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    } else {
        if (!is_int8(p.in.dtype) || p.w_dtype != CLDNN_B200_I8 || !is_int8(p.out.dtype)) return no("fp16, or 8-bit activations, weights and output");
        if (!(p.quantization || p.calibration || p.has_o_qf)) return no("quantised epilogue only");
        if (!act_is_simple(p.act, p.act_m)) return no("activation not in the fast set");
        if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_I32 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    }
    if (p.groups != 1 || p.fused_eltw) return no("plain convolution only");
    if (p.out.pf != 1) return no("output must be byxf");
    if (p.kh < 1 || p.kw < 1 || p.stride_x < 1 || p.stride_y < 1 || p.dil_x < 1 || p.dil_y < 1) return no("filter geometry");
    if ((int64_t)p.ifm * p.kh * ftc_qpr(p) > 2 * firsttc::kMaxCores) return no("too many filter rows (C * kh * 8-byte quanta per row above 512)");
    if ((p.kh - 1) * p.dil_y > 4095 || (ftc_qpr(p) * (8 / ftc_esize(p))) * p.dil_x > 4095) return no("filter extent");
    if (p.ofm % 32 || p.ofm > firsttc::kMaxOfm || p.out.f != p.ofm || p.in.f != p.ifm) return no("output features: multiple of 32, at most 256");
    const int es = ftc_esize(p);
    if ((p.out.px * es) % 16 || (p.out.py * es) % 16 || (p.out.pb * es) % 16 || (p.out.offset * es) % 16) return no("output pitches must be 16-byte aligned");
    const int P_ = (p.in.y + 2 * p.pad_y - ((p.kh - 1) * p.dil_y + 1)) / p.stride_y + 1;
    const int Q_ = (p.in.x + 2 * p.pad_x - ((p.kw - 1) * p.dil_x + 1)) / p.stride_x + 1;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");
    if (ftc_smem(p) > 200 * 1024) return no("weights do not fit in shared memory");
    if ((int64_t)p.out.b * p.out.y * p.out.x + 128 >= 0x7fffffffLL) return no("too many output pixels");
    // the gather table holds 32-bit element offsets from the window origin
    if ((int64_t)p.ifm * p.in.pf + (int64_t)p.kh * p.dil_y * p.in.py + (int64_t)p.kw * p.dil_x * p.in.px > 0x7fffffffLL) return no("input too large");
    return true;
}
// tuning variants: 0 / 1 the gather kernel of this file; 2 / 3 the row form of conv_i8_first_rows.cu (fp16 here; 8-bit layers reach
// it through conv_i8_first) with two / four epilogue warp groups
static bool ftc_rows(const cldnn_b200_conv_params& p) { return p.tune >= 2 && p.in.dtype == CLDNN_B200_F16; }
static bool ftc_supports(const void* vp)
{
    const cldnn_b200_conv_params& p = *(const cldnn_b200_conv_params*)vp;
    if (p.tune >= 2) return ftc_rows(p) && first_rows_plan(p, nullptr);
    return ftc_plan(p, nullptr);
}
static int ftc_tune_count(const void*) { return 4; }
// packed weights followed by the gather table
static size_t ftc_table_offset(const cldnn_b200_conv_params& p) { return ((size_t)p.ofm * ftc_cores(p) * 16 + 255) / 256 * 256; }
static size_t ftc_scratch(const void* vp)
{
    const auto& p = *(const cldnn_b200_conv_params*)vp;
    if (ftc_rows(p)) return first_rows_scratch(p);
    return ftc_table_offset(p) + (size_t)ftc_cores(p) * 2 * sizeof(int4);
}

static int32_t ftc_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    if (((const cldnn_b200_conv_params*)vp)->tune >= 2) {
        const cldnn_b200_conv_params& pr = *(const cldnn_b200_conv_params*)vp;
        if (!ftc_rows(pr)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_first_tc: the row form is the fp16 variant here");
        return first_rows_prepare(ctx, pr, a, out, pr.tune == 3 ? 4 : 2);
    }
    const cldnn_b200_conv_params p = simplified_conv_params(*(const cldnn_b200_conv_params*)vp);
    std::string why;
    if (!ftc_plan(p, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_first_tc: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: bias_dtype set but no bias pointer");
    if (p.quantization && !a->weights_quantization_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: quantization set but no factors");
    if (p.calibration && !a->output_calibration_factors) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: calibration set but no factors");
    const size_t need = ftc_scratch(&p);
    if (!a->scratch || a->scratch_bytes < need) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: needs " + std::to_string(need) + " bytes of scratch for the packed weights");
    if (((uintptr_t)a->scratch | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: scratch and output must be 16-byte aligned");
    const bool half = p.in.dtype == CLDNN_B200_F16;
    const int es = ftc_esize(p);
    if ((uintptr_t)a->input0 & (uintptr_t)(es - 1)) return fail(CLDNN_B200_INVALID_ARG, "conv_first_tc: input must be aligned to its element size");

    Params P{};
    P.N = p.in.b; P.H = p.in.y; P.W = p.in.x; P.Pn = p.out.y; P.Q = p.out.x; P.ofm = p.ofm;
    P.runs = p.ifm * p.kh * ftc_qpr(p); P.cores = ftc_cores(p); P.chunks = (P.cores + 7) / 8;
    P.run_len = ftc_qpr(p) * (8 / ftc_esize(p)); P.dil_x = p.dil_x;
    // contiguous, undilated filter rows of elements aligned to their size: the shifted-word gather applies
    P.fast_ok = (p.in.px == 1 && p.dil_x == 1) ? 1 : 0;
    P.sx = p.stride_x; P.sy = p.stride_y; P.pad_x = p.pad_x; P.pad_y = p.pad_y;
    P.ext_x = (p.kw - 1) * p.dil_x; P.ext_y = (p.kh - 1) * p.dil_y;
    P.M_total = (int64_t)P.N * P.Pn * P.Q;
    P.total_tiles = (int)((P.M_total + 127) / 128);
    P.in_pb = p.in.pb; P.in_py = p.in.py; P.in_px = p.in.px; P.in_off = p.in.offset;
    P.out_px = p.out.px; P.out_py = p.out.py; P.out_pb = p.out.pb; P.out_off = p.out.offset;
    if (half) P.idesc = (1u << 4) | ((uint32_t)(p.ofm >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);          // f16 x f16 -> f32
    else P.idesc = (2u << 4) | ((p.in.dtype == CLDNN_B200_U8 ? 0u : 1u) << 7) | (1u << 10) | ((uint32_t)(p.ofm >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    // CTAs per SM and accumulator buffers: two CTAs (when shared memory holds two) with at least two accumulators each
    // inside half of the SM's 512 columns of tensor memory, else one CTA with up to four
    const size_t smem = ftc_smem(p);
    if (smem > (size_t)ctx->prop.sharedMemPerBlockOptin) return fail(CLDNN_B200_OUT_OF_RESOURCES, "conv_first_tc: not enough shared memory");
    int per_sm = (ctx->prop.sharedMemPerMultiprocessor / (smem + 1024) >= 2 && 256 / p.ofm >= 2 &&
                  2 * firsttc::kThreads <= ctx->prop.maxThreadsPerMultiProcessor) ? 2 : 1;
    P.nacc = std::min(firsttc::kAccBufs, (per_sm == 2 ? 256 : 512) / p.ofm);
    uint32_t cols = 32; while (cols < (uint32_t)(P.nacc * p.ofm)) cols <<= 1;
    P.tmem_cols = cols;
    P.sbo_b = (uint32_t)P.cores * 128u;
    P.bias_dtype = p.bias_dtype; P.act = p.act; P.act_m = p.act_m; P.act_n = p.act_n;
    P.epi = make_epi_cfg(p);
    P.mul_iqf = p.i_qf != 1.0f ? 1 : 0; P.mul_oqf = (p.calibration || p.o_qf != 1.0f) ? 1 : 0;
    P.lean = (!half && p.quantization && !P.mul_iqf && (!P.mul_oqf || !p.calibration) && !P.epi.dont_dequantize_bias &&
              (p.act == CLDNN_B200_ACT_NONE || p.act == CLDNN_B200_ACT_RELU)) ? 1 : 0;
    P.in = a->input0; P.out = a->output; P.wpacked = (const uint8_t*)a->scratch;
    P.table = (const int4*)((const uint8_t*)a->scratch + ftc_table_offset(p));
    P.bias = a->bias; P.quant = a->weights_quantization_factors; P.calib = a->output_calibration_factors;
    P.status = ctx->d_status;

    // pack the weights and build the table once, on the context's stream, before anything that is prepared here can run
    const int pack_blocks = (p.ofm * P.cores * (16 / es) + 255) / 256;
    if (half) {
        B200_CUDA(raise_smem_limit((const void*)firsttc::conv_first_tc_kernel<__half>, ctx->device, smem));
        firsttc::first_tc_pack<__half><<<pack_blocks, 256, 0, ctx->stream>>>((const __half*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset, p.ofm, p.ifm, p.kh, p.kw,
                                                                              P.cores, (__half*)a->scratch, (int4*)P.table, p.in.pf, p.in.py, p.in.px, p.dil_x, p.dil_y);
    } else {
        B200_CUDA(raise_smem_limit((const void*)firsttc::conv_first_tc_kernel<uint8_t>, ctx->device, smem));
        firsttc::first_tc_pack<uint8_t><<<pack_blocks, 256, 0, ctx->stream>>>((const uint8_t*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset, p.ofm, p.ifm, p.kh, p.kw,
                                                                               P.cores, (uint8_t*)a->scratch, (int4*)P.table, p.in.pf, p.in.py, p.in.px, p.dil_x, p.dil_y);
    }
    B200_CUDA(cudaGetLastError());
    int grid = ctx->prop.multiProcessorCount * per_sm;
    if (grid > P.total_tiles) grid = P.total_tiles;
    out->fn = [P, grid, smem, half](cudaStream_t s) {
        if (half) firsttc::conv_first_tc_kernel<__half><<<grid, firsttc::kThreads, smem, s>>>(P);
        else firsttc::conv_first_tc_kernel<uint8_t><<<grid, firsttc::kThreads, smem, s>>>(P);
        return cudaGetLastError();
    };
    out->launches = 1;
    return CLDNN_B200_SUCCESS;
}

const KernelDef kdef_conv_first_tc = {"conv_first_tc", sizeof(cldnn_b200_conv_params), ftc_supports, ftc_tune_count, ftc_scratch, ftc_prepare};

}  // namespace b200
