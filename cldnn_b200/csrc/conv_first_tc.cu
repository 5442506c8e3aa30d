// conv_first_tc: the first convolution of a network in its general form -- few
// input features (3 for images), any filter size / stride / dilation (VGG's
// 3x3, AlexNet's 11x11 stride 4), fp16 or 8-bit -- on the tensor cores, read
// straight from the caller's input layout (planar bfyx as images arrive, or any
// other pitches) with no padded or reordered copy of the input in HBM.  With 3
// input features the generic tensor-core kernels would pad every filter tap to
// 16 / 32 features and multiply mostly zeros; here K = C*kh*kw is packed densely.
// It stands where the reference uses its first-layer kernels
// (cl_kernels/convolution_gpu_bfyx_os_iyx_osv16.cl for fp16 images,
// convolution_gpu_byxf_fs_bs_yx_bsv4_fsv32.cl for 8-bit ones) behind a reorder.
//
// M = N*P*Q output pixels, 128 consecutive ones per tile (= TMEM lanes); K is
// cut into chunks of 8 core matrices (128 bytes per pixel).  Warps 0..7 gather:
// thread (pixel m, half h) assembles every second 16-byte core of its pixel's
// im2col row -- element k = (c*kh + r)*kw + s read at an offset taken from a
// table in shared memory, zero outside the image -- into a ring of operand
// stages in the K-major no-swizzle core-matrix layout; warp 12 issues
// tcgen05.mma (kind::f16 / kind::i8) against the resident weight image, two
// accumulator buffers in tensor memory; warps 8..11 run the epilogue (fp16:
// bias + activation; 8-bit: the quantised epilogue of
// fused_conv_eltwise_gpu_ref.cl:148-198) and write byxf for the next layer.
// Every barrier wait is bounded and reports through the device status word.
#include <cuda.h>
#include <cuda_fp16.h>
#include <string>
#include "engine.hpp"
#include "sm100_ptx.cuh"
#include "conv_epilogue.cuh"

namespace b200 {

using namespace ptx;

namespace firsttc {

constexpr int kBuildWarps = 8, kEpiWarps = 4;
constexpr int kBuilders = kBuildWarps * 32;
constexpr int kMmaWarp = kBuildWarps + kEpiWarps;
constexpr int kThreads = (kBuildWarps + kEpiWarps + 1) * 32;
constexpr int kStages = 4;
constexpr int kAccBufs = 4;                       // most accumulator buffers in tensor memory (ofm columns each)
constexpr int kStageBytes = 128 * 128;            // 128 pixels x 8 cores x 16 bytes
constexpr int kMaxK = 1024;                       // table entries (elements of K)
constexpr int kMaxOfm = 256;
constexpr uint32_t kErr = 0x70u;

struct Params {
    int32_t N, H, W, Pn, Q, ofm, K, cores, chunks;   // cores = 16-byte groups of the padded K (even), chunks = ceil(cores / 8)
    int32_t sx, sy, pad_x, pad_y, ext_x, ext_y;      // ext = (kw-1)*dil_x, (kh-1)*dil_y
    int32_t total_tiles;
    int64_t M_total;
    int64_t in_pb, in_py, in_px, in_off;             // elements
    int64_t out_px, out_py, out_pb, out_off;         // elements
    uint32_t idesc, tmem_cols, sbo_b;
    int32_t bias_dtype, act; float act_m, act_n;     // fp16 epilogue
    int32_t nacc;                                    // accumulator buffers in tensor memory: up to kAccBufs of ofm columns each
    int32_t debug;                                   // diagnostic builds (-DCONV_TC_DEBUG): what-if switches, 0 otherwise
    int32_t mul_iqf, mul_oqf, lean;                  // 8-bit epilogue (lean: per-feature scale, optional uniform O_QF, NONE / ReLU, integer bias)
    const void* in; void* out; const uint8_t* wpacked; const int2* table; const void* bias; const float* quant; const float* calib;
    uint32_t* status;
    EpiCfg epi;
};

#ifdef CONV_TC_DEBUG
#define FTC_DEBUG(P, bit) (((P).debug >> (bit)) & 1)
#else
#define FTC_DEBUG(P, bit) 0
#endif

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

// weights [ofm][C][kh][kw] (any pitches) -> shared-memory image: element (n, k), k = (c*kh + r)*kw + s, at
// (n/8)*sbo + (k/EPC)*128 + (n%8)*16 + (k%EPC)*sizeof(T), zero for k >= K; and the gather table: entry k = (offset of
// the tap from the window origin in elements, row shift | column shift << 16)
template <typename T>
__global__ void first_tc_pack(const T* __restrict__ w, int64_t po, int64_t pi, int64_t py, int64_t px, int64_t off,
                              int ofm, int C, int kh, int kw, int cores, T* __restrict__ dst,
                              int2* __restrict__ table, int64_t in_pf, int64_t in_py, int64_t in_px, int dil_x, int dil_y)
{
    constexpr int EPC = 16 / (int)sizeof(T);
    const int K = C * kh * kw, Kp = cores * EPC;
    const int sbo = cores * 128 / (int)sizeof(T);                       // in elements
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ofm * Kp; i += gridDim.x * blockDim.x) {
        const int n = i / Kp, k = i - n * Kp;
        T v = T(0);
        if (k < K) { const int s = k % kw, t = k / kw; const int r = t % kh, c = t / kh; v = w[off + n * po + c * pi + r * py + s * px]; }
        dst[(n >> 3) * sbo + (k / EPC) * (128 / (int)sizeof(T)) + (n & 7) * EPC + (k % EPC)] = v;
    }
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < Kp; k += gridDim.x * blockDim.x) {
        int2 e = make_int2(0, 0);
        if (k < K) {
            const int s = k % kw, t = k / kw; const int r = t % kh, c = t / kh;
            e.x = (int)(c * in_pf + (int64_t)r * dil_y * in_py + (int64_t)s * dil_x * in_px);
            e.y = (r * dil_y) | ((s * dil_x) << 16);
        }
        table[k] = e;
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
__global__ void __launch_bounds__(kThreads, 2)
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
    int2* sTab = reinterpret_cast<int2*>(sB + b_bytes);
    Aux* aux = reinterpret_cast<Aux*>(reinterpret_cast<uint8_t*>(sTab) + (size_t)P.cores * EPC * sizeof(int2));
    volatile uint32_t* s_abort = &aux->abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const EpiCfg& c = P.epi;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(smem_u32(&aux->a_full[i]), kBuildWarps); mbar_init(smem_u32(&aux->a_empty[i]), 1); }
        for (int i = 0; i < kAccBufs; ++i) { mbar_init(smem_u32(&aux->tmem_full[i]), 1); mbar_init(smem_u32(&aux->tmem_empty[i]), kEpiWarps); }
        aux->abort = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp) { tmem_alloc(smem_u32(&aux->tmem_base), P.tmem_cols); tmem_relinquish(); }
    // weights image, gather table and per-feature constants: once per CTA
    for (int i = tid; i < b_bytes / 16; i += kThreads) reinterpret_cast<uint4*>(sB)[i] = __ldg(reinterpret_cast<const uint4*>(P.wpacked) + i);
    for (int i = tid; i < P.cores * EPC; i += kThreads) sTab[i] = __ldg(P.table + i);
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
        const int m = tid & 127, half = tid >> 7;
        const T* in = reinterpret_cast<const T*>(P.in) + P.in_off;
        uint8_t* dst0 = sA + (m >> 3) * 1024 + (m & 7) * 16;
        int stage = 0; uint32_t phase = 0; bool ok = true;
        PixelWalk px; px.init(blockIdx.x * 128u + (uint32_t)m, gridDim.x * 128u, P.Pn, P.Q);      // the host admits fewer than 2^31 pixels
        for (int it = 0; it < my_tiles && ok; ++it, px.next()) {
            const bool valid = px.n < P.N;
            const int n = px.n, p = px.p, q = px.q;
            const int y0 = p * P.sy - P.pad_y, x0 = q * P.sx - P.pad_x;
            const T* src = in + (int64_t)n * P.in_pb + (int64_t)y0 * P.in_py + (int64_t)x0 * P.in_px;   // dereferenced only at taps inside the image
            const bool interior = valid && y0 >= 0 && y0 + P.ext_y < P.H && x0 >= 0 && x0 + P.ext_x < P.W;
            for (int ch = 0; ch < P.chunks; ++ch) {
                // one lane per warp polls the barrier, and one arrives for the warp: 256 threads on one shared-memory word serialise
                if (lane == 0) ok = mbar_wait(smem_u32(&aux->a_empty[stage]), phase ^ 1u, s_abort, P.status, kErr + 1u);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                __syncwarp();
                if (!ok) break;
                const int ncore = min(8, P.cores - ch * 8);
                uint8_t* dst = dst0 + stage * kStageBytes;
                for (int j = half; j < ncore; j += 2) {
                    const int kb = (ch * 8 + j) * EPC;
                    uint32_t e[EPC];
                    if (FTC_DEBUG(P, 0)) {
#pragma unroll
                        for (int i = 0; i < EPC; ++i) e[i] = (uint32_t)(kb + i);
                    } else if (interior && kb + EPC <= P.K) {
#pragma unroll
                        for (int i = 0; i < EPC; i += 2) {
                            const int4 t = *reinterpret_cast<const int4*>(&sTab[kb + i]);
                            e[i] = load_elem(src + t.x); e[i + 1] = load_elem(src + t.z);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < EPC; ++i) {
                            const int2 t = sTab[kb + i];
                            const int iy = y0 + (t.y & 0xffff), ix = x0 + (t.y >> 16);
                            e[i] = (valid && kb + i < P.K && iy >= 0 && iy < P.H && ix >= 0 && ix < P.W) ? load_elem(src + t.x) : 0u;
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
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->a_full[stage]));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0; bool ok = true;
            for (int it = 0; it < my_tiles && ok; ++it) {
                const int buf = it % P.nacc; const uint32_t par = (uint32_t)(it / P.nacc) & 1u;
                if (!mbar_wait(smem_u32(&aux->tmem_empty[buf]), par ^ 1u, s_abort, P.status, kErr + 2u)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P.ofm);
                for (int ch = 0; ch < P.chunks; ++ch) {
                    if (!mbar_wait(smem_u32(&aux->a_full[stage]), phase, s_abort, P.status, kErr + 3u)) { ok = false; break; }
                    tc_fence_after();
                    const int nm = min(8, P.cores - ch * 8) >> 1;           // one instruction consumes two cores along K
                    const uint64_t adesc = desc_interleaved(smem_u32(sA + stage * kStageBytes), 128u, 1024u);
                    const uint64_t bdesc = desc_interleaved(smem_u32(sB + ch * 8 * 128), 128u, P.sbo_b);
                    for (int i = 0; i < nm; ++i) {
                        if (FTC_DEBUG(P, 2)) break;
                        if (kHalf) mma_f16_ss(d_tmem, adesc + (uint64_t)(i * 16), bdesc + (uint64_t)(i * 16), P.idesc, (ch | i) ? 1u : 0u);
                        else mma_i8_ss(d_tmem, adesc + (uint64_t)(i * 16), bdesc + (uint64_t)(i * 16), P.idesc, (ch | i) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&aux->a_empty[stage]));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(smem_u32(&aux->tmem_full[buf]));
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quad = warp & 3;                              // warps 8..11 -> TMEM lanes 32*quad ..
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
                if (!valid || FTC_DEBUG(P, 1)) continue;
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
static int ftc_cores(const cldnn_b200_conv_params& p)
{
    const int epc = 16 / ftc_esize(p);
    const int cores = (p.ifm * p.kh * p.kw + epc - 1) / epc;
    return (cores + 1) / 2 * 2;                                        // one instruction consumes two cores
}
static size_t ftc_smem(const cldnn_b200_conv_params& p)
{
    const int cores = ftc_cores(p);
    return 128 + (size_t)firsttc::kStages * firsttc::kStageBytes + (size_t)p.ofm * cores * 16 + (size_t)cores * (16 / ftc_esize(p)) * sizeof(int2) + sizeof(firsttc::Aux);
}

static bool ftc_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
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
    if ((int64_t)p.ifm * p.kh * p.kw > firsttc::kMaxK) return no("C*kh*kw must not exceed 1024");
    if ((p.kh - 1) * p.dil_y > 32767 || (p.kw - 1) * p.dil_x > 32767) return no("filter extent");
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
static bool ftc_supports(const void* vp) { return ftc_plan(*(const cldnn_b200_conv_params*)vp, nullptr); }
static int ftc_tune_count(const void*) { return 1; }
// packed weights followed by the gather table
static size_t ftc_table_offset(const cldnn_b200_conv_params& p) { return ((size_t)p.ofm * ftc_cores(p) * 16 + 255) / 256 * 256; }
static size_t ftc_scratch(const void* vp)
{
    const auto& p = *(const cldnn_b200_conv_params*)vp;
    return ftc_table_offset(p) + (size_t)ftc_cores(p) * (16 / ftc_esize(p)) * sizeof(int2);
}

static int32_t ftc_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
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
    P.K = p.ifm * p.kh * p.kw; P.cores = ftc_cores(p); P.chunks = (P.cores + 7) / 8;
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
    int per_sm = (ctx->prop.sharedMemPerMultiprocessor / (smem + 1024) >= 2 && 256 / p.ofm >= 2) ? 2 : 1;
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
    P.table = (const int2*)((const uint8_t*)a->scratch + ftc_table_offset(p));
    P.bias = a->bias; P.quant = a->weights_quantization_factors; P.calib = a->output_calibration_factors;
    P.status = ctx->d_status;
#ifdef CONV_TC_DEBUG
    if (const char* e = getenv("CLDNN_B200_TC_DEBUG")) P.debug = atoi(e);
#endif

    // pack the weights and build the table once, on the context's stream, before anything that is prepared here can run
    const int pack_blocks = (p.ofm * P.cores * (16 / es) + 255) / 256;
    if (half) {
        B200_CUDA(cudaFuncSetAttribute(firsttc::conv_first_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        firsttc::first_tc_pack<__half><<<pack_blocks, 256, 0, ctx->stream>>>((const __half*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset, p.ofm, p.ifm, p.kh, p.kw,
                                                                              P.cores, (__half*)a->scratch, (int2*)P.table, p.in.pf, p.in.py, p.in.px, p.dil_x, p.dil_y);
    } else {
        B200_CUDA(cudaFuncSetAttribute(firsttc::conv_first_tc_kernel<uint8_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        firsttc::first_tc_pack<uint8_t><<<pack_blocks, 256, 0, ctx->stream>>>((const uint8_t*)a->weights, p.w_po, p.w_pi, p.w_py, p.w_px, p.w_offset, p.ofm, p.ifm, p.kh, p.kw,
                                                                               P.cores, (uint8_t*)a->scratch, (int2*)P.table, p.in.pf, p.in.py, p.in.px, p.dil_x, p.dil_y);
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
