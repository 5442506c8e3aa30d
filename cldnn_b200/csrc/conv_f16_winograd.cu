// conv_f16_winograd: Winograd F(2x2, 3x3) for fp16 3x3 stride-1 convolutions
// -- the B200 counterpart of the reference's
// cl_kernels/convolution_gpu_winograd_2x3_s1.cl / _fused.cl and of the weight
// transform its generic_layer performs at build time
// (kernel_selector .. winograd_2x3_s1_weights).  Three launches:
//   1. input transform   V[xi][t][c] = (B^T d B)[xi]  for every 4x4 input tile t
//      (tiles step by 2 pixels) -- bandwidth-bound, 16-byte accesses;
//   2. 16 independent GEMMs M[xi] = V[xi] (tiles x C) * U[xi]^T (C x K) as one
//      batched launch of the tcgen05 fp16 kernel (fp32 accumulation);
//   3. output transform  Y = A^T M A -> 2x2 outputs per tile, + bias, activation.
// U = G g G^T is computed once at prepare time.  2.25x fewer multiplications
// than the direct form at the price of ~10x its memory traffic: it pays on the
// deep, small-map layers and the tuner decides per layer.
// The input transform is additions only and runs on packed halves; the weight and
// output transforms are evaluated in fp32; V, U and M are stored as fp16 (the
// reference works in half throughout).  Results agree with the direct path within
// the fp16 tolerance.
#include <cuda_fp16.h>
#include <functional>
#include <string>
#include "engine.hpp"

namespace b200 {

int32_t f16_batched_gemm_prepare(cldnn_b200_ctx_impl* ctx, const void* A, const void* B, void* D, int batches, int rows, int cs, int ofm,
                                 std::function<cudaError_t(cudaStream_t)>& fn);

namespace {

struct WinoParams {
    int32_t N, H, W, P, Q, cs, ofm, ofm_s;      // cs / ofm_s: stored input / transformed-output feature counts
    int32_t pad_x, pad_y, tiles_x, tiles_y, T, Tp;
    int64_t in_px, in_py, in_pb, in_off, out_px, out_py, out_pb, out_off;
    int32_t bias_dtype, act; float act_m, act_n;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8])
{
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8])
{
    uint4 v; __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

// weights oyxi [K][3][3][cs] -> U[16][K][cs],  U = G g G^T,  G = [1 0 0; .5 .5 .5; .5 -.5 .5; 0 0 1]
__global__ void wino_weight_transform(const __half* __restrict__ w, int64_t w_po, int64_t w_py, int64_t w_px, int K, int Ks, int cs, __half* __restrict__ U)
{
    const int total = K * cs;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i / cs, c = i - k * cs;
        float g[3][3];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int s = 0; s < 3; ++s) g[r][s] = __half2float(w[k * w_po + r * w_py + s * w_px + c]);
        float t[4][3];
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            t[0][s] = g[0][s]; t[1][s] = 0.5f * (g[0][s] + g[1][s] + g[2][s]); t[2][s] = 0.5f * (g[0][s] - g[1][s] + g[2][s]); t[3][s] = g[2][s];
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float u0 = t[r][0], u1 = 0.5f * (t[r][0] + t[r][1] + t[r][2]), u2 = 0.5f * (t[r][0] - t[r][1] + t[r][2]), u3 = t[r][2];
            U[((size_t)(r * 4 + 0) * Ks + k) * cs + c] = __float2half_rn(u0);
            U[((size_t)(r * 4 + 1) * Ks + k) * cs + c] = __float2half_rn(u1);
            U[((size_t)(r * 4 + 2) * Ks + k) * cs + c] = __float2half_rn(u2);
            U[((size_t)(r * 4 + 3) * Ks + k) * cs + c] = __float2half_rn(u3);
        }
    }
}

// V[xi][t][c] = (B^T d B)[xi],  B^T = [1 0 -1 0; 0 1 1 0; 0 -1 1 0; 0 1 0 -1];  thread = (tile, 8 features)
__global__ void __launch_bounds__(256) wino_input_transform(const __grid_constant__ WinoParams p, const __half* __restrict__ in, __half* __restrict__ V)
{
    const int c8n = p.cs / 8;
    const int64_t total = (int64_t)p.Tp * c8n;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int c8 = (int)(idx % c8n); const int t = (int)(idx / c8n);
        // additions only: carried out on packed halves (the result is stored as fp16 anyway)
        __half2 d[4][4][4];
        const bool live = t < p.T;
        int n = 0, ty = 0, tx = 0;
        if (live) { tx = t % p.tiles_x; const int t2 = t / p.tiles_x; ty = t2 % p.tiles_y; n = t2 / p.tiles_y; }
        const int y0 = ty * 2 - p.pad_y, x0 = tx * 2 - p.pad_x;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int y = y0 + i, x = x0 + j;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (live && y >= 0 && y < p.H && x >= 0 && x < p.W)
                    v = __ldg(reinterpret_cast<const uint4*>(in + p.in_off + (int64_t)n * p.in_pb + (int64_t)y * p.in_py + (int64_t)x * p.in_px + c8 * 8));
                const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) d[i][j][e] = h[e];
            }
        // rows: tr = B^T d
        __half2 tr[4][4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                tr[0][j][e] = __hsub2(d[0][j][e], d[2][j][e]); tr[1][j][e] = __hadd2(d[1][j][e], d[2][j][e]);
                tr[2][j][e] = __hsub2(d[2][j][e], d[1][j][e]); tr[3][j][e] = __hsub2(d[1][j][e], d[3][j][e]);
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 o[4][4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[0][e] = __hsub2(tr[i][0][e], tr[i][2][e]); o[1][e] = __hadd2(tr[i][1][e], tr[i][2][e]);
                o[2][e] = __hsub2(tr[i][2][e], tr[i][1][e]); o[3][e] = __hsub2(tr[i][1][e], tr[i][3][e]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 v; __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = o[j][e];
                *reinterpret_cast<uint4*>(V + ((size_t)(i * 4 + j) * p.Tp + t) * p.cs + c8 * 8) = v;
            }
        }
    }
}

// Y = A^T M A,  A^T = [1 1 1 0; 0 1 -1 -1];  thread = (tile, 8 output features); + bias, activation, store byxf
__global__ void __launch_bounds__(256) wino_output_transform(const __grid_constant__ WinoParams p, const __half* __restrict__ M, const void* __restrict__ bias,
                                                             __half* __restrict__ out)
{
    const int k8n = p.ofm_s / 8;
    const int64_t total = (int64_t)p.T * k8n;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int k8 = (int)(idx % k8n); const int t = (int)(idx / k8n);
        const int tx = t % p.tiles_x; const int t2 = t / p.tiles_x; const int ty = t2 % p.tiles_y; const int n = t2 / p.tiles_y;
        float b[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) { const int f = k8 * 8 + e; b[e] = (p.bias_dtype != CLDNN_B200_NONE && f < p.ofm) ? load_as_float(bias, p.bias_dtype, f) : 0.0f; }
        // columns first: r = A^T m, one column of the 4x4 tile at a time
        float r[2][4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float m[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(M + ((size_t)(i * 4 + j) * p.Tp + t) * p.ofm_s + k8 * 8));
                unpack8(v, m[i]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) { r[0][j][e] = m[0][e] + m[1][e] + m[2][e]; r[1][j][e] = m[1][e] - m[2][e] - m[3][e]; }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int y = ty * 2 + i; if (y >= p.P) continue;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int x = tx * 2 + j; if (x >= p.Q) continue;
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float v = (j == 0 ? r[i][0][e] + r[i][1][e] + r[i][2][e] : r[i][1][e] - r[i][2][e] - r[i][3][e]) + b[e];
                    o[e] = p.act == CLDNN_B200_ACT_NONE ? v : (p.act == CLDNN_B200_ACT_RELU ? fmaxf(v, 0.0f) : act_float(p.act, v, p.act_m, p.act_n));
                }
                __half* dst = out + p.out_off + (int64_t)n * p.out_pb + (int64_t)y * p.out_py + (int64_t)x * p.out_px + k8 * 8;
                if (k8 * 8 + 8 <= p.ofm) *reinterpret_cast<uint4*>(dst) = pack8(o);
                else for (int e = 0; e < 8 && k8 * 8 + e < p.ofm; ++e) dst[e] = __float2half_rn(o[e]);
            }
        }
    }
}

bool wino_plan(const cldnn_b200_conv_params& p, std::string* why)
{
    auto no = [&](const char* m) { if (why) *why = m; return false; };
    if (p.in.dtype != CLDNN_B200_F16 || p.w_dtype != CLDNN_B200_F16 || p.out.dtype != CLDNN_B200_F16) return no("fp16 only");
    if (p.kh != 3 || p.kw != 3 || p.stride_x != 1 || p.stride_y != 1 || p.dil_x != 1 || p.dil_y != 1 || p.groups != 1) return no("3x3 stride-1 undilated ungrouped filters only");
    if (p.fused_eltw || p.quantization || p.calibration || p.has_o_qf) return no("plain convolution only");
    if (p.out.f != p.ofm || p.in.f != p.ifm) return no("feature counts");
    if (p.in.pf != 1 || p.in.px % 16 || p.in.py % 8 || p.in.pb % 8 || p.in.offset % 8 || p.in.px < p.in.f) return no("input must be byxf with the stored feature count a multiple of 16");
    if (p.out.pf != 1 || p.out.px % 8 || p.out.py % 8 || p.out.pb % 8 || p.out.offset % 8 || p.out.px < (p.ofm + 7) / 8 * 8) return no("output must be byxf, 16-byte aligned, features stored in whole groups of 8");
    if (p.w_pi != 1 || p.w_px != p.in.px || p.w_py != p.w_px * 3) return no("weights must be oyxi with the input's stored feature count");
    if (p.bias_dtype != CLDNN_B200_NONE && p.bias_dtype != CLDNN_B200_F16 && p.bias_dtype != CLDNN_B200_F32) return no("bias type");
    const int P_ = p.in.y + 2 * p.pad_y - 2, Q_ = p.in.x + 2 * p.pad_x - 2;
    if (p.out.y != P_ || p.out.x != Q_ || p.out.b != p.in.b) return no("output size does not match the sliding-window rule");
    return true;
}

struct WinoSizes { int tiles_x, tiles_y, T, Tp, ofm_s; size_t u_bytes, v_bytes, m_bytes; };
WinoSizes wino_sizes(const cldnn_b200_conv_params& p)
{
    WinoSizes s{};
    s.tiles_x = (p.out.x + 1) / 2; s.tiles_y = (p.out.y + 1) / 2;
    s.T = p.out.b * s.tiles_x * s.tiles_y; s.Tp = (s.T + 127) / 128 * 128;
    s.ofm_s = (p.ofm + 7) / 8 * 8;
    const size_t cs = (size_t)p.in.px;
    s.u_bytes = ((size_t)16 * s.ofm_s * cs * 2 + 255) / 256 * 256;
    s.v_bytes = ((size_t)16 * s.Tp * cs * 2 + 255) / 256 * 256;
    s.m_bytes = ((size_t)16 * s.Tp * s.ofm_s * 2 + 255) / 256 * 256;
    return s;
}

bool wino_supports(const void* vp) { return wino_plan(*(const cldnn_b200_conv_params*)vp, nullptr); }
int wino_tune_count(const void*) { return 1; }
size_t wino_scratch(const void* vp)
{
    const auto& p = *(const cldnn_b200_conv_params*)vp;
    if (!wino_plan(p, nullptr)) return 0;
    const WinoSizes s = wino_sizes(p);
    return s.u_bytes + s.v_bytes + s.m_bytes;
}

int32_t wino_prepare(cldnn_b200_ctx_impl* ctx, const void* vp, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out)
{
    const cldnn_b200_conv_params& p = *(const cldnn_b200_conv_params*)vp;
    std::string why;
    if (!wino_plan(p, &why)) return fail(CLDNN_B200_UNSUPPORTED_FORMAT, "conv_f16_winograd: " + why);
    if (!a->input0 || !a->output || !a->weights) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_winograd: input, output and weights are required");
    if (p.bias_dtype != CLDNN_B200_NONE && !a->bias) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_winograd: bias_dtype set but no bias pointer");
    const WinoSizes s = wino_sizes(p);
    const size_t need = s.u_bytes + s.v_bytes + s.m_bytes;
    if (!a->scratch || a->scratch_bytes < need) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_winograd: needs " + std::to_string(need) + " bytes of scratch");
    if (((uintptr_t)a->scratch | (uintptr_t)a->input0 | (uintptr_t)a->output) & 15) return fail(CLDNN_B200_INVALID_ARG, "conv_f16_winograd: buffers must be 16-byte aligned");
    __half* U = (__half*)a->scratch;
    __half* V = (__half*)((char*)a->scratch + s.u_bytes);
    __half* M = (__half*)((char*)a->scratch + s.u_bytes + s.v_bytes);

    WinoParams W{};
    W.N = p.in.b; W.H = p.in.y; W.W = p.in.x; W.P = p.out.y; W.Q = p.out.x; W.cs = (int32_t)p.in.px; W.ofm = p.ofm; W.ofm_s = s.ofm_s;
    W.pad_x = p.pad_x; W.pad_y = p.pad_y; W.tiles_x = s.tiles_x; W.tiles_y = s.tiles_y; W.T = s.T; W.Tp = s.Tp;
    W.in_px = p.in.px; W.in_py = p.in.py; W.in_pb = p.in.pb; W.in_off = p.in.offset;
    W.out_px = p.out.px; W.out_py = p.out.py; W.out_pb = p.out.pb; W.out_off = p.out.offset;
    W.bias_dtype = p.bias_dtype; W.act = p.act; W.act_m = p.act_m; W.act_n = p.act_n;

    // transformed weights: once, on the context's stream, before anything prepared here can run.  Rows of U beyond ofm stay zero.
    B200_CUDA(cudaMemsetAsync(U, 0, s.u_bytes, ctx->stream));
    {
        // U is laid out [16][ofm_s][cs]; the transform writes K = ofm rows of it
        const __half* w = (const __half*)a->weights + p.w_offset;
        const int total = p.ofm * W.cs;
        wino_weight_transform<<<(total + 255) / 256, 256, 0, ctx->stream>>>(w, p.w_po, p.w_py, p.w_px, p.ofm, s.ofm_s, W.cs, U);
        B200_CUDA(cudaGetLastError());
    }
    std::function<cudaError_t(cudaStream_t)> gemm;
    const int32_t st = f16_batched_gemm_prepare(ctx, V, U, M, 16, s.Tp, W.cs, s.ofm_s, gemm);
    if (st != CLDNN_B200_SUCCESS) return st;
    const int sms = ctx->prop.multiProcessorCount;
    const int64_t in_items = (int64_t)s.Tp * (W.cs / 8), out_items = (int64_t)s.T * (s.ofm_s / 8);
    const int g1 = (int)std::min<int64_t>((in_items + 255) / 256, (int64_t)sms * 16), g3 = (int)std::min<int64_t>((out_items + 255) / 256, (int64_t)sms * 16);
    const __half* in = (const __half*)a->input0; __half* o = (__half*)a->output; const void* bias = a->bias;
    out->fn = [W, in, V, M, o, bias, gemm, g1, g3](cudaStream_t st_) {
        wino_input_transform<<<g1, 256, 0, st_>>>(W, in, V);
        cudaError_t e = cudaGetLastError(); if (e != cudaSuccess) return e;
        e = gemm(st_); if (e != cudaSuccess) return e;
        wino_output_transform<<<g3, 256, 0, st_>>>(W, M, bias, o);
        return cudaGetLastError();
    };
    out->launches = 3;
    return CLDNN_B200_SUCCESS;
}

}  // namespace

const KernelDef kdef_conv_f16_winograd = {"conv_f16_winograd", sizeof(cldnn_b200_conv_params), wino_supports, wino_tune_count, wino_scratch, wino_prepare};

}  // namespace b200
