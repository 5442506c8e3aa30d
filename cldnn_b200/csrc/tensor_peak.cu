// Measured tensor-core peak of the device this library runs on: the denominator the convolution
// kernels' roofline fractions are quoted against.  One CTA per SM; a single thread issues a long run
// of tcgen05.mma instructions (M = 128, N = 64 / 128 / 256, 32 bytes of K each) whose operands stay
// resident in shared memory in the 128-byte-swizzled K-major layout the convolution kernels use, with
// the accumulator in tensor memory -- no global-memory traffic, no epilogue: what the tensor pipe itself
// sustains.  Timed with CUDA events on the context's stream.
#include <algorithm>
#include <string>
#include "engine.hpp"
#include "sm100_ptx.cuh"

namespace b200 {

using namespace ptx;

constexpr int kPeakThreads = 128;
constexpr int kPeakOperandBytes = 16 * 1024 + 32 * 1024;      // A: 128 rows x 128 B, B: up to 256 rows x 128 B

template <bool kHalf>
__global__ void __launch_bounds__(kPeakThreads, 1) tensor_peak_kernel(int n, int iters, uint32_t* status)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    // small operand values: the accumulators stay finite (fp16) and far from wrapping (s32) over the whole run
    for (int i = threadIdx.x; i < kPeakOperandBytes / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem)[i] = kHalf ? 0x10001000u : ((i & 1) ? 0x01ff01ffu : 0xff01ff01u);
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); mbar_fence_init(); }
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_slot), 256); tmem_relinquish(); }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;
    if (threadIdx.x == 0) {
        // instruction descriptor: s32 (i8) or f32 (f16) accumulator, K-major operands, N >> 3, M >> 4
        const uint32_t idesc = kHalf ? ((1u << 4) | ((uint32_t)(n >> 3) << 17) | (8u << 24))
                                     : ((2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (8u << 24));
        uint64_t ad[4], bd[4];
        for (int k = 0; k < 4; ++k) {                             // the four 32-byte K slices of one swizzle atom
            ad[k] = make_smem_desc(base + 32u * k, 1024u, 2u);
            bd[k] = make_smem_desc(base + 16u * 1024u + 32u * k, 1024u, 2u);
        }
        for (int it = 0; it < iters; it += 4) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (kHalf) mma_f16_ss(tm, ad[k], bd[k], idesc, (it | k) ? 1u : 0u);
                else mma_i8_ss(tm, ad[k], bd[k], idesc, (it | k) ? 1u : 0u);
            }
        }
        tc_commit(smem_u32(&bar));
        const uint64_t t0 = globaltimer();
        while (!mbar_try_wait(smem_u32(&bar), 0u)) {
            if (globaltimer() - t0 > kWaitLimitNs) { atomicCAS(status, 0u, 0x50u); break; }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 256); }
}

}  // namespace b200

extern "C" int32_t cldnn_b200_tensor_peak(cldnn_b200_ctx ctx, int32_t dtype, int32_t n, double* tera_ops_per_second)
{
    using namespace b200;
    if (!ctx || !tera_ops_per_second) return fail(CLDNN_B200_INVALID_ARG, "tensor_peak: null argument");
    if (dtype != CLDNN_B200_I8 && dtype != CLDNN_B200_F16) return fail(CLDNN_B200_INVALID_ARG, "tensor_peak: dtype must be i8 or f16");
    if (n != 64 && n != 128 && n != 256) return fail(CLDNN_B200_INVALID_ARG, "tensor_peak: n must be 64, 128 or 256");
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); prev = -1; }
    if (prev != ctx->device) B200_CUDA(cudaSetDevice(ctx->device));
    struct Restore { int prev, cur; ~Restore() { if (prev >= 0 && prev != cur) (void)cudaSetDevice(prev); } } restore{prev, ctx->device};

    const bool half = dtype == CLDNN_B200_F16;
    const size_t smem = 1024 + kPeakOperandBytes;
    if (half) B200_CUDA(cudaFuncSetAttribute(tensor_peak_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else B200_CUDA(cudaFuncSetAttribute(tensor_peak_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = ctx->prop.multiProcessorCount;
    // ~2 ms per timed launch: an N = 256 instruction occupies the pipe for about 128 clocks
    const int iters = 32768 * (256 / n);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    B200_CUDA(cudaEventCreate(&e0));
    B200_CUDA(cudaEventCreate(&e1));
    float best_ms = 0.0f;
    cudaError_t err = cudaSuccess;
    for (int rep = 0; rep < 4 && err == cudaSuccess; ++rep) {    // the first launch warms up
        cudaEventRecord(e0, ctx->stream);
        if (half) tensor_peak_kernel<true><<<grid, kPeakThreads, smem, ctx->stream>>>(n, iters, ctx->d_status);
        else tensor_peak_kernel<false><<<grid, kPeakThreads, smem, ctx->stream>>>(n, iters, ctx->d_status);
        err = cudaGetLastError();
        cudaEventRecord(e1, ctx->stream);
        if (err == cudaSuccess) err = cudaEventSynchronize(e1);
        float ms = 0.0f;
        if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
        ctx->launches += 1;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (err != cudaSuccess) return cuda_fail(err, "tensor_peak");
    if (!(best_ms > 0.0f)) return fail(CLDNN_B200_DEVICE_ERROR, "tensor_peak: no time measured");
    const double k_elems = half ? 16.0 : 32.0;                   // elements of K per instruction
    const double ops = 2.0 * 128.0 * n * k_elems * (double)iters * grid;
    *tera_ops_per_second = ops / (best_ms * 1e-3) / 1e12;
    return CLDNN_B200_SUCCESS;
}
