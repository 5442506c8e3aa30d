/*
 * cldnn_b200.h -- thin C ABI of the B200 (sm_100a) CUDA engine that stands where
 * clDNN's OpenCL runtime layer stood.
 *
 * Everything in the clDNN graph core that used to talk to OpenCL (gpu_toolkit,
 * kernels_cache, gpu::kernel, gpu_buffer, base_event, kernel_runner) talks to
 * the functions declared here instead.  The ABI is plain C: opaque handles,
 * POD parameter blocks, device/host pointers and sizes; no C++ or torch types
 * cross it and no exception leaves it.  Every function returns a cldnn_status
 * compatible code (api/C/cldnn.h:70-82) and records a thread-local message
 * retrievable with cldnn_b200_last_error() (the convention of
 * cldnn_get_last_error_message, src/cldnn.cpp:29-33,746).
 *
 * Parameter blocks restate, as runtime PODs, the JIT "#define" blocks the
 * reference's kernel_selector generated per kernel instance
 * (kernel_selector/core/common/jitter.cpp:186-300 for tensors,
 * actual_kernels/convolution/convolution_kernel_base.cpp:51-127 for the
 * convolution constants).  Kernels are ahead-of-time compiled for sm_100a and
 * resolved by name; there is no run-time compilation.
 */
#ifndef CLDNN_B200_H
#define CLDNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define CLDNN_B200_API
#else
#define CLDNN_B200_API __attribute__((visibility("default")))
#endif

/* ---- status codes: same values as CLDNN_SUCCESS .. CLDNN_GLOBAL_SIZE_EXCEEDED
 *      (api/C/cldnn.h:70-79) ------------------------------------------------ */
#define CLDNN_B200_SUCCESS               0
#define CLDNN_B200_ERROR                -1
#define CLDNN_B200_INVALID_ARG          -2
#define CLDNN_B200_OUT_OF_RESOURCES     -3
#define CLDNN_B200_DEVICE_ERROR         -4
#define CLDNN_B200_UNSUPPORTED_SIZE     -5
#define CLDNN_B200_UNSUPPORTED_FORMAT   -6
#define CLDNN_B200_DIMENSION_MISMATCH   -7
#define CLDNN_B200_ALLOC_SIZE_EXCEEDED  -8
#define CLDNN_B200_GLOBAL_SIZE_EXCEEDED -9

/* ---- element types: same values as cldnn_data_type (api/C/cldnn.h:349-358) - */
#define CLDNN_B200_I8   0x01
#define CLDNN_B200_U8   0x41
#define CLDNN_B200_I32  0x04
#define CLDNN_B200_F16  0x82
#define CLDNN_B200_F32  0x84
#define CLDNN_B200_NONE 0x00

/* ---- activation functions (subset of kernel_selector ActivationFunction,
 *      kernel_selector/common/common_types.h; formulas in
 *      kernel_selector/core/common/jitter.cpp:366-397) ----------------------- */
#define CLDNN_B200_ACT_NONE                 0
#define CLDNN_B200_ACT_RELU                 1   /* max(0, x)                              */
#define CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE  2   /* max(x,0) + m*min(x,0); isinf(m) special */
#define CLDNN_B200_ACT_CLAMP                3   /* max(m, min(n, x))   (ReLU6 = clamp 0,6) */
#define CLDNN_B200_ACT_LOGISTIC             4
#define CLDNN_B200_ACT_TANH                 5
#define CLDNN_B200_ACT_ABS                  6
#define CLDNN_B200_ACT_LINEAR               7   /* m*x + n */
#define CLDNN_B200_ACT_SQUARE               8
#define CLDNN_B200_ACT_SQRT                 9
#define CLDNN_B200_ACT_ELU                 10

/* Operation order of the quantised epilogue.  The reference's kernels do not agree on it; the parity target is the
 * reference-order kernel, the other two are offered for callers whose models were calibrated against the optimised kernels:
 *   REF   fused_conv_eltwise_gpu_ref.cl:148-232  (i32 bias | dequantise, f32 bias) -> activation -> * calib|O_QF -> round
 *                                                 [-> + residual * scale -> activation -> * eltw_calib -> round] -> saturate
 *   MMAD  convolution_gpu_mmad.cl:106-132        round(((float)acc * q * I_QF + bias_f32) * calib|O_QF) -> convert to the 8-bit
 *                                                 type -> activation on the 8-bit value.  No residual.  Needs an f32 bias.
 *   IMAD  fused_conv_eltwise_gpu_imad.cl:171-207 round(((float)acc * q * I_QF + bias_f32) * calib|O_QF) -> 8-bit -> activation
 *                                                 [-> saturate(round(((int)a + (int)residual) * eltw_calib)) -> activation].
 *                                                 Needs an f32 bias and, when fused, eltwise calibration factors.
 * The conversion "to the 8-bit type" of MMAD / IMAD does not saturate in the reference (convert_char / TO_UNIT_TYPE on a value
 * that may be out of range, which OpenCL leaves to the implementation); here it keeps the low 8 bits of the rounded integer.
 * Both take a signed 8-bit output (the kernels' unit type is char).  For values inside the 8-bit range, ReLU or no
 * activation and positive factors all three orders give the same result.                                                   */
#define CLDNN_B200_EPILOGUE_REF  0
#define CLDNN_B200_EPILOGUE_MMAD 1
#define CLDNN_B200_EPILOGUE_IMAD 2

/* A 4-D activation tensor as the reference kernels see it: logical sizes plus
 * element pitches and the offset of element (0,0,0,0) -- the INPUT0_* /
 * OUTPUT_* macro family of jitter.cpp:229-262 and GET_DATA_INDEX of
 * cl_kernels/include/fetch.cl:19-31.  Any of bfyx / byxf / yxfb, with or
 * without padding, is expressible. */
typedef struct cldnn_b200_tensor {
    int32_t dtype;
    int32_t b, f, y, x;          /* logical sizes                         */
    int64_t pb, pf, py, px;      /* pitches, in elements                  */
    int64_t offset;              /* element offset of logical (0,0,0,0)   */
} cldnn_b200_tensor;

/* Convolution / fused_conv_eltwise launch constants.
 * Restates cldnn_convolution_desc (api/C/convolution.h:36-74) +
 * cldnn_fused_conv_eltwise_desc (api_extension/C/fused_conv_eltwise.h:35-97)
 * after convolution_gpu::create (src/gpu/convolution_gpu.cpp:71-162) and
 * fused_conv_eltwise_gpu::create (src/gpu/fused_conv_eltwise_gpu.cpp:70-199)
 * have turned them into kernel_selector params. */
typedef struct cldnn_b200_conv_params {
    cldnn_b200_tensor in;        /* INPUT0                                 */
    cldnn_b200_tensor out;       /* OUTPUT                                 */
    cldnn_b200_tensor eltw;      /* INPUT1 of fused_conv_eltwise           */
    /* weights: [groups*ofm][ifm][kh][kw] logical; pitches in elements      */
    int32_t w_dtype;
    int32_t ofm, ifm;            /* per group                              */
    int32_t kh, kw;
    int64_t w_po, w_pi, w_py, w_px, w_offset;
    int32_t stride_x, stride_y;
    int32_t pad_x, pad_y;        /* = max(-input_offset, 0)                */
    int32_t dil_x, dil_y;
    int32_t groups;              /* >=1; group g owns ofm*g..ofm*(g+1)-1   */
    int32_t bias_dtype;          /* NONE, I32 or F32 (or the input type)   */
    int32_t quantization;        /* QUANTIZATION_TERM                      */
    float   i_qf;                /* I_QF                                   */
    int32_t calibration;         /* CALIBRATION_TERM                       */
    int32_t has_o_qf;            /* O_QF emitted                           */
    float   o_qf;
    int32_t act;  float act_m, act_n;
    /* fused eltwise (sum) part                                             */
    int32_t fused_eltw;
    int32_t has_non_conv_scale;  float non_conv_scale;
    int32_t eltw_act; float eltw_m, eltw_n;
    int32_t eltw_calibration;    /* ELTW_CALIBRATION_TERM                  */
    int32_t eltw_stride_x, eltw_stride_y;
    int32_t in_out_opt;          /* second input lives in the output       */
    /* implementation choice (tuning index of the selected kernel)          */
    int32_t tune;
    int32_t epilogue_order;      /* CLDNN_B200_EPILOGUE_*: whose operation order the quantised epilogue follows */
    int32_t reserved[6];
} cldnn_b200_conv_params;

/* Arguments by role, in the order of kernel_selector's ArgumentDescriptor
 * (kernel_selector/core/kernel_selector_common.h:131-172): all are device
 * pointers owned by the caller. */
typedef struct cldnn_b200_args {
    const void* input0;
    const void* input1;          /* eltwise second input / fused residual  */
    void*       output;
    const void* weights;
    const void* bias;
    const float* weights_quantization_factors;
    const float* output_calibration_factors;
    const float* eltw_output_calibration_factors;
    void*       scratch;         /* kernel-specific workspace, may be NULL */
    size_t      scratch_bytes;
} cldnn_b200_args;

/* Pooling constants: cldnn_pooling_desc (api/C/pooling.h) after
 * pooling_gpu::create (src/gpu/pooling_gpu.cpp:98-160). */
#define CLDNN_B200_POOL_MAX 0
#define CLDNN_B200_POOL_AVG 1
#define CLDNN_B200_DIV_FIXED 0
#define CLDNN_B200_DIV_DYNAMIC 1
#define CLDNN_B200_DIV_DYNAMIC_WITH_PADDING 2
typedef struct cldnn_b200_pool_params {
    cldnn_b200_tensor in, out;
    int32_t mode, div_mode;
    int32_t size_x, size_y, stride_x, stride_y, pad_x, pad_y;
    int32_t act; float act_m, act_n;
    int32_t reserved[4];
} cldnn_b200_pool_params;

/* fully_connected constants (fully_connected_gpu::create,
 * src/gpu/fully_connected_gpu.cpp:59-112; arithmetic of
 * cl_kernels/fully_connected_gpu_bfyx_ref.cl:18-84). Weights [ofm][f][y][x]. */
typedef struct cldnn_b200_fc_params {
    cldnn_b200_tensor in, out;
    int32_t w_dtype;
    int64_t w_po, w_pi, w_py, w_px, w_offset;
    int32_t bias_dtype;
    int32_t quantization; float i_qf;
    int32_t calibration;  float o_qf;
    int32_t act; float act_m, act_n;
    int32_t reserved[4];
} cldnn_b200_fc_params;

/* softmax (cl_kernels/softmax_gpu_ref.cl:22-58).  `dimension` is the scope of normalisation, with the values of
 * cldnn_softmax_dimension (api/C/softmax.h:34-40): 0 over f for each (b, y, x), 1 over x for each (b, f, y),
 * 2 over y for each (b, f, x), 3 over the whole f*y*x image of each batch. */
#define CLDNN_B200_SOFTMAX_F 0
#define CLDNN_B200_SOFTMAX_X 1
#define CLDNN_B200_SOFTMAX_Y 2
#define CLDNN_B200_SOFTMAX_FYX 3
typedef struct cldnn_b200_softmax_params {
    cldnn_b200_tensor in, out;
    int32_t dimension;
    int32_t reserved[3];
} cldnn_b200_softmax_params;

/* eltwise (sum / prod / max / min / sub) of two tensors with the optional
 * int8 requantisation epilogue (cl_kernels/generic_eltwise_ref.cl:198-330). */
#define CLDNN_B200_ELTW_SUM 0
#define CLDNN_B200_ELTW_SUB 1
#define CLDNN_B200_ELTW_MAX 2
#define CLDNN_B200_ELTW_PROD 3
#define CLDNN_B200_ELTW_MIN 4
typedef struct cldnn_b200_eltwise_params {
    cldnn_b200_tensor in0, in1, out;
    int32_t mode;
    int32_t stride_x0, stride_y0, stride_x1, stride_y1;
    int32_t quantization;        /* QUANTIZATION_TERM: int op, *factor, round, convert_char_sat */
    int32_t calibration;         /* factor = calibrations[f], else o_qf    */
    float   o_qf;
    int32_t act; float act_m, act_n;
    int32_t reserved[4];
} cldnn_b200_eltwise_params;

/* reorder: layout and/or type conversion (cl_kernels/reorder_data.cl:72-128);
 * integer destinations saturate, float->int rounds toward zero like
 * convert_<t>_sat. */
typedef struct cldnn_b200_reorder_params {
    cldnn_b200_tensor in, out;
    int32_t has_mean; float mean[4];  /* per-feature subtract, up to 4 feats */
    int32_t reserved[4];
} cldnn_b200_reorder_params;

/* lrn across channel (cl_kernels/lrn_gpu_across_channel_ref.cl:26-66). */
typedef struct cldnn_b200_lrn_params {
    cldnn_b200_tensor in, out;
    int32_t size; float k, alpha, beta;
    int32_t reserved[4];
} cldnn_b200_lrn_params;

/* standalone activation (cl_kernels/activation_ref.cl). */
typedef struct cldnn_b200_activation_params {
    cldnn_b200_tensor in, out;
    int32_t act; float act_m, act_n;
    int32_t reserved[4];
} cldnn_b200_activation_params;

/* ---- opaque handles ----------------------------------------------------- */
typedef struct cldnn_b200_ctx_impl*      cldnn_b200_ctx;
typedef struct cldnn_b200_mem_impl*      cldnn_b200_mem;
typedef struct cldnn_b200_event_impl*    cldnn_b200_event;
typedef struct cldnn_b200_kernel_impl*   cldnn_b200_kernel;
typedef struct cldnn_b200_prepared_impl* cldnn_b200_prepared;
typedef struct cldnn_b200_graph_impl*    cldnn_b200_graph;

/* engine_info_internal (src/gpu/engine_info.cpp:190-231) */
typedef struct cldnn_b200_engine_info {
    uint32_t cores_count;        /* SM count (computeUnitsCount)           */
    uint32_t core_frequency;     /* MHz                                    */
    uint64_t max_alloc_mem_size;
    uint64_t max_global_mem_size;
    uint64_t max_local_mem_size; /* opt-in shared memory per block         */
    uint32_t max_work_group_size;
    uint32_t supports_fp16, supports_imad, supports_immad;
    uint32_t compute_major, compute_minor;
    char     name[64];
} cldnn_b200_engine_info;

/* ---- error text ---------------------------------------------------------- */
/* replaces cldnn_get_last_error_message (src/cldnn.cpp:746) for this layer. */
CLDNN_B200_API const char* cldnn_b200_last_error(void);

/* ---- context: replaces gpu_toolkit::create and the queue it owns
 *      (src/gpu/ocl_toolkit.cpp:75-151) -------------------------------------- */
/* number of CUDA devices visible to the process (0 without a driver): cldnn_get_engine_count, src/cldnn.cpp:179-190 */
CLDNN_B200_API int32_t cldnn_b200_device_count(int32_t* count);
CLDNN_B200_API int32_t cldnn_b200_ctx_create(int32_t device, uint32_t enable_profiling, cldnn_b200_ctx* out);
CLDNN_B200_API int32_t cldnn_b200_ctx_destroy(cldnn_b200_ctx ctx);
CLDNN_B200_API int32_t cldnn_b200_ctx_info(cldnn_b200_ctx ctx, cldnn_b200_engine_info* info);
/* gpu_toolkit::flush / finish (src/gpu/ocl_toolkit.cpp:260-265) */
CLDNN_B200_API int32_t cldnn_b200_ctx_flush(cldnn_b200_ctx ctx);
CLDNN_B200_API int32_t cldnn_b200_ctx_sync(cldnn_b200_ctx ctx);
/* raw cudaStream_t of the context's queue (for callers that interoperate). */
CLDNN_B200_API int32_t cldnn_b200_ctx_stream(cldnn_b200_ctx ctx, void** stream);
/* number of kernel launches issued by this context since creation          */
CLDNN_B200_API int32_t cldnn_b200_ctx_launch_count(cldnn_b200_ctx ctx, uint64_t* count);

/* ---- memory: replaces gpu_buffer (src/gpu/memory_gpu.cpp:37-89) ----------- */
CLDNN_B200_API int32_t cldnn_b200_mem_alloc(cldnn_b200_ctx ctx, size_t bytes, cldnn_b200_mem* out); /* zero filled */
/* cldnn_attach_memory (api/C/cldnn.h:770-772), for device memory: wraps a device pointer the caller owns; the caller keeps
 * it alive for the lifetime of the memory object and of every launch prepared on it.  mem_free releases the wrapper only. */
CLDNN_B200_API int32_t cldnn_b200_mem_attach(cldnn_b200_ctx ctx, void* device_ptr, size_t bytes, cldnn_b200_mem* out);
CLDNN_B200_API int32_t cldnn_b200_mem_free(cldnn_b200_mem mem);
CLDNN_B200_API int32_t cldnn_b200_mem_size(cldnn_b200_mem mem, size_t* bytes);
CLDNN_B200_API int32_t cldnn_b200_mem_devptr(cldnn_b200_mem mem, void** dev);
/* lock()/unlock(): blocking map to a host pointer and write-back            */
CLDNN_B200_API int32_t cldnn_b200_mem_map(cldnn_b200_mem mem, void** host);
CLDNN_B200_API int32_t cldnn_b200_mem_unmap(cldnn_b200_mem mem);
CLDNN_B200_API int32_t cldnn_b200_mem_fill(cldnn_b200_mem mem, uint8_t pattern);
/* explicit stream-ordered copies (host memory may be pinned or pageable)    */
CLDNN_B200_API int32_t cldnn_b200_mem_write(cldnn_b200_mem mem, size_t offset, const void* host, size_t bytes);
CLDNN_B200_API int32_t cldnn_b200_mem_read(cldnn_b200_mem mem, size_t offset, void* host, size_t bytes);
CLDNN_B200_API int32_t cldnn_b200_mem_write_async(cldnn_b200_mem mem, size_t offset, const void* pinned_host, size_t bytes);
CLDNN_B200_API int32_t cldnn_b200_mem_read_async(cldnn_b200_mem mem, size_t offset, void* pinned_host, size_t bytes);
/* pinned host staging buffers                                               */
CLDNN_B200_API int32_t cldnn_b200_host_alloc(size_t bytes, void** host);
CLDNN_B200_API int32_t cldnn_b200_host_free(void* host);

/* ---- events: replaces base_event / user_event
 *      (src/gpu/ocl_base_event.cpp:68-159) ---------------------------------- */
CLDNN_B200_API int32_t cldnn_b200_event_create(cldnn_b200_ctx ctx, cldnn_b200_event* out);
CLDNN_B200_API int32_t cldnn_b200_event_record(cldnn_b200_event ev);
CLDNN_B200_API int32_t cldnn_b200_event_wait(cldnn_b200_event ev);
CLDNN_B200_API int32_t cldnn_b200_event_query(cldnn_b200_event ev, int32_t* is_set);
CLDNN_B200_API int32_t cldnn_b200_event_elapsed_ns(cldnn_b200_event start, cldnn_b200_event end, uint64_t* ns);
CLDNN_B200_API int32_t cldnn_b200_event_destroy(cldnn_b200_event ev);

/* ---- kernels: replaces kernels_cache::set_kernel_source/get_kernel
 *      (src/gpu/kernels_cache.cpp:189-215,310-321) and gpu::kernel::run
 *      (src/gpu/kernel.cpp:233-247) ------------------------------------------ */
CLDNN_B200_API int32_t cldnn_b200_kernel_count(void);
CLDNN_B200_API const char* cldnn_b200_kernel_name(int32_t index);
CLDNN_B200_API int32_t cldnn_b200_kernel_lookup(cldnn_b200_ctx ctx, const char* name, cldnn_b200_kernel* out);
/* does this implementation accept these constants? (KernelBase::Validate)   */
CLDNN_B200_API int32_t cldnn_b200_kernel_supports(cldnn_b200_kernel k, const void* params, size_t params_size, int32_t* yes);
/* how many tuning variants it offers for these constants
 * (GetKernelsDataForAutoTune)                                               */
CLDNN_B200_API int32_t cldnn_b200_kernel_tune_count(cldnn_b200_kernel k, const void* params, size_t params_size, int32_t* count);
/* bytes of scratch the kernel needs for these constants                     */
CLDNN_B200_API int32_t cldnn_b200_kernel_scratch_bytes(cldnn_b200_kernel k, const void* params, size_t params_size, size_t* bytes);
/* immediate launch on the context's stream                                  */
CLDNN_B200_API int32_t cldnn_b200_launch(cldnn_b200_kernel k, const void* params, size_t params_size, const cldnn_b200_args* args);
/* prepared launch: validates, encodes tensor maps and fixes the grid once;
 * replaying it costs one kernel launch (what a network's exec order holds)  */
CLDNN_B200_API int32_t cldnn_b200_prepare(cldnn_b200_kernel k, const void* params, size_t params_size, const cldnn_b200_args* args, cldnn_b200_prepared* out);
CLDNN_B200_API int32_t cldnn_b200_run(cldnn_b200_prepared p);
CLDNN_B200_API int32_t cldnn_b200_prepared_destroy(cldnn_b200_prepared p);
/* kernel_runner::run_kernels (src/gpu/kernel_runner.cpp:112-196): warm-up +
 * `runs` timed replays with CUDA events, average nanoseconds per run         */
CLDNN_B200_API int32_t cldnn_b200_time(cldnn_b200_prepared p, int32_t warmup, int32_t runs, uint64_t* avg_ns);
/* Execution-order replay: everything run between graph_begin and graph_end is
 * recorded instead of executed (CUDA stream capture) and becomes one launchable
 * object.  This is what network_impl::execute's per-primitive enqueue loop
 * (src/network.cpp:217-275) collapses to for a fixed-shape network: one
 * submission per inference.                                                  */
CLDNN_B200_API int32_t cldnn_b200_graph_begin(cldnn_b200_ctx ctx);
CLDNN_B200_API int32_t cldnn_b200_graph_end(cldnn_b200_ctx ctx, cldnn_b200_graph* out);
CLDNN_B200_API int32_t cldnn_b200_graph_launch(cldnn_b200_graph g);
CLDNN_B200_API int32_t cldnn_b200_graph_destroy(cldnn_b200_graph g);
/* First-layer convolution for callers that cannot allocate device memory -- it has no counterpart in the reference.
 * Some embedders run where cudaMalloc is off limits: a serving process whose device memory is carved up once at start-up
 * by another allocator, or a latency-critical section that must not take cudaMalloc's device-wide synchronisation.  The
 * kernel "conv_i8_first" needs a workspace for its packed weights (kernel_scratch_bytes); this entry point keeps that
 * workspace in a fixed 32 KiB array inside the library image instead, so it calls no cudaMalloc / cudaFree and no
 * allocating library routine.  The caller passes the same constants and the same input / output / weights / bias /
 * factor pointers as for "conv_i8_first" (args->scratch is ignored); the two kernels (weights packing, convolution)
 * are enqueued on the context's stream and the call returns without waiting.
 *   - Constants whose packed weights exceed 32 KiB (output features x padded C*kh*8) are refused with
 *     CLDNN_B200_UNSUPPORTED_SIZE; everything "conv_i8_first" refuses is refused here with the same codes.
 *   - params->tune selects among the kernel's CTAs-per-SM variants (1..3) only: the row form (tune 4 / 5 of "conv_i8_first")
 *     needs a far larger workspace and is not offered here; those values run the default variant.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
 *     before starting any stream capture on the device.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Each call rewrites every
 *     byte it later reads, so sequential calls are independent; calls whose kernels may overlap on the GPU (other
 *     streams or contexts of the same process on the same device using this entry point) race on it.  Another
 *     process loads its own copy of the library image and therefore its own array.                               */
CLDNN_B200_API int32_t cldnn_b200_conv_first_noalloc(cldnn_b200_ctx ctx, const cldnn_b200_conv_params* params, const cldnn_b200_args* args);
/* Measured tensor-core peak of the context's device, in tera-operations per second (2 per multiply-add): one CTA per
 * SM issues tcgen05.mma (M = 128, N = n in {64, 128, 256}, 32 bytes of K) on operands resident in shared memory, the
 * accumulator in tensor memory, a few milliseconds per call.  dtype: CLDNN_B200_I8 (s8 x s8 -> s32) or CLDNN_B200_F16
 * (f16 x f16 -> f32).  It is the denominator roofline fractions of the convolution kernels are quoted against; it plays
 * the part of the reference's device capability query (engine_info_internal, src/gpu/engine_info.cpp:190-231), which
 * reports core counts and clock only.                                                                              */
CLDNN_B200_API int32_t cldnn_b200_tensor_peak(cldnn_b200_ctx ctx, int32_t dtype, int32_t n, double* tera_ops_per_second);
/* device-side status word: 0 when the last launches completed normally,
 * otherwise a code written by a kernel whose bounded wait gave up           */
CLDNN_B200_API int32_t cldnn_b200_ctx_device_status(cldnn_b200_ctx ctx, uint32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* CLDNN_B200_H */
