/*
 * cldnn_host.h -- flat C interface to the host side of the B200 engine
 * (topology / program / network), for callers that bind through an FFI.
 *
 * It exposes the same objects and primitive descriptors as clDNN's public API
 * for the convolution path -- cldnn_engine, cldnn_memory, cldnn_topology,
 * cldnn_network and the convolution / fused_conv_eltwise / pooling /
 * fully_connected / softmax / eltwise / reorder / activation / lrn primitives
 * (api/C/cldnn.h:537-805 and api/C/<primitive>.h, api_extension/C/
 * fused_conv_eltwise.h) -- with scalar arguments instead of nested descriptor
 * structs, so a ctypes / cgo / JNI binding needs no struct marshalling.
 * Argument meaning is the reference's: input_offset is negative for padding,
 * tensors are given as x, y (spatial[0], spatial[1]), empty strings stand for
 * absent optional primitive ids, data types are cldnn_data_type values.
 *
 * Every function returns a cldnn_status-compatible code; the message of the
 * last failure on the calling thread is cldnn_host_last_error().
 */
#ifndef CLDNN_HOST_H
#define CLDNN_HOST_H
#include <stddef.h>
#include <stdint.h>
#include "cldnn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cldnn_host_engine_impl*   cldnn_host_engine;
typedef struct cldnn_host_memory_impl*   cldnn_host_memory;
typedef struct cldnn_host_topology_impl* cldnn_host_topology;
typedef struct cldnn_host_network_impl*  cldnn_host_network;

/* formats: values of cldnn_format_type (api/C/cldnn.h:271-317) */
#define CLDNN_HOST_FORMAT_YXFB 0
#define CLDNN_HOST_FORMAT_BYXF 1
#define CLDNN_HOST_FORMAT_BFYX 2
#define CLDNN_HOST_FORMAT_BYXF_AF32 21

/* cldnn_get_last_error_message, src/cldnn.cpp:746 */
CLDNN_B200_API const char* cldnn_host_last_error(void);

/* cldnn_create_engine / cldnn_release_engine / cldnn_get_engine_info, api/C/cldnn.h:560-600 */
CLDNN_B200_API int32_t cldnn_host_engine_create(int32_t device, uint32_t enable_profiling, cldnn_host_engine* out);
CLDNN_B200_API int32_t cldnn_host_engine_release(cldnn_host_engine e);
CLDNN_B200_API int32_t cldnn_host_engine_info(cldnn_host_engine e, cldnn_b200_engine_info* info);
/* the engine's queue as a cudaStream_t, for callers that order their own copies with the network's work */
CLDNN_B200_API int32_t cldnn_host_engine_stream(cldnn_host_engine e, void** stream);

/* cldnn_allocate_memory / cldnn_release_memory / cldnn_lock_memory (as explicit copies), api/C/cldnn.h:760-800 */
CLDNN_B200_API int32_t cldnn_host_memory_allocate(cldnn_host_engine e, int32_t data_type, int32_t format, int32_t b, int32_t f, int32_t x, int32_t y, cldnn_host_memory* out);
/* cldnn_attach_memory, api/C/cldnn.h:770-772, for a device pointer owned by the caller */
CLDNN_B200_API int32_t cldnn_host_memory_attach(cldnn_host_engine e, int32_t data_type, int32_t format, int32_t b, int32_t f, int32_t x, int32_t y, void* device_ptr, cldnn_host_memory* out);
CLDNN_B200_API int32_t cldnn_host_memory_release(cldnn_host_memory m);
CLDNN_B200_API int32_t cldnn_host_memory_write(cldnn_host_memory m, const void* host, size_t bytes);
CLDNN_B200_API int32_t cldnn_host_memory_read(cldnn_host_memory m, void* host, size_t bytes);
CLDNN_B200_API int32_t cldnn_host_memory_layout(cldnn_host_memory m, int32_t* data_type, int32_t* format, int32_t* b, int32_t* f, int32_t* x, int32_t* y, size_t* bytes);
CLDNN_B200_API int32_t cldnn_host_memory_device_ptr(cldnn_host_memory m, void** dev);

/* cldnn_create_topology / cldnn_add_primitive / cldnn_release_topology, api/C/cldnn.h:606-640 */
CLDNN_B200_API int32_t cldnn_host_topology_create(cldnn_host_topology* out);
CLDNN_B200_API int32_t cldnn_host_topology_release(cldnn_host_topology t);
/* input_layout (api/C/input_layout.h), data (api/C/data.h), reorder (api/C/reorder.h) */
CLDNN_B200_API int32_t cldnn_host_add_input_layout(cldnn_host_topology t, const char* id, int32_t data_type, int32_t format, int32_t b, int32_t f, int32_t x, int32_t y);
CLDNN_B200_API int32_t cldnn_host_add_data(cldnn_host_topology t, const char* id, cldnn_host_memory m);
CLDNN_B200_API int32_t cldnn_host_add_reorder(cldnn_host_topology t, const char* id, const char* input, int32_t out_format, int32_t out_data_type,
                                              const float* subtract_per_feature, size_t subtract_count);
/* convolution, api/C/convolution.h:36-74 */
CLDNN_B200_API int32_t cldnn_host_add_convolution(cldnn_host_topology t, const char* id, const char* input, const char* weights, const char* bias,
                                                  const char* weights_quantization_factors, const char* output_calibration_factors,
                                                  float input_quantization_factor, float output_quantization_factor, int32_t output_data_type,
                                                  int32_t stride_x, int32_t stride_y, int32_t input_offset_x, int32_t input_offset_y,
                                                  int32_t dilation_x, int32_t dilation_y, uint32_t with_activation, float activation_negative_slope,
                                                  uint32_t groups);
/* fused_conv_eltwise, api_extension/C/fused_conv_eltwise.h:35-97 */
CLDNN_B200_API int32_t cldnn_host_add_fused_conv_eltwise(cldnn_host_topology t, const char* id, const char* input, const char* input2,
                                                         const char* weights, const char* bias, const char* conv_weights_quantization_factors,
                                                         const char* conv_output_calibration_factors, float conv_input_quantization_factor,
                                                         float non_conv_scale, const char* eltw_output_calibration_factors,
                                                         int32_t eltw_stride_x, int32_t eltw_stride_y, int32_t stride_x, int32_t stride_y,
                                                         int32_t input_offset_x, int32_t input_offset_y, int32_t dilation_x, int32_t dilation_y,
                                                         uint32_t conv_with_activation, float conv_activation_negative_slope,
                                                         uint32_t eltw_with_activation, float eltw_activation_negative_slope, int32_t output_data_type);
/* eltwise (api/C/eltwise.h), activation (api/C/activation.h), pooling (api/C/pooling.h), fully_connected
 * (api/C/fully_connected.h), softmax (api/C/softmax.h), lrn (api/C/lrn.h) */
CLDNN_B200_API int32_t cldnn_host_add_eltwise(cldnn_host_topology t, const char* id, const char* input, const char* input2, int32_t mode,
                                              uint32_t with_activation, float activation_negative_slope, const char* output_calibration_factors,
                                              float output_quantization_factor, uint32_t quantized);
CLDNN_B200_API int32_t cldnn_host_add_activation(cldnn_host_topology t, const char* id, const char* input, int32_t func, float a, float b);
CLDNN_B200_API int32_t cldnn_host_add_pooling(cldnn_host_topology t, const char* id, const char* input, int32_t mode, uint32_t global_pooling,
                                              int32_t size_x, int32_t size_y, int32_t stride_x, int32_t stride_y, int32_t input_offset_x, int32_t input_offset_y);
CLDNN_B200_API int32_t cldnn_host_add_fully_connected(cldnn_host_topology t, const char* id, const char* input, const char* weights, const char* bias,
                                                      const char* weights_quantization_factors, const char* output_calibration_factors,
                                                      float input_quantization_factor, float output_quantization_factor,
                                                      uint32_t with_activation, float activation_negative_slope);
CLDNN_B200_API int32_t cldnn_host_add_softmax(cldnn_host_topology t, const char* id, const char* input);   /* normalize_fyx, the reference's default */
/* dimension: cldnn_softmax_dimension (api/C/softmax.h:34-40): 0 normalize_f, 1 normalize_x, 2 normalize_y, 3 normalize_fyx */
CLDNN_B200_API int32_t cldnn_host_add_softmax_dim(cldnn_host_topology t, const char* id, const char* input, int32_t dimension);
CLDNN_B200_API int32_t cldnn_host_add_lrn(cldnn_host_topology t, const char* id, const char* input, uint32_t size, float k, float alpha, float beta);
/* Checks a tuning cache file (the reference's cache.json schema, kernel_selector/core/auto_tuner.cpp:72-118): *entries receives
 * the number of entries stored for `compute_units` streaming multiprocessors (0 when the file has no such section); malformed
 * JSON or a malformed entry gives CLDNN_B200_INVALID_ARG with the position in the last-error text.  Needs no device.      */
CLDNN_B200_API int32_t cldnn_host_tuning_cache_check(const char* path, uint32_t compute_units, size_t* entries);
/* cldnn::concatenation (api/CPP/concatenation.hpp:40-78): `inputs` is a comma-separated list of ids, axis 0 batch, 1 feature, 2 x, 3 y */
CLDNN_B200_API int32_t cldnn_host_add_concatenation(cldnn_host_topology t, const char* id, const char* inputs, int32_t axis);

/* build options, api/C/cldnn.h:207-232 */
typedef struct cldnn_host_build_options {
    uint32_t optimize_data;
    uint32_t fuse_any_conv_eltwise;
    uint32_t tuning_mode;                 /* 0 disabled, 1 use cache, 2 tune and cache */
    const char* tuning_cache_path;        /* may be NULL */
    const char* outputs;                  /* comma separated primitive ids, NULL = primitives without users */
    uint32_t use_graph;
    const char* force_kernel;             /* "<id>=<kernel>[:tune],..." or NULL */
} cldnn_host_build_options;

/* cldnn_build_network / cldnn_release_network / cldnn_set_network_input / cldnn_execute_network /
 * cldnn_get_network_output, api/C/cldnn.h:690-750 */
CLDNN_B200_API int32_t cldnn_host_network_build(cldnn_host_engine e, cldnn_host_topology t, const cldnn_host_build_options* options, cldnn_host_network* out);
CLDNN_B200_API int32_t cldnn_host_network_release(cldnn_host_network n);
CLDNN_B200_API int32_t cldnn_host_network_set_input(cldnn_host_network n, const char* id, cldnn_host_memory m);
CLDNN_B200_API int32_t cldnn_host_network_execute(cldnn_host_network n);
CLDNN_B200_API int32_t cldnn_host_network_wait(cldnn_host_network n);
/* the returned memory handle is owned by the caller (release it); it views the network's output buffer */
CLDNN_B200_API int32_t cldnn_host_network_get_output(cldnn_host_network n, const char* id, cldnn_host_memory* out);
/* executed primitives, one per line: "id|type|kernel|tune|format|dtype|b,f,y,x|fused ids|is_output"; cldnn_get_primitive_info */
CLDNN_B200_API int32_t cldnn_host_network_info(cldnn_host_network n, char* buffer, size_t buffer_bytes, size_t* needed);
/* per-primitive device time of the last execute on a profiling engine, one "id|nanoseconds" per line;
 * cldnn_get_event_profiling_info, src/cldnn.cpp:356 */
CLDNN_B200_API int32_t cldnn_host_network_profiling(cldnn_host_network n, char* buffer, size_t buffer_bytes, size_t* needed);
CLDNN_B200_API int32_t cldnn_host_network_stats(cldnn_host_network n, uint64_t* launches_per_execute, size_t* pool_bytes);

#ifdef __cplusplus
}
#endif
#endif /* CLDNN_HOST_H */
