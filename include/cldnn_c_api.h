/* The public C boundary of clDNN for the convolution hot path, as libclDNN64.so of this repository exports it.
 *
 * clDNN's applications (its header-only C++ API under api/CPP, its tests, the Inference-Engine plugin) reach the library
 * through the C entry points and plain-data descriptors of api/C/cldnn.h and api/C/<primitive>.h.  This header declares
 * the same symbols with the same binary layout, so that code compiled against the reference's own headers links against
 * this library unchanged; it exists so that the library itself can be built without the reference tree.  Each block
 * names the reference declaration it stands for.  Layout equality with the reference headers is a test
 * (tests/test_public_api_layout.py).
 *
 * Covered: engine, memory, topology, program, network, event, and the primitives of the hot path -- input_layout, data,
 * reorder, convolution, fused_conv_eltwise, eltwise, activation, pooling, fully_connected, softmax, lrn, concatenation.
 * Anything else (other primitive types, image formats, training options) is answered with an error status
 * (CLDNN_UNSUPPORTED_FORMAT / CLDNN_INVALID_ARG); nothing falls back to another implementation.
 *
 * Conventions (api/C/cldnn.h:70-119, src/cldnn.cpp:29-33): every function takes a trailing `cldnn_status*` that may be
 * NULL and returns a default value on failure; the message of the last failure of the calling thread is
 * cldnn_get_last_error_message().  Handles are reference counted: created with one reference, cldnn_retain_ / cldnn_release_.
 */
#ifndef CLDNN_C_API_H
#define CLDNN_C_API_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CLDNN_API __attribute__((visibility("default")))
#else
#define CLDNN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: api/C/cldnn.h:70-79 ---- */
#define CLDNN_SUCCESS                0
#define CLDNN_ERROR                 -1
#define CLDNN_INVALID_ARG           -2
#define CLDNN_OUT_OF_RESOURCES      -3
#define CLDNN_DEVICE_ERROR          -4
#define CLDNN_UNSUPPORTED_SIZE      -5
#define CLDNN_UNSUPPORTED_FORMAT    -6
#define CLDNN_DIMENSION_MISMATCH    -7
#define CLDNN_ALLOC_SIZE_EXCEEDED   -8
#define CLDNN_GLOBAL_SIZE_EXCEEDED  -9
typedef int32_t cldnn_status;

/* api/C/cldnn.h:88-94 */
typedef struct { int32_t major, minor, build, revision; } cldnn_version;

/* ---- opaque handles: api/C/cldnn.h:99-119 ---- */
typedef struct cldnn_engine_impl* cldnn_engine;
typedef struct cldnn_event_impl* cldnn_event;
typedef struct cldnn_topology_impl* cldnn_topology;
typedef struct cldnn_program_impl* cldnn_program;
typedef struct cldnn_network_impl* cldnn_network;
typedef struct cldnn_memory_impl* cldnn_memory;

/* api/C/cldnn.h:125-128: the only engine type; the CUDA engine answers to it */
typedef enum { cldnn_engine_ocl } cldnn_engine_type;

/* ---- engine configuration and capabilities: api/C/cldnn.h:150-188 ---- */
typedef struct {
    uint32_t enable_profiling;
    uint32_t meaningful_kernels_names;
    uint32_t dump_custom_program;
    const char* compiler_options;          /* OpenCL-only: must be empty */
    const char* single_kernel_name;
    uint32_t enable_parallelisation;
    const char* engine_log;
    const char* sources_dumps_dir;
    int16_t priority_mode;
    int16_t throttle_mode;
    uint32_t enable_memory_pool;
    void* context;                         /* OpenCL-only: must be NULL */
    const char* tuning_cache_path;
} cldnn_engine_configuration;

typedef struct {
    uint32_t cores_count;                  /* streaming multiprocessors */
    uint32_t core_frequency;               /* MHz */
    uint64_t max_work_group_size;
    uint64_t max_local_mem_size;
    uint64_t max_global_mem_size;
    uint64_t max_alloc_mem_size;
    uint64_t max_image2d_width;
    uint64_t max_image2d_height;
    uint8_t supports_fp16, supports_fp16_denorms, supports_subgroups_short, supports_image, supports_imad, supports_immad;
} cldnn_engine_info;

/* api/C/cldnn.h:193-201 */
typedef void (*cldnn_event_handler)(void*);
typedef struct { const char* name; uint64_t nanoseconds; } cldnn_profiling_interval;

/* ---- build options: api/C/cldnn.h:206-250 ---- */
typedef enum {
    cldnn_build_option_fusing, cldnn_build_option_optimize_data, cldnn_build_option_debug, cldnn_build_option_outputs,
    cldnn_build_option_tuning_config, cldnn_build_option_graph_dumps_dir, cldnn_build_option_learning_config,
    cldnn_build_option_detection_output_gpu
} cldnn_build_option_type;
typedef enum { cldnn_tuning_disabled, cldnn_tuning_use_cache, cldnn_tuning_tune_and_cache } cldnn_tuning_mode_type;
struct cldnn_tuning_config { const int32_t mode; const char* cache_file_path; };
typedef struct { int32_t type; const void* data; } cldnn_build_option;
typedef struct { cldnn_event event; cldnn_memory memory; } cldnn_network_output;

/* ---- memory formats: the values of cldnn_format_type (api/C/cldnn.h:271-317) this library accepts ---- */
typedef enum {
    cldnn_format_yxfb = 0, cldnn_format_byxf = 1, cldnn_format_bfyx = 2, cldnn_format_byxf_af32 = 21,
    cldnn_format_format_num = 35, cldnn_format_any = -1
} cldnn_format_type;

/* ---- element types: api/C/cldnn.h:360-368 (size in the low bits, 0x80 float, 0x40 unsigned) ---- */
typedef enum { cldnn_i8 = 1, cldnn_f16 = 2 | 0x80, cldnn_f32 = 4 | 0x80, cldnn_u8 = 1 | 0x40, cldnn_i32 = 4, cldnn_i64 = 8 } cldnn_data_type;

/* ---- tensor, padding, layout: api/C/cldnn.h:322-378.  sizes[]: batch, feature, x, y, z, two local dimensions ---- */
#define CLDNN_TENSOR_DIM_MAX 8
typedef struct { size_t batch_num, feature_num, spatial_num, local_num; int32_t sizes[CLDNN_TENSOR_DIM_MAX]; } cldnn_tensor;
typedef struct { cldnn_tensor lower_size, upper_size; float filling_value; } cldnn_padding;
typedef struct { size_t data_type; int32_t format; cldnn_tensor size; cldnn_padding padding; } cldnn_layout;

/* ---- small arrays: api/C/cldnn.h:381-415 ---- */
typedef struct { const float* data; size_t size; } cldnn_float_arr;
typedef struct { const cldnn_tensor* data; size_t size; } cldnn_tensor_arr;
typedef const struct cldnn_primitive_type* cldnn_primitive_type_id;
typedef const char* cldnn_primitive_id;
typedef struct { const cldnn_primitive_id* data; size_t size; } cldnn_primitive_id_arr;
typedef struct { cldnn_data_type data_type; char enabled; } cldnn_optional_data_type;

/* api/C/cldnn.h:445-475: the activation functions this library implements keep the reference's values */
typedef enum {
    activation_none = 0, activation_logistic = 1, activation_hyperbolic_tan = 2, activation_relu = 3, activation_relu_negative_slope = 4,
    activation_clamp = 5, activation_abs = 7, activation_linear = 8, activation_square = 9, activation_sqrt = 10, activation_elu = 11
} cldnn_activation_func;
typedef struct { float a, b; } cldnn_activation_additional_params;
typedef enum { mean_none, mean_subtract, mean_mul, mean_div } cldnn_reorder_mean_mode;

/* ---- primitive descriptors.  Every descriptor starts with the fields of api/C/cldnn.h:511-516 ---- */
#define CLDNN_DESC_HEAD                     \
    cldnn_primitive_type_id type;           \
    cldnn_primitive_id id;                  \
    cldnn_primitive_id_arr input;           \
    cldnn_padding output_padding;           \
    cldnn_optional_data_type output_data_type;

struct cldnn_primitive_desc { CLDNN_DESC_HEAD };

/* api/C/input_layout.h:35-38, api/C/data.h:35-38 */
struct cldnn_input_layout_desc { CLDNN_DESC_HEAD cldnn_layout layout; };
struct cldnn_data_desc { CLDNN_DESC_HEAD cldnn_memory mem; };

/* api/C/reorder.h:35-44 */
struct cldnn_reorder_desc {
    CLDNN_DESC_HEAD
    cldnn_format_type output_format;
    cldnn_primitive_id mean_subtract;
    cldnn_float_arr subtract_per_feature;
    cldnn_reorder_mean_mode mean_mode;
};

/* api/C/convolution.h:36-74.  One id per split in each array; input_offset is negative for zero padding. */
struct cldnn_convolution_desc {
    CLDNN_DESC_HEAD
    cldnn_tensor input_offset, stride, dilation;
    uint32_t with_activation;
    float activation_negative_slope;
    uint32_t split;
    uint32_t with_output_size;
    cldnn_tensor output_size;
    cldnn_primitive_id_arr weights, bias, weights_quantization_factors, output_calibration_factors;
    float input_quantization_factor, output_quantization_factor;
    uint32_t groups;
    cldnn_tensor padding_above, padding_below;
};

/* api_extension/C/fused_conv_eltwise.h:35-97 (a C++ structure in the reference: bool member, nested structs) */
struct cldnn_fused_conv_eltwise_desc {
    CLDNN_DESC_HEAD
    struct {
        cldnn_tensor input_offset, stride, dilation;
        uint32_t with_activation;
        float activation_negative_slope;
        uint32_t split;
        uint32_t with_output_size;
        cldnn_tensor output_size;
        cldnn_primitive_id_arr weights, bias, weights_quantization_factors, output_calibration_factors;
        float input_quantization_factor, output_quantization_factor;
    } conv;
    struct {
        cldnn_primitive_id output_calibration_factors;
        float output_quantization_factor;
        int32_t mode;                                     /* cldnn_eltwise_mode: only the sum is honoured */
        cldnn_float_arr coefficients;
        uint32_t with_activation;
        float activation_negative_slope;
        cldnn_tensor_arr stride;
    } eltw;
    float non_conv_scale;
    uint8_t second_input_in_output;                       /* `bool` in the reference */
};

/* api/C/eltwise.h:34-80 */
typedef enum { cldnn_eltwise_sum, cldnn_eltwise_sub, cldnn_eltwise_max, cldnn_eltwise_prod, cldnn_eltwise_div, cldnn_eltwise_min } cldnn_eltwise_mode;
struct cldnn_eltwise_desc {
    CLDNN_DESC_HEAD
    cldnn_primitive_id output_calibration_factors;
    float output_quantization_factor;
    int32_t mode;
    cldnn_float_arr coefficients;
    uint32_t with_activation;
    float activation_negative_slope;
    cldnn_tensor_arr stride;
};

/* api/C/activation.h:35-44 */
struct cldnn_activation_desc {
    CLDNN_DESC_HEAD
    cldnn_activation_func activation_func;
    cldnn_activation_additional_params additional_params;
    cldnn_primitive_id additional_params_input;
};

/* api/C/pooling.h:34-69 */
typedef enum { cldnn_pooling_max, cldnn_pooling_average, cldnn_pooling_average_no_padding, cldnn_pooling_max_with_argmax, cldnn_pooling_bilinear } cldnn_pooling_mode;
struct cldnn_pooling_desc {
    CLDNN_DESC_HEAD
    cldnn_primitive_id argmax;
    int32_t mode;
    int8_t global_pooling;
    cldnn_tensor input_offset, stride, size;
    uint32_t with_output_size;
    cldnn_tensor output_size;
};

/* api/C/fully_connected.h:35-56 */
struct cldnn_fully_connected_desc {
    CLDNN_DESC_HEAD
    uint32_t with_activation;
    float activation_negative_slope;
    cldnn_primitive_id weights, bias, weights_quantization_factors, output_calibration_factors;
    float input_quantization_factor, output_quantization_factor;
};

/* api/C/softmax.h:34-52 */
typedef enum { cldnn_softmax_normalize_f, cldnn_softmax_normalize_x, cldnn_softmax_normalize_y, cldnn_softmax_normalize_fyx } cldnn_softmax_dimension;
struct cldnn_softmax_desc { CLDNN_DESC_HEAD cldnn_softmax_dimension dimension; };

/* api/C/lrn.h:33-58 */
typedef enum { cldnn_lrn_norm_region_across_channel, cldnn_lrn_norm_region_within_channel } cldnn_lrn_norm_region;
struct cldnn_lrn_desc { CLDNN_DESC_HEAD uint32_t size; float k, alpha, beta; cldnn_lrn_norm_region norm_region; };

/* api/C/concatenation.h:33-62: the axis is the index into cldnn_tensor::sizes */
typedef enum { cldnn_concatenation_along_b = 0, cldnn_concatenation_along_f = 1, cldnn_concatenation_along_x = 2, cldnn_concatenation_along_y = 3, cldnn_concatenation_along_z = 4 } cldnn_concatenation_axis;
struct cldnn_concatenation_desc { CLDNN_DESC_HEAD cldnn_concatenation_axis axis; };

/* ---- entry points: api/C/cldnn.h:537-805 ---- */
CLDNN_API cldnn_version cldnn_get_version(cldnn_status* status);

CLDNN_API cldnn_topology cldnn_create_topology(cldnn_status* status);
CLDNN_API void cldnn_add_primitive(cldnn_topology topology, const struct cldnn_primitive_desc* dto, cldnn_status* status);
CLDNN_API void cldnn_change_input_layout(cldnn_topology topology, cldnn_primitive_id id, cldnn_layout new_layout, cldnn_status* status);
/* names are returned back to back, each ended by a zero, the list by one more zero; with too small a buffer the needed
 * size comes back in *size_ret and the status is CLDNN_INVALID_ARG (src/cldnn.cpp:110-150) */
CLDNN_API void cldnn_get_primitive_ids(cldnn_topology topology, char* ids, size_t size, size_t* size_ret, cldnn_status* status);
CLDNN_API void cldnn_retain_topology(cldnn_topology topology, cldnn_status* status);
CLDNN_API void cldnn_release_topology(cldnn_topology topology, cldnn_status* status);

CLDNN_API uint32_t cldnn_get_engine_count(int32_t type, cldnn_status* status);
CLDNN_API void cldnn_release_pending_memory(cldnn_engine engine, cldnn_status* status);
CLDNN_API cldnn_engine cldnn_create_engine(int32_t type, uint32_t engine_num, const cldnn_engine_configuration* configuration, cldnn_status* status);
CLDNN_API void cldnn_retain_engine(cldnn_engine engine, cldnn_status* status);
CLDNN_API void cldnn_release_engine(cldnn_engine engine, cldnn_status* status);
CLDNN_API cldnn_engine_info cldnn_get_engine_info(cldnn_engine engine, cldnn_status* status);
CLDNN_API int32_t cldnn_get_engine_type(cldnn_engine engine, cldnn_status* status);
CLDNN_API int64_t cldnn_get_temp_used_device_memory_size(cldnn_engine engine, cldnn_status* status);
CLDNN_API int64_t cldnn_get_max_used_device_memory_size(cldnn_engine engine, cldnn_status* status);

CLDNN_API cldnn_event cldnn_create_user_event(cldnn_engine engine, cldnn_status* status);
CLDNN_API int32_t cldnn_is_user_event(cldnn_event event, cldnn_status* status);
CLDNN_API void cldnn_retain_event(cldnn_event event, cldnn_status* status);
CLDNN_API void cldnn_release_event(cldnn_event event, cldnn_status* status);
CLDNN_API void cldnn_wait_for_event(cldnn_event event, cldnn_status* status);
CLDNN_API void cldnn_set_event(cldnn_event event, cldnn_status* status);
CLDNN_API void cldnn_add_event_handler(cldnn_event event, cldnn_event_handler handler, void* param, cldnn_status* status);
CLDNN_API void cldnn_get_event_profiling_info(cldnn_event event, cldnn_profiling_interval* profiling, size_t size, size_t* size_ret, cldnn_status* status);

CLDNN_API cldnn_program cldnn_build_program(cldnn_engine engine, cldnn_topology topology, cldnn_build_option* options, size_t options_num, cldnn_status* status);
CLDNN_API void cldnn_retain_program(cldnn_program program, cldnn_status* status);
CLDNN_API void cldnn_release_program(cldnn_program program, cldnn_status* status);

CLDNN_API cldnn_network cldnn_build_network(cldnn_engine engine, cldnn_topology topology, cldnn_build_option* options, size_t options_num, cldnn_status* status);
CLDNN_API cldnn_network cldnn_allocate_network(cldnn_program program, cldnn_status* status);
CLDNN_API void cldnn_retain_network(cldnn_network network, cldnn_status* status);
CLDNN_API void cldnn_release_network(cldnn_network network, cldnn_status* status);
CLDNN_API void cldnn_set_network_input(cldnn_network network, cldnn_primitive_id id, cldnn_memory mem, cldnn_status* status);
CLDNN_API void cldnn_set_learning_rate(cldnn_network network, float lr, cldnn_status* status);
CLDNN_API float cldnn_get_learning_rate(cldnn_network network, cldnn_status* status);
CLDNN_API void cldnn_get_primitive_info(cldnn_network network, cldnn_primitive_id id, char* info, size_t size, size_t* size_ret, cldnn_status* status);
CLDNN_API cldnn_engine cldnn_get_network_engine(cldnn_network network, cldnn_status* status);
CLDNN_API cldnn_program cldnn_get_network_program(cldnn_network network, cldnn_status* status);
CLDNN_API void cldnn_get_network_output_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status);
CLDNN_API void cldnn_get_network_executed_primitive_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status);
CLDNN_API void cldnn_get_network_all_primitive_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status);
CLDNN_API void cldnn_get_network_all_primitive_org_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status);
/* enqueues and returns; the caller waits on the event of a cldnn_network_output (api/C/cldnn.h:250-255) */
CLDNN_API void cldnn_execute_network(cldnn_network network, cldnn_event* dependencies, size_t deps_num, cldnn_status* status);
CLDNN_API cldnn_network_output cldnn_get_network_output(cldnn_network network, const char* name, cldnn_status* status);
CLDNN_API cldnn_memory cldnn_get_network_output_memory(cldnn_network network, const char* name, cldnn_status* status);
CLDNN_API cldnn_event cldnn_get_network_output_event(cldnn_network network, const char* name, cldnn_status* status);

CLDNN_API cldnn_memory cldnn_allocate_memory(cldnn_engine engine, cldnn_layout layout, cldnn_status* status);
/* wraps a host buffer of the caller, which must outlive the memory object (api/C/cldnn.h:770-772) */
CLDNN_API cldnn_memory cldnn_attach_memory(cldnn_layout layout, void* pointer, size_t size, cldnn_status* status);
CLDNN_API int32_t cldnn_is_the_same_buffer(cldnn_memory mem1, cldnn_memory mem2, cldnn_status* status);
CLDNN_API void cldnn_retain_memory(cldnn_memory memory, cldnn_status* status);
CLDNN_API void cldnn_release_memory(cldnn_memory memory, cldnn_status* status);
/* host view of the buffer, valid until the matching unlock; locks nest (api/C/cldnn.h:781-783) */
CLDNN_API void* cldnn_lock_memory(cldnn_memory memory, cldnn_status* status);
CLDNN_API void cldnn_unlock_memory(cldnn_memory memory, cldnn_status* status);
CLDNN_API cldnn_layout cldnn_get_memory_layout(cldnn_memory memory, cldnn_status* status);
CLDNN_API cldnn_engine cldnn_get_memory_engine(cldnn_memory memory, cldnn_status* status);

CLDNN_API uint16_t cldnn_float_to_half(float value, cldnn_status* status);
CLDNN_API float cldnn_half_to_float(uint16_t value, cldnn_status* status);
CLDNN_API const char* cldnn_get_last_error_message(void);

/* ---- primitive type identifiers: api/C/cldnn.h:814-819 and the DECLARE line of each api/C/<primitive>.h ---- */
CLDNN_API cldnn_primitive_type_id cldnn_input_layout_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_data_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_reorder_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_convolution_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_fused_conv_eltwise_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_eltwise_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_activation_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_pooling_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_fully_connected_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_softmax_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_lrn_type_id(cldnn_status* status);
CLDNN_API cldnn_primitive_type_id cldnn_concatenation_type_id(cldnn_status* status);

#ifdef __cplusplus
}
#endif
#endif /* CLDNN_C_API_H */
