// Prints the size of every structure of clDNN's public C boundary and the offset of every field this repository reads,
// plus the enumeration values it relies on.  Compiled twice by the tests: against include/cldnn_c_api.h of this repository,
// and (with -DUSE_REFERENCE_HEADERS and -I<clDNN tree>) against the reference's own api/C headers; the two outputs must
// be identical, and equal to tests/golden/cldnn_c_abi_layout.txt.
#include <cstddef>
#include <cstdio>
#ifdef USE_REFERENCE_HEADERS
#include "api/C/cldnn.h"
#include "api/C/convolution.h"
#include "api_extension/C/fused_conv_eltwise.h"
#include "api/C/pooling.h"
#include "api/C/fully_connected.h"
#include "api/C/softmax.h"
#include "api/C/eltwise.h"
#include "api/C/reorder.h"
#include "api/C/activation.h"
#include "api/C/lrn.h"
#include "api/C/data.h"
#include "api/C/input_layout.h"
#include "api/C/concatenation.h"
#else
#include "cldnn_c_api.h"
#endif

#define S(T) std::printf("sizeof %s %zu\n", #T, sizeof(T))
#define O(T, f) std::printf("offsetof %s.%s %zu\n", #T, #f, offsetof(T, f))
#define V(e) std::printf("value %s %d\n", #e, (int)(e))

int main()
{
    V(CLDNN_SUCCESS); V(CLDNN_ERROR); V(CLDNN_INVALID_ARG); V(CLDNN_OUT_OF_RESOURCES); V(CLDNN_DEVICE_ERROR); V(CLDNN_UNSUPPORTED_SIZE);
    V(CLDNN_UNSUPPORTED_FORMAT); V(CLDNN_DIMENSION_MISMATCH); V(CLDNN_ALLOC_SIZE_EXCEEDED); V(CLDNN_GLOBAL_SIZE_EXCEEDED);
    V(cldnn_format_yxfb); V(cldnn_format_byxf); V(cldnn_format_bfyx); V(cldnn_format_byxf_af32); V(cldnn_format_format_num); V(cldnn_format_any);
    V(cldnn_i8); V(cldnn_f16); V(cldnn_f32); V(cldnn_u8); V(cldnn_i32); V(cldnn_i64);
    V(cldnn_build_option_fusing); V(cldnn_build_option_optimize_data); V(cldnn_build_option_outputs); V(cldnn_build_option_tuning_config);
    V(cldnn_build_option_detection_output_gpu); V(cldnn_tuning_tune_and_cache);
    V(activation_none); V(activation_logistic); V(activation_hyperbolic_tan); V(activation_abs); V(activation_linear); V(activation_square); V(activation_sqrt); V(activation_elu); V(activation_relu); V(activation_relu_negative_slope); V(activation_clamp); V(mean_subtract);
    V(cldnn_eltwise_sum); V(cldnn_eltwise_sub); V(cldnn_eltwise_max); V(cldnn_eltwise_prod); V(cldnn_eltwise_div); V(cldnn_eltwise_min);
    V(cldnn_pooling_max); V(cldnn_pooling_average); V(cldnn_pooling_average_no_padding); V(cldnn_pooling_max_with_argmax);
    V(cldnn_softmax_normalize_f); V(cldnn_softmax_normalize_fyx); V(cldnn_lrn_norm_region_across_channel);
    V(cldnn_concatenation_along_b); V(cldnn_concatenation_along_f); V(cldnn_concatenation_along_x); V(cldnn_concatenation_along_y);
    V(CLDNN_TENSOR_DIM_MAX);
    S(cldnn_version); S(cldnn_tensor); S(cldnn_padding); S(cldnn_layout); S(cldnn_engine_configuration); S(cldnn_engine_info); S(cldnn_build_option);
    S(cldnn_tuning_config); S(cldnn_network_output); S(cldnn_profiling_interval); S(cldnn_float_arr); S(cldnn_tensor_arr); S(cldnn_primitive_id_arr);
    S(cldnn_optional_data_type); S(cldnn_activation_additional_params);
    S(cldnn_primitive_desc); S(cldnn_convolution_desc); S(cldnn_fused_conv_eltwise_desc); S(cldnn_pooling_desc); S(cldnn_fully_connected_desc);
    S(cldnn_softmax_desc); S(cldnn_eltwise_desc); S(cldnn_reorder_desc); S(cldnn_activation_desc); S(cldnn_lrn_desc); S(cldnn_data_desc);
    S(cldnn_input_layout_desc); S(cldnn_concatenation_desc);
    O(cldnn_tensor, sizes); O(cldnn_padding, upper_size); O(cldnn_padding, filling_value); O(cldnn_layout, format); O(cldnn_layout, size); O(cldnn_layout, padding);
    O(cldnn_engine_configuration, enable_profiling); O(cldnn_engine_configuration, compiler_options); O(cldnn_engine_configuration, priority_mode);
    O(cldnn_engine_configuration, context); O(cldnn_engine_configuration, tuning_cache_path);
    O(cldnn_engine_info, cores_count); O(cldnn_engine_info, core_frequency); O(cldnn_engine_info, max_alloc_mem_size); O(cldnn_engine_info, supports_fp16);
    O(cldnn_engine_info, supports_immad);
    O(cldnn_primitive_desc, type); O(cldnn_primitive_desc, id); O(cldnn_primitive_desc, input); O(cldnn_primitive_desc, output_padding); O(cldnn_primitive_desc, output_data_type);
    O(cldnn_convolution_desc, input_offset); O(cldnn_convolution_desc, stride); O(cldnn_convolution_desc, dilation); O(cldnn_convolution_desc, with_activation);
    O(cldnn_convolution_desc, activation_negative_slope); O(cldnn_convolution_desc, split); O(cldnn_convolution_desc, with_output_size); O(cldnn_convolution_desc, output_size);
    O(cldnn_convolution_desc, weights); O(cldnn_convolution_desc, bias); O(cldnn_convolution_desc, weights_quantization_factors);
    O(cldnn_convolution_desc, output_calibration_factors); O(cldnn_convolution_desc, input_quantization_factor); O(cldnn_convolution_desc, output_quantization_factor);
    O(cldnn_convolution_desc, groups); O(cldnn_convolution_desc, padding_above); O(cldnn_convolution_desc, padding_below);
    O(cldnn_fused_conv_eltwise_desc, conv); O(cldnn_fused_conv_eltwise_desc, conv.weights); O(cldnn_fused_conv_eltwise_desc, conv.output_quantization_factor);
    O(cldnn_fused_conv_eltwise_desc, eltw); O(cldnn_fused_conv_eltwise_desc, eltw.mode); O(cldnn_fused_conv_eltwise_desc, eltw.coefficients);
    O(cldnn_fused_conv_eltwise_desc, eltw.with_activation); O(cldnn_fused_conv_eltwise_desc, eltw.stride); O(cldnn_fused_conv_eltwise_desc, non_conv_scale);
    O(cldnn_fused_conv_eltwise_desc, second_input_in_output);
    O(cldnn_pooling_desc, argmax); O(cldnn_pooling_desc, mode); O(cldnn_pooling_desc, global_pooling); O(cldnn_pooling_desc, input_offset); O(cldnn_pooling_desc, stride);
    O(cldnn_pooling_desc, size); O(cldnn_pooling_desc, with_output_size); O(cldnn_pooling_desc, output_size);
    O(cldnn_fully_connected_desc, with_activation); O(cldnn_fully_connected_desc, weights); O(cldnn_fully_connected_desc, bias);
    O(cldnn_fully_connected_desc, weights_quantization_factors); O(cldnn_fully_connected_desc, output_calibration_factors);
    O(cldnn_fully_connected_desc, input_quantization_factor); O(cldnn_fully_connected_desc, output_quantization_factor);
    O(cldnn_eltwise_desc, output_calibration_factors); O(cldnn_eltwise_desc, output_quantization_factor); O(cldnn_eltwise_desc, mode); O(cldnn_eltwise_desc, coefficients);
    O(cldnn_eltwise_desc, with_activation); O(cldnn_eltwise_desc, activation_negative_slope); O(cldnn_eltwise_desc, stride);
    O(cldnn_reorder_desc, output_format); O(cldnn_reorder_desc, mean_subtract); O(cldnn_reorder_desc, subtract_per_feature); O(cldnn_reorder_desc, mean_mode);
    O(cldnn_activation_desc, activation_func); O(cldnn_activation_desc, additional_params); O(cldnn_activation_desc, additional_params_input);
    O(cldnn_lrn_desc, size); O(cldnn_lrn_desc, k); O(cldnn_lrn_desc, alpha); O(cldnn_lrn_desc, beta); O(cldnn_lrn_desc, norm_region);
    O(cldnn_softmax_desc, dimension); O(cldnn_data_desc, mem); O(cldnn_input_layout_desc, layout); O(cldnn_concatenation_desc, axis);
    return 0;
}
