// Host side of the B200 engine: a C++ mirror of the part of clDNN's public API
// and graph core that the convolution hot path needs -- engine, memory, layout,
// topology of primitives, program build (fusing, layout selection, weights
// pre-packing, kernel selection / tuning) and network execution.  Names and
// argument meaning follow the reference (api/CPP/*.hpp, api_extension/CPP/
// fused_conv_eltwise.hpp); the implementation is new and sits on the C ABI of
// include/cldnn_b200.h -- it never touches CUDA directly.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../include/cldnn_b200.h"

namespace cldnn {

// error carrying a cldnn_status-compatible code (api/CPP/cldnn_defs.h `cldnn::error`)
struct error : std::runtime_error {
    int32_t status;
    error(const std::string& msg, int32_t st = CLDNN_B200_ERROR) : std::runtime_error(msg), status(st) {}
};

enum class data_types : int32_t { none = CLDNN_B200_NONE, i8 = CLDNN_B200_I8, u8 = CLDNN_B200_U8, i32 = CLDNN_B200_I32,
                                  f16 = CLDNN_B200_F16, f32 = CLDNN_B200_F32 };

// activation / weights memory formats (values of cldnn_format_type, api/C/cldnn.h:271-317)
struct format {
    enum type : int32_t { yxfb = 0, byxf = 1, bfyx = 2, byxf_af32 = 21, any = -1 };
    static const char* name(int32_t f);
};

// cldnn::tensor(batch, feature, x, y) -- api/CPP/tensor.hpp
struct tensor {
    int32_t batch = 1, feature = 1, x = 1, y = 1;
    tensor() {}
    tensor(int32_t b, int32_t f, int32_t x_, int32_t y_) : batch(b), feature(f), x(x_), y(y_) {}
    bool operator==(const tensor& o) const { return batch == o.batch && feature == o.feature && x == o.x && y == o.y; }
};

// spatial padding kept inside a buffer around the data (cldnn::padding, api/CPP/layout.hpp)
struct padding {
    int32_t lower_x = 0, lower_y = 0, upper_x = 0, upper_y = 0;
};

struct layout {
    data_types data_type = data_types::f32;
    int32_t fmt = format::bfyx;
    tensor size;
    padding data_padding;
    layout() {}
    layout(data_types dt, int32_t f, const tensor& s, const padding& p = padding()) : data_type(dt), fmt(f), size(s), data_padding(p) {}
    int32_t stored_features() const;            // feature count including format alignment
    size_t count() const;                       // elements in the buffer, padding included
    size_t bytes_count() const;
    cldnn_b200_tensor desc() const;             // pitches / offset as the kernels see them
    bool operator==(const layout& o) const;
};

class engine_impl;
class memory_impl;
class network_impl;

// cldnn::engine -- api/CPP/engine.hpp:55-200
class engine {
public:
    explicit engine(int32_t device = 0, bool enable_profiling = false);
    cldnn_b200_engine_info get_info() const;
    void* stream() const;                       // cudaStream_t of the engine's queue
    void sync() const;                          // waits for everything enqueued on the engine's queue
    uint32_t device_status() const;             // non-zero after a kernel gave up a bounded wait
    bool profiling() const;
    std::shared_ptr<engine_impl> impl;
};

// cldnn::memory -- api/CPP/memory.hpp
class memory {
public:
    memory() {}
    static memory allocate(const engine& e, const layout& l);
    // cldnn::memory::attach for device memory: the caller owns `device_ptr` and keeps it alive
    static memory attach(const engine& e, const layout& l, void* device_ptr);
    const layout& get_layout() const;
    size_t size() const;
    void write(const void* host, size_t bytes);         // set_values
    void read(void* host, size_t bytes) const;          // pointer<T>() read-back
    void* device_ptr() const;
    explicit operator bool() const { return (bool)impl; }
    std::shared_ptr<memory_impl> impl;
};

enum class eltwise_mode : int32_t { sum = CLDNN_B200_ELTW_SUM, sub = CLDNN_B200_ELTW_SUB, max = CLDNN_B200_ELTW_MAX,
                                    prod = CLDNN_B200_ELTW_PROD, min = CLDNN_B200_ELTW_MIN };
enum class pooling_mode : int32_t { max = 0, average = 1, average_no_padding = 2 };
enum class tuning_mode : int32_t { tuning_disabled = 0, tuning_use_cache = 1, tuning_tune_and_cache = 2 };

// One primitive of a topology.  `type` is the reference's primitive name; the
// fields are the union of the descriptors used on the hot path:
//   convolution          api/CPP/convolution.hpp:34-962
//   fused_conv_eltwise   api_extension/CPP/fused_conv_eltwise.hpp:33-281
//   eltwise              api/CPP/eltwise.hpp
//   activation           api/CPP/activation.hpp
//   pooling              api/CPP/pooling.hpp
//   fully_connected      api/CPP/fully_connected.hpp
//   softmax, lrn, reorder, concatenation (api/CPP/concatenation.hpp), data, input_layout
struct primitive {
    std::string type, id;
    std::vector<std::string> input;
    std::string weights, bias, weights_quantization_factors, output_calibration_factors, eltw_output_calibration_factors;
    float input_quantization_factor = 1.0f, output_quantization_factor = 1.0f;
    float non_conv_scale = 1.0f;
    tensor stride{1, 1, 1, 1}, input_offset{0, 0, 0, 0}, dilation{1, 1, 1, 1}, eltw_stride{1, 1, 1, 1};
    int32_t groups = 1;
    bool with_activation = false; float activation_negative_slope = 0.0f;
    bool eltw_activation = false; float eltw_activation_negative_slope = 0.0f;
    bool second_input_in_output = false;
    bool eltw_quantized = false;                          // eltwise: int8 requantising form (QUANTIZATION_TERM)
    data_types output_data_type = data_types::none;       // optional explicit output precision
    // eltwise / activation / pooling / lrn / reorder specifics
    eltwise_mode mode = eltwise_mode::sum;
    int32_t activation_func = CLDNN_B200_ACT_NONE; float act_a = 0.0f, act_b = 0.0f;
    pooling_mode pool_mode = pooling_mode::max; tensor size{1, 1, 1, 1}; bool global_pooling = false;
    uint32_t lrn_size = 5; float lrn_k = 1.0f, lrn_alpha = 1e-4f, lrn_beta = 0.75f;
    int32_t concat_axis = 1;                                        // concatenation: index into tensor sizes (0 batch, 1 feature, 2 x, 3 y), api/C/concatenation.h:33-40
    int32_t softmax_dimension = 3;                                  // softmax::dimension_t: normalize_f 0, _x 1, _y 2, _fyx 3 (the default, api/CPP/softmax.hpp:59)
    layout target;                                        // reorder output layout / input_layout layout
    std::vector<float> subtract_per_feature;              // reorder mean values
    memory mem;                                           // data
};

// constructors with the reference's argument order
primitive input_layout(const std::string& id, const layout& l);
primitive data(const std::string& id, const memory& m);
primitive reorder(const std::string& id, const std::string& input, int32_t out_format, data_types out_type,
                  const std::vector<float>& subtract_per_feature = {});
primitive convolution(const std::string& id, const std::string& input, const std::string& weights, const std::string& bias,
                      const std::string& w_quantization_factor, const std::string& output_calibration_factors,
                      float i_quantization_factor, data_types output_data_type, tensor stride = {1, 1, 1, 1},
                      tensor input_offset = {0, 0, 0, 0}, tensor dilation = {1, 1, 1, 1}, bool with_activation = false,
                      float activation_slp = 0.0f, int32_t groups = 1);
primitive fused_conv_eltwise(const std::string& id, const std::string& input, const std::string& input2, eltwise_mode mode,
                             const std::string& weights, const std::string& bias, const std::string& conv_w_quantization_factor,
                             const std::string& conv_output_calibration_factors, float conv_i_quantization_factor,
                             float non_conv_scale, const std::string& eltw_output_calibration_factors, tensor eltw_stride,
                             tensor stride, tensor input_offset, tensor dilation, bool conv_with_activation, float conv_activation_slp,
                             bool eltw_activation, float eltw_activation_slp, data_types output_data_type = data_types::none);
primitive eltwise(const std::string& id, const std::string& input, const std::string& input2, eltwise_mode mode,
                  bool with_activation = false, float activation_slp = 0.0f, const std::string& output_calibration_factors = "",
                  float output_quantization_factor = 1.0f, bool quantized = false);
primitive activation(const std::string& id, const std::string& input, int32_t func, float a = 0.0f, float b = 0.0f);
primitive pooling(const std::string& id, const std::string& input, pooling_mode mode, tensor size, tensor stride,
                  tensor input_offset = {0, 0, 0, 0});
primitive global_pooling(const std::string& id, const std::string& input, pooling_mode mode);
primitive fully_connected(const std::string& id, const std::string& input, const std::string& weights, const std::string& bias,
                          const std::string& w_quantization_factor, const std::string& output_calibration_factors,
                          float i_quantization_factor, bool with_activation = false, float activation_slp = 0.0f);
enum softmax_dimension : int32_t { normalize_f = 0, normalize_x = 1, normalize_y = 2, normalize_fyx = 3 };   // api/CPP/softmax.hpp:44-50
primitive softmax(const std::string& id, const std::string& input, int32_t dimension = normalize_fyx);
primitive lrn(const std::string& id, const std::string& input, uint32_t size, float k, float alpha, float beta);
enum concatenation_axis : int32_t { along_b = 0, along_f = 1, along_x = 2, along_y = 3 };
primitive concatenation(const std::string& id, const std::vector<std::string>& inputs, int32_t axis);

// cldnn::topology -- api/CPP/topology.hpp
class topology {
public:
    topology() {}
    template <class... Ps> explicit topology(const Ps&... ps) { (add(ps), ...); }
    void add(const primitive& p);
    const std::vector<primitive>& primitives() const { return prims; }
private:
    std::vector<primitive> prims;
};

// cldnn::build_options -- api/CPP/program.hpp:108-138 (the options the hot path reads)
struct build_options {
    bool optimize_data = false;                 // fusing + layout optimisation + weights pre-packing
    bool fuse_any_conv_eltwise = true;          // lift the reference's 1x1 / stride-1 restriction on conv+eltwise fusing
    bool conv_eltw_read_write_opt = true;       // a fused_conv_eltwise writes its result over its second input where that is safe
    tuning_mode tuning = tuning_mode::tuning_disabled;
    std::string tuning_cache_path;              // JSON: { "<SM count>": { "<params hash>": ["kernel", tune_index] } }
    std::vector<std::string> outputs;           // empty: every primitive without users
    bool use_graph = true;                      // replay the execution order as one CUDA graph launch
    std::string force_kernel;                   // debugging: "<primitive id>=<kernel name>[:tune],..."
};

struct primitive_info {
    std::string id, type, original_ids, kernel; int32_t tune = 0; layout output; bool is_output = false;
    bool in_place = false;                      // fused_conv_eltwise: the result overwrites the second input's buffer
};

// cldnn::network -- api/CPP/network.hpp
class network {
public:
    network() {}
    network(const engine& e, const topology& t, const build_options& o = build_options());
    void set_input_data(const std::string& id, const memory& m);
    void execute();                             // enqueue; returns immediately
    memory get_output(const std::string& id);   // waits for completion, returns the primitive's memory
    memory output_memory(const std::string& id) const;   // the same memory object without waiting (the caller waits on the event)
    std::vector<std::string> get_output_ids() const;
    std::vector<primitive_info> get_primitives_info() const;   // executed order, with chosen kernels
    uint64_t launches_per_execute() const;
    // per-primitive device time of the last execute() when the engine was created with profiling enabled
    // (event::get_profiling_info of the reference, src/gpu/ocl_base_event.cpp:68-92): (primitive id, nanoseconds)
    std::vector<std::pair<std::string, uint64_t>> get_profiling_info() const;
    size_t device_memory_bytes() const;         // bytes held by the memory pool for intermediates
    void wait();
    std::shared_ptr<network_impl> impl;
};

// The tuning cache file as text -> { "<compute units>": { "<hash>": (kernel, tuning index) } }; throws `error` on malformed JSON
// or on entries that are not ["kernel", index] (the schema of the reference's cache.json, auto_tuner.cpp:72-118).
std::map<std::string, std::map<std::string, std::pair<std::string, int>>> parse_tuning_cache(const std::string& text);

// output spatial size of a sliding window; convolution: src/include/sliding_window_utils.h:87-124 (range mode `all`),
// pooling: :126-230 + src/pooling.cpp:91-92 (range mode `exceed_once_data`)
int32_t conv_output_size(int32_t in, int32_t filter, int32_t input_offset, int32_t stride, int32_t dilation);
int32_t pool_output_size(int32_t in, int32_t window, int32_t input_offset, int32_t stride);

}  // namespace cldnn
