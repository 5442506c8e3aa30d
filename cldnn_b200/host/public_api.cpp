// libclDNN64.so: clDNN's public C boundary (api/C/cldnn.h:537-805 and the api/C/<primitive>.h descriptors) on top of the
// B200 host layer, so that code written against the reference's headers -- its header-only C++ API included -- links and
// runs unchanged on the convolution hot path.  Conventions follow src/cldnn.cpp and src/include/api_impl.h:60-150:
// every call resets *status to CLDNN_SUCCESS, failures come back as a status code plus a thread-local message, handles
// are reference counted.  Primitive types outside the hot path are refused with CLDNN_UNSUPPORTED_FORMAT.
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <mutex>
#include <sstream>
#include "../../include/cldnn_c_api.h"
#include "cldnn_host.hpp"

namespace host = cldnn;

namespace {

thread_local std::string g_last_error;

struct api_error : std::runtime_error {
    cldnn_status status;
    api_error(const std::string& m, cldnn_status s) : std::runtime_error(m), status(s) {}
};
[[noreturn]] void refuse(const std::string& what, cldnn_status st = CLDNN_UNSUPPORTED_FORMAT) { throw api_error(what, st); }

template <class T>
T guarded(cldnn_status* status, const T& fallback, const std::function<T()>& fn)
{
    if (status) *status = CLDNN_SUCCESS;
    try { return fn(); }
    catch (const api_error& e) { if (status) *status = e.status; g_last_error = e.what(); }
    catch (const host::error& e) { if (status) *status = e.status; g_last_error = e.what(); }
    catch (const std::exception& e) { if (status) *status = CLDNN_ERROR; g_last_error = e.what(); }
    catch (...) { if (status) *status = CLDNN_ERROR; g_last_error = "error unknown"; }
    return fallback;
}
void guarded(cldnn_status* status, const std::function<void()>& fn)
{
    guarded<int>(status, 0, [&]() { fn(); return 0; });
}
template <class P> void not_null(P p, const char* what) { if (!p) throw api_error(std::string(what) + " should not be null.", CLDNN_ERROR); }

struct refcounted {
    std::atomic<int> refs{1};
    virtual ~refcounted() {}
    void retain() { ++refs; }
    void release() { if (--refs == 0) delete this; }
};

std::string str(const char* s) { return s ? s : ""; }

// ---- layout translation -----------------------------------------------------------------------------------------------
int32_t spatial(const cldnn_tensor& t, int i) { return t.sizes[2 + i]; }

host::tensor to_host_tensor(const cldnn_tensor& t, int32_t neutral, const char* what)
{
    // batch, feature, x, y; a third spatial dimension and local dimensions are outside this path
    if (t.sizes[4] != neutral && t.sizes[4] != 1 && t.sizes[4] != 0) refuse(std::string(what) + ": 3-D tensors are not supported", CLDNN_UNSUPPORTED_SIZE);
    return host::tensor(t.sizes[0], t.sizes[1], spatial(t, 0), spatial(t, 1));
}
cldnn_tensor to_c_tensor(const host::tensor& t, int32_t fill)
{
    cldnn_tensor c{};
    c.batch_num = 1; c.feature_num = 1; c.spatial_num = 3; c.local_num = 2;
    for (int i = 0; i < CLDNN_TENSOR_DIM_MAX; ++i) c.sizes[i] = fill;
    c.sizes[0] = t.batch; c.sizes[1] = t.feature; c.sizes[2] = t.x; c.sizes[3] = t.y;
    return c;
}
// batch, feature, x, y: the dimensions this path knows (the reference's tensor(b, f, x, y) leaves the others at a default of 1)
bool no_padding(const cldnn_padding& p)
{
    for (int i = 0; i < 4; ++i) if (p.lower_size.sizes[i] || p.upper_size.sizes[i]) return false;
    return true;
}
host::data_types to_host_type(size_t dt)
{
    switch (dt) {
    case cldnn_i8: return host::data_types::i8;   case cldnn_u8: return host::data_types::u8;
    case cldnn_i32: return host::data_types::i32; case cldnn_f16: return host::data_types::f16;
    case cldnn_f32: return host::data_types::f32;
    }
    refuse("data type " + std::to_string(dt) + " is not supported on this path");
}
int32_t to_host_format(int32_t f)
{
    switch (f) {
    case cldnn_format_yxfb: return host::format::yxfb;   case cldnn_format_byxf: return host::format::byxf;
    case cldnn_format_bfyx: return host::format::bfyx;   case cldnn_format_byxf_af32: return host::format::byxf_af32;
    case cldnn_format_any: return host::format::any;
    }
    refuse("memory format " + std::to_string(f) + " is not supported on this path (yxfb, byxf, bfyx, byxf_af32)");
}
host::layout to_host_layout(const cldnn_layout& l)
{
    if (l.format < cldnn_format_any || l.format >= cldnn_format_format_num) throw api_error("Unknown format of layout.", CLDNN_ERROR);
    host::padding pad;
    const cldnn_padding& p = l.padding;
    if (p.lower_size.sizes[0] || p.lower_size.sizes[1] || p.upper_size.sizes[0] || p.upper_size.sizes[1])
        refuse("layout: batch / feature padding is not supported", CLDNN_UNSUPPORTED_SIZE);
    pad.lower_x = p.lower_size.sizes[2]; pad.lower_y = p.lower_size.sizes[3]; pad.upper_x = p.upper_size.sizes[2]; pad.upper_y = p.upper_size.sizes[3];
    return host::layout(to_host_type(l.data_type), to_host_format(l.format), to_host_tensor(l.size, 1, "layout"), pad);
}
cldnn_layout to_c_layout(const host::layout& l)
{
    cldnn_layout c{};
    c.data_type = (size_t)(int32_t)l.data_type;                // same codes as cldnn_data_type
    c.format = l.fmt;
    c.size = to_c_tensor(l.size, 1);
    c.padding.lower_size = to_c_tensor(host::tensor(0, 0, l.data_padding.lower_x, l.data_padding.lower_y), 0);
    c.padding.upper_size = to_c_tensor(host::tensor(0, 0, l.data_padding.upper_x, l.data_padding.upper_y), 0);
    c.padding.filling_value = 0.0f;
    return c;
}

}  // namespace

// ---- handle types ---------------------------------------------------------------------------------------------------------
struct cldnn_engine_impl : refcounted {
    host::engine eng;
    bool profiling;
    std::string tuning_cache_path;
    explicit cldnn_engine_impl(int32_t device, bool prof) : eng(device, prof), profiling(prof) {}
};

struct cldnn_memory_impl : refcounted {
    cldnn_layout lay{};
    cldnn_engine owner = nullptr;            // retained; null for a host buffer attached by the caller
    host::memory dev;                        // device memory (owner != null)
    void* attached = nullptr;                // caller's host buffer (owner == null)
    std::mutex lock_mutex;
    int locks = 0;
    std::vector<uint8_t> staging;            // host view while locked
    ~cldnn_memory_impl() override { if (owner) owner->release(); }
    size_t bytes() const { return owner ? dev.size() : to_host_layout(lay).bytes_count(); }
};

// one primitive of a topology: the host-layer description plus, for `data`, the memory object it refers to
struct topo_entry {
    host::primitive prim;
    cldnn_memory mem = nullptr;              // retained
};
struct cldnn_topology_impl : refcounted {
    std::vector<topo_entry> entries;
    ~cldnn_topology_impl() override { for (auto& e : entries) if (e.mem) e.mem->release(); }
};

struct cldnn_program_impl : refcounted {
    cldnn_engine eng;                        // retained
    host::topology topo;                     // constants resolved to device memory of `eng`
    host::build_options opts;
    std::vector<std::string> org_ids;        // ids of the topology, in the order they were added
    std::vector<cldnn_memory> keep;          // memory objects of the data primitives, retained
    std::unique_ptr<host::network> first;    // built by cldnn_build_program (validation happens there), handed to the first network
    ~cldnn_program_impl() override { first.reset(); for (auto m : keep) m->release(); eng->release(); }
};

struct cldnn_network_impl : refcounted {
    cldnn_program prog;                      // retained
    std::unique_ptr<host::network> net;
    std::map<std::string, cldnn_memory> inputs;      // bound inputs, retained
    std::map<std::string, cldnn_memory> staged;      // device copies of host buffers attached as inputs, retained
    ~cldnn_network_impl() override
    {
        net.reset();
        for (auto& kv : inputs) kv.second->release();
        for (auto& kv : staged) kv.second->release();
        prog->release();
    }
};

struct cldnn_event_impl : refcounted {
    cldnn_engine eng = nullptr;              // retained
    cldnn_network net = nullptr;             // retained: the execution this event stands for (null for a user event)
    std::string primitive;                   // output primitive the event belongs to
    bool user = false;
    std::mutex m; std::condition_variable cv; bool is_set = false;
    std::vector<std::pair<cldnn_event_handler, void*>> handlers;
    ~cldnn_event_impl() override { if (net) net->release(); if (eng) eng->release(); }
};

// ---- primitive types: cldnn_<primitive>_type_id() returns the address of one of these (api/C/cldnn.h:814-819); the
// descriptor -> primitive conversion is the registered part, the role of primitive_type::from_dto (src/include/primitive_type.h)
struct cldnn_primitive_type {
    const char* name;
    void (*from_dto)(const cldnn_primitive_desc* dto, topo_entry& out);
};

namespace {

std::vector<std::string> ids_of(const cldnn_primitive_id_arr& a)
{
    std::vector<std::string> v;
    for (size_t i = 0; i < a.size; ++i) v.push_back(str(a.data[i]));
    return v;
}
std::string single_id(const cldnn_primitive_id_arr& a, const std::string& who, const char* what)
{
    if (a.size == 0) return "";
    if (a.size != 1) refuse(who + ": " + what + " given per split; split convolutions are expressed with `groups` here", CLDNN_UNSUPPORTED_SIZE);
    return str(a.data[0]);
}
void common_head(const cldnn_primitive_desc* d, host::primitive& p, size_t inputs_min, size_t inputs_max)
{
    p.id = str(d->id);
    p.input = ids_of(d->input);
    if (p.input.size() < inputs_min || p.input.size() > inputs_max)
        refuse(p.id + ": " + std::to_string(p.input.size()) + " inputs (between " + std::to_string(inputs_min) + " and " + std::to_string(inputs_max) + " are supported)", CLDNN_INVALID_ARG);
    if (!no_padding(d->output_padding)) refuse(p.id + ": output padding is not supported", CLDNN_UNSUPPORTED_SIZE);
    p.output_data_type = d->output_data_type.enabled ? to_host_type((size_t)d->output_data_type.data_type) : host::data_types::none;
}
bool all_ones(const cldnn_tensor& t) { return spatial(t, 0) == 1 && spatial(t, 1) == 1; }
bool all_zero(const cldnn_tensor& t) { return spatial(t, 0) == 0 && spatial(t, 1) == 0; }

int32_t activation_of(int32_t func, const std::string& id)
{
    switch (func) {
    case activation_none: return CLDNN_B200_ACT_NONE;
    case activation_relu: return CLDNN_B200_ACT_RELU;
    case activation_relu_negative_slope: return CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE;
    case activation_clamp: return CLDNN_B200_ACT_CLAMP;
    case activation_logistic: return CLDNN_B200_ACT_LOGISTIC;
    case activation_hyperbolic_tan: return CLDNN_B200_ACT_TANH;
    case activation_abs: return CLDNN_B200_ACT_ABS;
    case activation_linear: return CLDNN_B200_ACT_LINEAR;
    case activation_square: return CLDNN_B200_ACT_SQUARE;
    case activation_sqrt: return CLDNN_B200_ACT_SQRT;
    case activation_elu: return CLDNN_B200_ACT_ELU;
    }
    refuse(id + ": activation function " + std::to_string(func) + " is not supported on this path");
}

void dto_input_layout(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_input_layout_desc*>(d);
    common_head(d, out.prim, 0, 0);
    out.prim.type = "input_layout";
    out.prim.target = to_host_layout(x->layout);
}
void dto_data(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_data_desc*>(d);
    common_head(d, out.prim, 0, 0);
    not_null(x->mem, "Data memory");
    out.prim.type = "data";
    out.mem = x->mem; out.mem->retain();
}
void dto_reorder(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_reorder_desc*>(d);
    host::primitive p; common_head(d, p, 1, 1);
    if (!str(x->mean_subtract).empty()) refuse(p.id + ": mean subtraction from a primitive is not supported; use subtract_per_feature");
    std::vector<float> sub(x->subtract_per_feature.data, x->subtract_per_feature.data + x->subtract_per_feature.size);
    if (!sub.empty() && x->mean_mode != mean_subtract) refuse(p.id + ": only the subtracting mean mode is supported");
    out.prim = host::reorder(p.id, p.input[0], to_host_format(x->output_format), p.output_data_type, sub);
}
void dto_convolution(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_convolution_desc*>(d);
    host::primitive h; common_head(d, h, 1, 1);
    if (x->with_output_size) refuse(h.id + ": a user-defined output size is not supported", CLDNN_UNSUPPORTED_SIZE);
    if (!all_zero(x->padding_above) || !all_zero(x->padding_below)) refuse(h.id + ": asymmetric padding is not supported", CLDNN_UNSUPPORTED_SIZE);
    if (x->split > 1) refuse(h.id + ": split > 1 is expressed with `groups` on this path", CLDNN_UNSUPPORTED_SIZE);
    host::primitive p = host::convolution(h.id, h.input[0], single_id(x->weights, h.id, "weights"), single_id(x->bias, h.id, "bias"),
                                          single_id(x->weights_quantization_factors, h.id, "quantization factors"),
                                          single_id(x->output_calibration_factors, h.id, "calibration factors"), x->input_quantization_factor,
                                          h.output_data_type, to_host_tensor(x->stride, 1, "stride"), to_host_tensor(x->input_offset, 0, "input_offset"),
                                          to_host_tensor(x->dilation, 1, "dilation"), x->with_activation != 0, x->activation_negative_slope,
                                          x->groups ? (int32_t)x->groups : 1);
    p.output_quantization_factor = x->output_quantization_factor;
    out.prim = p;
}
void dto_fused_conv_eltwise(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_fused_conv_eltwise_desc*>(d);
    host::primitive h; common_head(d, h, 2, 2);
    const auto& c = x->conv; const auto& e = x->eltw;
    if (c.with_output_size) refuse(h.id + ": a user-defined output size is not supported", CLDNN_UNSUPPORTED_SIZE);
    if (c.split > 1) refuse(h.id + ": split > 1 is not supported", CLDNN_UNSUPPORTED_SIZE);
    if (e.mode != cldnn_eltwise_sum) refuse(h.id + ": the fused eltwise honours the sum only (fused_conv_eltwise_gpu_ref.cl:200-233)");
    if (e.coefficients.size) refuse(h.id + ": eltwise coefficients are not supported");
    host::tensor es(1, 1, 1, 1);
    if (e.stride.size) {
        // one stride per eltwise input; the convolution's own result is never strided
        const cldnn_tensor& t = e.stride.data[e.stride.size - 1];
        es = host::tensor(1, 1, spatial(t, 0), spatial(t, 1));
        if (e.stride.size > 1 && !all_ones(e.stride.data[0])) refuse(h.id + ": a stride on the convolution side of the fused sum is not supported", CLDNN_UNSUPPORTED_SIZE);
    }
    host::primitive p = host::fused_conv_eltwise(h.id, h.input[0], h.input[1], host::eltwise_mode::sum, single_id(c.weights, h.id, "weights"),
                                                 single_id(c.bias, h.id, "bias"), single_id(c.weights_quantization_factors, h.id, "quantization factors"),
                                                 single_id(c.output_calibration_factors, h.id, "calibration factors"), c.input_quantization_factor,
                                                 x->non_conv_scale, str(e.output_calibration_factors), es, to_host_tensor(c.stride, 1, "stride"),
                                                 to_host_tensor(c.input_offset, 0, "input_offset"), to_host_tensor(c.dilation, 1, "dilation"),
                                                 c.with_activation != 0, c.activation_negative_slope, e.with_activation != 0, e.activation_negative_slope,
                                                 h.output_data_type);
    p.output_quantization_factor = c.output_quantization_factor;
    p.second_input_in_output = x->second_input_in_output != 0;
    out.prim = p;
}
void dto_eltwise(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_eltwise_desc*>(d);
    host::primitive h; common_head(d, h, 2, 2);
    host::eltwise_mode mode;
    switch (x->mode) {
    case cldnn_eltwise_sum: mode = host::eltwise_mode::sum; break;   case cldnn_eltwise_sub: mode = host::eltwise_mode::sub; break;
    case cldnn_eltwise_max: mode = host::eltwise_mode::max; break;   case cldnn_eltwise_prod: mode = host::eltwise_mode::prod; break;
    case cldnn_eltwise_min: mode = host::eltwise_mode::min; break;
    default: refuse(h.id + ": eltwise mode " + std::to_string(x->mode) + " is not supported on this path (sum, sub, max, prod, min)");
    }
    if (x->coefficients.size) refuse(h.id + ": eltwise coefficients are not supported");
    for (size_t i = 0; i < x->stride.size; ++i) if (!all_ones(x->stride.data[i])) refuse(h.id + ": strided eltwise inputs are not supported", CLDNN_UNSUPPORTED_SIZE);
    const std::string oc = str(x->output_calibration_factors);
    host::primitive p = host::eltwise(h.id, h.input[0], h.input[1], mode, x->with_activation != 0, x->activation_negative_slope, oc, x->output_quantization_factor,
                                      !oc.empty() || x->output_quantization_factor != 1.0f);
    p.output_data_type = h.output_data_type;
    out.prim = p;
}
void dto_activation(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_activation_desc*>(d);
    host::primitive h; common_head(d, h, 1, 1);
    if (!str(x->additional_params_input).empty()) refuse(h.id + ": activation parameters from a primitive are not supported");
    out.prim = host::activation(h.id, h.input[0], activation_of(x->activation_func, h.id), x->additional_params.a, x->additional_params.b);
}
void dto_pooling(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_pooling_desc*>(d);
    host::primitive h; common_head(d, h, 1, 1);
    if (!str(x->argmax).empty() || x->mode == cldnn_pooling_max_with_argmax || x->mode == cldnn_pooling_bilinear)
        refuse(h.id + ": pooling mode " + std::to_string(x->mode) + " is not supported on this path (max, average, average_no_padding)");
    if (x->with_output_size) refuse(h.id + ": a user-defined output size is not supported", CLDNN_UNSUPPORTED_SIZE);
    const host::pooling_mode mode = x->mode == cldnn_pooling_max ? host::pooling_mode::max
                                  : (x->mode == cldnn_pooling_average ? host::pooling_mode::average : host::pooling_mode::average_no_padding);
    if (x->global_pooling) out.prim = host::global_pooling(h.id, h.input[0], mode);
    else out.prim = host::pooling(h.id, h.input[0], mode, to_host_tensor(x->size, 1, "size"), to_host_tensor(x->stride, 1, "stride"),
                                  to_host_tensor(x->input_offset, 0, "input_offset"));
}
void dto_fully_connected(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_fully_connected_desc*>(d);
    host::primitive h; common_head(d, h, 1, 1);
    host::primitive p = host::fully_connected(h.id, h.input[0], str(x->weights), str(x->bias), str(x->weights_quantization_factors),
                                              str(x->output_calibration_factors), x->input_quantization_factor, x->with_activation != 0,
                                              x->activation_negative_slope);
    p.output_quantization_factor = x->output_quantization_factor;
    p.output_data_type = h.output_data_type;
    out.prim = p;
}
void dto_softmax(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_softmax_desc*>(d);
    host::primitive h; common_head(d, h, 1, 1);
    out.prim = host::softmax(h.id, h.input[0], (int32_t)x->dimension);
}
void dto_lrn(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_lrn_desc*>(d);
    host::primitive h; common_head(d, h, 1, 1);
    if (x->norm_region != cldnn_lrn_norm_region_across_channel) refuse(h.id + ": only the across-channel normalisation region is supported");
    out.prim = host::lrn(h.id, h.input[0], x->size, x->k, x->alpha, x->beta);
}
void dto_concatenation(const cldnn_primitive_desc* d, topo_entry& out)
{
    auto* x = reinterpret_cast<const cldnn_concatenation_desc*>(d);
    host::primitive h; common_head(d, h, 1, 64);
    if (x->axis < cldnn_concatenation_along_b || x->axis > cldnn_concatenation_along_y) refuse(h.id + ": concatenation axis must be b, f, x or y", CLDNN_INVALID_ARG);
    out.prim = host::concatenation(h.id, h.input, (int32_t)x->axis);
}

const cldnn_primitive_type k_input_layout = {"input_layout", dto_input_layout}, k_data = {"data", dto_data}, k_reorder = {"reorder", dto_reorder},
                           k_convolution = {"convolution", dto_convolution}, k_fused = {"fused_conv_eltwise", dto_fused_conv_eltwise},
                           k_eltwise = {"eltwise", dto_eltwise}, k_activation = {"activation", dto_activation}, k_pooling = {"pooling", dto_pooling},
                           k_fc = {"fully_connected", dto_fully_connected}, k_softmax = {"softmax", dto_softmax}, k_lrn = {"lrn", dto_lrn},
                           k_concat = {"concatenation", dto_concatenation};
const cldnn_primitive_type* const k_types[] = {&k_input_layout, &k_data, &k_reorder, &k_convolution, &k_fused, &k_eltwise, &k_activation,
                                               &k_pooling, &k_fc, &k_softmax, &k_lrn, &k_concat};

// names back to back, each ended by a zero, one more zero after the last; too small a buffer: needed size + CLDNN_INVALID_ARG
void pack_names(const std::vector<std::string>& names, char* out, size_t size, size_t* size_ret, cldnn_status* status)
{
    size_t need = 1;
    for (auto& n : names) need += n.size() + 1;
    if (size_ret) *size_ret = need;
    if (size < need || !out) { if (status) *status = CLDNN_INVALID_ARG; return; }
    size_t i = 0;
    for (auto& n : names) { std::memcpy(out + i, n.data(), n.size()); i += n.size(); out[i++] = 0; }
    out[i] = 0;
}

cldnn_memory wrap_device_memory(cldnn_engine eng, const host::memory& m)
{
    auto* mem = new cldnn_memory_impl();
    mem->owner = eng; eng->retain();
    mem->dev = m;
    mem->lay = to_c_layout(m.get_layout());
    return mem;
}

// device memory of `eng` holding what `mem` holds now (the object itself when it already lives there)
host::memory device_view(cldnn_engine eng, cldnn_memory mem)
{
    if (mem->owner) return mem->dev;
    const host::layout l = to_host_layout(mem->lay);
    host::memory m = host::memory::allocate(eng->eng, l);
    m.write(mem->attached, l.bytes_count());
    return m;
}

host::build_options read_options(cldnn_engine eng, const cldnn_build_option* options, size_t n)
{
    host::build_options o;
    o.tuning_cache_path = eng->tuning_cache_path;
    // the reference fuses conv + eltwise for 1x1 stride-1 convolutions only (prepare_primitive_fusing.cpp:197-217); keep that
    // default here so that a topology is rewritten as it would be there
    o.fuse_any_conv_eltwise = false;
    for (size_t i = 0; i < n; ++i) {
        const cldnn_build_option& b = options[i];
        switch (b.type) {
        case cldnn_build_option_fusing: break;                                       // activation fusing is part of optimize_data here
        case cldnn_build_option_optimize_data: o.optimize_data = reinterpret_cast<uintptr_t>(b.data) != 0; break;
        case cldnn_build_option_debug: break;
        case cldnn_build_option_outputs: {
            not_null(b.data, "output data");
            auto* arr = reinterpret_cast<const cldnn_primitive_id_arr*>(b.data);
            o.outputs = ids_of(*arr);
            break;
        }
        case cldnn_build_option_tuning_config: {
            not_null(b.data, "Tuning config data");
            auto* t = reinterpret_cast<const cldnn_tuning_config*>(b.data);
            o.tuning = (host::tuning_mode)t->mode;
            if (!str(t->cache_file_path).empty()) o.tuning_cache_path = str(t->cache_file_path);
            break;
        }
        case cldnn_build_option_graph_dumps_dir: break;                              // no graph dumps
        case cldnn_build_option_learning_config: refuse("training options are outside the inference path");
        case cldnn_build_option_detection_output_gpu: break;
        default: refuse("unknown build option " + std::to_string(b.type), CLDNN_INVALID_ARG);
        }
    }
    return o;
}

cldnn_network make_network(cldnn_program prog)
{
    auto* n = new cldnn_network_impl();
    n->prog = prog; prog->retain();
    try {
        if (prog->first) n->net = std::move(prog->first);
        else n->net.reset(new host::network(prog->eng->eng, prog->topo, prog->opts));
    } catch (...) { n->net.reset(); n->release(); throw; }
    return n;
}

}  // namespace

extern "C" {

cldnn_version cldnn_get_version(cldnn_status* status)
{
    return guarded<cldnn_version>(status, cldnn_version{}, []() { return cldnn_version{1, 4, 25, 0}; });   // the drop this boundary follows (14.1, v1.4.25)
}
const char* cldnn_get_last_error_message(void) { return g_last_error.c_str(); }

// ---- topology ------------------------------------------------------------------------------------------------------------
cldnn_topology cldnn_create_topology(cldnn_status* status)
{
    return guarded<cldnn_topology>(status, nullptr, []() { return new cldnn_topology_impl(); });
}
void cldnn_add_primitive(cldnn_topology topology, const struct cldnn_primitive_desc* dto, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(topology, "Topology"); not_null(dto, "Primitive"); not_null(dto->id, "Primitive id"); not_null(dto->type, "Primitive type");
        bool known = false;
        for (auto* t : k_types) known |= t == dto->type;
        if (!known) refuse(std::string("primitive '") + dto->id + "': this primitive type is outside the convolution path this library implements");
        for (auto& e : topology->entries) if (e.prim.id == dto->id) throw api_error(std::string("Different primitive with id '") + dto->id + "' exists already.", CLDNN_ERROR);
        topo_entry e;
        dto->type->from_dto(dto, e);
        topology->entries.push_back(e);
    });
}
void cldnn_change_input_layout(cldnn_topology topology, cldnn_primitive_id id, cldnn_layout new_layout, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(topology, "Topology"); not_null(id, "Input layout id");
        const host::layout l = to_host_layout(new_layout);
        for (auto& e : topology->entries) if (e.prim.id == id) {
            if (e.prim.type != "input_layout") throw api_error(std::string("Primitive: ") + id + " is not input_layout.", CLDNN_ERROR);
            e.prim.target = l; return;
        }
        throw api_error(std::string("Can't find primitive with id: ") + id, CLDNN_ERROR);
    });
}
void cldnn_get_primitive_ids(cldnn_topology topology, char* ids, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(topology, "Topology");
        std::vector<std::string> v;
        for (auto& e : topology->entries) v.push_back(e.prim.id);
        if (v.empty()) throw api_error("Primitives number should not equals 0.", CLDNN_ERROR);
        pack_names(v, ids, size, size_ret, status);
    });
}
void cldnn_retain_topology(cldnn_topology topology, cldnn_status* status) { guarded(status, [&]() { not_null(topology, "Topology"); topology->retain(); }); }
void cldnn_release_topology(cldnn_topology topology, cldnn_status* status) { guarded(status, [&]() { not_null(topology, "Topology"); topology->release(); }); }

// ---- engine --------------------------------------------------------------------------------------------------------------
uint32_t cldnn_get_engine_count(int32_t type, cldnn_status* status)
{
    return guarded<uint32_t>(status, 0u, [&]() -> uint32_t {
        if (type != cldnn_engine_ocl) throw api_error("Invalid engine type.", CLDNN_DEVICE_ERROR);
        int32_t n = 0;
        if (cldnn_b200_device_count(&n) != CLDNN_B200_SUCCESS) return 0u;
        return (uint32_t)n;
    });
}
cldnn_engine cldnn_create_engine(int32_t type, uint32_t engine_num, const cldnn_engine_configuration* configuration, cldnn_status* status)
{
    return guarded<cldnn_engine>(status, nullptr, [&]() -> cldnn_engine {
        if (type != cldnn_engine_ocl) throw api_error("Invalid engine type.", CLDNN_DEVICE_ERROR);
        bool prof = false; std::string cache;
        if (configuration) {
            if (configuration->context) refuse("engine configuration: an OpenCL context cannot be adopted by the CUDA engine", CLDNN_INVALID_ARG);
            if (!str(configuration->compiler_options).empty()) refuse("engine configuration: OpenCL compiler options have no meaning for the CUDA engine", CLDNN_INVALID_ARG);
            prof = configuration->enable_profiling != 0;
            cache = str(configuration->tuning_cache_path);
        }
        auto* e = new cldnn_engine_impl((int32_t)engine_num, prof);
        e->tuning_cache_path = cache;
        return e;
    });
}
void cldnn_retain_engine(cldnn_engine engine, cldnn_status* status) { guarded(status, [&]() { not_null(engine, "Engine"); engine->retain(); }); }
void cldnn_release_engine(cldnn_engine engine, cldnn_status* status) { guarded(status, [&]() { not_null(engine, "Engine"); engine->release(); }); }
void cldnn_release_pending_memory(cldnn_engine engine, cldnn_status* status) { guarded(status, [&]() { not_null(engine, "Engine"); engine->eng.sync(); }); }
cldnn_engine_info cldnn_get_engine_info(cldnn_engine engine, cldnn_status* status)
{
    return guarded<cldnn_engine_info>(status, cldnn_engine_info{}, [&]() {
        not_null(engine, "Engine");
        const cldnn_b200_engine_info i = engine->eng.get_info();
        cldnn_engine_info o{};
        o.cores_count = i.cores_count; o.core_frequency = i.core_frequency;
        o.max_work_group_size = i.max_work_group_size; o.max_local_mem_size = i.max_local_mem_size;
        o.max_global_mem_size = i.max_global_mem_size; o.max_alloc_mem_size = i.max_alloc_mem_size;
        o.supports_fp16 = 1; o.supports_fp16_denorms = 1; o.supports_imad = 1; o.supports_immad = 1;   // tensor cores: fp16 and 8-bit integer MMA
        return o;
    });
}
int32_t cldnn_get_engine_type(cldnn_engine engine, cldnn_status* status)
{
    return guarded<int32_t>(status, 0, [&]() { not_null(engine, "Engine"); return (int32_t)cldnn_engine_ocl; });
}
int64_t cldnn_get_temp_used_device_memory_size(cldnn_engine engine, cldnn_status* status)
{
    return guarded<int64_t>(status, 0, [&]() -> int64_t { not_null(engine, "Engine"); return 0; });
}
int64_t cldnn_get_max_used_device_memory_size(cldnn_engine engine, cldnn_status* status)
{
    return guarded<int64_t>(status, 0, [&]() -> int64_t { not_null(engine, "Engine"); return 0; });
}

// ---- events ----------------------------------------------------------------------------------------------------------------
cldnn_event cldnn_create_user_event(cldnn_engine engine, cldnn_status* status)
{
    return guarded<cldnn_event>(status, nullptr, [&]() -> cldnn_event {
        not_null(engine, "Engine");
        auto* e = new cldnn_event_impl(); e->eng = engine; engine->retain(); e->user = true; return e;
    });
}
int32_t cldnn_is_user_event(cldnn_event event, cldnn_status* status)
{
    return guarded<int32_t>(status, 0, [&]() { not_null(event, "Event"); return event->user ? 1 : 0; });
}
void cldnn_retain_event(cldnn_event event, cldnn_status* status) { guarded(status, [&]() { not_null(event, "Event"); event->retain(); }); }
void cldnn_release_event(cldnn_event event, cldnn_status* status) { guarded(status, [&]() { not_null(event, "Event"); event->release(); }); }
void cldnn_wait_for_event(cldnn_event event, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(event, "Event");
        if (event->user) {
            std::unique_lock<std::mutex> lk(event->m);
            event->cv.wait(lk, [&] { return event->is_set; });
            return;
        }
        // the execution this event stands for has finished once the engine's queue has drained
        event->eng->eng.sync();
        const uint32_t st = event->eng->eng.device_status();
        if (st) throw api_error("a kernel gave up a bounded wait (device status " + std::to_string(st) + ")", CLDNN_DEVICE_ERROR);
        std::vector<std::pair<cldnn_event_handler, void*>> hs;
        { std::lock_guard<std::mutex> lk(event->m); event->is_set = true; hs.swap(event->handlers); }
        for (auto& h : hs) h.first(h.second);
    });
}
void cldnn_set_event(cldnn_event event, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(event, "Event");
        if (!event->user) throw api_error("Event passed to cldnn_set_event should be an user event", CLDNN_ERROR);
        std::vector<std::pair<cldnn_event_handler, void*>> hs;
        { std::lock_guard<std::mutex> lk(event->m); event->is_set = true; hs.swap(event->handlers); }
        event->cv.notify_all();
        for (auto& h : hs) h.first(h.second);
    });
}
void cldnn_add_event_handler(cldnn_event event, cldnn_event_handler handler, void* param, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(event, "Event"); not_null(handler, "Handler");
        bool now = false;
        { std::lock_guard<std::mutex> lk(event->m); if (event->is_set) now = true; else event->handlers.push_back({handler, param}); }
        if (now) handler(param);
    });
}
void cldnn_get_event_profiling_info(cldnn_event event, cldnn_profiling_interval* profiling, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(event, "Event");
        // the three intervals of the reference (src/gpu/ocl_base_event.cpp:68-92); only the execution time exists on an in-order stream
        static const char* names[3] = {"submission", "starting", "executing"};
        uint64_t exec_ns = 0;
        const bool have = event->net && event->net->net && event->eng->profiling;
        if (have) for (auto& kv : event->net->net->get_profiling_info()) if (kv.first == event->primitive) exec_ns = kv.second;
        const size_t n = have ? 3 : 0;
        if (size_ret) *size_ret = n;
        if (size < n || (n && !profiling)) { if (status) *status = CLDNN_INVALID_ARG; return; }
        for (size_t i = 0; i < n; ++i) { profiling[i].name = names[i]; profiling[i].nanoseconds = i == 2 ? exec_ns : 0; }
    });
}

// ---- program / network -----------------------------------------------------------------------------------------------------
cldnn_program cldnn_build_program(cldnn_engine engine, cldnn_topology topology, cldnn_build_option* options, size_t options_num, cldnn_status* status)
{
    return guarded<cldnn_program>(status, nullptr, [&]() -> cldnn_program {
        not_null(engine, "Engine"); not_null(topology, "Topology");
        if (options_num) not_null(options, "Options");
        auto* p = new cldnn_program_impl();
        p->eng = engine; engine->retain();
        try {
            p->opts = read_options(engine, options, options_num);
            for (auto& e : topology->entries) {
                host::primitive prim = e.prim;
                if (prim.type == "data") {
                    prim = host::data(prim.id, device_view(engine, e.mem));
                    p->keep.push_back(e.mem); e.mem->retain();
                }
                p->topo.add(prim);
                p->org_ids.push_back(prim.id);
            }
            // the graph is built (validated, optimised, buffers allocated) here, as the reference's program build does
            p->first.reset(new host::network(engine->eng, p->topo, p->opts));
        } catch (...) { p->release(); throw; }
        return p;
    });
}
void cldnn_retain_program(cldnn_program program, cldnn_status* status) { guarded(status, [&]() { not_null(program, "Program"); program->retain(); }); }
void cldnn_release_program(cldnn_program program, cldnn_status* status) { guarded(status, [&]() { not_null(program, "Program"); program->release(); }); }

cldnn_network cldnn_allocate_network(cldnn_program program, cldnn_status* status)
{
    return guarded<cldnn_network>(status, nullptr, [&]() -> cldnn_network { not_null(program, "Program"); return make_network(program); });
}
cldnn_network cldnn_build_network(cldnn_engine engine, cldnn_topology topology, cldnn_build_option* options, size_t options_num, cldnn_status* status)
{
    cldnn_program prog = cldnn_build_program(engine, topology, options, options_num, status);
    if (!prog) return nullptr;
    cldnn_network net = cldnn_allocate_network(prog, status);
    prog->release();
    return net;
}
void cldnn_retain_network(cldnn_network network, cldnn_status* status) { guarded(status, [&]() { not_null(network, "Network"); network->retain(); }); }
void cldnn_release_network(cldnn_network network, cldnn_status* status) { guarded(status, [&]() { not_null(network, "Network"); network->release(); }); }

void cldnn_set_network_input(cldnn_network network, cldnn_primitive_id id, cldnn_memory mem, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(network, "Network"); not_null(id, "Id"); not_null(mem, "Mem");
        const std::string key = id;
        if (mem->owner) {
            network->net->set_input_data(key, mem->dev);
        } else {
            // a host buffer of the caller: its contents are copied into a device buffer now
            const host::layout l = to_host_layout(mem->lay);
            auto it = network->staged.find(key);
            if (it == network->staged.end() || !(it->second->dev.get_layout() == l)) {
                cldnn_memory d = wrap_device_memory(network->prog->eng, host::memory::allocate(network->prog->eng->eng, l));
                if (it != network->staged.end()) { it->second->release(); it->second = d; } else network->staged[key] = d;
                it = network->staged.find(key);
            }
            it->second->dev.write(mem->attached, l.bytes_count());
            network->net->set_input_data(key, it->second->dev);
        }
        mem->retain();
        auto old = network->inputs.find(key);
        if (old != network->inputs.end()) { old->second->release(); old->second = mem; } else network->inputs[key] = mem;
    });
}
void cldnn_set_learning_rate(cldnn_network network, float, cldnn_status* status)
{
    guarded(status, [&]() { not_null(network, "Network"); refuse("training is outside the inference path"); });
}
float cldnn_get_learning_rate(cldnn_network network, cldnn_status* status)
{
    return guarded<float>(status, 0.0f, [&]() -> float { not_null(network, "Network"); return 0.0f; });
}
void cldnn_get_primitive_info(cldnn_network network, cldnn_primitive_id id, char* info, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(network, "Network"); not_null(id, "Id");
        std::string text;
        for (auto& i : network->net->get_primitives_info()) {
            bool match = i.id == id;
            std::stringstream ss(i.original_ids); std::string f;
            while (std::getline(ss, f, ',')) match |= f == id;
            if (!match) continue;
            std::stringstream o;
            o << "id: " << i.id << ", type: " << i.type << ", kernel: " << (i.kernel.empty() ? "-" : i.kernel) << ", tune: " << i.tune << ", output: "
              << host::format::name(i.output.fmt) << " [b" << i.output.size.batch << " f" << i.output.size.feature << " y" << i.output.size.y << " x" << i.output.size.x
              << "]" << (i.original_ids.empty() ? "" : ", fused: " + i.original_ids);
            text = o.str();
        }
        if (text.empty()) throw api_error(std::string("primitive '") + id + "' is not in the network", CLDNN_INVALID_ARG);
        const size_t need = text.size() + 1;
        if (size_ret) *size_ret = need;
        if (size < need || !info) { if (status) *status = CLDNN_INVALID_ARG; return; }
        std::memcpy(info, text.c_str(), need);
    });
}
cldnn_engine cldnn_get_network_engine(cldnn_network network, cldnn_status* status)
{
    return guarded<cldnn_engine>(status, nullptr, [&]() { not_null(network, "Network"); network->prog->eng->retain(); return network->prog->eng; });
}
cldnn_program cldnn_get_network_program(cldnn_network network, cldnn_status* status)
{
    return guarded<cldnn_program>(status, nullptr, [&]() { not_null(network, "Network"); network->prog->retain(); return network->prog; });
}
void cldnn_get_network_output_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(network, "Network");
        const std::vector<std::string> ids = network->net->get_output_ids();
        if (ids.empty()) throw api_error("Output size should not equals 0.", CLDNN_ERROR);
        pack_names(ids, names, size, size_ret, status);
    });
}
void cldnn_get_network_executed_primitive_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(network, "Network");
        std::vector<std::string> v;
        for (auto& i : network->net->get_primitives_info()) if (!i.kernel.empty()) v.push_back(i.id);
        pack_names(v, names, size, size_ret, status);
    });
}
// one entry per primitive of the topology: its id, or "_optimized_" when the build folded it into another primitive
static std::vector<std::string> all_names(cldnn_network network, bool original)
{
    std::vector<std::string> alive;
    for (auto& i : network->net->get_primitives_info()) alive.push_back(i.id);
    std::vector<std::string> v;
    for (auto& id : network->prog->org_ids) {
        const bool here = std::find(alive.begin(), alive.end(), id) != alive.end();
        v.push_back(original || here ? id : "_optimized_");
    }
    return v;
}
void cldnn_get_network_all_primitive_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() { not_null(network, "Network"); pack_names(all_names(network, false), names, size, size_ret, status); });
}
void cldnn_get_network_all_primitive_org_names(cldnn_network network, char* names, size_t size, size_t* size_ret, cldnn_status* status)
{
    guarded(status, [&]() { not_null(network, "Network"); pack_names(all_names(network, true), names, size, size_ret, status); });
}
void cldnn_execute_network(cldnn_network network, cldnn_event* dependencies, size_t deps_num, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(network, "Network");
        // dependencies are waited for on the host, then the whole network is enqueued on the engine's stream
        for (size_t i = 0; i < deps_num; ++i) { cldnn_status st = CLDNN_SUCCESS; cldnn_wait_for_event(dependencies[i], &st); if (st != CLDNN_SUCCESS) throw api_error(g_last_error, st); }
        network->net->execute();
    });
}
static cldnn_event output_event(cldnn_network network, const std::string& name)
{
    auto* e = new cldnn_event_impl();
    e->eng = network->prog->eng; e->eng->retain();
    e->net = network; network->retain();
    e->primitive = name;
    return e;
}
cldnn_memory cldnn_get_network_output_memory(cldnn_network network, const char* name, cldnn_status* status)
{
    return guarded<cldnn_memory>(status, nullptr, [&]() -> cldnn_memory {
        not_null(network, "Network"); not_null(name, "ID of primitive");
        return wrap_device_memory(network->prog->eng, network->net->output_memory(name));
    });
}
cldnn_event cldnn_get_network_output_event(cldnn_network network, const char* name, cldnn_status* status)
{
    return guarded<cldnn_event>(status, nullptr, [&]() -> cldnn_event {
        not_null(network, "Network"); not_null(name, "ID of primitive");
        (void)network->net->output_memory(name);                      // validates the id
        return output_event(network, name);
    });
}
cldnn_network_output cldnn_get_network_output(cldnn_network network, const char* name, cldnn_status* status)
{
    cldnn_network_output out{nullptr, nullptr};
    out.memory = cldnn_get_network_output_memory(network, name, status);
    if (!out.memory) return out;
    out.event = cldnn_get_network_output_event(network, name, status);
    if (!out.event) { out.memory->release(); out.memory = nullptr; }
    return out;
}

// ---- memory ----------------------------------------------------------------------------------------------------------------
cldnn_memory cldnn_allocate_memory(cldnn_engine engine, cldnn_layout layout, cldnn_status* status)
{
    return guarded<cldnn_memory>(status, nullptr, [&]() -> cldnn_memory {
        not_null(engine, "Engine");
        cldnn_memory m = wrap_device_memory(engine, host::memory::allocate(engine->eng, to_host_layout(layout)));
        m->lay = layout;
        return m;
    });
}
cldnn_memory cldnn_attach_memory(cldnn_layout layout, void* pointer, size_t size, cldnn_status* status)
{
    return guarded<cldnn_memory>(status, nullptr, [&]() -> cldnn_memory {
        not_null(pointer, "Pointer");
        if (to_host_layout(layout).bytes_count() > size) throw api_error("buffer size does not match layout size", CLDNN_ERROR);
        auto* m = new cldnn_memory_impl(); m->lay = layout; m->attached = pointer; return m;
    });
}
int32_t cldnn_is_the_same_buffer(cldnn_memory mem1, cldnn_memory mem2, cldnn_status* status)
{
    return guarded<int32_t>(status, 0, [&]() -> int32_t {
        not_null(mem1, "Memory"); not_null(mem2, "Memory");
        if (mem1 == mem2) return 1;
        if (mem1->owner != mem2->owner) return 0;
        if (!mem1->owner) return mem1->attached == mem2->attached ? 1 : 0;
        return mem1->dev.device_ptr() == mem2->dev.device_ptr() ? 1 : 0;
    });
}
void cldnn_retain_memory(cldnn_memory memory, cldnn_status* status) { guarded(status, [&]() { not_null(memory, "Memory"); memory->retain(); }); }
void cldnn_release_memory(cldnn_memory memory, cldnn_status* status) { guarded(status, [&]() { not_null(memory, "Memory"); memory->release(); }); }
void* cldnn_lock_memory(cldnn_memory memory, cldnn_status* status)
{
    return guarded<void*>(status, nullptr, [&]() -> void* {
        not_null(memory, "Memory");
        if (!memory->owner) return memory->attached;
        std::lock_guard<std::mutex> lk(memory->lock_mutex);
        if (memory->locks++ == 0) {
            // blocking map (gpu_buffer::lock, src/gpu/memory_gpu.cpp:49-60): device contents into a host view
            memory->staging.resize(memory->dev.size());
            memory->dev.read(memory->staging.data(), memory->staging.size());
        }
        return memory->staging.data();
    });
}
void cldnn_unlock_memory(cldnn_memory memory, cldnn_status* status)
{
    guarded(status, [&]() {
        not_null(memory, "Memory");
        if (!memory->owner) return;
        std::lock_guard<std::mutex> lk(memory->lock_mutex);
        if (memory->locks <= 0) throw api_error("memory is not locked", CLDNN_ERROR);
        if (--memory->locks == 0) {
            memory->dev.write(memory->staging.data(), memory->staging.size());     // unmap: the host view goes back to the device
            std::vector<uint8_t>().swap(memory->staging);
        }
    });
}
cldnn_layout cldnn_get_memory_layout(cldnn_memory memory, cldnn_status* status)
{
    cldnn_layout none{}; none.data_type = cldnn_f32; none.format = cldnn_format_bfyx;
    return guarded<cldnn_layout>(status, none, [&]() { not_null(memory, "Memory"); return memory->lay; });
}
cldnn_engine cldnn_get_memory_engine(cldnn_memory memory, cldnn_status* status)
{
    return guarded<cldnn_engine>(status, nullptr, [&]() -> cldnn_engine { not_null(memory, "Memory"); if (memory->owner) memory->owner->retain(); return memory->owner; });
}

// ---- half precision helpers (src/half.cpp) ---------------------------------------------------------------------------------
uint16_t cldnn_float_to_half(float value, cldnn_status* status)
{
    return guarded<uint16_t>(status, 0, [&]() -> uint16_t {
        uint32_t x; std::memcpy(&x, &value, 4);
        const uint32_t sign = (x >> 16) & 0x8000u;
        const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
        uint32_t man = x & 0x7fffffu;
        if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0u));          // inf / nan
        if (exp >= 31) return (uint16_t)(sign | 0x7c00u);                                                  // overflow -> inf
        if (exp <= 0) {                                                                                     // subnormal or zero
            if (exp < -10) return (uint16_t)sign;
            man |= 0x800000u;
            const int shift = 14 - exp;
            uint32_t h = man >> shift;
            const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
            if (rem > halfway || (rem == halfway && (h & 1))) ++h;
            return (uint16_t)(sign | h);
        }
        uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
        const uint32_t rem = man & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;                                             // round to nearest even (may carry into the exponent)
        return (uint16_t)(sign | h);
    });
}
float cldnn_half_to_float(uint16_t value, cldnn_status* status)
{
    return guarded<float>(status, 0.0f, [&]() -> float {
        const uint32_t sign = (uint32_t)(value & 0x8000u) << 16;
        uint32_t exp = (value >> 10) & 0x1f, man = value & 0x3ffu, x;
        if (exp == 31) x = sign | 0x7f800000u | (man << 13);
        else if (exp == 0) {
            if (!man) x = sign;
            else { int e = -1; do { ++e; man <<= 1; } while (!(man & 0x400u)); x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13); }
        } else x = sign | ((exp + 127 - 15) << 23) | (man << 13);
        float f; std::memcpy(&f, &x, 4); return f;
    });
}

// ---- primitive type identifiers --------------------------------------------------------------------------------------------
#define TYPE_ID(NAME, OBJ) cldnn_primitive_type_id cldnn_##NAME##_type_id(cldnn_status* status) { if (status) *status = CLDNN_SUCCESS; return &OBJ; }
TYPE_ID(input_layout, k_input_layout)
TYPE_ID(data, k_data)
TYPE_ID(reorder, k_reorder)
TYPE_ID(convolution, k_convolution)
TYPE_ID(fused_conv_eltwise, k_fused)
TYPE_ID(eltwise, k_eltwise)
TYPE_ID(activation, k_activation)
TYPE_ID(pooling, k_pooling)
TYPE_ID(fully_connected, k_fc)
TYPE_ID(softmax, k_softmax)
TYPE_ID(lrn, k_lrn)
TYPE_ID(concatenation, k_concat)
#undef TYPE_ID

}  // extern "C"
