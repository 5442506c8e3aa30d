// Program build and network execution for the convolution hot path: the host
// logic of clDNN's graph core (src/program.cpp, src/network.cpp, the passes in
// src/graph_optimizer/) re-done for the B200 engine.  Everything device-side
// goes through the C ABI of include/cldnn_b200.h.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <functional>
#include <set>
#include <sstream>
#include "cldnn_host.hpp"

namespace cldnn {

static void check(int32_t st, const std::string& what)
{
    if (st != CLDNN_B200_SUCCESS) throw error(what + ": " + cldnn_b200_last_error(), st);
}

// --------------------------------------------------------------------------------------
// layout
// --------------------------------------------------------------------------------------
const char* format::name(int32_t f)
{
    switch (f) { case yxfb: return "yxfb"; case byxf: return "byxf"; case bfyx: return "bfyx"; case byxf_af32: return "byxf_af32"; }
    return "any";
}
static int dtype_bytes(data_types d) { return (int)d & 0x0f; }
static bool is_int8(data_types d) { return d == data_types::i8 || d == data_types::u8; }

int32_t layout::stored_features() const { return fmt == format::byxf_af32 ? (size.feature + 31) / 32 * 32 : size.feature; }
size_t layout::count() const
{
    return (size_t)size.batch * stored_features() * (size.y + data_padding.lower_y + data_padding.upper_y) * (size.x + data_padding.lower_x + data_padding.upper_x);
}
size_t layout::bytes_count() const { return count() * dtype_bytes(data_type); }
bool layout::operator==(const layout& o) const
{
    return data_type == o.data_type && fmt == o.fmt && size == o.size && data_padding.lower_x == o.data_padding.lower_x &&
           data_padding.lower_y == o.data_padding.lower_y && data_padding.upper_x == o.data_padding.upper_x && data_padding.upper_y == o.data_padding.upper_y;
}
cldnn_b200_tensor layout::desc() const
{
    cldnn_b200_tensor t{};
    const int64_t fs = stored_features();
    const int64_t ys = size.y + data_padding.lower_y + data_padding.upper_y, xs = size.x + data_padding.lower_x + data_padding.upper_x;
    t.dtype = (int32_t)data_type; t.b = size.batch; t.f = size.feature; t.y = size.y; t.x = size.x;
    switch (fmt) {
    case format::bfyx: t.px = 1; t.py = xs; t.pf = xs * ys; t.pb = xs * ys * fs; break;
    case format::byxf: case format::byxf_af32: t.pf = 1; t.px = fs; t.py = fs * xs; t.pb = fs * xs * ys; break;
    case format::yxfb: t.pb = 1; t.pf = size.batch; t.px = size.batch * fs; t.py = size.batch * fs * xs; break;
    default: throw error("layout: unsupported format", CLDNN_B200_UNSUPPORTED_FORMAT);
    }
    t.offset = data_padding.lower_y * t.py + data_padding.lower_x * t.px;
    return t;
}

int32_t conv_output_size(int32_t in, int32_t filter, int32_t input_offset, int32_t stride, int32_t dilation)
{
    const int32_t wes = (filter - 1) * dilation + 1;
    if (2 * input_offset + wes > in) return 0;
    return (in - 2 * input_offset - wes) / stride + 1;
}
int32_t pool_output_size(int32_t in, int32_t window, int32_t input_offset, int32_t stride)
{
    const int32_t ext = std::max(window, stride);
    const int32_t once = (2 * input_offset + ext <= in + stride - 1) ? (in - 2 * input_offset - ext + stride - 1) / stride + 1 : 1;
    const int32_t any = (input_offset <= in - 1) ? (in - input_offset - 1) / stride + 1 : 1;
    return std::min(once, any);
}

// --------------------------------------------------------------------------------------
// engine / memory
// --------------------------------------------------------------------------------------
class engine_impl {
public:
    cldnn_b200_ctx ctx = nullptr;
    cldnn_b200_engine_info info{};
    bool profiling = false;
    std::map<std::string, cldnn_b200_kernel> kernels;
    ~engine_impl() { if (ctx) cldnn_b200_ctx_destroy(ctx); }
    cldnn_b200_kernel kernel(const std::string& name)
    {
        auto it = kernels.find(name);
        if (it != kernels.end()) return it->second;
        cldnn_b200_kernel k = nullptr;
        check(cldnn_b200_kernel_lookup(ctx, name.c_str(), &k), "kernel_lookup");
        kernels[name] = k;
        return k;
    }
};

engine::engine(int32_t device, bool enable_profiling) : impl(std::make_shared<engine_impl>())
{
    check(cldnn_b200_ctx_create(device, enable_profiling ? 1u : 0u, &impl->ctx), "engine");
    check(cldnn_b200_ctx_info(impl->ctx, &impl->info), "engine info");
    impl->profiling = enable_profiling;
}
void* engine::stream() const { void* s = nullptr; check(cldnn_b200_ctx_stream(impl->ctx, &s), "engine stream"); return s; }
bool engine::profiling() const { return impl->profiling; }
void engine::sync() const { check(cldnn_b200_ctx_sync(impl->ctx), "engine sync"); }
uint32_t engine::device_status() const { uint32_t st = 0; check(cldnn_b200_ctx_device_status(impl->ctx, &st), "device status"); return st; }
cldnn_b200_engine_info engine::get_info() const { return impl->info; }

// one device allocation; several memory objects may view it over disjoint lifetimes (memory pool)
struct block {
    std::shared_ptr<engine_impl> eng;
    cldnn_b200_mem mem = nullptr; void* dev = nullptr; size_t bytes = 0;
    ~block() { if (mem) cldnn_b200_mem_free(mem); }
};
static std::shared_ptr<block> new_block(const std::shared_ptr<engine_impl>& eng, size_t bytes)
{
    auto b = std::make_shared<block>(); b->eng = eng; b->bytes = std::max<size_t>(bytes, 16);
    check(cldnn_b200_mem_alloc(eng->ctx, b->bytes, &b->mem), "memory allocation");
    check(cldnn_b200_mem_devptr(b->mem, &b->dev), "memory devptr");
    return b;
}

class memory_impl {
public:
    std::shared_ptr<block> blk;
    layout l;
};

memory memory::allocate(const engine& e, const layout& l)
{
    memory m; m.impl = std::make_shared<memory_impl>();
    m.impl->l = l; m.impl->blk = new_block(e.impl, l.bytes_count());
    return m;
}
memory memory::attach(const engine& e, const layout& l, void* device_ptr)
{
    memory m; m.impl = std::make_shared<memory_impl>();
    m.impl->l = l;
    auto b = std::make_shared<block>(); b->eng = e.impl; b->bytes = std::max<size_t>(l.bytes_count(), 16);
    check(cldnn_b200_mem_attach(e.impl->ctx, device_ptr, b->bytes, &b->mem), "memory::attach");
    b->dev = device_ptr;
    m.impl->blk = b;
    return m;
}
const layout& memory::get_layout() const { return impl->l; }
size_t memory::size() const { return impl->l.bytes_count(); }
void* memory::device_ptr() const { return impl->blk->dev; }
void memory::write(const void* host, size_t bytes)
{
    if (bytes > impl->blk->bytes) throw error("memory::write: more bytes than the memory object holds", CLDNN_B200_INVALID_ARG);
    check(cldnn_b200_mem_write(impl->blk->mem, 0, host, bytes), "memory::write");
}
void memory::read(void* host, size_t bytes) const
{
    if (bytes > impl->blk->bytes) throw error("memory::read: more bytes than the memory object holds", CLDNN_B200_INVALID_ARG);
    check(cldnn_b200_mem_read(impl->blk->mem, 0, host, bytes), "memory::read");
}

// --------------------------------------------------------------------------------------
// primitive constructors
// --------------------------------------------------------------------------------------
primitive input_layout(const std::string& id, const layout& l) { primitive p; p.type = "input_layout"; p.id = id; p.target = l; return p; }
primitive data(const std::string& id, const memory& m) { primitive p; p.type = "data"; p.id = id; p.mem = m; return p; }
primitive reorder(const std::string& id, const std::string& input, int32_t out_format, data_types out_type, const std::vector<float>& sub)
{
    primitive p; p.type = "reorder"; p.id = id; p.input = {input}; p.target.fmt = out_format; p.target.data_type = out_type; p.subtract_per_feature = sub; return p;
}
primitive convolution(const std::string& id, const std::string& input, const std::string& weights, const std::string& bias,
                      const std::string& wq, const std::string& oc, float iqf, data_types odt, tensor stride, tensor input_offset,
                      tensor dilation, bool with_activation, float slp, int32_t groups)
{
    primitive p; p.type = "convolution"; p.id = id; p.input = {input}; p.weights = weights; p.bias = bias;
    p.weights_quantization_factors = wq; p.output_calibration_factors = oc; p.input_quantization_factor = iqf; p.output_data_type = odt;
    p.stride = stride; p.input_offset = input_offset; p.dilation = dilation; p.with_activation = with_activation; p.activation_negative_slope = slp; p.groups = groups;
    return p;
}
primitive fused_conv_eltwise(const std::string& id, const std::string& input, const std::string& input2, eltwise_mode mode,
                             const std::string& weights, const std::string& bias, const std::string& wq, const std::string& oc, float iqf,
                             float non_conv_scale, const std::string& ec, tensor eltw_stride, tensor stride, tensor input_offset, tensor dilation,
                             bool conv_act, float conv_slp, bool eltw_act, float eltw_slp, data_types odt)
{
    primitive p; p.type = "fused_conv_eltwise"; p.id = id; p.input = {input, input2}; p.mode = mode; p.weights = weights; p.bias = bias;
    p.weights_quantization_factors = wq; p.output_calibration_factors = oc; p.input_quantization_factor = iqf; p.non_conv_scale = non_conv_scale;
    p.eltw_output_calibration_factors = ec; p.eltw_stride = eltw_stride; p.stride = stride; p.input_offset = input_offset; p.dilation = dilation;
    p.with_activation = conv_act; p.activation_negative_slope = conv_slp; p.eltw_activation = eltw_act; p.eltw_activation_negative_slope = eltw_slp;
    p.output_data_type = odt;
    return p;
}
primitive eltwise(const std::string& id, const std::string& input, const std::string& input2, eltwise_mode mode, bool with_activation,
                  float slp, const std::string& oc, float oqf, bool quantized)
{
    primitive p; p.type = "eltwise"; p.id = id; p.input = {input, input2}; p.mode = mode; p.with_activation = with_activation;
    p.activation_negative_slope = slp; p.output_calibration_factors = oc; p.output_quantization_factor = oqf;
    p.eltw_quantized = quantized || !oc.empty() || oqf != 1.0f;
    return p;
}
primitive activation(const std::string& id, const std::string& input, int32_t func, float a, float b)
{
    primitive p; p.type = "activation"; p.id = id; p.input = {input}; p.activation_func = func; p.act_a = a; p.act_b = b; return p;
}
primitive pooling(const std::string& id, const std::string& input, pooling_mode mode, tensor size, tensor stride, tensor input_offset)
{
    primitive p; p.type = "pooling"; p.id = id; p.input = {input}; p.pool_mode = mode; p.size = size; p.stride = stride; p.input_offset = input_offset; return p;
}
primitive global_pooling(const std::string& id, const std::string& input, pooling_mode mode)
{
    primitive p; p.type = "pooling"; p.id = id; p.input = {input}; p.pool_mode = mode; p.global_pooling = true; return p;
}
primitive fully_connected(const std::string& id, const std::string& input, const std::string& weights, const std::string& bias,
                          const std::string& wq, const std::string& oc, float iqf, bool with_activation, float slp)
{
    primitive p; p.type = "fully_connected"; p.id = id; p.input = {input}; p.weights = weights; p.bias = bias; p.weights_quantization_factors = wq;
    p.output_calibration_factors = oc; p.input_quantization_factor = iqf; p.with_activation = with_activation; p.activation_negative_slope = slp;
    return p;
}
primitive softmax(const std::string& id, const std::string& input, int32_t dimension)
{
    primitive p; p.type = "softmax"; p.id = id; p.input = {input}; p.softmax_dimension = dimension; return p;
}
primitive lrn(const std::string& id, const std::string& input, uint32_t size, float k, float alpha, float beta)
{
    primitive p; p.type = "lrn"; p.id = id; p.input = {input}; p.lrn_size = size; p.lrn_k = k; p.lrn_alpha = alpha; p.lrn_beta = beta; return p;
}

primitive concatenation(const std::string& id, const std::vector<std::string>& inputs, int32_t axis)
{
    primitive p; p.type = "concatenation"; p.id = id; p.input = inputs; p.concat_axis = axis; return p;
}

void topology::add(const primitive& p)
{
    if (p.id.empty()) throw error("topology: primitive without id", CLDNN_B200_INVALID_ARG);
    for (auto& q : prims) if (q.id == p.id) throw error("topology: primitive id '" + p.id + "' is not unique", CLDNN_B200_INVALID_ARG);
    prims.push_back(p);
}

// --------------------------------------------------------------------------------------
// program nodes
// --------------------------------------------------------------------------------------
struct block;
struct node {
    primitive p;
    std::vector<node*> deps;            // data inputs
    std::vector<node*> users;
    node *weights = nullptr, *bias = nullptr, *wq = nullptr, *oc = nullptr, *ec = nullptr;
    layout out;
    bool is_output = false;
    bool removed = false;
    bool in_place = false;              // fused_conv_eltwise: output written over the second input (second_input_in_output)
    std::string answers_for;            // user-visible id this node's output stands for (after fusing / reorder insertion)
    std::string fused_ids;              // ids of primitives folded into this one
    // fused activations (prepare_primitive_fusing)
    int32_t act = CLDNN_B200_ACT_NONE; float act_m = 0.f, act_n = 0.f;
    int32_t eltw_act = CLDNN_B200_ACT_NONE; float eltw_m = 0.f, eltw_n = 0.f;
    // execution
    memory mem;                         // output memory
    memory packed_weights;              // weights re-laid for the chosen kernel
    std::shared_ptr<struct block> scratch; // kernel workspace (kernel_scratch_bytes)
    std::string kernel; int32_t tune = 0;
    cldnn_b200_prepared prepared = nullptr;
    std::vector<cldnn_b200_prepared> more_prepared;   // further launches of the same primitive (concatenation: one copy per input)
    int order = -1;
    bool constant() const { return p.type == "data"; }
};

static int32_t act_from_slope(bool with, float slope, float& m)
{
    // convert_activation_func_params (src/include/kernel_selector_helper.h): slope 0 -> RELU, else RELU_NEGATIVE_SLOPE
    if (!with) return CLDNN_B200_ACT_NONE;
    m = slope;
    return slope == 0.0f ? CLDNN_B200_ACT_RELU : CLDNN_B200_ACT_RELU_NEGATIVE_SLOPE;
}

class network_impl {
public:
    std::shared_ptr<engine_impl> eng;
    build_options opts;
    std::vector<std::unique_ptr<node>> nodes;
    std::map<std::string, node*> by_id;
    std::vector<node*> order;
    std::vector<std::string> output_ids;
    cldnn_b200_graph graph = nullptr;
    bool inputs_changed = true;
    uint64_t launches = 0;
    size_t pool_bytes = 0;
    std::map<std::string, std::pair<std::string, int>> tuning_cache;   // hash -> (kernel, tune)
    std::map<std::string, std::map<std::string, std::pair<std::string, int>>> other_devices;   // sections of the cache file for other SM counts, written back untouched
    std::vector<std::pair<cldnn_b200_event, cldnn_b200_event>> prof_events;   // per node of `order`, profiling only
    bool cache_dirty = false;

    ~network_impl()
    {
        if (eng && eng->ctx) cldnn_b200_ctx_sync(eng->ctx);
        if (graph) cldnn_b200_graph_destroy(graph);
        for (auto& n : nodes) { if (n->prepared) cldnn_b200_prepared_destroy(n->prepared); for (auto pr : n->more_prepared) cldnn_b200_prepared_destroy(pr); }
        for (auto& pe : prof_events) { cldnn_b200_event_destroy(pe.first); cldnn_b200_event_destroy(pe.second); }
    }

    node* get(const std::string& id)
    {
        auto it = by_id.find(id);
        if (it == by_id.end()) throw error("primitive '" + id + "' is not in the topology", CLDNN_B200_INVALID_ARG);
        return it->second;
    }
    node* opt(const std::string& id) { return id.empty() ? nullptr : get(id); }
    node* add_node(const primitive& p)
    {
        nodes.emplace_back(new node()); node* n = nodes.back().get(); n->p = p; by_id[p.id] = n; return n;
    }

    void build(const topology& topo);
    void link();
    void sort();
    void relayout() { for (node* n : order) calc_layout(n); }
    void calc_layout(node* n);
    void fuse_activations();
    void fuse_conv_eltwise();
    void select_layouts();
    void conv_eltw_read_write_opt();
    void replace_dep(node* consumer, node* from, node* to) { for (auto& id : consumer->p.input) if (id == from->p.id) id = to->p.id; }
    void allocate_and_prepare();
    void prepare_kernel(node* n);
    void pick_kernel(node* n, const std::vector<std::string>& candidates, void* params, size_t params_size, const void* key_params,
                     const cldnn_b200_args& args, const std::function<void(int)>& set_tune, bool time_all = false);
    memory pack_conv_weights(node* n, int32_t stored_ifm, int32_t groups = 1);
    void load_cache(); void save_cache();
    void execute();
    void run_prepared(node* n)
    {
        if (n->prepared) check(cldnn_b200_run(n->prepared), "run " + n->p.id);
        for (auto pr : n->more_prepared) check(cldnn_b200_run(pr), "run " + n->p.id);
    }
};

void network_impl::link()
{
    for (auto& up : nodes) { up->deps.clear(); up->users.clear(); }
    for (auto& up : nodes) {
        node* n = up.get(); if (n->removed) continue;
        for (auto& id : n->p.input) { node* d = get(id); n->deps.push_back(d); d->users.push_back(n); }
        n->weights = opt(n->p.weights); n->bias = opt(n->p.bias); n->wq = opt(n->p.weights_quantization_factors);
        n->oc = opt(n->p.output_calibration_factors); n->ec = opt(n->p.eltw_output_calibration_factors);
    }
}

void network_impl::sort()
{
    // processing order: topological, stable with respect to the topology's own order
    order.clear();
    std::set<node*> done;
    std::function<void(node*)> visit = [&](node* n) {
        if (done.count(n) || n->removed) return;
        done.insert(n);
        for (node* d : n->deps) visit(d);
        for (node* d : {n->weights, n->bias, n->wq, n->oc, n->ec}) if (d) visit(d);
        order.push_back(n);
    };
    for (auto& up : nodes) visit(up.get());
    for (size_t i = 0; i < order.size(); ++i) order[i]->order = (int)i;
}

void network_impl::calc_layout(node* n)
{
    const primitive& p = n->p;
    if (p.type == "input_layout") { n->out = p.target; return; }
    if (p.type == "data") { n->out = p.mem.get_layout(); return; }
    const layout& in = n->deps.at(0)->out;
    layout o = in; o.data_padding = padding();
    if (p.type == "reorder") {
        o.fmt = p.target.fmt == format::any ? in.fmt : p.target.fmt;
        o.data_type = p.target.data_type == data_types::none ? in.data_type : p.target.data_type;
    } else if (p.type == "convolution" || p.type == "fused_conv_eltwise") {
        // convolution_inst::calc_output_layout, src/convolution.cpp:32-130
        if (!n->weights) throw error(p.id + ": weights are required", CLDNN_B200_INVALID_ARG);
        const layout& w = n->weights->out;
        if (p.stride.x < 1 || p.stride.y < 1) throw error(p.id + ": stride must be positive (>= 1)", CLDNN_B200_INVALID_ARG);
        if (p.dilation.x < 1 || p.dilation.y < 1) throw error(p.id + ": dilation must be positive (>= 1)", CLDNN_B200_INVALID_ARG);
        if (2 * p.input_offset.x > in.size.x || 2 * p.input_offset.y > in.size.y) throw error(p.id + ": input offset is greater than input data range", CLDNN_B200_INVALID_ARG);
        if (p.groups < 1 || w.size.feature * p.groups != in.size.feature)
            throw error(p.id + ": weights input features (" + std::to_string(w.size.feature) + " x groups " + std::to_string(p.groups) + ") do not match input features " + std::to_string(in.size.feature), CLDNN_B200_DIMENSION_MISMATCH);
        o.size.feature = w.size.batch;
        o.size.x = conv_output_size(in.size.x, w.size.x, p.input_offset.x, p.stride.x, p.dilation.x);
        o.size.y = conv_output_size(in.size.y, w.size.y, p.input_offset.y, p.stride.y, p.dilation.y);
        if (o.size.x <= 0 || o.size.y <= 0) throw error(p.id + ": filter does not fit the input", CLDNN_B200_UNSUPPORTED_SIZE);
        if (p.output_data_type != data_types::none) o.data_type = p.output_data_type;
        if (n->bias && (int)n->bias->out.count() != o.size.feature) throw error(p.id + ": bias size does not match output features", CLDNN_B200_DIMENSION_MISMATCH);
        if (n->wq && (int)n->wq->out.count() != o.size.feature) throw error(p.id + ": quantization factors do not match output features", CLDNN_B200_DIMENSION_MISMATCH);
    } else if (p.type == "pooling") {
        // pooling_inst::calc_output_layout, src/pooling.cpp:31-97
        const int sx = p.global_pooling ? in.size.x : p.size.x, sy = p.global_pooling ? in.size.y : p.size.y;
        if (p.stride.x < 1 || p.stride.y < 1 || sx < 1 || sy < 1) throw error(p.id + ": stride and window size must be positive (>= 1)", CLDNN_B200_INVALID_ARG);
        if (-p.input_offset.x > sx || -p.input_offset.y > sy) throw error(p.id + ": first pool is outside of image", CLDNN_B200_INVALID_ARG);
        o.size.x = p.global_pooling ? 1 : pool_output_size(in.size.x, sx, p.input_offset.x, p.stride.x);
        o.size.y = p.global_pooling ? 1 : pool_output_size(in.size.y, sy, p.input_offset.y, p.stride.y);
    } else if (p.type == "fully_connected") {
        // fully_connected_inst::calc_output_layout, src/fully_connected.cpp:59-80
        if (!n->weights) throw error(p.id + ": weights are required", CLDNN_B200_INVALID_ARG);
        const layout& w = n->weights->out;
        if ((int64_t)w.size.feature * w.size.x * w.size.y != (int64_t)in.size.feature * in.size.x * in.size.y)
            throw error(p.id + ": weights do not match the input size", CLDNN_B200_DIMENSION_MISMATCH);
        o.size = tensor(in.size.batch, w.size.batch, 1, 1);
        if (o.fmt == format::byxf) o.fmt = format::bfyx;
    } else if (p.type == "eltwise") {
        const layout& b = n->deps.at(1)->out;
        o.size.x = std::max(in.size.x, b.size.x); o.size.y = std::max(in.size.y, b.size.y);
        o.size.feature = std::max(in.size.feature, b.size.feature); o.size.batch = std::max(in.size.batch, b.size.batch);
    } else if (p.type == "concatenation") {
        // concatenation_inst::calc_output_layout (src/concatenation.cpp:34-63): the first input's layout with the sizes along the axis summed
        if (p.concat_axis < 0 || p.concat_axis > 3) throw error(p.id + ": concatenation axis must be b, f, x or y", CLDNN_B200_INVALID_ARG);
        auto dim = [&](tensor& t) -> int32_t& { return p.concat_axis == 0 ? t.batch : (p.concat_axis == 1 ? t.feature : (p.concat_axis == 2 ? t.x : t.y)); };
        int32_t total = 0;
        for (node* d : n->deps) {
            tensor a = d->out.size, b = in.size;
            total += dim(a);
            dim(a) = 0; dim(b) = 0;
            if (!(a == b)) throw error(p.id + ": inputs differ outside the concatenation axis", CLDNN_B200_DIMENSION_MISMATCH);
            if (d->out.data_type != in.data_type) throw error(p.id + ": inputs differ in data type", CLDNN_B200_INVALID_ARG);
        }
        dim(o.size) = total;
    } else if (p.type == "activation" || p.type == "softmax" || p.type == "lrn") {
        // same shape and type
    } else throw error("primitive type '" + p.type + "' is outside the supported path", CLDNN_B200_UNSUPPORTED_FORMAT);
    if (p.type == "fused_conv_eltwise") {
        const layout& r = n->deps.at(1)->out;
        if (r.size.feature != o.size.feature || r.size.batch != o.size.batch || r.size.x / std::max(1, p.eltw_stride.x) < o.size.x || r.size.y / std::max(1, p.eltw_stride.y) < o.size.y)
            throw error(p.id + ": second input does not match the convolution output", CLDNN_B200_DIMENSION_MISMATCH);
    }
    n->out = o;
}

// prepare_primitive_fusing::run, src/graph_optimizer/prepare_primitive_fusing.cpp:396-433: a standalone activation whose
// only producer has a single user and no activation of its own is folded into the producer.
void network_impl::fuse_activations()
{
    for (size_t i = 0; i < nodes.size(); ++i) {
        node* a = nodes[i].get();
        if (a->removed || a->p.type != "activation" || a->deps.size() != 1) continue;
        node* prod = a->deps[0];
        const std::string& t = prod->p.type;
        if (!(t == "convolution" || t == "fused_conv_eltwise" || t == "eltwise" || t == "fully_connected" || t == "pooling")) continue;
        if (prod->users.size() != 1 || prod->is_output) continue;
        const bool on_eltw = t == "fused_conv_eltwise";
        int32_t& slot = on_eltw ? prod->eltw_act : prod->act;
        const bool own = on_eltw ? prod->p.eltw_activation : prod->p.with_activation;
        if (slot != CLDNN_B200_ACT_NONE || own) continue;
        if (is_int8(prod->out.data_type) && (t == "pooling" || t == "fully_connected" || t == "eltwise") && a->p.activation_func != CLDNN_B200_ACT_RELU) continue;
        slot = a->p.activation_func;
        if (on_eltw) { prod->eltw_m = a->p.act_a; prod->eltw_n = a->p.act_b; } else { prod->act_m = a->p.act_a; prod->act_n = a->p.act_b; }
        for (auto& vp : nodes) for (auto& id : vp->p.input) if (id == a->p.id) id = prod->p.id;
        prod->fused_ids += (prod->fused_ids.empty() ? "" : ",") + a->p.id;
        if (a->is_output) { prod->is_output = true; prod->answers_for = a->answers_for.empty() ? a->p.id : a->answers_for; }
        by_id[a->p.id] = prod;
        a->removed = true;
        link();
    }
    sort(); relayout();
}

// prepare_conv_eltw_fusing::fuse_conv_eltwise, src/graph_optimizer/prepare_primitive_fusing.cpp:181-337:
// convolution -> eltwise(sum) [-> relu, already folded into the eltwise] becomes one fused_conv_eltwise.  The reference
// restricts this to 1x1 stride-1 convolutions in five (format, type) pairs (:197-217); fuse_any_conv_eltwise lifts the
// restriction because the fused kernel here handles every filter.
void network_impl::fuse_conv_eltwise()
{
    for (size_t i = 0; i < nodes.size(); ++i) {
        node* e = nodes[i].get();
        if (e->removed || e->p.type != "eltwise" || e->p.mode != eltwise_mode::sum || e->deps.size() != 2) continue;
        node* a = e->deps[0]; node* b = e->deps[1];
        auto fusable = [&](node* c) {
            if (c->p.type != "convolution" || c->users.size() != 1 || c->is_output || c->p.groups != 1) return false;
            if (!opts.fuse_any_conv_eltwise) {
                const layout& w = c->weights->out;
                if (w.size.x != 1 || w.size.y != 1 || c->p.stride.x != 1 || c->p.stride.y != 1) return false;
            }
            return c->out.size == e->out.size;
        };
        // fuse the input that executes later (:246-262) so the other one is already computed
        node* conv = nullptr;
        if (fusable(a) && fusable(b)) conv = a->order > b->order ? a : b;
        else if (fusable(a)) conv = a;
        else if (fusable(b)) conv = b;
        if (!conv) continue;
        node* other = conv == a ? b : a;
        if (!(other->out.size == e->out.size)) continue;
        const bool int8 = is_int8(conv->deps[0]->out.data_type);
        if (int8 && conv->p.weights_quantization_factors.empty()) continue;
        primitive f = conv->p;
        f.type = "fused_conv_eltwise"; f.id = e->p.id;
        f.input = {conv->p.input[0], other->p.id};
        f.eltw_output_calibration_factors = e->p.output_calibration_factors;
        f.eltw_activation = e->p.with_activation; f.eltw_activation_negative_slope = e->p.activation_negative_slope;
        f.output_data_type = e->out.data_type;
        f.non_conv_scale = 1.0f; f.eltw_stride = tensor(1, 1, 1, 1);
        const std::string conv_fused = conv->fused_ids, e_fused = e->fused_ids, conv_id = conv->p.id;
        const int32_t ca = conv->act; const float cm = conv->act_m, cn = conv->act_n;
        const int32_t ea = e->act; const float em = e->act_m, en = e->act_n;
        const bool e_out = e->is_output; const std::string e_ans = e->answers_for;
        conv->removed = true; e->removed = true;
        node* nf = add_node(f);                                     // may reallocate `nodes`; a, b, e, conv stay valid (unique_ptr)
        nf->act = ca; nf->act_m = cm; nf->act_n = cn;
        nf->eltw_act = ea; nf->eltw_m = em; nf->eltw_n = en;
        nf->is_output = e_out; nf->answers_for = e_ans;
        nf->fused_ids = conv_id + (conv_fused.empty() ? "" : "," + conv_fused) + (e_fused.empty() ? "" : "," + e_fused);
        link(); sort(); relayout();
    }
}

// layout_optimizer::get_expected_layout + reorder_inputs::run (src/layout_optimizer.cpp:187-291,
// src/graph_optimizer/reorder_inputs.cpp:43-318), extended with a rule for 8-bit data, which the reference leaves in the
// caller's format (:239-249): quantised 8-bit convolutions, and the pooling / eltwise / activation between them, run in
// byxf_af32 (features innermost, padded to 32), the layout the tensor-core kernel reads with TMA.
void network_impl::select_layouts()
{
    // an inner product whose weights have the input's feature and map sizes is a GEMM over the flattened byxf input
    auto fc_weights_match = [&](node* n) {
        if (!n->weights) return false;
        const layout& in = n->deps[0]->out; const layout& w = n->weights->out;
        return w.size.feature == in.size.feature && w.size.x == in.size.x && w.size.y == in.size.y;
    };
    auto conv_like = [&](node* n) {
        const std::string& t = n->p.type;
        if (n->deps.empty()) return false;
        // fp16 convolutions and inner products run on the tensor cores from the same feature-innermost padded layout
        if (n->deps[0]->out.data_type == data_types::f16) {
            if (t == "fully_connected") return n->weights && n->weights->out.data_type == data_types::f16 && !n->wq && fc_weights_match(n);
            return (t == "convolution" || t == "fused_conv_eltwise") && n->p.groups >= 1 && n->p.groups <= 4 && n->weights && n->weights->out.data_type == data_types::f16 && !n->wq;
        }
        if (!is_int8(n->deps[0]->out.data_type)) return false;
        // dense convolutions go to the tensor cores, depthwise ones (one feature per group) to the byxf depthwise kernel
        if (t == "convolution" && n->p.groups > 4) return n->wq != nullptr && n->weights && n->weights->out.size.feature == 1 && n->p.groups == n->deps[0]->out.size.feature &&
                                                          n->weights->out.size.batch == n->p.groups && n->p.groups % 4 == 0;
        if (t == "convolution" || t == "fused_conv_eltwise") return n->p.groups >= 1 && n->p.groups <= 4 && n->wq != nullptr;
        if (t == "fully_connected") return n->wq && n->bias && n->bias->out.data_type == data_types::f32 && fc_weights_match(n);
        return false;
    };
    // a convolution over a planar few-feature input (the image) has a kernel that builds its operand from bfyx itself
    // (conv_i8_first: 8-bit, filters up to 8 taps wide; conv_first_tc: fp16 or 8-bit, K = C*kh*kw packed densely)
    auto first_layer = [&](node* n, node* d) {
        if (n->p.type != "convolution" || d->out.fmt != format::bfyx || !n->weights || n->p.groups != 1) return false;
        const layout& w = n->weights->out;
        const bool i8 = is_int8(d->out.data_type) && n->wq != nullptr && w.data_type == data_types::i8;
        const bool f16 = d->out.data_type == data_types::f16 && w.data_type == data_types::f16 && !n->wq;
        if ((!i8 && !f16) || w.size.batch % 32 || w.size.batch > 256) return false;
        const bool simple_act = (n->act == CLDNN_B200_ACT_NONE || n->act == CLDNN_B200_ACT_RELU || n->act == CLDNN_B200_ACT_CLAMP) && !n->p.activation_negative_slope;
        if (i8 && w.size.x <= 8 && d->out.size.feature * w.size.y * 8 <= 256 && n->p.dilation.x == 1 && n->p.dilation.y == 1 && simple_act) return true;
        const int64_t qe = f16 ? 4 : 8;                                                  // taps per 8-byte quantum of a padded filter row
        const int64_t cores = ((int64_t)d->out.size.feature * w.size.y * ((w.size.x + qe - 1) / qe) + 3) / 4 * 2;
        const int64_t image = w.size.batch * cores * 16;                                  // resident weights in shared memory
        return d->out.size.feature <= 4 && cores <= 256 && image <= 120 * 1024 && (f16 || simple_act);
    };
    std::set<node*> chosen;
    for (node* n : order) {
        if (n->removed || n->constant() || n->p.type == "input_layout" || n->deps.empty()) continue;
        if (conv_like(n)) chosen.insert(n);
        else if ((n->p.type == "pooling" || n->p.type == "eltwise" || n->p.type == "activation" || n->p.type == "lrn" || n->p.type == "concatenation") &&
                 (is_int8(n->deps[0]->out.data_type) || n->deps[0]->out.data_type == data_types::f16)) {
            bool all = true; for (node* d : n->deps) all &= chosen.count(d) > 0;
            if (all) chosen.insert(n);
        }
    }
    std::vector<node*> snapshot(order);
    for (node* n : snapshot) {
        if (!chosen.count(n)) continue;
        for (node* d : std::vector<node*>(n->deps)) {
            if (chosen.count(d) || d->out.fmt == format::byxf_af32) continue;
            if (first_layer(n, d)) continue;                        // conv_i8_first reads the planar input directly
            const std::string rid = d->p.id + "_to_byxf_af32";
            node* r = by_id.count(rid) ? by_id[rid] : add_node(reorder(rid, d->p.id, format::byxf_af32, data_types::none));
            replace_dep(n, d, r);
        }
        // a reorder consumer reads any layout through pitches: it needs no conversion back in front of it
        bool back = n->is_output;
        for (node* u : n->users) back |= chosen.count(u) == 0 && u->p.type != "reorder";
        if (back) {
            const int32_t user_fmt = n->out.fmt == format::byxf_af32 ? (int32_t)format::bfyx : n->out.fmt;
            node* r = add_node(reorder(n->p.id + "_from_byxf_af32", n->p.id, user_fmt, data_types::none));
            for (node* u : std::vector<node*>(n->users)) if (!chosen.count(u) && u->p.type != "reorder") replace_dep(u, n, r);
            if (n->is_output) { r->is_output = true; r->answers_for = n->answers_for.empty() ? n->p.id : n->answers_for; n->is_output = false; }
        }
    }
    link(); sort();
    for (node* n : order) { calc_layout(n); if (chosen.count(n)) n->out.fmt = format::byxf_af32; }
}

// prepare_conv_eltw_read_write_opt (src/graph_optimizer/prepare_primitive_fusing.cpp:468-555): when the result of a
// fused_conv_eltwise has exactly the layout of its second input, the two share one buffer and the kernel reads the residual
// from the place it then writes (second_input_in_output).  The reference re-points every other reader of the second input at
// the shared buffer whatever its place in the execution order; here the buffer is shared only when every other reader runs
// before the fused primitive, so nobody can see the overwritten values.
void network_impl::conv_eltw_read_write_opt()
{
    for (node* n : order) {
        if (n->removed || n->p.type != "fused_conv_eltwise" || n->deps.size() != 2) continue;
        node* r = n->deps[1];
        if (r == n->deps[0] || r->constant() || r->p.type == "input_layout" || r->is_output) continue;
        if (!(r->out == n->out) || n->p.eltw_stride.x != 1 || n->p.eltw_stride.y != 1) continue;
        bool safe = true;
        for (node* u : r->users) safe &= u == n || u->order < n->order;
        if (!safe) continue;
        n->in_place = true;
    }
}

// --------------------------------------------------------------------------------------
// tuning cache: same schema as the reference's cache.json (kernel_selector/core/auto_tuner.cpp:72-118), keyed by the
// number of compute units (SMs) and a hash of the launch constants.
// --------------------------------------------------------------------------------------
static std::string fnv1a_hex(const void* data, size_t n, const std::string& salt)
{
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](const uint8_t* p, size_t k) { for (size_t i = 0; i < k; ++i) { h ^= p[i]; h *= 1099511628211ull; } };
    mix((const uint8_t*)salt.data(), salt.size()); mix((const uint8_t*)data, n);
    char buf[32]; snprintf(buf, sizeof(buf), "%016llx", (unsigned long long)h); return buf;
}

// A small JSON reader for the cache file (the reference parses cache.json with rapidjson, auto_tuner.cpp:72-104): values
// are objects, arrays, strings, numbers, true / false / null; anything malformed makes the whole file unusable (and says so)
// instead of silently dropping entries.
namespace {
struct json_value {
    enum kind_t { null_v, bool_v, number_v, string_v, array_v, object_v } kind = null_v;
    double number = 0.0; bool boolean = false; std::string text;
    std::vector<json_value> items;                              // array
    std::vector<std::pair<std::string, json_value>> members;    // object, in file order
    const json_value* find(const std::string& key) const { for (auto& m : members) if (m.first == key) return &m.second; return nullptr; }
};
struct json_reader {
    const std::string& s; size_t i = 0;
    explicit json_reader(const std::string& text) : s(text) {}
    [[noreturn]] void bad(const char* what) const { throw error(std::string("tuning cache: ") + what + " at offset " + std::to_string(i), CLDNN_B200_INVALID_ARG); }
    void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
    bool eat(char c) { ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
    std::string string_body()
    {
        std::string out;
        while (true) {
            if (i >= s.size()) bad("unterminated string");
            const char c = s[i++];
            if (c == '"') return out;
            if (c != '\\') { out.push_back(c); continue; }
            if (i >= s.size()) bad("unterminated escape");
            const char e = s[i++];
            switch (e) {
            case '"': out.push_back('"'); break; case '\\': out.push_back('\\'); break; case '/': out.push_back('/'); break;
            case 'b': out.push_back('\b'); break; case 'f': out.push_back('\f'); break; case 'n': out.push_back('\n'); break;
            case 'r': out.push_back('\r'); break; case 't': out.push_back('\t'); break;
            case 'u': {
                if (i + 4 > s.size()) bad("short \\u escape");
                const unsigned cp = (unsigned)std::strtoul(s.substr(i, 4).c_str(), nullptr, 16); i += 4;
                if (cp < 0x80) out.push_back((char)cp);
                else if (cp < 0x800) { out.push_back((char)(0xc0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3f))); }
                else { out.push_back((char)(0xe0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3f))); out.push_back((char)(0x80 | (cp & 0x3f))); }
                break;
            }
            default: bad("unknown escape");
            }
        }
    }
    json_value value(int depth = 0)
    {
        if (depth > 32) bad("nesting too deep");
        ws();
        if (i >= s.size()) bad("unexpected end");
        json_value v;
        const char c = s[i];
        if (c == '{') {
            ++i; v.kind = json_value::object_v;
            if (eat('}')) return v;
            do {
                ws();
                if (i >= s.size() || s[i] != '"') bad("object key expected");
                ++i;
                std::string key = string_body();
                if (!eat(':')) bad("':' expected");
                v.members.push_back({key, value(depth + 1)});
            } while (eat(','));
            if (!eat('}')) bad("'}' expected");
            return v;
        }
        if (c == '[') {
            ++i; v.kind = json_value::array_v;
            if (eat(']')) return v;
            do v.items.push_back(value(depth + 1)); while (eat(','));
            if (!eat(']')) bad("']' expected");
            return v;
        }
        if (c == '"') { ++i; v.kind = json_value::string_v; v.text = string_body(); return v; }
        if (s.compare(i, 4, "true") == 0) { i += 4; v.kind = json_value::bool_v; v.boolean = true; return v; }
        if (s.compare(i, 5, "false") == 0) { i += 5; v.kind = json_value::bool_v; return v; }
        if (s.compare(i, 4, "null") == 0) { i += 4; return v; }
        char* end = nullptr;
        v.number = std::strtod(s.c_str() + i, &end);
        if (end == s.c_str() + i) bad("value expected");
        i = (size_t)(end - s.c_str()); v.kind = json_value::number_v;
        return v;
    }
    json_value document() { json_value v = value(); ws(); if (i != s.size()) bad("trailing characters"); return v; }
};
}  // namespace

// { "<compute units>": { "<hash of the launch constants>": ["<kernel>", <tuning index>], ... }, ... }: the entries under this
// device's SM count are taken, other devices' sections are kept out.
std::map<std::string, std::map<std::string, std::pair<std::string, int>>> parse_tuning_cache(const std::string& text)
{
    std::map<std::string, std::map<std::string, std::pair<std::string, int>>> out;
    if (text.find_first_not_of(" \n\t\r") == std::string::npos) return out;   // an empty file is an empty cache
    const json_value doc = json_reader(text).document();
    if (doc.kind != json_value::object_v) throw error("tuning cache: the top level must be an object keyed by compute-unit count", CLDNN_B200_INVALID_ARG);
    for (auto& dev : doc.members) {
        if (dev.second.kind != json_value::object_v) throw error("tuning cache: device section '" + dev.first + "' must be an object", CLDNN_B200_INVALID_ARG);
        auto& section = out[dev.first];
        for (auto& m : dev.second.members) {
            const json_value& e = m.second;
            if (e.kind != json_value::array_v || e.items.size() != 2 || e.items[0].kind != json_value::string_v || e.items[1].kind != json_value::number_v)
                throw error("tuning cache: entry '" + m.first + "' must be [\"kernel\", index]", CLDNN_B200_INVALID_ARG);
            section[m.first] = {e.items[0].text, (int)e.items[1].number};
        }
    }
    return out;
}

void network_impl::load_cache()
{
    tuning_cache.clear(); other_devices.clear();
    if (opts.tuning_cache_path.empty()) return;
    std::ifstream f(opts.tuning_cache_path);
    if (!f) return;
    std::stringstream ss; ss << f.rdbuf();
    other_devices = parse_tuning_cache(ss.str());
    const std::string mine = std::to_string(eng->info.cores_count);
    auto it = other_devices.find(mine);
    if (it != other_devices.end()) { tuning_cache = it->second; other_devices.erase(it); }
}

void network_impl::save_cache()
{
    if (opts.tuning_cache_path.empty() || !cache_dirty) return;
    std::ofstream f(opts.tuning_cache_path);
    if (!f) throw error("cannot write tuning cache '" + opts.tuning_cache_path + "'", CLDNN_B200_ERROR);
    auto section = [&](const std::string& key, const std::map<std::string, std::pair<std::string, int>>& entries, bool last) {
        f << "  \"" << key << "\": {\n";
        size_t k = 0;
        for (auto& e : entries)
            f << "    \"" << e.first << "\": [\"" << e.second.first << "\", " << e.second.second << "]" << (++k < entries.size() ? "," : "") << "\n";
        f << "  }" << (last ? "" : ",") << "\n";
    };
    f << "{\n";
    for (auto& o : other_devices) section(o.first, o.second, false);
    section(std::to_string(eng->info.cores_count), tuning_cache, true);
    f << "}\n";
    cache_dirty = false;
}

// kernel_selector_base::GetNaiveBestKernel / GetAutoTuneBestKernel (kernel_selector/core/kernel_selector.cpp:80-280):
// candidates are tried in priority order and the first whose Validate() accepts the constants wins, unless tuning is on,
// in which case every (kernel, tuning variant) is timed on the device and the fastest is kept and cached.
// `time_all`: the candidates are alternatives of equal standing (direct and Winograd convolution), all of them are timed;
// otherwise later candidates are fallbacks that are only reached when the earlier ones refuse the constants.
void network_impl::pick_kernel(node* n, const std::vector<std::string>& candidates, void* params, size_t psize, const void* key_params,
                               const cldnn_b200_args& args, const std::function<void(int)>& set_tune, bool time_all)
{
    if (!opts.force_kernel.empty()) {                               // "<primitive id>=<kernel>[:tune],..."
        std::stringstream ss(opts.force_kernel); std::string item;
        while (std::getline(ss, item, ',')) {
            const size_t eq = item.find('='); if (eq == std::string::npos || item.substr(0, eq) != n->p.id) continue;
            std::string k = item.substr(eq + 1); int tune = 0; const size_t colon = k.find(':');
            if (colon != std::string::npos) { tune = std::atoi(k.substr(colon + 1).c_str()); k = k.substr(0, colon); }
            bool known = false; for (auto& c : candidates) known |= c == k;
            if (!known) throw error(n->p.id + ": forced kernel '" + k + "' does not implement " + n->p.type, CLDNN_B200_INVALID_ARG);
            n->kernel = k; n->tune = tune; set_tune(tune); return;
        }
    }
    set_tune(0);
    // the key carries the generation of the kernel set: timings taken on older kernels must not be reused.  `key_params`:
    // the constants with the fields that do not bear on the choice cleared (same size as `params`)
    const std::string hash = fnv1a_hex(key_params ? key_params : params, psize, n->p.type + "#g3");
    if (opts.tuning != tuning_mode::tuning_disabled) {
        auto it = tuning_cache.find(hash);
        if (it != tuning_cache.end()) {
            bool known = false; for (auto& c : candidates) known |= c == it->second.first;
            set_tune(it->second.second);
            int32_t yes = 0;
            if (known && cldnn_b200_kernel_supports(eng->kernel(it->second.first), params, psize, &yes) == CLDNN_B200_SUCCESS && yes) {
                n->kernel = it->second.first; n->tune = it->second.second; return;
            }
            set_tune(0);
        }
    }
    if (opts.tuning == tuning_mode::tuning_tune_and_cache) {
        uint64_t best_ns = ~0ull; std::string best_k; int best_t = 0;
        for (auto& cand : candidates) {
            cldnn_b200_kernel k = eng->kernel(cand);
            set_tune(0);
            int32_t count = 0;
            if (cldnn_b200_kernel_tune_count(k, params, psize, &count) != CLDNN_B200_SUCCESS || count <= 0) continue;
            for (int t = count > 1 ? 1 : 0; t < count; ++t) {
                set_tune(t);
                int32_t yes = 0;
                if (cldnn_b200_kernel_supports(k, params, psize, &yes) != CLDNN_B200_SUCCESS || !yes) continue;
                cldnn_b200_prepared pr = nullptr;
                if (cldnn_b200_prepare(k, params, psize, &args, &pr) != CLDNN_B200_SUCCESS) continue;
                uint64_t ns = 0;
                // kernel_runner times 3 runs (src/gpu/kernel_runner.h:37-38); launches here last tens of microseconds, so more
                // runs are averaged to keep the choice stable
                const int32_t st = cldnn_b200_time(pr, 3, 12, &ns);
                cldnn_b200_prepared_destroy(pr);
                if (st == CLDNN_B200_SUCCESS && ns < best_ns) { best_ns = ns; best_k = cand; best_t = t; }
            }
            if (!best_k.empty() && !time_all) break;                 // a preferred kernel took the job: the fallback is not timed
        }
        if (!best_k.empty()) {
            n->kernel = best_k; n->tune = best_t; set_tune(best_t);
            tuning_cache[hash] = {best_k, best_t}; cache_dirty = true;
            return;
        }
    }
    set_tune(0);
    for (auto& cand : candidates) {
        int32_t yes = 0;
        if (cldnn_b200_kernel_supports(eng->kernel(cand), params, psize, &yes) == CLDNN_B200_SUCCESS && yes) { n->kernel = cand; n->tune = 0; return; }
    }
    throw error(n->p.id + ": cannot find a proper kernel with these arguments", CLDNN_B200_ERROR);
}

// post_optimize_weights (src/graph_optimizer/post_optimize_weights.cpp:36-64) + generic_layer: the chosen kernel's
// weights layout (oyxi, input features padded to the activation's stored count) is produced once, at build time, by the
// reorder kernel.
memory network_impl::pack_conv_weights(node* n, int32_t stored_ifm, int32_t groups)
{
    const layout& w = n->weights->out;                            // [o = batch][i = feature][y][x], caller's format (bfyx)
    layout packed(w.data_type, format::byxf, tensor(w.size.batch, stored_ifm, w.size.x, w.size.y));
    memory m; m.impl = std::make_shared<memory_impl>(); m.impl->l = packed; m.impl->blk = new_block(eng, packed.bytes_count());
    cldnn_b200_args a{}; a.input0 = n->weights->mem.device_ptr(); a.output = m.device_ptr();
    if (groups <= 1) {
        cldnn_b200_reorder_params rp{};
        rp.in = w.desc(); rp.out = packed.desc();
        check(cldnn_b200_launch(eng->kernel("reorder_ref"), &rp, sizeof(rp), &a), n->p.id + ": weights pre-packing");
        return m;
    }
    // grouped convolution as a dense one: block-diagonal weights over all input features, zeros off the diagonal
    // (the tensor cores multiply the zeros, which for a few groups costs less than leaving the tensor-core kernel)
    check(cldnn_b200_mem_fill(m.impl->blk->mem, 0), n->p.id + ": weights pre-packing (zero fill)");
    const int32_t ofm = w.size.batch / groups, ifm = w.size.feature;
    for (int32_t g = 0; g < groups; ++g) {
        cldnn_b200_reorder_params rp{};
        rp.in = w.desc(); rp.out = packed.desc();
        rp.in.b = ofm; rp.in.offset += (int64_t)g * ofm * rp.in.pb;
        rp.out.b = ofm; rp.out.f = ifm; rp.out.offset += (int64_t)g * ofm * rp.out.pb + (int64_t)g * ifm * rp.out.pf;
        check(cldnn_b200_launch(eng->kernel("reorder_ref"), &rp, sizeof(rp), &a), n->p.id + ": weights pre-packing (group)");
    }
    return m;
}

void network_impl::prepare_kernel(node* n)
{
    const primitive& p = n->p;
    const std::string& t = p.type;
    cldnn_b200_args a{};
    if (!n->deps.empty()) a.input0 = n->deps[0]->mem.device_ptr();
    if (n->deps.size() > 1) a.input1 = n->deps[1]->mem.device_ptr();
    a.output = n->mem.device_ptr();
    if (n->weights) a.weights = n->weights->mem.device_ptr();
    if (n->bias) a.bias = n->bias->mem.device_ptr();
    if (n->wq) a.weights_quantization_factors = (const float*)n->wq->mem.device_ptr();
    if (n->oc) a.output_calibration_factors = (const float*)n->oc->mem.device_ptr();
    if (n->ec) a.eltw_output_calibration_factors = (const float*)n->ec->mem.device_ptr();
    for (node* f : {n->wq, n->oc, n->ec}) if (f && f->out.data_type != data_types::f32) throw error(p.id + ": quantization / calibration factors must be f32", CLDNN_B200_INVALID_ARG);

    auto finish = [&](const std::vector<std::string>& cands, void* params, size_t size, const std::function<void(int)>& set_tune, bool time_all = false,
                      const void* key_params = nullptr) {
        pick_kernel(n, cands, params, size, key_params, a, set_tune, time_all);
        check(cldnn_b200_prepare(eng->kernel(n->kernel), params, size, &a, &n->prepared), p.id + " (" + n->kernel + ")");
    };

    if (t == "convolution" || t == "fused_conv_eltwise" || t == "fully_connected") {
        const bool fc = t == "fully_connected";
        const layout& in = n->deps[0]->out; const layout& w = n->weights->out;
        cldnn_b200_conv_params cp{};
        cp.in = in.desc(); cp.out = n->out.desc();
        cp.groups = fc ? 1 : p.groups;
        cp.ofm = w.size.batch / cp.groups; cp.ifm = w.size.feature;
        cp.kh = fc ? 1 : w.size.y; cp.kw = fc ? 1 : w.size.x;       // inner product over a 1x1 map = 1x1 convolution
        {
            const cldnn_b200_tensor wd = w.desc();
            cp.w_dtype = wd.dtype; cp.w_po = wd.pb; cp.w_pi = wd.pf; cp.w_py = wd.py; cp.w_px = wd.px; cp.w_offset = wd.offset;
        }
        cp.stride_x = fc ? 1 : p.stride.x; cp.stride_y = fc ? 1 : p.stride.y;
        cp.pad_x = fc ? 0 : std::max(-p.input_offset.x, 0); cp.pad_y = fc ? 0 : std::max(-p.input_offset.y, 0);
        cp.dil_x = fc ? 1 : p.dilation.x; cp.dil_y = fc ? 1 : p.dilation.y;
        if (!fc && (p.input_offset.x > 0 || p.input_offset.y > 0)) {   // positive offset: the window starts inside the buffer
            cp.in.offset += p.input_offset.x * cp.in.px + p.input_offset.y * cp.in.py; cp.in.x -= 2 * p.input_offset.x; cp.in.y -= 2 * p.input_offset.y;
        }
        cp.bias_dtype = n->bias ? (int32_t)n->bias->out.data_type : CLDNN_B200_NONE;
        cp.quantization = n->wq ? 1 : 0; cp.i_qf = p.input_quantization_factor;
        cp.calibration = n->oc ? 1 : 0; cp.o_qf = p.output_quantization_factor;
        // O_QF is emitted by the plain convolution only when it differs from 1 (convolution_kernel_base.cpp:96-113) and
        // always under quantisation by the fused primitive (fused_conv_eltwise_kernel_base.cpp:139-151)
        cp.has_o_qf = (t == "fused_conv_eltwise") ? cp.quantization : ((!cp.calibration && cp.o_qf != 1.0f) ? 1 : 0);
        cp.act = n->act != CLDNN_B200_ACT_NONE ? n->act : act_from_slope(p.with_activation, p.activation_negative_slope, cp.act_m);
        if (n->act != CLDNN_B200_ACT_NONE) { cp.act_m = n->act_m; cp.act_n = n->act_n; }
        cp.eltw_stride_x = cp.eltw_stride_y = 1;
        if (t == "fused_conv_eltwise") {
            cp.fused_eltw = 1; cp.eltw = n->deps[1]->out.desc();
            cp.has_non_conv_scale = p.non_conv_scale != 1.0f ? 1 : 0; cp.non_conv_scale = p.non_conv_scale;
            cp.eltw_act = n->eltw_act != CLDNN_B200_ACT_NONE ? n->eltw_act : act_from_slope(p.eltw_activation, p.eltw_activation_negative_slope, cp.eltw_m);
            if (n->eltw_act != CLDNN_B200_ACT_NONE) { cp.eltw_m = n->eltw_m; cp.eltw_n = n->eltw_n; }
            cp.eltw_calibration = n->ec ? 1 : 0;
            cp.eltw_stride_x = p.eltw_stride.x; cp.eltw_stride_y = p.eltw_stride.y;
            cp.in_out_opt = n->in_place ? 1 : 0;
            if (n->in_place) a.input1 = nullptr;
        }
        std::function<void()> fc_fallback;
        if (fc) {
            // fully_connected_gpu_bfyx_ref.cl:68-81: round(((float)acc*q*I_QF + bias) * calib|O_QF), activation on the 8-bit
            // value.  With a float bias this is the convolution epilogue with DONT_DEQUANTIZE_BIAS; ReLU commutes with
            // the rounding and the saturating store.  The fp16 form is bias + activation, the fp16 convolution's epilogue.
            // A byxf input without padding between pixels is one row of y*x*stored-features values per image, and the
            // weights packed oyxi are the matching rows: the inner product is a 1x1 convolution over a 1x1 map.
            const bool flat = cp.in.pf == 1 && cp.in.py == cp.in.px * cp.in.x && cp.in.pb == cp.in.py * cp.in.y && cp.out.pf == 1 &&
                              w.size.feature == in.size.feature && w.size.x == in.size.x && w.size.y == in.size.y;
            // (the reference saturates the rounded value to s8 whatever the output type; written to an unsigned output that
            // leaves 0..127 -- the bytes an s8 store after a ReLU produces)
            const bool i8_conv = cp.quantization && n->bias && n->bias->out.data_type == data_types::f32 && is_int8(n->out.data_type) &&
                                 (cp.act == CLDNN_B200_ACT_NONE || cp.act == CLDNN_B200_ACT_RELU) && is_int8(in.data_type);
            const bool f16_conv = in.data_type == data_types::f16 && w.data_type == data_types::f16 && n->out.data_type == data_types::f16 && !cp.quantization &&
                                  !cp.calibration && cp.o_qf == 1.0f;
            const bool as_conv = flat && (i8_conv || f16_conv);
            auto plain_fc = [&]() {
                cldnn_b200_fc_params fp{};
                fp.in = in.desc(); fp.out = n->out.desc();
                const cldnn_b200_tensor wd = w.desc();
                fp.w_dtype = wd.dtype; fp.w_po = wd.pb; fp.w_pi = wd.pf; fp.w_py = wd.py; fp.w_px = wd.px; fp.w_offset = wd.offset;
                fp.bias_dtype = cp.bias_dtype; fp.quantization = cp.quantization; fp.i_qf = cp.i_qf; fp.calibration = cp.calibration; fp.o_qf = cp.o_qf;
                fp.act = cp.act; fp.act_m = cp.act_m; fp.act_n = cp.act_n;
                finish({"fc_ref"}, &fp, sizeof(fp), [](int) {});
            };
            fc_fallback = plain_fc;
            if (!as_conv) { plain_fc(); return; }
            cp.has_o_qf = (!cp.calibration && cp.o_qf != 1.0f) ? 1 : 0;
            if (i8_conv && n->out.data_type == data_types::u8) { cp.out.dtype = CLDNN_B200_I8; cp.act = CLDNN_B200_ACT_RELU; }
        }
        // first layer: planar input as the caller provides it, byxf output
        if (!fc && (is_int8(in.data_type) || in.data_type == data_types::f16) && cp.in.px == 1 && cp.out.pf == 1) {
            for (const char* kn : {"conv_i8_first", "conv_first_tc"}) {
                int32_t yes = 0; size_t sbytes = 0;
                cldnn_b200_kernel k = eng->kernel(kn);
                if (cldnn_b200_kernel_supports(k, &cp, sizeof(cp), &yes) == CLDNN_B200_SUCCESS && yes &&
                    cldnn_b200_kernel_scratch_bytes(k, &cp, sizeof(cp), &sbytes) == CLDNN_B200_SUCCESS) {
                    // the workspace serves whichever tuning variant is chosen: the variants pack the weights differently
                    int32_t variants = 0;
                    if (cldnn_b200_kernel_tune_count(k, &cp, sizeof(cp), &variants) != CLDNN_B200_SUCCESS) variants = 0;
                    for (int32_t t = 1; t < variants; ++t) {
                        cp.tune = t; size_t b = 0; int32_t ok_t = 0;
                        if (cldnn_b200_kernel_supports(k, &cp, sizeof(cp), &ok_t) == CLDNN_B200_SUCCESS && ok_t &&
                            cldnn_b200_kernel_scratch_bytes(k, &cp, sizeof(cp), &b) == CLDNN_B200_SUCCESS && b > sbytes) sbytes = b;
                    }
                    cp.tune = 0;
                    n->scratch = new_block(eng, sbytes);
                    a.scratch = n->scratch->dev; a.scratch_bytes = n->scratch->bytes;
                    finish({kn}, &cp, sizeof(cp), [&](int tn) { cp.tune = tn; });
                    return;
                }
            }
        }
        // tensor-core kernel: needs byxf activations and oyxi weights padded like the activations
        const bool half_tc = in.data_type == data_types::f16 && w.data_type == data_types::f16 && n->out.data_type == data_types::f16;
        const int32_t stored_ifm = (int32_t)cp.in.px;
        if (fc) {                                                       // the flattened view (the weights are packed from the original one)
            const int64_t kflat = cp.in.pb;
            cp.in.f = (int32_t)kflat; cp.in.x = cp.in.y = 1; cp.in.px = cp.in.py = kflat; cp.ifm = (int32_t)kflat;
        }
        // a convolution in 2..4 groups runs as a dense one on block-diagonal weights (AlexNet's split layers)
        const bool dense_groups = cp.groups >= 2 && cp.groups <= 4 && !fc;
        const bool try_tc = ((is_int8(in.data_type) && w.data_type == data_types::i8) || half_tc) && (cp.groups == 1 || dense_groups) && cp.in.pf == 1 && cp.in.px % 32 == 0 && cp.out.pf == 1;
        const char* tc_kernel = half_tc ? "conv_f16_tc" : "conv_i8_tc";
        if (try_tc) {
            cldnn_b200_conv_params tp = cp;
            if (dense_groups) { tp.ofm = cp.ofm * cp.groups; tp.ifm = cp.ifm * cp.groups; tp.groups = 1; }
            n->packed_weights = pack_conv_weights(n, stored_ifm, dense_groups ? cp.groups : 1);
            const cldnn_b200_tensor pd = n->packed_weights.get_layout().desc();
            tp.w_po = pd.pb; tp.w_pi = 1; tp.w_py = pd.py; tp.w_px = pd.px; tp.w_offset = 0;
            if (fc) tp.w_px = tp.w_py = pd.pb;                         // one tap holding the whole flattened row
            cldnn_b200_args ta = a; ta.weights = n->packed_weights.device_ptr();
            int32_t yes = 0;
            if (cldnn_b200_kernel_supports(eng->kernel(tc_kernel), &tp, sizeof(tp), &yes) == CLDNN_B200_SUCCESS && yes) {
                a = ta; cp = tp;
                // Winograd F(2x2, 3x3) beside the direct form, behind a gate modelled on should_use_winograd_2x3_s1
                // (src/layout_optimizer.cpp:34-53): 3x3 stride-1 undilated ungrouped fp16 convolutions whose feature counts are
                // multiples of 64, maps of at least 8x8, an input that is neither tiny nor so large that the transformed
                // operands (16/4 x input + 16/4 x output, in a workspace) get out of hand.  Where the reference rewrites the graph
                // (reorder_inputs.cpp:179-277) the two forms are alternatives of one primitive here: with tuning on both are timed
                // and the faster one is kept; without tuning the direct form runs.
                std::vector<std::string> cands = {tc_kernel};
                int32_t wino_yes = 0; size_t wino_bytes = 0;
                const int64_t in_count = (int64_t)in.size.batch * in.size.feature * in.size.x * in.size.y;
                const bool gate = half_tc && !fc && t == "convolution" && cp.groups == 1 && w.size.x == 3 && w.size.y == 3 && cp.stride_x == 1 && cp.stride_y == 1 &&
                                  cp.dil_x == 1 && cp.dil_y == 1 && in.size.feature % 64 == 0 && w.size.batch % 64 == 0 && in.size.x >= 8 && in.size.y >= 8 &&
                                  in_count >= 50000;
                if (gate && cldnn_b200_kernel_supports(eng->kernel("conv_f16_winograd"), &cp, sizeof(cp), &wino_yes) == CLDNN_B200_SUCCESS && wino_yes &&
                    cldnn_b200_kernel_scratch_bytes(eng->kernel("conv_f16_winograd"), &cp, sizeof(cp), &wino_bytes) == CLDNN_B200_SUCCESS &&
                    wino_bytes && wino_bytes <= ((size_t)1 << 31)) {
                    n->scratch = new_block(eng, wino_bytes);
                    a.scratch = n->scratch->dev; a.scratch_bytes = n->scratch->bytes;
                    cands.push_back("conv_f16_winograd");
                }
                // the tile shape does not depend on whether the residual is read from the output buffer: one cache entry for both
                cldnn_b200_conv_params key = cp; key.in_out_opt = 0; key.tune = 0;
                finish(cands, &cp, sizeof(cp), [&](int tn) { cp.tune = tn; }, cands.size() > 1, &key);
                if (n->kernel != "conv_f16_winograd" && n->scratch) {      // the direct form won: the workspace goes back
                    // (the prepared launch of the direct kernel never looks at the scratch pointer)
                    n->scratch.reset();
                }
                return;
            }
            n->packed_weights = memory();
        }
        if (fc) { fc_fallback(); return; }
        {   // the depthwise kernel keeps its weights as one word per (tap, feature) in a scratch buffer
            int32_t yes = 0; size_t sbytes = 0;
            cldnn_b200_kernel k = eng->kernel("conv_i8_dw");
            if (cldnn_b200_kernel_supports(k, &cp, sizeof(cp), &yes) == CLDNN_B200_SUCCESS && yes &&
                cldnn_b200_kernel_scratch_bytes(k, &cp, sizeof(cp), &sbytes) == CLDNN_B200_SUCCESS && sbytes) {
                n->scratch = new_block(eng, sbytes);
                a.scratch = n->scratch->dev; a.scratch_bytes = n->scratch->bytes;
            }
        }
        finish({"conv_i8_dw", "conv_ref"}, &cp, sizeof(cp), [&](int tn) { cp.tune = tn; });
        return;
    }
    if (t == "pooling") {
        const layout& in = n->deps[0]->out;
        cldnn_b200_pool_params pp{};
        pp.in = in.desc(); pp.out = n->out.desc();
        pp.size_x = p.global_pooling ? in.size.x : p.size.x; pp.size_y = p.global_pooling ? in.size.y : p.size.y;
        pp.stride_x = p.global_pooling ? 1 : p.stride.x; pp.stride_y = p.global_pooling ? 1 : p.stride.y;
        pp.pad_x = std::max(-p.input_offset.x, 0); pp.pad_y = std::max(-p.input_offset.y, 0);
        pp.mode = p.pool_mode == pooling_mode::max ? CLDNN_B200_POOL_MAX : CLDNN_B200_POOL_AVG;
        // pooling_gpu::create, src/gpu/pooling_gpu.cpp:122-130: when the last window runs past input + padding the
        // average divides by the clipped window
        const bool dyn = ((n->out.size.x - 1) * pp.stride_x + pp.size_x) > 2 * pp.pad_x + in.size.x ||
                         ((n->out.size.y - 1) * pp.stride_y + pp.size_y) > 2 * pp.pad_y + in.size.y;
        if (p.pool_mode == pooling_mode::average && dyn) pp.div_mode = CLDNN_B200_DIV_DYNAMIC_WITH_PADDING;
        else pp.div_mode = p.pool_mode == pooling_mode::average_no_padding ? CLDNN_B200_DIV_DYNAMIC : CLDNN_B200_DIV_FIXED;
        pp.act = n->act; pp.act_m = n->act_m; pp.act_n = n->act_n;
        finish({"pooling_i8_byxf", "pooling_f16_byxf", "pooling_ref"}, &pp, sizeof(pp), [](int) {});
        return;
    }
    if (t == "softmax") {
        cldnn_b200_softmax_params sp{}; sp.in = n->deps[0]->out.desc(); sp.out = n->out.desc();
        if (p.softmax_dimension < 0 || p.softmax_dimension > 3) throw error(p.id + ": wrong API - no such softmax dimension", CLDNN_B200_INVALID_ARG);
        sp.dimension = p.softmax_dimension;
        finish({"softmax"}, &sp, sizeof(sp), [](int) {});
        return;
    }
    if (t == "eltwise") {
        cldnn_b200_eltwise_params ep{};
        ep.in0 = n->deps[0]->out.desc(); ep.in1 = n->deps[1]->out.desc(); ep.out = n->out.desc();
        ep.mode = (int32_t)p.mode; ep.stride_x0 = ep.stride_y0 = ep.stride_x1 = ep.stride_y1 = 1;
        ep.quantization = p.eltw_quantized ? 1 : 0; ep.calibration = n->oc ? 1 : 0; ep.o_qf = p.output_quantization_factor;
        ep.act = n->act != CLDNN_B200_ACT_NONE ? n->act : act_from_slope(p.with_activation, p.activation_negative_slope, ep.act_m);
        if (n->act != CLDNN_B200_ACT_NONE) { ep.act_m = n->act_m; ep.act_n = n->act_n; }
        finish({"eltwise_byxf", "eltwise_ref"}, &ep, sizeof(ep), [](int) {});
        return;
    }
    if (t == "reorder") {
        cldnn_b200_reorder_params rp{};
        rp.in = n->deps[0]->out.desc(); rp.out = n->out.desc();
        rp.out.f = n->out.stored_features();                        // feature padding of the destination is written as zero
        if (!p.subtract_per_feature.empty()) {
            if (p.subtract_per_feature.size() > 4) throw error(p.id + ": at most 4 per-feature mean values are supported", CLDNN_B200_UNSUPPORTED_SIZE);
            rp.has_mean = 1; for (size_t i = 0; i < 4; ++i) rp.mean[i] = p.subtract_per_feature[std::min(i, p.subtract_per_feature.size() - 1)];
        }
        finish({"reorder_ref"}, &rp, sizeof(rp), [](int) {});
        return;
    }
    if (t == "concatenation") {
        // concatenation_gpu (src/gpu/concatenation_gpu.cpp): one copy launch per input, each writing its slice of the output;
        // the copy kernel addresses both sides through pitches, so any of the supported layouts works on either side
        const cldnn_b200_tensor od = n->out.desc();
        int64_t at = 0;
        n->kernel = "reorder_ref"; n->tune = 0;
        for (node* d : n->deps) {
            cldnn_b200_reorder_params rp{};
            rp.in = d->out.desc(); rp.out = od;
            rp.out.b = rp.in.b; rp.out.f = rp.in.f; rp.out.y = rp.in.y; rp.out.x = rp.in.x;
            const int64_t pitch = p.concat_axis == 0 ? od.pb : (p.concat_axis == 1 ? od.pf : (p.concat_axis == 2 ? od.px : od.py));
            const int64_t len = p.concat_axis == 0 ? rp.in.b : (p.concat_axis == 1 ? rp.in.f : (p.concat_axis == 2 ? rp.in.x : rp.in.y));
            rp.out.offset += at * pitch;
            at += len;
            cldnn_b200_args ca{}; ca.input0 = d->mem.device_ptr(); ca.output = n->mem.device_ptr();
            cldnn_b200_prepared pr = nullptr;
            check(cldnn_b200_prepare(eng->kernel("reorder_ref"), &rp, sizeof(rp), &ca, &pr), p.id + " (concatenation copy)");
            if (!n->prepared) n->prepared = pr; else n->more_prepared.push_back(pr);
        }
        return;
    }
    if (t == "lrn") {
        cldnn_b200_lrn_params lp{}; lp.in = n->deps[0]->out.desc(); lp.out = n->out.desc();
        lp.size = (int32_t)p.lrn_size; lp.k = p.lrn_k; lp.alpha = p.lrn_alpha; lp.beta = p.lrn_beta;
        finish({"lrn_f16_byxf", "lrn_ref"}, &lp, sizeof(lp), [](int) {});
        return;
    }
    if (t == "activation") {
        cldnn_b200_activation_params ap{}; ap.in = n->deps[0]->out.desc(); ap.out = n->out.desc();
        ap.act = p.activation_func; ap.act_m = p.act_a; ap.act_n = p.act_b;
        finish({"activation_ref"}, &ap, sizeof(ap), [](int) {});
        return;
    }
    throw error("primitive type '" + t + "' is outside the supported path", CLDNN_B200_UNSUPPORTED_FORMAT);
}

// network_impl::allocate_primitives + memory_pool (src/network.cpp:173-190, src/memory_pool.cpp:182-260): an intermediate
// buffer is handed on to a later primitive once its last reader has been enqueued; kernels run in order on one stream,
// so the reuse needs no further synchronisation.  Network inputs, constants and outputs are never pooled.
void network_impl::allocate_and_prepare()
{
    std::vector<int> last_use(order.size(), -1);
    for (node* n : order) {
        for (node* d : n->deps) last_use[d->order] = std::max(last_use[d->order], n->order);
        if (n->is_output) last_use[n->order] = 1 << 30;
    }
    std::multimap<size_t, std::shared_ptr<block>> free_blocks;
    std::vector<std::pair<int, std::shared_ptr<block>>> live;       // (last use, block)
    for (node* n : order) {
        if (n->p.type == "data") { n->mem = n->p.mem; continue; }
        if (n->p.type == "input_layout") continue;                  // bound by set_input_data
        if (n->in_place) {
            // the second input's buffer becomes the output: it now lives until this node's last reader
            node* r = n->deps[1];
            n->mem = memory(); n->mem.impl = std::make_shared<memory_impl>(); n->mem.impl->l = n->out; n->mem.impl->blk = r->mem.impl->blk;
            for (auto& lv : live) if (lv.second == r->mem.impl->blk) lv.first = std::max(lv.first, last_use[n->order]);
            continue;
        }
        for (auto it = live.begin(); it != live.end();) {
            if (it->first < n->order) { free_blocks.insert({it->second->bytes, it->second}); it = live.erase(it); } else ++it;
        }
        const size_t need = std::max<size_t>(n->out.bytes_count(), 16);
        std::shared_ptr<block> blk;
        // fp16 tensors whose stored feature count exceeds the real one: the kernels write the real features only and the
        // consumer multiplies the padded lanes by zero weights, which is only safe while those lanes hold zeros (a previous
        // tenant's Inf or NaN times zero is NaN).  Such a tensor keeps a zero-filled block of its own for the network's life.
        const bool private_block = n->out.data_type == data_types::f16 && n->out.stored_features() != n->out.size.feature;
        if (!n->is_output && !private_block) {
            auto it = free_blocks.lower_bound(need);
            if (it != free_blocks.end() && it->first <= 2 * need + 65536) { blk = it->second; free_blocks.erase(it); }
        }
        if (!blk) { blk = new_block(eng, need); if (!n->is_output) pool_bytes += blk->bytes; }
        n->mem = memory(); n->mem.impl = std::make_shared<memory_impl>(); n->mem.impl->l = n->out; n->mem.impl->blk = blk;
        if (!n->is_output && !private_block) live.push_back({last_use[n->order], blk});
    }
}

void network_impl::build(const topology& topo)
{
    for (auto& p : topo.primitives()) add_node(p);
    link(); sort();
    // outputs: requested ids, else every primitive without users (trim_to_outputs)
    if (!opts.outputs.empty()) for (auto& id : opts.outputs) get(id)->is_output = true;
    else for (node* n : order) if (n->users.empty() && !n->constant() && n->p.type != "input_layout") {
        bool param = false;
        for (auto& up : nodes) for (node* d : {up->weights, up->bias, up->wq, up->oc, up->ec}) param |= d == n;
        if (!param) n->is_output = true;
    }
    for (node* n : order) if (n->is_output) { n->answers_for = n->p.id; output_ids.push_back(n->p.id); }
    relayout();
    if (opts.optimize_data) {
        fuse_activations();
        fuse_conv_eltwise();
        fuse_activations();                                         // relu behind a freshly fused conv+eltwise
        select_layouts();
        if (opts.conv_eltw_read_write_opt) conv_eltw_read_write_opt();
    }
    load_cache();
    allocate_and_prepare();
}

void network_impl::execute()
{
    for (node* n : order) if (n->p.type == "input_layout" && !n->mem) throw error("input '" + n->p.id + "' has not been set", CLDNN_B200_INVALID_ARG);
    if (inputs_changed) {
        // (re)build the launches: pointers of the inputs are baked into the prepared kernels
        if (graph) { cldnn_b200_graph_destroy(graph); graph = nullptr; }
        for (node* n : order) {
            if (n->prepared) { cldnn_b200_prepared_destroy(n->prepared); n->prepared = nullptr; }
            for (auto pr : n->more_prepared) cldnn_b200_prepared_destroy(pr);
            n->more_prepared.clear();
        }
        for (node* n : order) if (n->p.type != "data" && n->p.type != "input_layout") prepare_kernel(n);
        save_cache();
        check(cldnn_b200_ctx_sync(eng->ctx), "sync");
        launches = 0; for (node* n : order) if (n->prepared) launches += 1 + n->more_prepared.size();
        if (opts.use_graph && !eng->profiling) {
            check(cldnn_b200_graph_begin(eng->ctx), "graph begin");
            try { for (node* n : order) run_prepared(n); }
            catch (...) { cldnn_b200_graph cg = nullptr; cldnn_b200_graph_end(eng->ctx, &cg); if (cg) cldnn_b200_graph_destroy(cg); throw; }
            check(cldnn_b200_graph_end(eng->ctx, &graph), "graph end");
        }
        inputs_changed = false;
    }
    if (graph) { check(cldnn_b200_graph_launch(graph), "graph launch"); return; }
    if (!eng->profiling) { for (node* n : order) run_prepared(n); return; }
    // profiling: one event pair per primitive, no graph
    if (prof_events.size() != order.size()) {
        for (auto& pe : prof_events) { cldnn_b200_event_destroy(pe.first); cldnn_b200_event_destroy(pe.second); }
        prof_events.assign(order.size(), {nullptr, nullptr});
        for (auto& pe : prof_events) { check(cldnn_b200_event_create(eng->ctx, &pe.first), "event"); check(cldnn_b200_event_create(eng->ctx, &pe.second), "event"); }
    }
    for (size_t i = 0; i < order.size(); ++i) {
        if (!order[i]->prepared) continue;
        check(cldnn_b200_event_record(prof_events[i].first), "event record");
        run_prepared(order[i]);
        check(cldnn_b200_event_record(prof_events[i].second), "event record");
    }
}

// --------------------------------------------------------------------------------------
// network facade
// --------------------------------------------------------------------------------------
network::network(const engine& e, const topology& t, const build_options& o) : impl(std::make_shared<network_impl>())
{
    impl->eng = e.impl; impl->opts = o;
    impl->build(t);
}
void network::set_input_data(const std::string& id, const memory& m)
{
    node* n = impl->get(id);
    if (n->p.type != "input_layout") throw error("primitive '" + id + "' is not an input_layout", CLDNN_B200_INVALID_ARG);
    if (!(m.get_layout() == n->out)) throw error("set_input_data: layout of '" + id + "' does not match the topology", CLDNN_B200_DIMENSION_MISMATCH);
    if (!n->mem || n->mem.device_ptr() != m.device_ptr()) impl->inputs_changed = true;
    n->mem = m;
}
void network::execute() { impl->execute(); }
void network::wait() { check(cldnn_b200_ctx_sync(impl->eng->ctx), "wait"); }
memory network::get_output(const std::string& id)
{
    wait();
    uint32_t st = 0; check(cldnn_b200_ctx_device_status(impl->eng->ctx, &st), "device status");
    if (st) throw error("a kernel gave up waiting (device status 0x" + std::to_string(st) + ")", CLDNN_B200_DEVICE_ERROR);
    return output_memory(id);
}
memory network::output_memory(const std::string& id) const
{
    for (node* n : impl->order) if (n->is_output && (n->answers_for == id || n->p.id == id)) return n->mem;
    node* n = impl->get(id);
    if (!n->mem) throw error("primitive '" + id + "' has no memory (fused away); request it as an output", CLDNN_B200_INVALID_ARG);
    return n->mem;
}
std::vector<std::string> network::get_output_ids() const { return impl->output_ids; }
std::vector<primitive_info> network::get_primitives_info() const
{
    std::vector<primitive_info> v;
    for (node* n : impl->order) {
        primitive_info i; i.id = n->p.id; i.type = n->p.type; i.original_ids = n->fused_ids; i.kernel = n->kernel; i.tune = n->tune; i.output = n->out; i.is_output = n->is_output; i.in_place = n->in_place;
        v.push_back(i);
    }
    return v;
}
uint64_t network::launches_per_execute() const { return impl->launches; }
std::vector<std::pair<std::string, uint64_t>> network::get_profiling_info() const
{
    std::vector<std::pair<std::string, uint64_t>> v;
    if (impl->prof_events.size() != impl->order.size()) return v;
    check(cldnn_b200_ctx_sync(impl->eng->ctx), "sync");
    for (size_t i = 0; i < impl->order.size(); ++i) {
        if (!impl->order[i]->prepared) continue;
        uint64_t ns = 0;
        check(cldnn_b200_event_elapsed_ns(impl->prof_events[i].first, impl->prof_events[i].second, &ns), "event elapsed");
        v.push_back({impl->order[i]->p.id, ns});
    }
    return v;
}
size_t network::device_memory_bytes() const { return impl->pool_bytes; }

}  // namespace cldnn
