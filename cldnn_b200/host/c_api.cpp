// Flat C interface over the C++ host layer (include/cldnn_host.h).  Exceptions
// are turned into status codes with a thread-local message, as exception_handler
// does for the reference's C API (src/include/api_impl.h:61-140).
#include <cstring>
#include <fstream>
#include <sstream>
#include "../../include/cldnn_host.h"
#include "cldnn_host.hpp"

using namespace cldnn;

struct cldnn_host_engine_impl { engine e; };
struct cldnn_host_memory_impl { memory m; };
struct cldnn_host_topology_impl { topology t; };
struct cldnn_host_network_impl { network n; };

static thread_local std::string g_err;

template <class F>
static int32_t guarded(F&& f)
{
    try { f(); return CLDNN_B200_SUCCESS; }
    catch (const error& e) { g_err = e.what(); return e.status; }
    catch (const std::bad_alloc&) { g_err = "out of host memory"; return CLDNN_B200_OUT_OF_RESOURCES; }
    catch (const std::exception& e) { g_err = e.what(); return CLDNN_B200_ERROR; }
    catch (...) { g_err = "unknown error"; return CLDNN_B200_ERROR; }
}
static void need(const void* p, const char* what) { if (!p) throw error(std::string(what) + ": null argument", CLDNN_B200_INVALID_ARG); }
static std::string str(const char* s) { return s ? s : ""; }

extern "C" {

const char* cldnn_host_last_error(void) { return g_err.c_str(); }

int32_t cldnn_host_engine_create(int32_t device, uint32_t prof, cldnn_host_engine* out)
{
    return guarded([&] { need(out, "engine_create"); *out = nullptr; *out = new cldnn_host_engine_impl{engine(device, prof != 0)}; });
}
int32_t cldnn_host_engine_release(cldnn_host_engine e) { delete e; return CLDNN_B200_SUCCESS; }
int32_t cldnn_host_engine_stream(cldnn_host_engine e, void** stream)
{
    return guarded([&] { need(e, "engine_stream"); need(stream, "engine_stream"); *stream = e->e.stream(); });
}
int32_t cldnn_host_engine_info(cldnn_host_engine e, cldnn_b200_engine_info* info)
{
    return guarded([&] { need(e, "engine_info"); need(info, "engine_info"); *info = e->e.get_info(); });
}

int32_t cldnn_host_memory_allocate(cldnn_host_engine e, int32_t dt, int32_t fmt, int32_t b, int32_t f, int32_t x, int32_t y, cldnn_host_memory* out)
{
    return guarded([&] {
        need(e, "memory_allocate"); need(out, "memory_allocate"); *out = nullptr;
        if (b < 1 || f < 1 || x < 1 || y < 1) throw error("memory_allocate: sizes must be positive", CLDNN_B200_INVALID_ARG);
        *out = new cldnn_host_memory_impl{memory::allocate(e->e, layout((data_types)dt, fmt, tensor(b, f, x, y)))};
    });
}
int32_t cldnn_host_memory_attach(cldnn_host_engine e, int32_t dt, int32_t fmt, int32_t b, int32_t f, int32_t x, int32_t y, void* dev, cldnn_host_memory* out)
{
    return guarded([&] {
        need(e, "memory_attach"); need(out, "memory_attach"); need(dev, "memory_attach"); *out = nullptr;
        *out = new cldnn_host_memory_impl{memory::attach(e->e, layout((data_types)dt, fmt, tensor(b, f, x, y)), dev)};
    });
}
int32_t cldnn_host_memory_release(cldnn_host_memory m) { delete m; return CLDNN_B200_SUCCESS; }
int32_t cldnn_host_memory_write(cldnn_host_memory m, const void* host, size_t bytes)
{
    return guarded([&] { need(m, "memory_write"); need(host, "memory_write"); m->m.write(host, bytes); });
}
int32_t cldnn_host_memory_read(cldnn_host_memory m, void* host, size_t bytes)
{
    return guarded([&] { need(m, "memory_read"); need(host, "memory_read"); m->m.read(host, bytes); });
}
int32_t cldnn_host_memory_layout(cldnn_host_memory m, int32_t* dt, int32_t* fmt, int32_t* b, int32_t* f, int32_t* x, int32_t* y, size_t* bytes)
{
    return guarded([&] {
        need(m, "memory_layout");
        const layout& l = m->m.get_layout();
        if (dt) *dt = (int32_t)l.data_type; if (fmt) *fmt = l.fmt; if (b) *b = l.size.batch; if (f) *f = l.size.feature;
        if (x) *x = l.size.x; if (y) *y = l.size.y; if (bytes) *bytes = l.bytes_count();
    });
}
int32_t cldnn_host_memory_device_ptr(cldnn_host_memory m, void** dev)
{
    return guarded([&] { need(m, "memory_device_ptr"); need(dev, "memory_device_ptr"); *dev = m->m.device_ptr(); });
}

int32_t cldnn_host_topology_create(cldnn_host_topology* out)
{
    return guarded([&] { need(out, "topology_create"); *out = new cldnn_host_topology_impl(); });
}
int32_t cldnn_host_topology_release(cldnn_host_topology t) { delete t; return CLDNN_B200_SUCCESS; }

int32_t cldnn_host_add_input_layout(cldnn_host_topology t, const char* id, int32_t dt, int32_t fmt, int32_t b, int32_t f, int32_t x, int32_t y)
{
    return guarded([&] { need(t, "add_input_layout"); t->t.add(input_layout(str(id), layout((data_types)dt, fmt, tensor(b, f, x, y)))); });
}
int32_t cldnn_host_add_data(cldnn_host_topology t, const char* id, cldnn_host_memory m)
{
    return guarded([&] { need(t, "add_data"); need(m, "add_data"); t->t.add(data(str(id), m->m)); });
}
int32_t cldnn_host_add_reorder(cldnn_host_topology t, const char* id, const char* input, int32_t fmt, int32_t dt, const float* sub, size_t nsub)
{
    return guarded([&] {
        need(t, "add_reorder");
        std::vector<float> s; if (sub) s.assign(sub, sub + nsub);
        t->t.add(reorder(str(id), str(input), fmt, (data_types)dt, s));
    });
}
int32_t cldnn_host_add_convolution(cldnn_host_topology t, const char* id, const char* input, const char* weights, const char* bias, const char* wq,
                                   const char* oc, float iqf, float oqf, int32_t odt, int32_t sx, int32_t sy, int32_t ox, int32_t oy, int32_t dx, int32_t dy,
                                   uint32_t act, float slope, uint32_t groups)
{
    return guarded([&] {
        need(t, "add_convolution");
        primitive p = convolution(str(id), str(input), str(weights), str(bias), str(wq), str(oc), iqf, (data_types)odt, tensor(1, 1, sx, sy),
                                  tensor(0, 0, ox, oy), tensor(1, 1, dx, dy), act != 0, slope, (int32_t)(groups ? groups : 1));
        p.output_quantization_factor = oqf;
        t->t.add(p);
    });
}
int32_t cldnn_host_add_fused_conv_eltwise(cldnn_host_topology t, const char* id, const char* input, const char* input2, const char* weights, const char* bias,
                                          const char* wq, const char* oc, float iqf, float ncs, const char* ec, int32_t esx, int32_t esy, int32_t sx, int32_t sy,
                                          int32_t ox, int32_t oy, int32_t dx, int32_t dy, uint32_t cact, float cslope, uint32_t eact, float eslope, int32_t odt)
{
    return guarded([&] {
        need(t, "add_fused_conv_eltwise");
        t->t.add(fused_conv_eltwise(str(id), str(input), str(input2), eltwise_mode::sum, str(weights), str(bias), str(wq), str(oc), iqf, ncs, str(ec),
                                    tensor(1, 1, esx, esy), tensor(1, 1, sx, sy), tensor(0, 0, ox, oy), tensor(1, 1, dx, dy), cact != 0, cslope, eact != 0, eslope,
                                    (data_types)odt));
    });
}
int32_t cldnn_host_add_eltwise(cldnn_host_topology t, const char* id, const char* input, const char* input2, int32_t mode, uint32_t act, float slope,
                               const char* oc, float oqf, uint32_t quantized)
{
    return guarded([&] { need(t, "add_eltwise"); t->t.add(eltwise(str(id), str(input), str(input2), (eltwise_mode)mode, act != 0, slope, str(oc), oqf, quantized != 0)); });
}
int32_t cldnn_host_add_activation(cldnn_host_topology t, const char* id, const char* input, int32_t func, float a, float b)
{
    return guarded([&] { need(t, "add_activation"); t->t.add(activation(str(id), str(input), func, a, b)); });
}
int32_t cldnn_host_add_pooling(cldnn_host_topology t, const char* id, const char* input, int32_t mode, uint32_t global, int32_t zx, int32_t zy,
                               int32_t sx, int32_t sy, int32_t ox, int32_t oy)
{
    return guarded([&] {
        need(t, "add_pooling");
        if (global) t->t.add(global_pooling(str(id), str(input), (pooling_mode)mode));
        else t->t.add(pooling(str(id), str(input), (pooling_mode)mode, tensor(1, 1, zx, zy), tensor(1, 1, sx, sy), tensor(0, 0, ox, oy)));
    });
}
int32_t cldnn_host_add_fully_connected(cldnn_host_topology t, const char* id, const char* input, const char* weights, const char* bias, const char* wq,
                                       const char* oc, float iqf, float oqf, uint32_t act, float slope)
{
    return guarded([&] {
        need(t, "add_fully_connected");
        primitive p = fully_connected(str(id), str(input), str(weights), str(bias), str(wq), str(oc), iqf, act != 0, slope);
        p.output_quantization_factor = oqf;
        t->t.add(p);
    });
}
int32_t cldnn_host_add_softmax(cldnn_host_topology t, const char* id, const char* input)
{
    return guarded([&] { need(t, "add_softmax"); t->t.add(softmax(str(id), str(input))); });
}
int32_t cldnn_host_add_softmax_dim(cldnn_host_topology t, const char* id, const char* input, int32_t dimension)
{
    return guarded([&] { need(t, "add_softmax_dim"); t->t.add(softmax(str(id), str(input), dimension)); });
}
int32_t cldnn_host_add_lrn(cldnn_host_topology t, const char* id, const char* input, uint32_t size, float k, float alpha, float beta)
{
    return guarded([&] { need(t, "add_lrn"); t->t.add(lrn(str(id), str(input), size, k, alpha, beta)); });
}

int32_t cldnn_host_tuning_cache_check(const char* path, uint32_t compute_units, size_t* entries)
{
    return guarded([&] {
        need(path, "tuning_cache_check"); need(entries, "tuning_cache_check");
        std::ifstream f(path);
        if (!f) throw error(std::string("cannot read '") + path + "'", CLDNN_B200_INVALID_ARG);
        std::stringstream ss; ss << f.rdbuf();
        const auto all = parse_tuning_cache(ss.str());
        auto it = all.find(std::to_string(compute_units));
        *entries = it == all.end() ? 0 : it->second.size();
    });
}

int32_t cldnn_host_add_concatenation(cldnn_host_topology t, const char* id, const char* inputs, int32_t axis)
{
    return guarded([&] {
        need(t, "add_concatenation");
        std::vector<std::string> ins; std::stringstream ss(str(inputs)); std::string item;
        while (std::getline(ss, item, ',')) if (!item.empty()) ins.push_back(item);
        t->t.add(concatenation(str(id), ins, axis));
    });
}

int32_t cldnn_host_network_build(cldnn_host_engine e, cldnn_host_topology t, const cldnn_host_build_options* o, cldnn_host_network* out)
{
    return guarded([&] {
        need(e, "network_build"); need(t, "network_build"); need(out, "network_build"); *out = nullptr;
        build_options bo;
        if (o) {
            bo.optimize_data = o->optimize_data != 0; bo.fuse_any_conv_eltwise = o->fuse_any_conv_eltwise != 0;
            bo.tuning = (tuning_mode)o->tuning_mode; bo.tuning_cache_path = str(o->tuning_cache_path);
            bo.use_graph = o->use_graph != 0; bo.force_kernel = str(o->force_kernel);
            std::stringstream ss(str(o->outputs)); std::string item;
            while (std::getline(ss, item, ',')) if (!item.empty()) bo.outputs.push_back(item);
        }
        *out = new cldnn_host_network_impl{network(e->e, t->t, bo)};
    });
}
int32_t cldnn_host_network_release(cldnn_host_network n) { return guarded([&] { delete n; }); }
int32_t cldnn_host_network_set_input(cldnn_host_network n, const char* id, cldnn_host_memory m)
{
    return guarded([&] { need(n, "network_set_input"); need(m, "network_set_input"); n->n.set_input_data(str(id), m->m); });
}
int32_t cldnn_host_network_execute(cldnn_host_network n) { return guarded([&] { need(n, "network_execute"); n->n.execute(); }); }
int32_t cldnn_host_network_wait(cldnn_host_network n) { return guarded([&] { need(n, "network_wait"); n->n.wait(); }); }
int32_t cldnn_host_network_get_output(cldnn_host_network n, const char* id, cldnn_host_memory* out)
{
    return guarded([&] { need(n, "network_get_output"); need(out, "network_get_output"); *out = nullptr; *out = new cldnn_host_memory_impl{n->n.get_output(str(id))}; });
}
int32_t cldnn_host_network_info(cldnn_host_network n, char* buffer, size_t buffer_bytes, size_t* needed)
{
    return guarded([&] {
        need(n, "network_info");
        std::stringstream ss;
        for (auto& i : n->n.get_primitives_info())
            ss << i.id << "|" << i.type << "|" << i.kernel << "|" << i.tune << "|" << format::name(i.output.fmt) << "|" << (int)i.output.data_type << "|"
               << i.output.size.batch << "," << i.output.size.feature << "," << i.output.size.y << "," << i.output.size.x << "|" << i.original_ids << "|"
               << (i.is_output ? 1 : 0) << "|" << (i.in_place ? 1 : 0) << "\n";
        const std::string s = ss.str();
        if (needed) *needed = s.size() + 1;
        if (buffer && buffer_bytes) { const size_t k = std::min(buffer_bytes - 1, s.size()); std::memcpy(buffer, s.data(), k); buffer[k] = 0; }
    });
}
int32_t cldnn_host_network_profiling(cldnn_host_network n, char* buffer, size_t buffer_bytes, size_t* needed)
{
    return guarded([&] {
        need(n, "network_profiling");
        std::stringstream ss;
        for (auto& i : n->n.get_profiling_info()) ss << i.first << "|" << i.second << "\n";
        const std::string s = ss.str();
        if (needed) *needed = s.size() + 1;
        if (buffer && buffer_bytes) { const size_t k = std::min(buffer_bytes - 1, s.size()); std::memcpy(buffer, s.data(), k); buffer[k] = 0; }
    });
}
int32_t cldnn_host_network_stats(cldnn_host_network n, uint64_t* launches, size_t* pool_bytes)
{
    return guarded([&] { need(n, "network_stats"); if (launches) *launches = n->n.launches_per_execute(); if (pool_bytes) *pool_bytes = n->n.device_memory_bytes(); });
}

}  // extern "C"
