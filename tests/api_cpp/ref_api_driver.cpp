// A small interpreter that drives clDNN through its own header-only C++ API (api/CPP/*.hpp of the clDNN tree, unmodified,
// found through -I at compile time) and therefore through the public C boundary the headers call.  Linked against
// libclDNN64.so of this repository it shows that an application written for the reference runs on the B200 engine
// unchanged.  Test infrastructure: built by tests/api_cpp/Makefile when the clDNN tree is present.
//
// usage: ref_api_driver <script>      (paths inside the script are relative to the script's directory)
// script lines (tokens separated by blanks, '-' = empty / default):
//   mem NAME DTYPE B F X Y FILE                      memory::allocate(engine, {dtype, bfyx, tensor(B,F,X,Y)}) filled from FILE
//   attach NAME DTYPE B F X Y FILE                   memory::attach over a host buffer read from FILE
//   input_layout ID MEM | data ID MEM
//   convolution ID IN W BIAS QUANT OUT_DTYPE SX SY OX OY DX DY ACT
//   fused_conv_eltwise ID IN IN2 W BIAS QUANT OUT_DTYPE SX SY OX OY CONV_ACT ELTW_ACT
//   pooling ID IN max|average KX KY SX SY OX OY
//   fully_connected ID IN W BIAS QUANT CALIB ACT      softmax ID IN      activation ID IN relu|clamp A B
//   eltwise ID IN IN2 sum|max ACT                     reorder ID IN FORMAT DTYPE        concatenation ID AXIS IN...
//   option optimize_data 0|1 | option outputs ID...
//   build | set_input ID MEM | execute | save OUTPUT_ID FILE | info ID | expect_build_error
// exit code 0 when every command succeeded.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <limits>      // the reference headers use std::numeric_limits without including it
#include <map>
#include <memory>
#include <sstream>
#include <api/CPP/memory.hpp>
#include <api/CPP/topology.hpp>
#include <api/CPP/network.hpp>
#include <api/CPP/engine.hpp>
#include <api/CPP/input_layout.hpp>
#include <api/CPP/data.hpp>
#include <api/CPP/reorder.hpp>
#include <api/CPP/convolution.hpp>
#include <api/CPP/pooling.hpp>
#include <api/CPP/fully_connected.hpp>
#include <api/CPP/softmax.hpp>
#include <api/CPP/eltwise.hpp>
#include <api/CPP/activation.hpp>
#include <api/CPP/concatenation.hpp>
#include <api_extension/CPP/fused_conv_eltwise.hpp>

using namespace cldnn;

static data_types dtype_of(const std::string& s)
{
    if (s == "u8") return data_types::u8;
    if (s == "i8") return data_types::i8;
    if (s == "i32") return data_types::i32;
    if (s == "f16") return data_types::f16;
    if (s == "f32") return data_types::f32;
    throw std::runtime_error("unknown data type " + s);
}
static format format_of(const std::string& s)
{
    if (s == "bfyx") return format::bfyx;
    if (s == "byxf") return format::byxf;
    if (s == "yxfb") return format::yxfb;
    if (s == "byxf_af32") return format::byxf_af32;
    throw std::runtime_error("unknown format " + s);
}
static std::vector<char> read_file(const std::string& path)
{
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot read " + path);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
static std::vector<primitive_id> opt_list(const std::string& s) { return s == "-" ? std::vector<primitive_id>{} : std::vector<primitive_id>{s}; }
static primitive_id opt_id(const std::string& s) { return s == "-" ? "" : s; }

int main(int argc, char** argv)
{
    if (argc < 2) { std::fprintf(stderr, "usage: ref_api_driver <script>\n"); return 2; }
    const std::string script = argv[1];
    const std::string dir = script.find('/') == std::string::npos ? "." : script.substr(0, script.rfind('/'));
    std::ifstream in(script);
    if (!in) { std::fprintf(stderr, "cannot read %s\n", script.c_str()); return 2; }
    try {
        engine eng;
        std::map<std::string, memory> mems;
        std::map<std::string, std::vector<char>> host_buffers;
        topology topo;
        build_options opts;
        std::unique_ptr<network> net;
        std::map<primitive_id, network_output> outputs;
        std::string line;
        int lineno = 0;
        while (std::getline(in, line)) {
            ++lineno;
            std::istringstream ss(line);
            std::vector<std::string> t;
            for (std::string w; ss >> w;) t.push_back(w);
            if (t.empty() || t[0][0] == '#') continue;
            const std::string& c = t[0];
            auto I = [&](size_t i) { return std::stoi(t.at(i)); };
            if (c == "mem" || c == "attach") {
                layout l(dtype_of(t.at(2)), format::bfyx, tensor(I(3), I(4), I(5), I(6)));
                std::vector<char> bytes = read_file(dir + "/" + t.at(7));
                if (bytes.size() != l.bytes_count()) throw std::runtime_error(t[1] + ": file size does not match the layout");
                if (c == "mem") {
                    memory m = memory::allocate(eng, l);
                    { auto p = m.pointer<char>(); std::memcpy(p.data(), bytes.data(), bytes.size()); }
                    mems.emplace(t[1], m);
                } else {
                    host_buffers[t[1]] = bytes;
                    mems.emplace(t[1], memory::attach(l, host_buffers[t[1]].data(), host_buffers[t[1]].size()));
                }
            } else if (c == "input_layout") topo.add(input_layout(t.at(1), mems.at(t.at(2)).get_layout()));
            else if (c == "data") topo.add(data(t.at(1), mems.at(t.at(2))));
            else if (c == "convolution") {
                const tensor stride(1, 1, I(7), I(8)), offset(0, 0, I(9), I(10)), dil(1, 1, I(11), I(12));
                if (t.at(5) != "-")
                    topo.add(convolution(t[1], t[2], {t[3]}, opt_list(t[4]), {t[5]}, dtype_of(t[6]), stride, offset, dil, I(13) != 0));
                else
                    topo.add(convolution(t[1], t[2], {t[3]}, opt_list(t[4]), stride, offset, dil, I(13) != 0));
            } else if (c == "fused_conv_eltwise") {
                const tensor stride(1, 1, I(8), I(9)), offset(0, 0, I(10), I(11));
                topo.add(fused_conv_eltwise(t[1], t[2], t[3], eltwise_mode::sum, {t[4]}, opt_list(t[5]), opt_list(t[6]), {}, 1.0f, 1.0f, "",
                                            {tensor(1, 1, 1, 1), tensor(1, 1, 1, 1)}, stride, offset, tensor(1, 1, 1, 1), I(12) != 0, 0.0f, I(13) != 0, 0.0f,
                                            padding(), optional_data_type{dtype_of(t[7])}));
            } else if (c == "pooling") {
                topo.add(pooling(t[1], t[2], t[3] == "max" ? pooling_mode::max : pooling_mode::average, tensor(1, 1, I(4), I(5)), tensor(1, 1, I(6), I(7)),
                                 tensor(0, 0, I(8), I(9))));
            } else if (c == "fully_connected") {
                if (t.at(5) != "-") topo.add(fully_connected(t[1], t[2], t[3], opt_id(t[4]), t[5], opt_id(t[6]), 1.0f, I(7) != 0));
                else topo.add(fully_connected(t[1], t[2], t[3], opt_id(t[4]), I(7) != 0));
            } else if (c == "softmax") topo.add(softmax(t.at(1), t.at(2)));
            else if (c == "activation") {
                topo.add(activation(t[1], t[2], t[3] == "relu" ? activation_relu : activation_clamp, {std::stof(t.at(4)), std::stof(t.at(5))}));
            } else if (c == "eltwise") topo.add(eltwise(t[1], t[2], t[3], t[4] == "sum" ? eltwise_mode::sum : eltwise_mode::max, I(5) != 0));
            else if (c == "reorder") topo.add(reorder(t[1], t[2], format_of(t.at(3)), dtype_of(t.at(4))));
            else if (c == "concatenation") {
                std::vector<primitive_id> ins(t.begin() + 3, t.end());
                topo.add(concatenation(t[1], ins, t[2] == "f" ? concatenation::along_f : (t[2] == "b" ? concatenation::along_b : (t[2] == "x" ? concatenation::along_x : concatenation::along_y))));
            } else if (c == "option") {
                if (t.at(1) == "optimize_data") opts.set_option(build_option::optimize_data(I(2) != 0));
                else if (t[1] == "outputs") opts.set_option(build_option::outputs(std::vector<primitive_id>(t.begin() + 2, t.end())));
                else throw std::runtime_error("unknown option " + t[1]);
            } else if (c == "build") net.reset(new network(eng, topo, opts));
            else if (c == "expect_build_error") {
                bool threw = false;
                try { network n(eng, topo, opts); } catch (const std::exception& e) { threw = true; std::printf("build refused: %s\n", e.what()); }
                if (!threw) throw std::runtime_error("the build was expected to fail");
            } else if (c == "set_input") net->set_input_data(t.at(1), mems.at(t.at(2)));
            else if (c == "execute") outputs = net->execute();
            else if (c == "save") {
                memory m = outputs.at(t.at(1)).get_memory();
                const layout l = m.get_layout();
                auto p = m.pointer<char>();
                std::ofstream f(dir + "/" + t.at(2), std::ios::binary);
                f.write(p.data(), (std::streamsize)l.bytes_count());
                std::printf("saved %s: format %d, b %d f %d y %d x %d, %zu bytes\n", t[1].c_str(), (int)l.format.value, l.size.batch[0], l.size.feature[0],
                            l.size.spatial[1], l.size.spatial[0], l.bytes_count());
            } else if (c == "info") std::printf("%s\n", net->get_primitive_info(t.at(1)).c_str());
            else throw std::runtime_error("line " + std::to_string(lineno) + ": unknown command " + c);
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_api_driver: %s\n", e.what());
        return 1;
    }
    return 0;
}
