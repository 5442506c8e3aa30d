// Row form of the first-layer convolution (conv_i8_first_rows.cu): tuning variants 4 / 5 of conv_i8_first (8-bit) and 2 / 3 of
// conv_first_tc (fp16).
#pragma once
#include <string>
#include "engine.hpp"

namespace b200 {
bool first_rows_plan(const cldnn_b200_conv_params& p, std::string* why);
size_t first_rows_scratch(const cldnn_b200_conv_params& p);
// `groups`: 2 or 4 epilogue warp groups
int32_t first_rows_prepare(cldnn_b200_ctx_impl* ctx, const cldnn_b200_conv_params& p, const cldnn_b200_args* a, cldnn_b200_prepared_impl* out, int groups);
}
