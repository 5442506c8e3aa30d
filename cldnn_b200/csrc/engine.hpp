// Internal interfaces of the CUDA engine: context, prepared launches and the
// table of ahead-of-time compiled kernels that kernel_lookup resolves by name
// (the role kernels_cache played for JIT-compiled OpenCL programs,
// src/gpu/kernels_cache.cpp:189-215).
#pragma once
#include <cuda_runtime.h>
#include <functional>
#include <stdint.h>
#include "common.cuh"

struct cldnn_b200_ctx_impl {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool profiling = false;
    uint64_t launches = 0;
    bool capturing = false;
    uint64_t capture_start_launches = 0;
    uint32_t* d_status = nullptr;     // device word written by kernels whose bounded wait gave up
    cudaDeviceProp prop{};
};

struct cldnn_b200_mem_impl {
    cldnn_b200_ctx_impl* ctx = nullptr;
    void* dev = nullptr;
    size_t bytes = 0;
    bool attached = false;            // wraps memory owned by the caller
    void* mapped = nullptr;           // pinned staging while locked
    int map_count = 0;
};

struct cldnn_b200_event_impl {
    cldnn_b200_ctx_impl* ctx = nullptr;
    cudaEvent_t ev = nullptr;
};

struct cldnn_b200_prepared_impl {
    cldnn_b200_ctx_impl* ctx = nullptr;
    std::function<cudaError_t(cudaStream_t)> fn;   // enqueues the kernel(s)
    int launches = 1;
};

struct cldnn_b200_graph_impl {
    cldnn_b200_ctx_impl* ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
};

namespace b200 {

// Raises the dynamic shared-memory limit of kernel `fn` on `device` (which must be current) to at least `bytes`.  The limit
// is a property of (function, device) shared by every prepared launch, so it only ever grows: a later, smaller shape must
// not lower it under an earlier launch that is still alive.
cudaError_t raise_smem_limit(const void* fn, int device, size_t bytes);

struct KernelDef {
    const char* name;
    size_t params_size;
    bool (*supports)(const void* params);
    int (*tune_count)(const void* params);
    size_t (*scratch_bytes)(const void* params);
    int32_t (*prepare)(cldnn_b200_ctx_impl* ctx, const void* params, const cldnn_b200_args* args,
                       cldnn_b200_prepared_impl* out);
};

// one definition per kernel file
extern const KernelDef kdef_conv_ref;
extern const KernelDef kdef_conv_i8_tc;
extern const KernelDef kdef_conv_i8_first;
extern const KernelDef kdef_conv_first_tc;
extern const KernelDef kdef_conv_f16_tc;
extern const KernelDef kdef_conv_f16_winograd;
extern const KernelDef kdef_conv_i8_dw;
extern const KernelDef kdef_pooling_ref;
extern const KernelDef kdef_pooling_i8_byxf;
extern const KernelDef kdef_pooling_f16_byxf;
extern const KernelDef kdef_lrn_f16_byxf;
extern const KernelDef kdef_fc_ref;
extern const KernelDef kdef_softmax;
extern const KernelDef kdef_eltwise_ref;
extern const KernelDef kdef_eltwise_byxf;
extern const KernelDef kdef_reorder_ref;
extern const KernelDef kdef_lrn_ref;
extern const KernelDef kdef_activation_ref;

}  // namespace b200

struct cldnn_b200_kernel_impl {
    cldnn_b200_ctx_impl* ctx = nullptr;
    const b200::KernelDef* def = nullptr;
};
