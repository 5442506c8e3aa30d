// Shared declarations of the tensor-core 8-bit convolution kernels: the launch
// parameter block the host fills once per prepared launch.
#pragma once
#include <cuda.h>
#include "engine.hpp"
#include "sm100_ptx.cuh"

namespace b200 {

using namespace ptx;

constexpr int kBM = 128;                 // pixels per tile = TMEM lanes
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kStoreWarp = 2 + kEpiWarps;  // warp that issues the TMA stores of finished tiles
constexpr int kThreads = 64 + kEpiThreads + 32;
constexpr int kMaxStages = 8;
constexpr int kMaxBN = 256;
constexpr int kMaxBufs = 8;               // accumulator / staging buffers in flight per CTA (512 columns of tensor memory / feature tile)
constexpr uint32_t kErrProducer = 0x10u, kErrMma = 0x20u, kErrEpilogue = 0x30u, kErrDrain = 0x40u;

enum AMode { A_FLAT = 0, A_IM2COL = 1, A_TILED = 2, A_PATCH = 3 };

struct alignas(64) TcParams {
    CUtensorMap tmA;                     // activations
    CUtensorMap tmB;                     // weights
    CUtensorMap tmO;                     // output (staged epilogue)
    CUtensorMap tmE;                     // residual input (staged epilogue, fused)
    int32_t a_mode;
    int32_t N, P, Q;                     // output batch, rows, columns
    int32_t kh, kw, stride_x, stride_y, pad_x, pad_y, dil_x, dil_y;
    int32_t bk, chunks, k_steps;         // bytes of K per stage, channel chunks per tap, stages per tile
    int32_t bn, n_tiles, m_tiles, total_tiles;
    int64_t M_total;
    int32_t bw, bh, bb, tiles_w, tiles_h; // tiled mode: box of bw x bh x bb pixels
    int32_t stages, a_stage_bytes, b_stage_bytes, a_tx_bytes, b_tx_bytes;
    uint32_t sbo, layout_type, idesc, tmem_cols;
    int32_t ofm;
    // epilogue
    int32_t staged;                      // 1: shared-memory tile + TMA store, 0: direct stores
    int32_t fast_epi;                    // quantised, 8-bit output and residual, simple activations
    int32_t cw, col_blocks, sw_shift, sw_mask, stage_rows;   // staging tile: column block width, 16-byte chunk swizzle
    int32_t mul_iqf, mul_oqf;
    int32_t lean;                        // epilogue configuration covered by the hoisted fast body
    int32_t nbuf;                        // accumulator and staging buffers in flight: 512 / feature tile, at most 8
    int32_t nstg;                        // conv_i8_tc_fast: staging tiles (>= nbuf when a fused residual is prefetched into them)
    // patch mode: all weights resident in shared memory, one activation patch per (filter column, channel chunk)
    int32_t ring_bytes, b_total_bytes;   // operand area: activation ring (+ weight ring or resident weights)
    int32_t patch_alloc;                 // bytes reserved per filter column's patch inside a stage (a stage holds the kw patches of one channel chunk)
    int32_t fast_variant;                // conv_i8_tc_fast: (output kind << 1) | ReLU before the residual sum
    int32_t epi_groups;                  // conv_i8_tc_fast: epilogue warp groups per CTA, 2 or 4
    int32_t b_resident;                  // conv_i8_tc_fast, modes other than patch: the weights of every step and feature tile stay in shared memory
    int32_t pair;                        // conv_i8_tc_fast: CTA pairs (cta_group::2): m_tiles is even, the weight box holds bn / 2 rows
    float acc_bound;                     // K * max|activation| * 128: no accumulator can exceed it in magnitude
    // output / residual addressing for the direct path, in elements
    int64_t out_px, out_py, out_pb, out_off;
    int64_t el_px, el_py, el_pb, el_off;
    int32_t el_sx, el_sy;
    void* out; const void* eltw; const void* bias; const float* quant; const float* calib; const float* ecal;
    uint32_t* status;
    EpiCfg epi;
};

// conv_i8_tc_fast.cu: the specialised kernels for the common network configuration.
bool tc_fast_eligible(const TcParams& P);
cudaError_t tc_fast_configure(const TcParams& P, int max_smem);
cudaError_t tc_fast_launch(const TcParams& P, int grid, size_t smem_bytes, cudaStream_t stream);
size_t tc_fast_aux_bytes();

}  // namespace b200
