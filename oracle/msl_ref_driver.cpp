// Test infrastructure: runs the reference's scalar shader kernels on the CPU.
//
// The kernels are the reference's own text (cut out of h3_shaders.metal by
// extract_msl.py into _ref/msl_kernels.inc at build time) compiled through
// msl_shim.h.  This file only plays the GPU's part: it walks the dispatch grid
// the reference's op wrappers use and calls the kernel once per thread.
//   h3_gpu_head_rms_norm_bf16 / qw_gpu_head_rms_norm_bf16: grid (sequence, heads)
//     (h3_gpu.m:4478-4493, :5258-5275)
//   qw_gpu_qk_rope_bf16: grid (head_dim/2, heads, sequence) (h3_gpu.m:5159-5193)
//   qw_gpu_layer_norm_mod_bf16: one threadgroup per row, 256 threads
//     (h3_gpu.m:357-378, :5100-5124); the threads of a group run as real threads
//     that meet at the kernel's own barriers
//   h3_gpu_gate_bf16: grid (width, rows) (h3_gpu.m:3865-3889)
#include "msl_shim.h"

#include <thread>
#include <vector>

namespace msl_emulation {
thread_local std::barrier<> *group_barrier = nullptr;
}

#include "_ref/msl_kernels.inc"

extern "C" {

void msl_head_rms_norm_bf16(uint16_t *tensor, const uint16_t *weight, uint32_t sequence,
                            uint32_t heads, uint32_t head_dim, float epsilon, int double_round) {
    head_norm_args args = {sequence, heads, head_dim, epsilon};
    for (uint32_t row = 0; row < sequence; row++)
        for (uint32_t head = 0; head < heads; head++) {
            uint2 gid = {row, head};
            if (double_round) qw_head_rms_norm_bf16(tensor, weight, args, gid);
            else h3_head_rms_norm_bf16(tensor, weight, args, gid);
        }
}

void msl_qk_rope_bf16(uint16_t *q_out, uint16_t *k_out, const uint16_t *q_in, const uint16_t *k_in,
                      const float *rope_cos, const float *rope_sin, uint32_t sequence,
                      uint32_t heads, uint32_t head_dim) {
    qkv_args args = {sequence, heads, head_dim, head_dim / 2, 0, 0.0f};
    for (uint32_t row = 0; row < sequence; row++)
        for (uint32_t head = 0; head < heads; head++)
            for (uint32_t pair = 0; pair < head_dim / 2; pair++) {
                uint3 gid = {pair, head, row};
                qw_qk_rope_bf16(q_in, k_in, rope_cos, rope_sin, q_out, k_out, args, gid);
            }
}

void msl_layer_norm_mod_bf16(uint16_t *out, const uint16_t *in, const uint16_t *modulation,
                             const uint32_t *row_map, uint32_t rows, uint32_t width,
                             uint32_t slots, uint32_t scale_slot, float epsilon,
                             uint32_t threads) {
    qw_mod_args args = {rows, width, slots, scale_slot, epsilon};
    // One threadgroup (= one row) at a time; its threads are real threads so the
    // kernel's barriers and its shared reduction array behave as on the GPU.
    std::barrier<> sync((std::ptrdiff_t)threads);
    std::barrier<> next_row((std::ptrdiff_t)threads);
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < threads; t++)
        pool.emplace_back([&, t]() {
            msl_emulation::group_barrier = &sync;
            for (uint32_t row = 0; row < rows; row++) {
                uint3 group = {row, 0, 0}, tid = {t, 0, 0}, size = {threads, 1, 1};
                qw_layer_norm_mod_bf16(in, modulation, row_map, out, args, group, tid, size);
                next_row.arrive_and_wait();  // the shared array is reused by the next group
            }
            msl_emulation::group_barrier = nullptr;
        });
    for (auto &th : pool) th.join();
}

void msl_gate_bf16(uint16_t *out, const uint16_t *residual, const uint16_t *branch,
                   const uint16_t *modulation, const uint32_t *row_map, uint32_t rows,
                   uint32_t width, uint32_t slots, uint32_t gate_slot) {
    gate_args args = {rows, width, slots, gate_slot};
    for (uint32_t row = 0; row < rows; row++)
        for (uint32_t column = 0; column < width; column++) {
            uint2 gid = {column, row};
            h3_gate_bf16(residual, branch, modulation, row_map, out, args, gid);
        }
}

}  // extern "C"
