// The two element-wise neighbours of the attention path in the DiT block, both
// HBM-bound: the AdaLN norm in front of the QKV projection and the gated
// residual behind the output projection.
//
//   layer_norm_mod : out = bf16((x - mean) * rsqrt(var + eps) * (1 + scale[row_map[row]]))
//                    (reference h3_shaders.metal:4767-4813)
//   gate           : out = bf16(residual + branch * gate[row_map[row]])
//                    (reference h3_shaders.metal:3583-3599)
//
// The norm keeps a row in registers (one warp per row, 16-byte loads, all of
// them in flight before the first use), so every input byte is read once and
// every output byte written once; mean and variance are the reference's two
// passes, done on the register copy.  Rows wider than the register budget, or
// not a multiple of 8 columns, take a plain loop that re-reads the row from
// cache.  The modulation rows are shared by all rows of a segment and stay in L2.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../qw_cuda.h"

namespace {

// (128-thread CTAs: the row copy plus the prefetched modulation vectors take up to
// about 150 registers per thread, and three to four such CTAs fit on an SM)
constexpr int kWarpsPerBlock = 4;
constexpr int kMaxVecs = 16;  // 16-byte vectors per lane: rows up to 32 * 16 * 8 = 4096 columns

__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ uint16_t round_bf16(float v) {
    return (uint16_t)(pack_bf16(v, 0.0f) & 0xffffu);
}

// The modulation row of a token: row_map[row] indexes [maps][slots][width].  An
// index outside the tensor is recorded in the status words (the submit then
// fails) and row 0 is used instead, so a stale map cannot read out of bounds.
__device__ __forceinline__ uint32_t checked_map(const uint32_t *row_map, uint32_t row,
                                                uint32_t maps, uint32_t *status) {
    const uint32_t map = row_map[row];
    if (map < maps) return map;
    if (status && atomicCAS(status, 0u, (uint32_t)QWCU_STATUS_BAD_ARGUMENT) == 0u) {
        status[1] = 0x40000u;  // where: modulation row index
        status[2] = row;
        status[3] = map;
    }
    return 0u;
}

struct NormArgs {
    const uint16_t *in;
    const uint16_t *modulation;
    const uint32_t *row_map;
    uint16_t *out;
    uint32_t rows, width, slots, scale_slot;
    float epsilon;
    uint32_t maps;
    uint32_t *status;
};

// width % 8 == 0 and width <= 32 * kVecs * 8.  A warp walks rows (stride = warps
// in the grid); the grid holds a few resident CTAs per SM, so no time goes into
// launching a CTA per handful of rows.
template <int kVecs>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qw_layer_norm_mod_kernel(const NormArgs a) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t vecs = a.width >> 3;  // 16-byte vectors per row
    const uint32_t warps = gridDim.x * kWarpsPerBlock;
    for (uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); row < a.rows;
         row += warps) {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.in + (size_t)row * a.width);
        uint4 x[kVecs];
#pragma unroll
        for (int i = 0; i < kVecs; ++i) {
            const uint32_t v = lane + 32u * i;
            x[i] = v < vecs ? __ldcs(src + v) : make_uint4(0, 0, 0, 0);
        }
        const uint32_t map = checked_map(a.row_map, row, a.maps, a.status);
        const uint4 *scale = reinterpret_cast<const uint4 *>(
            a.modulation + ((size_t)map * a.slots + a.scale_slot) * a.width);

        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kVecs; ++i) {
            const uint32_t w[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) sum += bf16_lo(w[k]) + bf16_hi(w[k]);
        }
        const float mean = warp_sum(sum) / (float)a.width;
        float square = 0.0f;
#pragma unroll
        for (int i = 0; i < kVecs; ++i) {
            if (lane + 32u * i < vecs) {  // padding vectors hold zeros, not (0 - mean)
                const uint32_t w[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float c0 = bf16_lo(w[k]) - mean, c1 = bf16_hi(w[k]) - mean;
                    square = fmaf(c0, c0, square);
                    square = fmaf(c1, c1, square);
                }
            }
        }
        const float inverse = rsqrtf(warp_sum(square) / (float)a.width + a.epsilon);

        uint4 *dst = reinterpret_cast<uint4 *>(a.out + (size_t)row * a.width);
#pragma unroll
        for (int i = 0; i < kVecs; ++i) {
            const uint32_t v = lane + 32u * i;
            if (v < vecs) {
                const uint4 s = __ldg(scale + v);
                const uint32_t w[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
                const uint32_t g[4] = {s.x, s.y, s.z, s.w};
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float n0 = __fmul_rn(__fsub_rn(bf16_lo(w[k]), mean), inverse);
                    const float n1 = __fmul_rn(__fsub_rn(bf16_hi(w[k]), mean), inverse);
                    o[k] = pack_bf16(__fmul_rn(n0, __fadd_rn(1.0f, bf16_lo(g[k]))),
                                     __fmul_rn(n1, __fadd_rn(1.0f, bf16_hi(g[k]))));
                }
                __stcs(dst + v, make_uint4(o[0], o[1], o[2], o[3]));
            }
        }
    }
}

// Any width: one warp per row, three passes over the (cached) row.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qw_layer_norm_mod_generic_kernel(const NormArgs a) {
    const uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint16_t *x = a.in + (size_t)row * a.width;
    float sum = 0.0f;
    for (uint32_t c = lane; c < a.width; c += 32) sum += __uint_as_float((uint32_t)x[c] << 16);
    const float mean = warp_sum(sum) / (float)a.width;
    float square = 0.0f;
    for (uint32_t c = lane; c < a.width; c += 32) {
        const float centered = __uint_as_float((uint32_t)x[c] << 16) - mean;
        square = fmaf(centered, centered, square);
    }
    const float inverse = rsqrtf(warp_sum(square) / (float)a.width + a.epsilon);
    const uint16_t *scale =
        a.modulation +
        ((size_t)checked_map(a.row_map, row, a.maps, a.status) * a.slots + a.scale_slot) * a.width;
    for (uint32_t c = lane; c < a.width; c += 32) {
        const float n = __fmul_rn(__fsub_rn(__uint_as_float((uint32_t)x[c] << 16), mean), inverse);
        const float s = __uint_as_float((uint32_t)scale[c] << 16);
        a.out[(size_t)row * a.width + c] = round_bf16(__fmul_rn(n, __fadd_rn(1.0f, s)));
    }
}

struct GateArgs {
    const uint16_t *residual;
    const uint16_t *branch;
    const uint16_t *modulation;
    const uint32_t *row_map;
    uint16_t *out;
    uint32_t rows, width, slots, gate_slot;
    uint32_t maps;
    uint32_t *status;
};

// width % 8 == 0: one 16-byte vector per thread and step.
__global__ void __launch_bounds__(256) qw_gate_kernel(const GateArgs a) {
    const uint32_t vecs = a.width >> 3;
    const size_t total = (size_t)a.rows * vecs;
    const uint4 *residual = reinterpret_cast<const uint4 *>(a.residual);
    const uint4 *branch = reinterpret_cast<const uint4 *>(a.branch);
    uint4 *out = reinterpret_cast<uint4 *>(a.out);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / vecs);
        const uint32_t v = (uint32_t)(i - (size_t)row * vecs);
        const uint4 r = __ldcs(residual + i);
        const uint4 b = __ldcs(branch + i);
        const uint4 g = __ldg(reinterpret_cast<const uint4 *>(
                                  a.modulation +
                                  ((size_t)checked_map(a.row_map, row, a.maps, a.status) * a.slots +
                                   a.gate_slot) * a.width) +
                              v);
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w}, bw[4] = {b.x, b.y, b.z, b.w},
                       gw[4] = {g.x, g.y, g.z, g.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            o[k] = pack_bf16(__fadd_rn(bf16_lo(rw[k]), __fmul_rn(bf16_lo(bw[k]), bf16_lo(gw[k]))),
                             __fadd_rn(bf16_hi(rw[k]), __fmul_rn(bf16_hi(bw[k]), bf16_hi(gw[k]))));
        __stcs(out + i, make_uint4(o[0], o[1], o[2], o[3]));
    }
}

__global__ void __launch_bounds__(256) qw_gate_generic_kernel(const GateArgs a) {
    const size_t total = (size_t)a.rows * a.width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / a.width);
        const uint32_t c = (uint32_t)(i - (size_t)row * a.width);
        const float gate = __uint_as_float(
            (uint32_t)a.modulation[((size_t)checked_map(a.row_map, row, a.maps, a.status) * a.slots +
                                    a.gate_slot) * a.width + c]
            << 16);
        const float value = __fadd_rn(__uint_as_float((uint32_t)a.residual[i] << 16),
                                      __fmul_rn(__uint_as_float((uint32_t)a.branch[i] << 16), gate));
        a.out[i] = round_bf16(value);
    }
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

extern "C" int qwcu_layer_norm_mod_launch(const qwcu_rowwise_args *a, int sm_count,
                                          qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a->rows || !a->width) return (int)cudaErrorInvalidValue;
    NormArgs k;
    k.in = static_cast<const uint16_t *>(a->input);
    k.modulation = static_cast<const uint16_t *>(a->modulation);
    k.row_map = a->row_map;
    k.out = static_cast<uint16_t *>(a->output);
    k.rows = a->rows;
    k.width = a->width;
    k.slots = a->slots;
    k.scale_slot = a->slot;
    k.epsilon = a->epsilon;
    k.maps = a->maps;
    k.status = a->status;
    if (!a->maps) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (a->rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const bool vector = a->width % 8 == 0 && a->width <= 32u * kMaxVecs * 8u &&
                        aligned16(k.in) && aligned16(k.out) && aligned16(k.modulation);
    if (!vector) {
        qw_layer_norm_mod_generic_kernel<<<blocks, kWarpsPerBlock * 32, 0, stream>>>(k);
        return (int)cudaGetLastError();
    }
    // A few resident CTAs per SM, each warp walking rows.
    const unsigned cap = (unsigned)(sm_count > 0 ? sm_count : 148) * 4u;
    const unsigned grid = blocks < cap ? blocks : cap;
    const uint32_t vecs_per_lane = (a->width / 8 + 31) / 32;
    if (vecs_per_lane <= 4)
        qw_layer_norm_mod_kernel<4><<<grid, kWarpsPerBlock * 32, 0, stream>>>(k);
    else if (vecs_per_lane <= 8)
        qw_layer_norm_mod_kernel<8><<<grid, kWarpsPerBlock * 32, 0, stream>>>(k);
    else if (vecs_per_lane <= 12)
        qw_layer_norm_mod_kernel<12><<<grid, kWarpsPerBlock * 32, 0, stream>>>(k);
    else
        qw_layer_norm_mod_kernel<kMaxVecs><<<grid, kWarpsPerBlock * 32, 0, stream>>>(k);
    return (int)cudaGetLastError();
}

extern "C" int qwcu_gate_launch(const qwcu_rowwise_args *a, int sm_count, qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a->rows || !a->width) return (int)cudaErrorInvalidValue;
    GateArgs k;
    k.residual = static_cast<const uint16_t *>(a->input);
    k.branch = static_cast<const uint16_t *>(a->branch);
    k.modulation = static_cast<const uint16_t *>(a->modulation);
    k.row_map = a->row_map;
    k.out = static_cast<uint16_t *>(a->output);
    k.rows = a->rows;
    k.width = a->width;
    k.slots = a->slots;
    k.gate_slot = a->slot;
    k.maps = a->maps;
    k.status = a->status;
    if (!a->maps) return (int)cudaErrorInvalidValue;
    const bool vector = a->width % 8 == 0 && aligned16(k.residual) && aligned16(k.branch) &&
                        aligned16(k.out) && aligned16(k.modulation);
    const size_t items = vector ? (size_t)a->rows * (a->width / 8) : (size_t)a->rows * a->width;
    // Enough CTAs to cover the work once, capped at a few waves of the device.
    size_t blocks = (items + 255) / 256;
    const size_t cap = (size_t)(sm_count > 0 ? sm_count : 148) * 32;
    if (blocks > cap) blocks = cap;
    if (vector)
        qw_gate_kernel<<<(unsigned)blocks, 256, 0, stream>>>(k);
    else
        qw_gate_generic_kernel<<<(unsigned)blocks, 256, 0, stream>>>(k);
    return (int)cudaGetLastError();
}
