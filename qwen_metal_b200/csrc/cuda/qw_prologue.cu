// Fused per-head QK RMSNorm + interleaved 3-axis RoPE (HBM-bound prologue).
//
// A head is 128 bf16 = 256 B = sixteen 16-byte vectors, so a half-warp owns one
// (row, head) of one tensor: one 16-byte load per lane (8 elements = 4 whole
// RoPE pairs), a 4-step shuffle reduction for the sum of squares, then the
// rotation from two 16-byte f32 table loads, one 16-byte store.  Q and K each
// cross HBM exactly once in each direction.
//
// Arithmetic follows the reference's three separate kernels including the bf16
// store between norm and rotation: n = bf16(x * inv * w) (h3_shaders.metal:
// 4309-4329; bf16(bf16(x*inv)*w) for the double-rounding variant :4975-4997),
// then (e, o) <- bf16(e*c - o*s), bf16(e*s + o*c) (h3_shaders.metal:4864-4890),
// products and sums as separate fp32 operations.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../qw_cuda.h"

namespace {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Round-to-nearest-even by the integer trick the reference uses on every
// path (h3_shaders.metal:15-19); NaN handling is irrelevant here.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
    uint32_t bits = __float_as_uint(v);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return bits >> 16;
}
__device__ __forceinline__ float round_bf16(float v) {
    return __uint_as_float(f32_to_bf16_bits(v) << 16);
}

struct Params {
    const uint4 *q_in;
    const uint4 *k_in;
    uint4 *q_out;
    uint4 *k_out;
    const uint4 *wq;
    const uint4 *wk;
    const float4 *cos_t;
    const float4 *sin_t;
    uint32_t rows, table_rows, heads;
    float eps;
    int double_round;
    unsigned long long units;  // rows * heads * tensors
    int tensors;
};

__global__ void __launch_bounds__(256) qw_prologue_kernel(const Params p) {
    const int lane16 = threadIdx.x & 15;
    unsigned long long unit = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const unsigned long long stride = ((unsigned long long)gridDim.x * blockDim.x) >> 4;
    // All 16 lanes of a half-warp share `unit`; both halves of a warp stay in
    // the loop together because units is padded to an even count by the host.
    for (; unit < p.units; unit += stride) {
        // Unit order: (row, tensor, head) so q and k of a row share table lines.
        const unsigned long long per_row = (unsigned long long)p.heads * p.tensors;
        const uint32_t row = (uint32_t)(unit / per_row);
        const uint32_t rem = (uint32_t)(unit % per_row);
        const int is_k = rem >= p.heads;
        const uint32_t head = is_k ? rem - p.heads : rem;
        const bool live = row < p.rows;
        const size_t vec = ((size_t)row * p.heads + head) * 16 + lane16;
        const uint4 *src = is_k ? p.k_in : p.q_in;
        uint4 *dst = is_k ? p.k_out : p.q_out;
        const uint4 *w = is_k ? p.wk : p.wq;

        uint4 x = live ? src[vec] : make_uint4(0, 0, 0, 0);
        float v[8] = {bf16_lo(x.x), bf16_hi(x.x), bf16_lo(x.y), bf16_hi(x.y),
                      bf16_lo(x.z), bf16_hi(x.z), bf16_lo(x.w), bf16_hi(x.w)};
        if (w) {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off, 16);
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.0f), p.eps)));
            uint4 wv = w[lane16];
            float wf[8] = {bf16_lo(wv.x), bf16_hi(wv.x), bf16_lo(wv.y), bf16_hi(wv.y),
                           bf16_lo(wv.z), bf16_hi(wv.z), bf16_lo(wv.w), bf16_hi(wv.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float n = __fmul_rn(v[i], inv);
                if (p.double_round) n = round_bf16(n);
                v[i] = round_bf16(__fmul_rn(n, wf[i]));
            }
        }
        if (p.cos_t) {
            const size_t t = (size_t)(row % p.table_rows) * 16 + lane16;
            float4 c = live ? p.cos_t[t] : make_float4(1, 1, 1, 1);
            float4 s = live ? p.sin_t[t] : make_float4(0, 0, 0, 0);
            const float cc[4] = {c.x, c.y, c.z, c.w};
            const float sn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float e = v[2 * i], o = v[2 * i + 1];
                v[2 * i] = __fsub_rn(__fmul_rn(e, cc[i]), __fmul_rn(o, sn[i]));
                v[2 * i + 1] = __fadd_rn(__fmul_rn(e, sn[i]), __fmul_rn(o, cc[i]));
            }
        }
        if (live) {
            uint4 y;
            y.x = f32_to_bf16_bits(v[0]) | (f32_to_bf16_bits(v[1]) << 16);
            y.y = f32_to_bf16_bits(v[2]) | (f32_to_bf16_bits(v[3]) << 16);
            y.z = f32_to_bf16_bits(v[4]) | (f32_to_bf16_bits(v[5]) << 16);
            y.w = f32_to_bf16_bits(v[6]) | (f32_to_bf16_bits(v[7]) << 16);
            dst[vec] = y;
        }
    }
}

__global__ void qw_scale_bf16_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *in, size_t n,
                                     float scale) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = __uint_as_float((uint32_t)__bfloat16_as_ushort(in[i]) << 16);
        out[i] = __ushort_as_bfloat16((unsigned short)f32_to_bf16_bits(__fmul_rn(v, scale)));
    }
}

int sm_count_cached() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

}  // namespace

extern "C" int qwcu_prologue_launch(const qwcu_prologue_args *a, qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a->rows || !a->heads || !a->q_in || !a->q_out) return (int)cudaErrorInvalidValue;
    Params p;
    p.q_in = static_cast<const uint4 *>(a->q_in);
    p.k_in = static_cast<const uint4 *>(a->k_in);
    p.q_out = static_cast<uint4 *>(a->q_out);
    p.k_out = static_cast<uint4 *>(a->k_out);
    p.wq = static_cast<const uint4 *>(a->norm_weight_q);
    p.wk = static_cast<const uint4 *>(a->norm_weight_k);
    p.cos_t = reinterpret_cast<const float4 *>(a->rope_cos);
    p.sin_t = reinterpret_cast<const float4 *>(a->rope_sin);
    p.rows = a->rows;
    p.table_rows = a->table_rows ? a->table_rows : a->rows;
    p.heads = a->heads;
    p.eps = a->epsilon;
    p.double_round = a->double_round;
    p.tensors = a->k_in ? 2 : 1;
    unsigned long long units = (unsigned long long)a->rows * a->heads * p.tensors;
    p.units = (units + 1ull) & ~1ull;  // whole warps iterate together
    const int threads = 256;
    unsigned long long want = (p.units * 16 + threads - 1) / threads;
    // Persistent-ish grid: a multiple of the SM count, 8 resident CTAs per SM.
    unsigned long long cap = (unsigned long long)sm_count_cached() * 8ull * 4ull;
    unsigned int blocks = (unsigned int)(want < cap ? want : cap);
    if (!blocks) blocks = 1;
    qw_prologue_kernel<<<blocks, threads, 0, stream>>>(p);
    return (int)cudaGetLastError();
}

extern "C" int qwcu_scale_bf16_launch(void *out, const void *in, size_t elements, float scale,
                                      qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!elements) return 0;
    size_t want = (elements + 255) / 256;
    size_t cap = (size_t)sm_count_cached() * 16;
    unsigned int blocks = (unsigned int)(want < cap ? want : cap);
    qw_scale_bf16_kernel<<<blocks, 256, 0, stream>>>(static_cast<__nv_bfloat16 *>(out),
                                                     static_cast<const __nv_bfloat16 *>(in),
                                                     elements, scale);
    return (int)cudaGetLastError();
}

extern "C" int qwcu_device_sm_count(int device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    return sms;
}

extern "C" int qwcu_device_cc(int device) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess)
        return 0;
    return major * 10 + minor;
}
