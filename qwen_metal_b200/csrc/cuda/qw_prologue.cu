// Fused per-head QK RMSNorm + interleaved 3-axis RoPE (HBM-bound prologue).
//
// A head is 128 bf16 = 256 B = sixteen 16-byte vectors, so a half-warp owns one
// head at a time: one 16-byte load per lane (8 elements = 4 whole RoPE pairs), a
// 4-step shuffle reduction for the sum of squares, then the rotation, one
// 16-byte store.  Each half-warp walks all heads of one (row, tensor) strip with
// its slice of the norm weight and of the row's cos/sin held in registers, four
// heads in flight at a time.  Q and K each cross HBM exactly once in each
// direction.  The kernel was instruction-bound before it was HBM-bound, so the
// bf16 roundings use cvt.rn.bf16x2.f32 and the inverse norm uses rsqrtf.
//
// Arithmetic follows the reference's three separate kernels including the bf16
// store between norm and rotation: n = bf16(x * inv * w) (h3_shaders.metal:
// 4309-4329; bf16(bf16(x*inv)*w) for the double-rounding variant :4975-4997),
// then (e, o) <- bf16(e*c - o*s), bf16(e*s + o*c) (h3_shaders.metal:4864-4890),
// products and sums as separate fp32 operations.  The sum of squares is reduced
// as a tree and 1/sqrt is within 2 ulp, where the reference shader runs a serial
// fma chain and its own rsqrt: a normalised value differs from a serial CPU
// restatement by one bf16 step in about 1 element in 10^5.

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

struct Params {
    const uint4 *q_in;
    const uint4 *k_in;
    uint4 *q_out;
    uint4 *k_out;
    const uint4 *v_in;  // optional third tensor: copied as is (K/V cache update)
    uint4 *v_out;
    const uint4 *wq;
    const uint4 *wk;
    const float4 *cos_t;
    const float4 *sin_t;
    uint32_t rows, table_rows, heads;
    float eps;
    int double_round;
    uint32_t strips;  // rows * tensors: one half-warp walks the heads of one (row, tensor)
    int tensors;
    float *bound_out;  // optional: [0], [1] = upper bounds of the 2-norm of any q row, k row
};

// Two floats -> packed bf16 pair, round to nearest even in one instruction
// (the same rounding as the integer trick for every finite value).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Heads a half-warp has in flight at once (independent 16-byte loads; the
// kernel is HBM-bound once the instruction count is small enough).
constexpr int kHeadsPerTrip = 4;

// A half-warp owns one (row, tensor) strip: it keeps its 8-element slice of the
// norm weight and of the row's cos/sin in registers and walks the heads, four at
// a time.  Lane l holds elements [8l, 8l+8) of every head = RoPE pairs 4l..4l+3.
// The two half-warps of a warp may hold different tensors (a normed key strip
// next to a copied value strip), so the reductions name their own 16 lanes.
__global__ void __launch_bounds__(256) qw_prologue_kernel(const Params p) {
    const int lane16 = threadIdx.x & 15;
    const uint32_t half_mask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
    const uint32_t half_warps = (gridDim.x * blockDim.x) >> 4;
    // Both half-warps of a warp run the same number of trips (the strip count is
    // padded to an even number by the host): the shuffles need the whole warp.
    for (uint32_t strip = (blockIdx.x * blockDim.x + threadIdx.x) >> 4; strip < p.strips;
         strip += half_warps) {
        const uint32_t row = strip / (uint32_t)p.tensors;
        const uint32_t which = strip - row * (uint32_t)p.tensors;  // 0 query, 1 key, 2 value
        const bool live = row < p.rows;
        const uint4 *src = (which == 0 ? p.q_in : which == 1 ? p.k_in : p.v_in) +
                           (size_t)row * p.heads * 16 + lane16;
        uint4 *dst = (which == 0 ? p.q_out : which == 1 ? p.k_out : p.v_out) +
                     (size_t)row * p.heads * 16 + lane16;
        const uint4 *w = which == 0 ? p.wq : which == 1 ? p.wk : nullptr;
        const bool rotate = p.cos_t && which < 2;
        float wf[8], cc[4], sn[4];
        if (w) {
            const uint4 wv = w[lane16];
            wf[0] = bf16_lo(wv.x); wf[1] = bf16_hi(wv.x); wf[2] = bf16_lo(wv.y); wf[3] = bf16_hi(wv.y);
            wf[4] = bf16_lo(wv.z); wf[5] = bf16_hi(wv.z); wf[6] = bf16_lo(wv.w); wf[7] = bf16_hi(wv.w);
        }
        if (p.bound_out && strip < 2u && w) {
            // The first two strips are row 0 of q and of k.  A normalised head has
            // sum (x*inv)^2 <= 128, so after the weight its 2-norm is at most
            // sqrt(128) * max|w|; the two bf16 roundings (norm, rotation) and the
            // f32 tables add well under 1 %.  The rotation itself preserves it.
            float wmax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) wmax = fmaxf(wmax, fabsf(wf[i]));
#pragma unroll
            for (int off = 8; off > 0; off >>= 1)
                wmax = fmaxf(wmax, __shfl_xor_sync(half_mask, wmax, off, 16));
            if (lane16 == 0) p.bound_out[which] = 11.313708499f * 1.01f * wmax;
        }
        if (rotate) {
            const size_t t = (size_t)((live ? row : 0u) % p.table_rows) * 16 + lane16;
            const float4 c = p.cos_t[t], s4 = p.sin_t[t];
            cc[0] = c.x; cc[1] = c.y; cc[2] = c.z; cc[3] = c.w;
            sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
        }
        for (uint32_t head0 = 0; head0 < p.heads; head0 += kHeadsPerTrip) {
            uint4 x[kHeadsPerTrip];
#pragma unroll
            for (int u = 0; u < kHeadsPerTrip; ++u)
                x[u] = (live && head0 + u < p.heads) ? src[(size_t)(head0 + u) * 16]
                                                     : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < kHeadsPerTrip; ++u) {
                float v[8] = {bf16_lo(x[u].x), bf16_hi(x[u].x), bf16_lo(x[u].y), bf16_hi(x[u].y),
                              bf16_lo(x[u].z), bf16_hi(x[u].z), bf16_lo(x[u].w), bf16_hi(x[u].w)};
                uint32_t y[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
                if (w) {
                    float ss = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1)
                        ss += __shfl_xor_sync(half_mask, ss, off, 16);
                    // mean = ss / 128 exactly; 1/sqrt to within 2 ulp of the reference's rsqrt
                    const float inv = rsqrtf(__fadd_rn(ss * 0.0078125f, p.eps));
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        float n0 = __fmul_rn(v[i], inv), n1 = __fmul_rn(v[i + 1], inv);
                        if (p.double_round) {
                            const uint32_t r = pack_bf16x2(n0, n1);
                            n0 = bf16_lo(r);
                            n1 = bf16_hi(r);
                        }
                        y[i >> 1] = pack_bf16x2(__fmul_rn(n0, wf[i]), __fmul_rn(n1, wf[i + 1]));
                    }
                    if (rotate) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {  // the bf16 store between norm and rotation
                            v[2 * i] = bf16_lo(y[i]);
                            v[2 * i + 1] = bf16_hi(y[i]);
                        }
                    }
                }
                if (rotate) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float e = v[2 * i], o = v[2 * i + 1];
                        y[i] = pack_bf16x2(__fsub_rn(__fmul_rn(e, cc[i]), __fmul_rn(o, sn[i])),
                                           __fadd_rn(__fmul_rn(e, sn[i]), __fmul_rn(o, cc[i])));
                    }
                }
                if (live && head0 + u < p.heads)
                    dst[(size_t)(head0 + u) * 16] = make_uint4(y[0], y[1], y[2], y[3]);
            }
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

// SM count of the current device (a process may drive several devices).
int sm_count_cached() {
    static int sms[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        if (sms[dev] <= 0) sms[dev] = 148;
    }
    return sms[dev];
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
    p.v_in = static_cast<const uint4 *>(a->v_in);
    p.v_out = static_cast<uint4 *>(a->v_out);
    p.bound_out = a->bound_out;
    if (a->bound_out && (!a->k_in || a->v_in || !a->norm_weight_q || !a->norm_weight_k))
        return (int)cudaErrorInvalidValue;
    if (a->v_in && (!a->k_in || !a->v_out)) return (int)cudaErrorInvalidValue;
    p.tensors = a->v_in ? 3 : a->k_in ? 2 : 1;
    unsigned long long strips = (unsigned long long)a->rows * p.tensors;
    strips = (strips + 1ull) & ~1ull;  // whole warps iterate together
    if (strips > 0xffffffffull) return (int)cudaErrorInvalidValue;
    p.strips = (uint32_t)strips;
    const int threads = 256;
    unsigned long long want = (strips * 16 + threads - 1) / threads;
    // Grid: at most 8 resident CTAs per SM, a multiple of the SM count when capped.
    unsigned long long cap = (unsigned long long)sm_count_cached() * 8ull;
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
