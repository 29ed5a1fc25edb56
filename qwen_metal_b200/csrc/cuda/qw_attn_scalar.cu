// Diagnostic fp32 attention kernel: one CTA per (row, head, batch), scores in
// shared memory, three passes (scores + max, exp + sum, weighted V sum) like the
// reference's scalar causal kernel (h3_shaders.metal:5003-5069) but with the
// prefix-limit / key-padding mask of the flash path.  It exists so the tensor
// memory kernel can be cross-checked on the GPU at sizes where a CPU check is
// slow, and to serve degenerate scales (0, negative, non-finite).  It is not a
// performance path.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../qw_cuda.h"

namespace {

constexpr int kThreads = 128;
constexpr int kHeadDim = 128;

__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) {
    return __uint_as_float((uint32_t)__bfloat16_as_ushort(v) << 16);
}
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16(float v) {
    uint32_t bits = __float_as_uint(v);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return __ushort_as_bfloat16((unsigned short)(bits >> 16));
}

__device__ float block_reduce(float v, bool is_max, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float o = __shfl_xor_sync(0xffffffffu, v, off);
        v = is_max ? fmaxf(v, o) : v + o;
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int w = 1; w < kThreads / 32; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
    return r;
}

__global__ void __launch_bounds__(kThreads) qw_attn_scalar_kernel(const qwcu_attn_args a) {
    extern __shared__ float scores[];
    __shared__ float q_sh[kHeadDim];
    __shared__ float red[kThreads / 32];
    const uint32_t r = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const uint32_t kvh = (uint32_t)((unsigned long long)h * a.kv_heads / a.heads);
    const __nv_bfloat16 *q = static_cast<const __nv_bfloat16 *>(a.q);
    const __nv_bfloat16 *k = static_cast<const __nv_bfloat16 *>(a.k);
    const __nv_bfloat16 *v = static_cast<const __nv_bfloat16 *>(a.v);
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(a.out);
    const int tid = threadIdx.x;

    int limit;
    if (a.kv_limit) {
        limit = a.kv_limit[a.per_batch_limits ? (size_t)b * a.q_rows + r : r];
        limit = max(limit, 0);
    } else if (a.causal) {
        unsigned long long c = (unsigned long long)r + 1ull + a.causal_offset;
        limit = (int)min(c, (unsigned long long)a.kv_rows);
    } else {
        limit = (int)a.kv_rows;
    }
    limit = min(limit, (int)a.kv_rows);
    const int pad_lo = a.text_pad ? (int)a.text_len[b] : 0;
    const int pad_hi = (int)a.text_pad;
    if (a.text_pad && (int)r >= pad_lo && (int)r < pad_hi) limit = 0;

    const size_t o_index = a.head_major_out
                               ? (((size_t)b * a.heads + h) * a.q_rows + r) * kHeadDim
                               : (((size_t)b * a.q_rows + r) * a.heads + h) * kHeadDim;
    {
        float qv = bf16_to_f32(q[(((size_t)b * a.q_rows + r) * a.heads + h) * kHeadDim + tid]);
        if (a.scale_in_q) qv = bf16_to_f32(f32_to_bf16(qv * a.scale));
        q_sh[tid] = qv;
    }
    __syncthreads();

    float local_max = -INFINITY;
    for (int s = tid; s < limit; s += kThreads) {
        float score = -INFINITY;
        if (!(s >= pad_lo && s < pad_hi)) {
            const __nv_bfloat16 *kr = k + (((size_t)b * a.kv_rows + s) * a.kv_heads + kvh) * kHeadDim;
            float dot = 0.0f;
            for (int d = 0; d < kHeadDim; ++d) dot = fmaf(q_sh[d], bf16_to_f32(kr[d]), dot);
            score = a.scale_in_q ? dot : dot * a.scale;
        }
        scores[s] = score;
        local_max = fmaxf(local_max, score);
    }
    const float m = block_reduce(local_max, true, red);
    if (m == -INFINITY) {  // no visible key
        out[o_index + tid] = f32_to_bf16(0.0f);
        return;
    }
    float local_sum = 0.0f;
    for (int s = tid; s < limit; s += kThreads) {
        float p = scores[s] == -INFINITY ? 0.0f : expf(scores[s] - m);
        scores[s] = p;
        local_sum += p;
    }
    const float denom = block_reduce(local_sum, false, red);
    const float inv = 1.0f / denom;
    float acc = 0.0f;
    for (int s = 0; s < limit; ++s) {
        float p = scores[s];
        if (p != 0.0f)
            acc = fmaf(p * inv,
                       bf16_to_f32(v[(((size_t)b * a.kv_rows + s) * a.kv_heads + kvh) * kHeadDim + tid]),
                       acc);
    }
    out[o_index + tid] = f32_to_bf16(acc);
}

}  // namespace

extern "C" int qwcu_attn_scalar_launch(const qwcu_attn_args *a, qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a->batch || a->batch > 8 || !a->q_rows || !a->kv_rows || !a->heads || !a->kv_heads)
        return (int)cudaErrorInvalidValue;
    size_t smem = (size_t)a->kv_rows * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(qw_attn_scalar_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(a->q_rows, a->heads, a->batch);
    qw_attn_scalar_kernel<<<grid, kThreads, smem, stream>>>(*a);
    return (int)cudaGetLastError();
}
