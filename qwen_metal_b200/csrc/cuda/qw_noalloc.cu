// h3_gpu_gqa_causal_noalloc_bf16: the token-causal attention op whose query is
// pre-scaled and re-rounded to bf16 (the arithmetic of h3_gpu_gqa_causal_bf16),
// for callers that must not allocate device memory when they call it.
//
// The regular op keeps the pre-scaled query in a scratch block it obtains from
// the CUDA allocator on demand.  That is a problem for a host program that has
// handed the whole GPU to its own arena at start-up (a later cudaMalloc simply
// fails there), and for a steady-state loop that cannot afford the device-wide
// synchronisation an allocation or a free may imply.  This variant keeps the
// scratch in a fixed array that is part of the library image instead:
//
//   * capacity: kMaxElements bf16 values (8 MiB) = sequence * query_heads * 128;
//     larger calls are refused with an error, nothing is launched;
//   * every GPU that loads the library carries the array until the process ends;
//   * the array is shared by every call and keeps the previous call's bytes.  The
//     part a call uses is rewritten before it is read, so nothing has to be
//     cleared; two calls that overlap on the same GPU (different streams or
//     contexts) race on it and must be serialised by the caller;
//   * the first call on a device resolves the array's device address (one
//     cudaGetSymbolAddress with that device current).  Make that first call
//     before starting any stream capture on the device.
//
// No cudaMalloc, cudaFree or other allocating routine is called on this path.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

extern "C" {
#include "../qw_internal.h"
}

namespace {

constexpr size_t kMaxElements = 4u * 1024u * 1024u;  // 8 MiB of bf16
constexpr int kMaxDevices = 64;

// Host code must never hand this name to a kernel: on the host it is only a
// stand-in.  The device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned short g_prescaled_query[kMaxElements];

std::mutex g_setup_lock;
unsigned short *g_device_address[kMaxDevices];  // per device, resolved on first use

// Resolve (once per device) the device address of the scratch array.  The
// caller's context has already made its device current.
cudaError_t scratch_address(int device, unsigned short **out) {
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(g_setup_lock);
    if (!g_device_address[device]) {
        void *address = nullptr;
        cudaError_t code = cudaGetSymbolAddress(&address, g_prescaled_query);
        if (code != cudaSuccess) return code;
        g_device_address[device] = static_cast<unsigned short *>(address);
    }
    *out = g_device_address[device];
    return cudaSuccess;
}

// q' = bf16(q * scale), the rounding of h3_shaders.metal:4396-4402.
__global__ void __launch_bounds__(256)
qw_prescale_query_kernel(unsigned short *__restrict__ scaled,
                         const unsigned short *__restrict__ query, size_t count, float scale) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float v = __uint_as_float((uint32_t)query[i] << 16);
        uint32_t bits = __float_as_uint(__fmul_rn(v, scale));
        bits += 0x7fffu + ((bits >> 16) & 1u);
        scaled[i] = (unsigned short)(bits >> 16);
    }
}

}  // namespace

extern "C" int h3_gpu_gqa_causal_noalloc_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                              const h3_gpu_tensor *query,
                                              const h3_gpu_tensor *key,
                                              const h3_gpu_tensor *value, uint32_t sequence,
                                              uint32_t query_heads, uint32_t kv_heads,
                                              uint32_t head_dim, float scale) {
    if (!gpu) return 0;
    if (!sequence || !query_heads || !kv_heads || query_heads % kv_heads || head_dim != 128) {
        qw_set_error(gpu, "GQA (no-alloc): unsupported geometry");
        return 0;
    }
    const size_t query_count = (size_t)sequence * query_heads * head_dim;
    const size_t kv_count = (size_t)sequence * kv_heads * head_dim;
    if (query_count > kMaxElements) {
        qw_set_error(gpu,
                     "GQA (no-alloc): sequence * query_heads * head_dim = %zu exceeds the fixed "
                     "scratch of %zu elements; use h3_gpu_gqa_causal_bf16",
                     query_count, (size_t)kMaxElements);
        return 0;
    }
    if (!(scale > 0.0f) || !isfinite(scale)) {
        qw_set_error(gpu, "GQA (no-alloc): scale must be positive and finite");
        return 0;
    }
    if (!qw_require_dtype(gpu, query, query_count, H3_GPU_BF16, "GQA (no-alloc) query") ||
        !qw_require_dtype(gpu, key, kv_count, H3_GPU_BF16, "GQA (no-alloc) key") ||
        !qw_require_dtype(gpu, value, kv_count, H3_GPU_BF16, "GQA (no-alloc) value") ||
        !qw_require_dtype(gpu, output, query_count, H3_GPU_BF16, "GQA (no-alloc) output") ||
        !qw_require_command(gpu) || !qw_bind(gpu))
        return 0;

    unsigned short *scaled = nullptr;
    cudaError_t code = scratch_address(gpu->device, &scaled);
    if (code != cudaSuccess) {
        qw_set_error(gpu, "GQA (no-alloc): cannot resolve the scratch array: %s",
                     cudaGetErrorString(code));
        return 0;
    }
    const unsigned int blocks =
        (unsigned int)((query_count + 255) / 256 < 148 * 16 ? (query_count + 255) / 256 : 148 * 16);
    qw_prescale_query_kernel<<<blocks, 256, 0, gpu->stream>>>(
        scaled, static_cast<const unsigned short *>(query->dev), query_count, scale);
    int rc = (int)cudaGetLastError();
    qw_count_launch(gpu, rc, "query pre-scale (no-alloc)");
    if (rc) return 0;

    qwcu_attn_args args;
    memset(&args, 0, sizeof(args));
    args.q = scaled;
    args.k = key->dev;
    args.v = value->dev;
    args.out = output->dev;
    args.causal = 1;
    args.batch = 1;
    args.q_rows = sequence;
    args.kv_rows = sequence;
    args.heads = query_heads;
    args.kv_heads = kv_heads;
    args.scale = 1.0f;  // already folded into the query
    args.status = gpu->status_dev;
    args.whole_units = gpu->attn_kernel == QW_ATTN_SM100_WHOLE;
    rc = gpu->attn_kernel == QW_ATTN_SCALAR ? qwcu_attn_scalar_launch(&args, gpu->stream)
                                            : qwcu_attn_sm100_launch(&args, gpu->stream);
    qw_count_launch(gpu, rc, "GQA (no-alloc)");
    return rc == 0;
}
