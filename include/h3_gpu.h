/* h3_gpu.h -- C ABI of the B200 attention library: context, tensors, command
 * chain and the h3_* attention ops.
 *
 * The declarations keep the names, argument order and return conventions of
 * the reference's h3_gpu.h so that a caller of the reference (qwen_dit.m,
 * the tests under tests/) links against this library unchanged for the ops on
 * the attention path.  Each declaration cites the reference interface it
 * replaces (path:line inside the reference project).
 *
 * Conventions (reference h3_gpu.m:267-289, 975-1053):
 *   - every op returns 1 on success and 0 on failure; the reason is available
 *     from h3_gpu_error(); creators return NULL on failure;
 *   - ops only enqueue work; an op called without an open chain fails with
 *     "h3_gpu_begin() was not called"; errors raised on the device surface at
 *     h3_gpu_submit();
 *   - a tensor may be larger than an op needs ("absent or too small" is the
 *     only size failure), the caller owns every handle, a context is used from
 *     one thread.
 */
#ifndef H3_GPU_H
#define H3_GPU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference h3_gpu.h:7-8 */
typedef struct h3_gpu h3_gpu;
typedef struct h3_gpu_tensor h3_gpu_tensor;

/* reference h3_gpu.h:14-19 */
typedef enum {
    H3_GPU_F32 = 0,
    H3_GPU_BF16,
    H3_GPU_I8,
    H3_GPU_U32
} h3_gpu_dtype;

/* reference h3_gpu.h:21-37.  Filled here: allocated/live/peak bytes, tensor
 * allocations, direct_dispatches (kernel launches), blit_copies,
 * submissions, command_wait_seconds, gpu_seconds (CUDA events around each
 * chain).  The mps_* counters stay 0. */
typedef struct {
    uint64_t allocated_bytes;
    uint64_t live_bytes;
    uint64_t peak_live_bytes;
    uint64_t tensor_allocations;
    uint64_t direct_dispatches;
    uint64_t mps_linear_dispatches;
    uint64_t mps_conv_dispatches;
    uint64_t mps_sdpa_dispatches;
    uint64_t blit_copies;
    uint64_t submissions;
    double command_encode_seconds;
    double command_wait_seconds;
    double gpu_seconds;
} h3_gpu_stats;

/* reference h3_gpu.h:39-44, h3_gpu.m:380-579.  The shader path is ignored.
 * The context binds the CUDA device named by QW_CUDA_DEVICE (default: the
 * calling thread's current device) and owns one stream.  Fails (NULL + message)
 * when no sm_100 device is present: there is no CPU fallback. */
h3_gpu *h3_gpu_create(const char *shader_source_path, char *error, size_t error_size);
void h3_gpu_free(h3_gpu *gpu);
int h3_gpu_is_m5(const h3_gpu *gpu);        /* always 0 */
int h3_gpu_has_nax_mlp(const h3_gpu *gpu);  /* always 0 */
int h3_gpu_has_int8_mlp(const h3_gpu *gpu); /* always 0 */
/* reference h3_gpu.h:10-12: nothing is cached per shape here; no-op. */
void h3_gpu_clear_graph_cache(h3_gpu *gpu);

/* reference h3_gpu.h:46-55, h3_gpu.m:621-647 */
h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_i8(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *gpu, const float *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *gpu, const uint16_t *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *values, size_t elements);
/* reference h3_gpu.h:73-75, h3_gpu.m:887-918; NULL-safe */
void h3_gpu_tensor_free(h3_gpu_tensor *tensor);
size_t h3_gpu_tensor_elements(const h3_gpu_tensor *tensor);
h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *tensor);

/* reference h3_gpu.h:76-91, h3_gpu.m:920-973.  The reference's tensors are
 * host-visible and these are raw memcpys; here a write is a host-to-device copy
 * ordered on the context's stream (the host buffer may be reused as soon as
 * the call returns unless it is pinned memory from qw_gpu_host_alloc, which is
 * consumed asynchronously), and a read drains the stream first.  Range and
 * dtype violations return 0. */
int h3_gpu_tensor_read_f32(const h3_gpu_tensor *tensor, float *values, size_t elements);
int h3_gpu_tensor_read_f32_range(const h3_gpu_tensor *tensor, size_t source_offset,
                                 float *values, size_t elements);
int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *tensor, uint16_t *values, size_t elements);
int h3_gpu_tensor_write_f32(h3_gpu_tensor *tensor, const float *values, size_t elements);
int h3_gpu_tensor_write_f32_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                  const float *values, size_t elements);
int h3_gpu_tensor_write_bf16(h3_gpu_tensor *tensor, const uint16_t *values, size_t elements);
int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                   const uint16_t *values, size_t elements);

/* reference h3_gpu.h:93-97, h3_gpu.m:975-1047.  begin fails when a chain is
 * already open; continue flushes without waiting; submit waits for the whole
 * chain and reports any launch error or device-side status. */
int h3_gpu_begin(h3_gpu *gpu);
int h3_gpu_continue(h3_gpu *gpu);
int h3_gpu_submit(h3_gpu *gpu);
/* reference h3_gpu.h:98, h3_gpu.m:1049-1053; never NULL */
const char *h3_gpu_error(const h3_gpu *gpu);
/* reference h3_gpu.h:99, h3_gpu.m:1055-1059 */
int h3_gpu_get_stats(const h3_gpu *gpu, h3_gpu_stats *stats);
/* reference h3_gpu.h:102-103; no-ops */
void h3_gpu_profile_set_label(h3_gpu *gpu, const char *label);
void h3_gpu_profile_mark(h3_gpu *gpu, const char *phase);

/* reference h3_gpu.h:135-142, h3_gpu.m:1384-1444: element-range copy between
 * tensors of the same dtype ("invalid BF16 blit range" / "invalid F32 blit
 * range" on any violation). */
int h3_gpu_copy_bf16(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                     const h3_gpu_tensor *source, size_t source_offset, size_t elements);
int h3_gpu_copy_f32(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                    const h3_gpu_tensor *source, size_t source_offset, size_t elements);

/* reference h3_gpu.h:497-507, h3_gpu.m:1698-1720: full bidirectional
 * self-attention over [sequence, heads, head_dim]; the second form stores
 * [heads, sequence, head_dim]. */
int h3_gpu_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                     const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                     uint32_t heads, uint32_t head_dim, float scale);
int h3_gpu_sdpa_bf16_head_major_output(h3_gpu *gpu, h3_gpu_tensor *output,
                                       const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                       const h3_gpu_tensor *value, uint32_t sequence,
                                       uint32_t heads, uint32_t head_dim, float scale);

/* reference h3_gpu.h:293-299, h3_gpu.m:2697-2812, h3_shaders.metal:788-822: bf16
 * linear layer, output[rows, output_dim] = bf16(bias + input . weight^T) with the
 * weight in its [output_dim, input_dim] checkpoint layout, fp32 accumulation;
 * bias may be NULL.  The DiT block's output projection behind the attention
 * (qwen_dit.m:1446).  Dimensions must be multiples of 8. */
int h3_gpu_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                       const h3_gpu_tensor *weight, const h3_gpu_tensor *bias, uint32_t rows,
                       uint32_t input_dim, uint32_t output_dim);

/* reference h3_gpu.h:527-530, h3_gpu.m:4478-4493, h3_shaders.metal:4309-4329:
 * in-place per-(row, head) RMSNorm, single bf16 rounding of x*inv*w. */
int h3_gpu_head_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *tensor, const h3_gpu_tensor *weight,
                              uint32_t sequence, uint32_t heads, uint32_t head_dim,
                              float epsilon);

/* reference h3_gpu.h:406-411, h3_gpu.m:3865-3889, h3_shaders.metal:3583-3599:
 * gated residual behind the attention / MLP branch of a DiT block,
 * output = bf16(residual + branch * modulation[row_map[row]][gate_slot][column]);
 * modulation is [maps][slots][width] bf16, row_map u32 per row. */
int h3_gpu_gate_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                     const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                     const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                     uint32_t slots, uint32_t gate_slot);

/* reference h3_gpu.h:537-543, h3_gpu.m:4642-4693, h3_shaders.metal:4375-4445:
 * token-causal attention; this variant folds the scale into Q and re-rounds Q
 * to bf16 before the dot products. */
int h3_gpu_gqa_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t sequence, uint32_t query_heads, uint32_t kv_heads,
                           uint32_t head_dim, float scale);

/* No counterpart in the reference.  Same arguments, arithmetic and result as
 * h3_gpu_gqa_causal_bf16, for callers that cannot allocate device memory at the
 * time of the call: a host that gave the whole GPU to its own arena at start-up
 * (a later allocation fails there) or a steady-state loop that must not hit the
 * device-wide synchronisation an allocation or free can imply.  The pre-scaled
 * query lives in a fixed 8 MiB array inside the library image instead of a
 * block from the CUDA allocator, so sequence * query_heads * head_dim may not
 * exceed 4,194,304 (larger calls fail with an error; use the regular op).  The
 * array is shared by all calls on a GPU: calls that overlap on one GPU race and
 * must be serialised by the caller.  The first call on a device resolves the
 * array's address; make it before starting any stream capture.  That first call
 * is also the one moment this entry point can need memory: with lazy module
 * loading it is when the driver loads this kernel's module and sets the 8 MiB
 * array aside, so make it (or run with CUDA_MODULE_LOADING=EAGER) before the
 * host's arena claims the GPU; every later call allocates nothing.  Requires
 * head_dim == 128 and a positive finite scale. */
int h3_gpu_gqa_causal_noalloc_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                   const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                   const h3_gpu_tensor *value, uint32_t sequence,
                                   uint32_t query_heads, uint32_t kv_heads, uint32_t head_dim,
                                   float scale);

#ifdef __cplusplus
}
#endif
#endif
