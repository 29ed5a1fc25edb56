/* qwen_gpu_ext.h -- the qw_* ops of the DiT attention path, same names,
 * argument order and conventions as the reference's qwen_gpu_ext.h, plus the
 * additive entry points this library introduces (marked NEW).  Citations are
 * path:line inside the reference project.  See h3_gpu.h for the shared
 * conventions (1 = success, 0 = failure + h3_gpu_error()).
 *
 * Layouts: activations are token-major [rows, heads, 128] bf16, contiguous;
 * RoPE tables are f32 [rows, 64]; norm weights bf16 [128]; kv_limit is a U32
 * tensor of per-row key counts.  head_dim must be 128 for the attention ops.
 */
#ifndef QWEN_GPU_EXT_H
#define QWEN_GPU_EXT_H

#include "h3_gpu.h"

#ifdef __cplusplus
extern "C" {
#endif

/* reference qwen_gpu_ext.h:28-36, h3_gpu.m:5159-5193, h3_shaders.metal:4864-4890:
 * interleaved complex RoPE on q and k with f32 cos/sin tables of
 * [row, head_dim/2].  In-place safe. */
int qw_gpu_qk_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query_output, h3_gpu_tensor *key_output,
                        const h3_gpu_tensor *query_input, const h3_gpu_tensor *key_input,
                        const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                        uint32_t sequence, uint32_t heads, uint32_t head_dim);

/* reference qwen_gpu_ext.h:10-16, h3_gpu.m:5100-5124, h3_shaders.metal:4767-4813:
 * the block's AdaLN norm in front of the QKV projection (and the MLP):
 * affine-free LayerNorm over `width`, then (1 + modulation[row_map[row]][scale_slot]). */
int qw_gpu_layer_norm_mod_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                               const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
                               uint32_t rows, uint32_t width, uint32_t slots,
                               uint32_t scale_slot, float epsilon);

/* reference qwen_gpu_ext.h:57-60, h3_gpu.m:5258-5275, h3_shaders.metal:4975-4997:
 * per-head RMSNorm with the normalised value rounded to bf16 before the
 * weight multiply (double rounding). */
int qw_gpu_head_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *tensor, const h3_gpu_tensor *weight,
                              uint32_t sequence, uint32_t heads, uint32_t head_dim,
                              float epsilon);

/* reference qwen_gpu_ext.h:202-210, h3_gpu.m:2918-3018: fused q/k/v projection in
 * front of the attention (qwen_dit.m:1270), three [dim, dim] weights in their
 * [out, in] layout sharing the input, one launch. */
int qw_gpu_qkv_bf16(h3_gpu *gpu, h3_gpu_tensor *query_out, h3_gpu_tensor *key_out,
                    h3_gpu_tensor *value_out, const h3_gpu_tensor *input,
                    const h3_gpu_tensor *query_weight, const h3_gpu_tensor *key_weight,
                    const h3_gpu_tensor *value_weight, uint32_t rows, uint32_t dim);

/* reference qwen_gpu_ext.h:116-123, h3_gpu.m:5745-5789: flash SDPA, every query
 * row sees every key; q_rows may differ from kv_rows. */
int qw_gpu_flash_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t q_rows, uint32_t kv_rows, uint32_t heads, uint32_t head_dim,
                           float scale);

/* reference qwen_gpu_ext.h:125-138, h3_gpu.m:5791-5844, h3_shaders.metal:3061-3272:
 * prefix-visible SDPA.  kv_limit[q_row] (U32 tensor, >= q_rows elements) caps
 * the key range of each query row; values are read as int32, negatives count
 * as 0 and everything is capped at kv_rows.  Grouped-query attention:
 * heads % kv_heads == 0, q head h reads kv head h * kv_heads / heads. */
int qw_gpu_flash_sdpa_prefix_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                                  const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                                  const h3_gpu_tensor *kv_limit, uint32_t q_rows,
                                  uint32_t kv_rows, uint32_t heads, uint32_t kv_heads,
                                  uint32_t head_dim, float scale);

/* reference qwen_gpu_ext.h:212-219, h3_gpu.m:5903-5953, h3_shaders.metal:5003-5069:
 * token-causal GQA, scale applied to the fp32 scores. */
int qw_gpu_gqa_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t sequence, uint32_t query_heads, uint32_t kv_heads,
                           uint32_t head_dim, float scale);

/* reference qwen_gpu_ext.h:221-228, h3_gpu.m:5972-6054: full SDPA whose query
 * length may differ from the key/value length. */
int qw_gpu_sdpa_rect_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                          const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                          uint32_t query_sequence, uint32_t kv_sequence, uint32_t heads,
                          uint32_t head_dim, float scale);

/* ---------------------------------------------------------------------- */
/* NEW entry points (no counterpart in the reference).                     */

/* Fused prologue: per-head RMSNorm of q and k (single rounding, the variant
 * the DiT block uses: qwen_dit.m:1273-1276) followed by the interleaved RoPE
 * (qwen_dit.m:1277) in one pass over q and k, in place.  Reproduces the bf16
 * store the reference has between the two stages.  `batch` items share the
 * tables: row r of every item uses table row r. */
int qw_gpu_qk_norm_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                             const h3_gpu_tensor *norm_weight_q,
                             const h3_gpu_tensor *norm_weight_k, const h3_gpu_tensor *rope_cos,
                             const h3_gpu_tensor *rope_sin, uint32_t batch, uint32_t sequence,
                             uint32_t heads, uint32_t head_dim, float epsilon);

/* Same, reading query_input/key_input and writing query_output/key_output (the
 * pairs may alias for in-place use, like qw_gpu_qk_rope_bf16). */
int qw_gpu_qk_norm_rope_out_bf16(h3_gpu *gpu, h3_gpu_tensor *query_output,
                                 h3_gpu_tensor *key_output, const h3_gpu_tensor *query_input,
                                 const h3_gpu_tensor *key_input,
                                 const h3_gpu_tensor *norm_weight_q,
                                 const h3_gpu_tensor *norm_weight_k,
                                 const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                 uint32_t batch, uint32_t sequence, uint32_t heads,
                                 uint32_t head_dim, float epsilon);

/* Same pass, which also writes two floats into score_bound (F32 tensor, >= 2
 * elements): upper bounds of the 2-norm of every output query row and of every
 * output key row (sqrt(128) * max|weight| plus rounding slack; the rotation
 * preserves the norm).  Hand them to qw_gpu_attn_block_causal_bounded_bf16.
 * epsilon must be >= 0. */
int qw_gpu_qk_norm_rope_bound_bf16(h3_gpu *gpu, h3_gpu_tensor *query_output,
                                   h3_gpu_tensor *key_output, const h3_gpu_tensor *query_input,
                                   const h3_gpu_tensor *key_input,
                                   const h3_gpu_tensor *norm_weight_q,
                                   const h3_gpu_tensor *norm_weight_k,
                                   const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                   h3_gpu_tensor *score_bound, uint32_t batch,
                                   uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                   float epsilon);

/* NEW: the q/k/v projection with the per-head QK RMSNorm and the interleaved RoPE
 * in the GEMM's epilogue: the reference's sequence qw_gpu_qkv_bf16, two
 * h3_gpu_head_rms_norm_bf16, qw_gpu_qk_rope_bf16 (qwen_dit.m:1270-1278) as one
 * launch, with the same bf16 roundings between the stages.  input [batch*sequence,
 * dim]; tables f32 [sequence, 64]; dim a multiple of 128 (whole heads).
 * score_bound (F32 tensor >= 2 elements, or NULL) as in
 * qw_gpu_qk_norm_rope_bound_bf16. */
int qw_gpu_qkv_norm_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query_out, h3_gpu_tensor *key_out,
                              h3_gpu_tensor *value_out, const h3_gpu_tensor *input,
                              const h3_gpu_tensor *query_weight, const h3_gpu_tensor *key_weight,
                              const h3_gpu_tensor *value_weight,
                              const h3_gpu_tensor *norm_weight_q,
                              const h3_gpu_tensor *norm_weight_k, const h3_gpu_tensor *rope_cos,
                              const h3_gpu_tensor *rope_sin, h3_gpu_tensor *score_bound,
                              uint32_t batch, uint32_t sequence, uint32_t dim, float epsilon);

/* NEW: the prologue of a target-only layer of the edit path, where only the
 * target image rows are recomputed against the per-layer K/V cache of an
 * earlier full pass (reference qwen_dit.m:1872-1904 runs two head norms, the
 * rotation and two h3_gpu_copy_bf16 scatters for this).  query [rows, heads,
 * 128] is normed and rotated in place; key_new is normed, rotated and written to
 * rows [cache_row_offset, cache_row_offset + rows) of key_cache [cache_rows,
 * heads, 128]; value_new is copied to the same rows of value_cache.  The tables
 * are the target rows' slices, [rows, 64] f32.  Follow it with
 * qw_gpu_sdpa_rect_bf16(out, query, key_cache, value_cache, rows, cache_rows, ...). */
int qw_gpu_qk_norm_rope_cache_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key_cache,
                                   h3_gpu_tensor *value_cache, const h3_gpu_tensor *key_new,
                                   const h3_gpu_tensor *value_new,
                                   const h3_gpu_tensor *norm_weight_q,
                                   const h3_gpu_tensor *norm_weight_k,
                                   const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                   uint32_t cache_rows, uint32_t cache_row_offset, uint32_t rows,
                                   uint32_t heads, uint32_t head_dim, float epsilon);

/* Batched block-causal attention with optional key padding (classifier-free
 * guidance runs cond/uncond as batch items whose text lengths differ).
 *   q, out [batch, rows, heads, 128]; k, v [batch, rows, kv_heads, 128]
 *   kv_limit  U32 tensor with `rows` entries (shared by the batch) or
 *             batch*rows entries (per item), or NULL for "every key".
 *   text_len  host array of `batch` entries or NULL; with text_pad != 0 the
 *             keys text_len[b] <= s < text_pad are invisible for item b and the
 *             query rows in that window store zeros.
 * Rows without any visible key store zeros.  batch <= 8. */
int qw_gpu_attn_block_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                  const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                  const h3_gpu_tensor *value, const h3_gpu_tensor *kv_limit,
                                  uint32_t batch, uint32_t rows, uint32_t heads,
                                  uint32_t kv_heads, uint32_t head_dim,
                                  const uint32_t *text_len, uint32_t text_pad, float scale);

/* The same op for inputs whose row norms are bounded, which is what the DiT
 * block's QK-norm guarantees.  score_bound (F32 tensor, two elements on the
 * device, e.g. from qw_gpu_qk_norm_rope_bound_bf16) is the caller's promise that
 * every query row has a 2-norm <= score_bound[0] and every key row <=
 * score_bound[1].  Then |q.k| * scale cannot exceed their product, and the kernel
 * computes P = exp2(score - bound) against that one fixed exponent: no running
 * row maximum, no rescaling of the accumulator.  The result is the same softmax
 * (a common factor cancels in O / l).  A product above 60 (log2 units), or a
 * non-finite one, is ignored and the running-maximum path runs instead; a bound
 * that the data violates by more than 2^60 can overflow the row sums. */
int qw_gpu_attn_block_causal_bounded_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                          const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                          const h3_gpu_tensor *value,
                                          const h3_gpu_tensor *kv_limit,
                                          const h3_gpu_tensor *score_bound, uint32_t batch,
                                          uint32_t rows, uint32_t heads, uint32_t kv_heads,
                                          uint32_t head_dim, const uint32_t *text_len,
                                          uint32_t text_pad, float scale);

/* Context bound to an explicit CUDA device. */
h3_gpu *qw_gpu_create_on_device(int device, char *error, size_t error_size);
int qw_gpu_device(const h3_gpu *gpu);
/* Interop handles: the tensor's device address and the context's cudaStream_t. */
void *qw_gpu_tensor_device_ptr(const h3_gpu_tensor *tensor);
void *qw_gpu_stream(const h3_gpu *gpu);
/* Pinned host memory for asynchronous tensor writes/reads. */
void *qw_gpu_host_alloc(size_t bytes);
void qw_gpu_host_free(void *pointer);
/* Asynchronous device-to-host read into pinned memory, ordered on the
 * context's stream; complete after the next h3_gpu_submit(). */
int qw_gpu_tensor_read_async(h3_gpu *gpu, const h3_gpu_tensor *tensor, void *host,
                             size_t elements);
/* Copy lanes: two more streams beside the context's own (lane 0, where every op
 * runs) that carry only copies, so that a host program can overlap the upload of
 * the next layer's inputs (lane 1), the compute of this layer (lane 0) and the
 * read-back of the last layer's output (lane 2).  qw_gpu_fence(from, to) orders
 * everything enqueued on lane `from` so far before whatever is enqueued on lane
 * `to` next.  Host buffers must be pinned (qw_gpu_host_alloc) and stay valid until
 * the next h3_gpu_submit, which waits for every lane.  Not inside a graph capture. */
int qw_gpu_fence(h3_gpu *gpu, int from_lane, int to_lane);
int qw_gpu_tensor_write_lane(h3_gpu *gpu, h3_gpu_tensor *tensor, const void *host,
                             size_t elements, int lane);
int qw_gpu_tensor_read_lane(h3_gpu *gpu, const h3_gpu_tensor *tensor, void *host,
                            size_t elements, int lane);
/* Select the attention kernel: "sm100" (default; the 256-row blocks of the last,
 * partly filled wave of CTAs run split in two), "sm100-whole" (same kernel, no
 * block is ever split), "sm100-row" (same kernel; with a score bound the softmax
 * keeps one thread per query row instead of pairing the warpgroups on each
 * sub-tile) or "scalar" (diagnostic fp32 kernel).  Returns 0 on an unknown name. */
int qw_gpu_set_attention_kernel(h3_gpu *gpu, const char *name);
/* Test hook for the attention kernel's bounded waits: later launches use a wait
 * budget of wait_cycles SM cycles and their TMA producer leaves out every key tile
 * from visited tile withhold_from_tile (>= 1) on; the waits behind the missing
 * tile run out, every role of the CTA leaves through its clean exit (loads
 * drained, TMEM freed) and h3_gpu_submit returns 0 with the place of the first
 * expiry.  (0, 0) restores normal operation. */
int qw_gpu_debug_attention_waits(h3_gpu *gpu, long long wait_cycles, int withhold_from_tile);
/* Launches enqueued by this context's ops since creation (own kernels only). */
uint64_t qw_gpu_kernel_launches(const h3_gpu *gpu);

/* Replayable graphs: ops enqueued between begin and end (inside an open chain)
 * are captured instead of run; qw_gpu_graph_launch replays them with one launch.
 * The first call of every op kind must have happened before a capture (one-time
 * kernel attribute set-up is not capturable). */
typedef struct qw_gpu_graph qw_gpu_graph;
int qw_gpu_graph_begin(h3_gpu *gpu);
qw_gpu_graph *qw_gpu_graph_end(h3_gpu *gpu);
int qw_gpu_graph_launch(h3_gpu *gpu, qw_gpu_graph *graph);
void qw_gpu_graph_free(qw_gpu_graph *graph);

/* ---- multi-GPU: one process per GPU -------------------------------------
 * The ranks form batch_groups x head_groups.  A batch group owns some of the
 * batch items (the reference runs the two classifier-free-guidance branches as two
 * separate forwards, qwen_pipeline.m:376-381 and :396-401, so a branch's output
 * is only ever needed by that branch); inside a batch group the attention heads
 * are sharded, nothing is exchanged before attention, and only the per-layer
 * [rows, heads*128] output is gathered over NVLink. */
typedef struct qw_gpu_group qw_gpu_group;
#define QW_GPU_GROUP_ID_BYTES 128
/* Rank 0 creates the rendezvous id and hands the bytes to every rank by any
 * host channel; each rank then joins with its own context (collective, at most
 * 8 ranks). */
int qw_gpu_group_new_id(void *id_bytes, char *error, size_t error_size);
qw_gpu_group *qw_gpu_group_join(h3_gpu *gpu, const void *id_bytes, int rank, int world,
                                char *error, size_t error_size);
void qw_gpu_group_free(qw_gpu_group *group);
int qw_gpu_group_rank(const qw_gpu_group *group);
int qw_gpu_group_world(const qw_gpu_group *group);
/* Split the ranks: rank = batch_index * head_groups + head_index with head_groups
 * = world / batch_groups.  Same value on every rank, before the first sharded
 * attention; the default is 1 (every rank shards the heads of every batch item). */
int qw_gpu_group_set_batch_groups(qw_gpu_group *group, int batch_groups);
int qw_gpu_group_batch_index(const qw_gpu_group *group);
int qw_gpu_group_head_index(const qw_gpu_group *group);
int qw_gpu_group_head_groups(const qw_gpu_group *group);
/* NCCL comparison path (one batch group only): gather the per-rank attention
 * outputs [rows, heads_local*128] into the full [rows, world*heads_local*128]
 * tensor on every rank (rank g owns head columns [g*heads_local, (g+1)*heads_local)).
 * Enqueued on the context's stream. */
int qw_gpu_group_all_gather_heads_bf16(qw_gpu_group *group, h3_gpu_tensor *full,
                                       const h3_gpu_tensor *local, uint32_t rows,
                                       uint32_t heads_local, uint32_t head_dim);

/* Sharded attention with this library's own gather.
 * qw_gpu_group_bind_output (collective, outside a graph capture) maps every rank's
 * `full` buffer into every process over the NVLink peer path.  After that
 * qw_gpu_group_attn_block_causal_bf16 runs this rank's heads_local heads of its
 * batch group's `batch` items into head columns [head_index*heads_local,
 * +heads_local) of its own `full` [batch*rows, head_groups*heads_local*128], and a
 * push kernel on the group's own stream copies that column slice into the same
 * place of every peer's `full`, under whatever the context's stream runs next.
 * Ranks hand-shake through epoch flags in peer-mapped memory (a rank stores into a
 * peer's buffer only after the peer's next attention on that buffer has begun,
 * i.e. after everything the peer enqueued to read the old contents; every wait is
 * bounded and reports through h3_gpu_submit).  No landing zone, no interleave pass,
 * no NCCL call per layer.
 * Up to 4 outputs can be bound; alternate between two so that layer L's gather
 * overlaps layer L+1.  score_bound as in qw_gpu_attn_block_causal_bounded_bf16, or
 * NULL.  The other arguments as qw_gpu_attn_block_causal_bf16 with this rank's
 * head counts and its batch group's items. */
int qw_gpu_group_bind_output(qw_gpu_group *group, h3_gpu_tensor *full);
int qw_gpu_group_barrier(qw_gpu_group *group);
/* Before enqueueing a consumer of `full`, make the context's stream wait until
 * every peer's columns have landed in it; h3_gpu_submit waits anyway. */
int qw_gpu_group_wait_output(qw_gpu_group *group, const h3_gpu_tensor *full);
int qw_gpu_group_attn_block_causal_bf16(qw_gpu_group *group, h3_gpu_tensor *full,
                                        const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                        const h3_gpu_tensor *value,
                                        const h3_gpu_tensor *kv_limit,
                                        const h3_gpu_tensor *score_bound, uint32_t batch,
                                        uint32_t rows, uint32_t heads_local,
                                        uint32_t kv_heads_local, uint32_t head_dim,
                                        const uint32_t *text_len, uint32_t text_pad, float scale);

#ifdef __cplusplus
}
#endif
#endif
