/* The attention-path ops of the C ABI: argument validation in the reference's
 * order and wording, then one asynchronous launch through the extern-"C" CUDA
 * layer.  No op allocates caller-visible memory and none falls back to the CPU.
 */
#include "qw_internal.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

/* ---- prologue ops -------------------------------------------------------- */

static int launch_prologue(h3_gpu *gpu, const qwcu_prologue_args *args, const char *what) {
    if (!qw_bind(gpu)) return 0;
    int rc = qwcu_prologue_launch(args, gpu->stream);
    qw_count_launch(gpu, rc, what);
    return rc == 0;
}

static int head_norm(h3_gpu *gpu, h3_gpu_tensor *tensor, const h3_gpu_tensor *weight,
                     uint32_t sequence, uint32_t heads, uint32_t head_dim, float epsilon,
                     int double_round) {
    size_t count = (size_t)sequence * heads * head_dim;
    if (!qw_require_dtype(gpu, tensor, count, H3_GPU_BF16, "head norm tensor") ||
        !qw_require_dtype(gpu, weight, head_dim, H3_GPU_BF16, "head norm weight"))
        return 0;
    if (!qw_require_command(gpu)) return 0;
    if (head_dim != 128) {
        qw_set_error(gpu, "head norm: unsupported geometry (head_dim must be 128)");
        return 0;
    }
    if (!count) return 1;
    qwcu_prologue_args args;
    memset(&args, 0, sizeof(args));
    args.q_in = tensor->dev;
    args.q_out = tensor->dev;
    args.norm_weight_q = weight->dev;
    args.rows = sequence;
    args.table_rows = sequence;
    args.heads = heads;
    args.epsilon = epsilon;
    args.double_round = double_round;
    return launch_prologue(gpu, &args, "head RMSNorm");
}

/* reference h3_gpu.m:4478-4493 */
int h3_gpu_head_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *tensor, const h3_gpu_tensor *weight,
                              uint32_t sequence, uint32_t heads, uint32_t head_dim,
                              float epsilon) {
    return head_norm(gpu, tensor, weight, sequence, heads, head_dim, epsilon, 0);
}

/* reference h3_gpu.m:5258-5275 */
int qw_gpu_head_rms_norm_bf16(h3_gpu *gpu, h3_gpu_tensor *tensor, const h3_gpu_tensor *weight,
                              uint32_t sequence, uint32_t heads, uint32_t head_dim,
                              float epsilon) {
    return head_norm(gpu, tensor, weight, sequence, heads, head_dim, epsilon, 1);
}

/* reference h3_gpu.m:5100-5124 */
int qw_gpu_layer_norm_mod_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                               const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
                               uint32_t rows, uint32_t width, uint32_t slots,
                               uint32_t scale_slot, float epsilon) {
    if (!gpu) return 0;
    size_t count = (size_t)rows * width;
    if (!qw_require_dtype(gpu, input, count, H3_GPU_BF16, "Qwen AdaLN input") ||
        !qw_require_dtype(gpu, modulation, 1, H3_GPU_BF16, "Qwen AdaLN modulation") ||
        !qw_require_dtype(gpu, row_map, rows, H3_GPU_U32, "Qwen AdaLN row map") ||
        !qw_require_dtype(gpu, output, count, H3_GPU_BF16, "Qwen AdaLN output"))
        return 0;
    if (scale_slot >= slots) {
        qw_set_error(gpu, "Qwen AdaLN: scale slot %u outside %u slots", scale_slot, slots);
        return 0;
    }
    if (!rows || !width) {
        qw_set_error(gpu, "Qwen AdaLN: empty geometry");
        return 0;
    }
    size_t maps = modulation->elements / ((size_t)slots * width);
    if (!maps) {
        qw_set_error(gpu, "Qwen AdaLN: the modulation tensor holds less than one [%u, %u] block",
                     slots, width);
        return 0;
    }
    if (!qw_require_command(gpu) || !qw_bind(gpu)) return 0;
    qwcu_rowwise_args args = {input->dev, NULL, modulation->dev, row_map->dev, output->dev,
                              rows, width, slots, scale_slot, epsilon,
                              maps > UINT32_MAX ? UINT32_MAX : (uint32_t)maps, gpu->status_dev};
    int rc = qwcu_layer_norm_mod_launch(&args, qwcu_device_sm_count(gpu->device), gpu->stream);
    qw_count_launch(gpu, rc, "Qwen AdaLN");
    return rc == 0;
}

/* reference h3_gpu.m:3865-3889 */
int h3_gpu_gate_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                     const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                     const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                     uint32_t slots, uint32_t gate_slot) {
    if (!gpu) return 0;
    size_t count = (size_t)rows * width;
    if (!qw_require_dtype(gpu, residual, count, H3_GPU_BF16, "gate residual") ||
        !qw_require_dtype(gpu, branch, count, H3_GPU_BF16, "gate branch") ||
        !qw_require_dtype(gpu, modulation, 1, H3_GPU_BF16, "gate modulation") ||
        !qw_require_dtype(gpu, row_map, rows, H3_GPU_U32, "gate row map") ||
        !qw_require_dtype(gpu, output, count, H3_GPU_BF16, "gate output"))
        return 0;
    if (gate_slot >= slots) {
        qw_set_error(gpu, "gate: slot %u outside %u slots", gate_slot, slots);
        return 0;
    }
    if (!rows || !width) {
        qw_set_error(gpu, "gate: empty geometry");
        return 0;
    }
    size_t maps = modulation->elements / ((size_t)slots * width);
    if (!maps) {
        qw_set_error(gpu, "gate: the modulation tensor holds less than one [%u, %u] block", slots,
                     width);
        return 0;
    }
    if (!qw_require_command(gpu) || !qw_bind(gpu)) return 0;
    qwcu_rowwise_args args = {residual->dev, branch->dev, modulation->dev, row_map->dev,
                              output->dev, rows, width, slots, gate_slot, 0.0f,
                              maps > UINT32_MAX ? UINT32_MAX : (uint32_t)maps, gpu->status_dev};
    int rc = qwcu_gate_launch(&args, qwcu_device_sm_count(gpu->device), gpu->stream);
    qw_count_launch(gpu, rc, "gate");
    return rc == 0;
}

/* reference h3_gpu.m:5159-5193 */
int qw_gpu_qk_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query_output, h3_gpu_tensor *key_output,
                        const h3_gpu_tensor *query_input, const h3_gpu_tensor *key_input,
                        const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                        uint32_t sequence, uint32_t heads, uint32_t head_dim) {
    size_t count = (size_t)sequence * heads * head_dim;
    size_t rope_count = (size_t)sequence * (head_dim / 2);
    if (!qw_require_dtype(gpu, query_input, count, H3_GPU_BF16, "Qwen QK rope query") ||
        !qw_require_dtype(gpu, key_input, count, H3_GPU_BF16, "Qwen QK rope key") ||
        !qw_require_dtype(gpu, rope_cos, rope_count, H3_GPU_F32, "Qwen QK rope cosine") ||
        !qw_require_dtype(gpu, rope_sin, rope_count, H3_GPU_F32, "Qwen QK rope sine") ||
        !qw_require_dtype(gpu, query_output, count, H3_GPU_BF16, "Qwen QK rope query output") ||
        !qw_require_dtype(gpu, key_output, count, H3_GPU_BF16, "Qwen QK rope key output") ||
        head_dim % 2 != 0)
        return 0;
    if (!qw_require_command(gpu)) return 0;
    if (head_dim != 128) {
        qw_set_error(gpu, "Qwen QK rope: unsupported geometry (head_dim must be 128)");
        return 0;
    }
    if (!count) return 1;
    qwcu_prologue_args args;
    memset(&args, 0, sizeof(args));
    args.q_in = query_input->dev;
    args.k_in = key_input->dev;
    args.q_out = query_output->dev;
    args.k_out = key_output->dev;
    args.rope_cos = rope_cos->dev;
    args.rope_sin = rope_sin->dev;
    args.rows = sequence;
    args.table_rows = sequence;
    args.heads = heads;
    return launch_prologue(gpu, &args, "QK rope");
}

/* NEW: fused norm(q), norm(k), rope(q, k) (reference sequence qwen_dit.m:1273-1278) */
static int qk_norm_rope(h3_gpu *gpu, h3_gpu_tensor *query_output, h3_gpu_tensor *key_output,
                        const h3_gpu_tensor *query_input, const h3_gpu_tensor *key_input,
                        const h3_gpu_tensor *norm_weight_q, const h3_gpu_tensor *norm_weight_k,
                        const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                        h3_gpu_tensor *score_bound, int want_bound, uint32_t batch,
                        uint32_t sequence, uint32_t heads, uint32_t head_dim, float epsilon) {
    if (!gpu) return 0;
    if (want_bound) {
        if (!qw_require_dtype(gpu, score_bound, 2, H3_GPU_F32, "QK norm+rope score bound")) return 0;
        if (!(epsilon >= 0.0f)) {
            qw_set_error(gpu, "QK norm+rope: the score bound needs epsilon >= 0");
            return 0;
        }
    }
    size_t count = (size_t)batch * sequence * heads * head_dim;
    size_t rope_count = (size_t)sequence * (head_dim / 2);
    if (!qw_require_dtype(gpu, query_input, count, H3_GPU_BF16, "QK norm+rope query") ||
        !qw_require_dtype(gpu, key_input, count, H3_GPU_BF16, "QK norm+rope key") ||
        !qw_require_dtype(gpu, query_output, count, H3_GPU_BF16, "QK norm+rope query output") ||
        !qw_require_dtype(gpu, key_output, count, H3_GPU_BF16, "QK norm+rope key output") ||
        !qw_require_dtype(gpu, norm_weight_q, head_dim, H3_GPU_BF16, "QK norm+rope query weight") ||
        !qw_require_dtype(gpu, norm_weight_k, head_dim, H3_GPU_BF16, "QK norm+rope key weight") ||
        !qw_require_dtype(gpu, rope_cos, rope_count, H3_GPU_F32, "QK norm+rope cosine") ||
        !qw_require_dtype(gpu, rope_sin, rope_count, H3_GPU_F32, "QK norm+rope sine"))
        return 0;
    if (!qw_require_command(gpu)) return 0;
    if (head_dim != 128 || !batch || !sequence || !heads) {
        qw_set_error(gpu, "QK norm+rope: unsupported geometry");
        return 0;
    }
    if ((uint64_t)batch * sequence > UINT32_MAX) {
        qw_set_error(gpu, "QK norm+rope: too many rows");
        return 0;
    }
    qwcu_prologue_args args;
    memset(&args, 0, sizeof(args));
    args.q_in = query_input->dev;
    args.k_in = key_input->dev;
    args.q_out = query_output->dev;
    args.k_out = key_output->dev;
    args.norm_weight_q = norm_weight_q->dev;
    args.norm_weight_k = norm_weight_k->dev;
    args.rope_cos = rope_cos->dev;
    args.rope_sin = rope_sin->dev;
    args.rows = batch * sequence;
    args.table_rows = sequence;
    args.heads = heads;
    args.epsilon = epsilon;
    args.bound_out = want_bound ? (float *)score_bound->dev : NULL;
    return launch_prologue(gpu, &args, "QK norm+rope");
}

int qw_gpu_qk_norm_rope_out_bf16(h3_gpu *gpu, h3_gpu_tensor *query_output,
                                 h3_gpu_tensor *key_output, const h3_gpu_tensor *query_input,
                                 const h3_gpu_tensor *key_input,
                                 const h3_gpu_tensor *norm_weight_q,
                                 const h3_gpu_tensor *norm_weight_k,
                                 const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                 uint32_t batch, uint32_t sequence, uint32_t heads,
                                 uint32_t head_dim, float epsilon) {
    return qk_norm_rope(gpu, query_output, key_output, query_input, key_input, norm_weight_q,
                        norm_weight_k, rope_cos, rope_sin, NULL, 0, batch, sequence, heads,
                        head_dim, epsilon);
}

/* NEW: the same pass, which also leaves in score_bound[0..1] (F32 tensor) upper
 * bounds of the 2-norm of every output query row and key row. */
int qw_gpu_qk_norm_rope_bound_bf16(h3_gpu *gpu, h3_gpu_tensor *query_output,
                                   h3_gpu_tensor *key_output, const h3_gpu_tensor *query_input,
                                   const h3_gpu_tensor *key_input,
                                   const h3_gpu_tensor *norm_weight_q,
                                   const h3_gpu_tensor *norm_weight_k,
                                   const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                   h3_gpu_tensor *score_bound, uint32_t batch,
                                   uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                   float epsilon) {
    return qk_norm_rope(gpu, query_output, key_output, query_input, key_input, norm_weight_q,
                        norm_weight_k, rope_cos, rope_sin, score_bound, 1, batch, sequence, heads,
                        head_dim, epsilon);
}

int qw_gpu_qk_norm_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                             const h3_gpu_tensor *norm_weight_q,
                             const h3_gpu_tensor *norm_weight_k, const h3_gpu_tensor *rope_cos,
                             const h3_gpu_tensor *rope_sin, uint32_t batch, uint32_t sequence,
                             uint32_t heads, uint32_t head_dim, float epsilon) {
    return qw_gpu_qk_norm_rope_out_bf16(gpu, query, key, query, key, norm_weight_q,
                                        norm_weight_k, rope_cos, rope_sin, batch, sequence,
                                        heads, head_dim, epsilon);
}

/* The target-only layer of the edit path (reference qwen_dit.m:1872-1904): the new
 * target rows' q is normed and rotated in place, their k is normed, rotated and
 * written straight into rows [cache_row_offset, +rows) of the layer's key cache,
 * and their v is copied into the same rows of the value cache -- one launch for
 * the reference's two norms, the rotation and the two scatter copies. */
int qw_gpu_qk_norm_rope_cache_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key_cache,
                                   h3_gpu_tensor *value_cache, const h3_gpu_tensor *key_new,
                                   const h3_gpu_tensor *value_new,
                                   const h3_gpu_tensor *norm_weight_q,
                                   const h3_gpu_tensor *norm_weight_k,
                                   const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                   uint32_t cache_rows, uint32_t cache_row_offset, uint32_t rows,
                                   uint32_t heads, uint32_t head_dim, float epsilon) {
    if (!gpu) return 0;
    size_t count = (size_t)rows * heads * head_dim;
    size_t cache_count = (size_t)cache_rows * heads * head_dim;
    size_t rope_count = (size_t)rows * (head_dim / 2);
    if (!qw_require_dtype(gpu, query, count, H3_GPU_BF16, "QK norm+rope cache query") ||
        !qw_require_dtype(gpu, key_new, count, H3_GPU_BF16, "QK norm+rope cache key") ||
        !qw_require_dtype(gpu, value_new, count, H3_GPU_BF16, "QK norm+rope cache value") ||
        !qw_require_dtype(gpu, key_cache, cache_count, H3_GPU_BF16, "QK norm+rope key cache") ||
        !qw_require_dtype(gpu, value_cache, cache_count, H3_GPU_BF16, "QK norm+rope value cache") ||
        !qw_require_dtype(gpu, norm_weight_q, head_dim, H3_GPU_BF16, "QK norm+rope cache query weight") ||
        !qw_require_dtype(gpu, norm_weight_k, head_dim, H3_GPU_BF16, "QK norm+rope cache key weight") ||
        !qw_require_dtype(gpu, rope_cos, rope_count, H3_GPU_F32, "QK norm+rope cache cosine") ||
        !qw_require_dtype(gpu, rope_sin, rope_count, H3_GPU_F32, "QK norm+rope cache sine"))
        return 0;
    if (!qw_require_command(gpu)) return 0;
    if (head_dim != 128 || !rows || !heads) {
        qw_set_error(gpu, "QK norm+rope cache: unsupported geometry");
        return 0;
    }
    if ((uint64_t)cache_row_offset + rows > cache_rows) {
        qw_set_error(gpu, "QK norm+rope cache: rows [%u, %u) lie outside the %u cached rows",
                     cache_row_offset, cache_row_offset + rows, cache_rows);
        return 0;
    }
    if (key_new == key_cache || value_new == value_cache) {
        qw_set_error(gpu, "QK norm+rope cache: the new rows and the cache must be distinct tensors");
        return 0;
    }
    size_t offset_bytes = (size_t)cache_row_offset * heads * head_dim * 2;
    qwcu_prologue_args args;
    memset(&args, 0, sizeof(args));
    args.q_in = query->dev;
    args.q_out = query->dev;
    args.k_in = key_new->dev;
    args.k_out = (char *)key_cache->dev + offset_bytes;
    args.v_in = value_new->dev;
    args.v_out = (char *)value_cache->dev + offset_bytes;
    args.norm_weight_q = norm_weight_q->dev;
    args.norm_weight_k = norm_weight_k->dev;
    args.rope_cos = rope_cos->dev;
    args.rope_sin = rope_sin->dev;
    args.rows = rows;
    args.table_rows = rows;
    args.heads = heads;
    args.epsilon = epsilon;
    return launch_prologue(gpu, &args, "QK norm+rope cache");
}

/* ---- attention ops ------------------------------------------------------- */

int qw_launch_attention(h3_gpu *gpu, qwcu_attn_args *args, const char *what) {
    if (!qw_bind(gpu)) return 0;
    args->status = gpu->status_dev;
    args->whole_units = gpu->attn_kernel == QW_ATTN_SM100_WHOLE;
    args->row_softmax = gpu->attn_kernel == QW_ATTN_SM100_ROW;
    args->wait_cycles = gpu->attn_wait_cycles;
    args->withhold_from = gpu->attn_withhold_tile;
    int scalar = gpu->attn_kernel == QW_ATTN_SCALAR;
    /* Degenerate scales cannot ride the exp2-domain fast path. */
    if (!(args->scale > 0.0f) || !isfinite(args->scale)) scalar = 1;
    if (scalar && args->n_out_peers) {
        qw_set_error(gpu, "%s: sharded output needs the sm100 kernel and a positive finite scale", what);
        return 0;
    }
    if (!scalar && args->scale_in_q) {
        /* h3 causal variant: q' = bf16(q * scale) into scratch, scores unscaled
         * (h3_shaders.metal:4396-4402). */
        size_t count = (size_t)args->batch * args->q_rows * args->heads * 128;
        void *scaled = qw_scratch(gpu, count * 2);
        if (!scaled) return 0; /* message set by qw_scratch */
        int rc = qwcu_scale_bf16_launch(scaled, args->q, count, args->scale, gpu->stream);
        qw_count_launch(gpu, rc, "query pre-scale");
        if (rc) return 0;
        args->q = scaled;
        args->scale = 1.0f;
        args->scale_in_q = 0;
    }
    int rc = scalar ? qwcu_attn_scalar_launch(args, gpu->stream)
                    : qwcu_attn_sm100_launch(args, gpu->stream);
    qw_count_launch(gpu, rc, what);
    return rc == 0;
}

/* reference h3_gpu.m:5745-5789 */
int qw_gpu_flash_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t q_rows, uint32_t kv_rows, uint32_t heads, uint32_t head_dim,
                           float scale) {
    if (!gpu) return 0;
    if (head_dim != 128 || !heads) {
        qw_set_error(gpu, "flash SDPA: unsupported geometry");
        return 0;
    }
    size_t q_count = (size_t)q_rows * heads * head_dim;
    size_t kv_count = (size_t)kv_rows * heads * head_dim;
    if (!q_rows || !kv_rows ||
        !qw_require_dtype(gpu, query, q_count, H3_GPU_BF16, "flash SDPA query") ||
        !qw_require_dtype(gpu, key, kv_count, H3_GPU_BF16, "flash SDPA key") ||
        !qw_require_dtype(gpu, value, kv_count, H3_GPU_BF16, "flash SDPA value") ||
        !qw_require_dtype(gpu, output, q_count, H3_GPU_BF16, "flash SDPA output") ||
        !qw_require_command(gpu))
        return 0;
    qwcu_attn_args args;
    memset(&args, 0, sizeof(args));
    args.q = query->dev;
    args.k = key->dev;
    args.v = value->dev;
    args.out = output->dev;
    args.batch = 1;
    args.q_rows = q_rows;
    args.kv_rows = kv_rows;
    args.heads = heads;
    args.kv_heads = heads;
    args.scale = scale;
    return qw_launch_attention(gpu, &args, "flash SDPA");
}

/* reference h3_gpu.m:5791-5844 */
int qw_gpu_flash_sdpa_prefix_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                                  const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                                  const h3_gpu_tensor *kv_limit, uint32_t q_rows,
                                  uint32_t kv_rows, uint32_t heads, uint32_t kv_heads,
                                  uint32_t head_dim, float scale) {
    if (!gpu) return 0;
    if (head_dim != 128 || !heads || !kv_heads || heads % kv_heads) {
        qw_set_error(gpu, "flash SDPA prefix: unsupported geometry");
        return 0;
    }
    size_t q_count = (size_t)q_rows * heads * head_dim;
    size_t kv_count = (size_t)kv_rows * kv_heads * head_dim;
    if (!q_rows || !kv_rows ||
        !qw_require_dtype(gpu, query, q_count, H3_GPU_BF16, "flash SDPA prefix query") ||
        !qw_require_dtype(gpu, key, kv_count, H3_GPU_BF16, "flash SDPA prefix key") ||
        !qw_require_dtype(gpu, value, kv_count, H3_GPU_BF16, "flash SDPA prefix value") ||
        !qw_require_dtype(gpu, output, q_count, H3_GPU_BF16, "flash SDPA prefix output") ||
        !qw_require_elements(gpu, kv_limit, q_rows, "flash SDPA prefix limit") ||
        kv_limit->dtype != H3_GPU_U32 || !qw_require_command(gpu))
        return 0;
    qwcu_attn_args args;
    memset(&args, 0, sizeof(args));
    args.q = query->dev;
    args.k = key->dev;
    args.v = value->dev;
    args.out = output->dev;
    args.kv_limit = kv_limit->dev;
    args.batch = 1;
    args.q_rows = q_rows;
    args.kv_rows = kv_rows;
    args.heads = heads;
    args.kv_heads = kv_heads;
    args.scale = scale;
    return qw_launch_attention(gpu, &args, "flash SDPA prefix");
}

/* reference h3_gpu.m:5972-6054 */
int qw_gpu_sdpa_rect_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                          const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                          uint32_t query_sequence, uint32_t kv_sequence, uint32_t heads,
                          uint32_t head_dim, float scale) {
    if (!gpu) return 0;
    size_t q_count = (size_t)query_sequence * heads * head_dim;
    size_t kv_count = (size_t)kv_sequence * heads * head_dim;
    if (!query_sequence || !kv_sequence || !heads || !head_dim || !qw_require_command(gpu) ||
        !qw_require_dtype(gpu, query, q_count, H3_GPU_BF16, "Rect SDPA query") ||
        !qw_require_dtype(gpu, key, kv_count, H3_GPU_BF16, "Rect SDPA key") ||
        !qw_require_dtype(gpu, value, kv_count, H3_GPU_BF16, "Rect SDPA value") ||
        !qw_require_dtype(gpu, output, q_count, H3_GPU_BF16, "Rect SDPA output"))
        return 0;
    if (head_dim != 128) {
        qw_set_error(gpu, "Rect SDPA: unsupported geometry (head_dim must be 128)");
        return 0;
    }
    qwcu_attn_args args;
    memset(&args, 0, sizeof(args));
    args.q = query->dev;
    args.k = key->dev;
    args.v = value->dev;
    args.out = output->dev;
    args.batch = 1;
    args.q_rows = query_sequence;
    args.kv_rows = kv_sequence;
    args.heads = heads;
    args.kv_heads = heads;
    args.scale = scale;
    return qw_launch_attention(gpu, &args, "Rect SDPA");
}

static int gqa_causal(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                      const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                      uint32_t query_heads, uint32_t kv_heads, uint32_t head_dim, float scale,
                      int scale_in_q, const char *label) {
    if (!gpu) return 0;
    size_t query_count = (size_t)sequence * query_heads * head_dim;
    size_t kv_count = (size_t)sequence * kv_heads * head_dim;
    char name[64];
    if (!sequence || !query_heads || !kv_heads || !head_dim || query_heads % kv_heads ||
        head_dim > 128)
        return 0;
    snprintf(name, sizeof(name), "%s query", label);
    if (!qw_require_dtype(gpu, query, query_count, H3_GPU_BF16, name)) return 0;
    snprintf(name, sizeof(name), "%s key", label);
    if (!qw_require_dtype(gpu, key, kv_count, H3_GPU_BF16, name)) return 0;
    snprintf(name, sizeof(name), "%s value", label);
    if (!qw_require_dtype(gpu, value, kv_count, H3_GPU_BF16, name)) return 0;
    snprintf(name, sizeof(name), "%s output", label);
    if (!qw_require_dtype(gpu, output, query_count, H3_GPU_BF16, name)) return 0;
    if (!qw_require_command(gpu)) return 0;
    if (head_dim != 128) {
        qw_set_error(gpu, "%s: unsupported geometry (head_dim must be 128)", label);
        return 0;
    }
    qwcu_attn_args args;
    memset(&args, 0, sizeof(args));
    args.q = query->dev;
    args.k = key->dev;
    args.v = value->dev;
    args.out = output->dev;
    args.causal = 1;
    args.batch = 1;
    args.q_rows = sequence;
    args.kv_rows = sequence;
    args.heads = query_heads;
    args.kv_heads = kv_heads;
    args.scale = scale;
    args.scale_in_q = scale_in_q;
    return qw_launch_attention(gpu, &args, label);
}

/* reference h3_gpu.m:4642-4693 */
int h3_gpu_gqa_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t sequence, uint32_t query_heads, uint32_t kv_heads,
                           uint32_t head_dim, float scale) {
    return gqa_causal(gpu, output, query, key, value, sequence, query_heads, kv_heads, head_dim,
                      scale, 1, "GQA");
}

/* reference h3_gpu.m:5903-5953 */
int qw_gpu_gqa_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t sequence, uint32_t query_heads, uint32_t kv_heads,
                           uint32_t head_dim, float scale) {
    return gqa_causal(gpu, output, query, key, value, sequence, query_heads, kv_heads, head_dim,
                      scale, 0, "Qwen GQA");
}

/* reference h3_gpu.m:1630-1682 (validation), :1698-1720 (entry points) */
static int sdpa_square(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                       const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                       uint32_t heads, uint32_t head_dim, float scale, int head_major_out) {
    if (!gpu) return 0;
    size_t count = (size_t)sequence * heads * head_dim;
    if (!sequence || !heads || !head_dim || !qw_require_command(gpu) ||
        !qw_require_elements(gpu, query, count, "SDPA query") ||
        !qw_require_elements(gpu, key, count, "SDPA key") ||
        !qw_require_elements(gpu, value, count, "SDPA value") ||
        !qw_require_elements(gpu, output, count, "SDPA output"))
        return 0;
    if (query->dtype != H3_GPU_BF16 || key->dtype != H3_GPU_BF16 || value->dtype != H3_GPU_BF16 ||
        output->dtype != H3_GPU_BF16) {
        qw_set_error(gpu, "SDPA tensor dtype mismatch");
        return 0;
    }
    if (head_dim != 128) {
        qw_set_error(gpu, "SDPA: unsupported geometry (head_dim must be 128)");
        return 0;
    }
    qwcu_attn_args args;
    memset(&args, 0, sizeof(args));
    args.q = query->dev;
    args.k = key->dev;
    args.v = value->dev;
    args.out = output->dev;
    args.batch = 1;
    args.q_rows = sequence;
    args.kv_rows = sequence;
    args.heads = heads;
    args.kv_heads = heads;
    args.scale = scale;
    args.head_major_out = head_major_out;
    return qw_launch_attention(gpu, &args, "SDPA");
}

int h3_gpu_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                     const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                     uint32_t heads, uint32_t head_dim, float scale) {
    return sdpa_square(gpu, output, query, key, value, sequence, heads, head_dim, scale, 0);
}

int h3_gpu_sdpa_bf16_head_major_output(h3_gpu *gpu, h3_gpu_tensor *output,
                                       const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                       const h3_gpu_tensor *value, uint32_t sequence,
                                       uint32_t heads, uint32_t head_dim, float scale) {
    return sdpa_square(gpu, output, query, key, value, sequence, heads, head_dim, scale, 1);
}

/* Validation + argument block of the batched block-causal op; `output` may be
 * NULL when the caller provides the destinations itself (sharded heads). */
int qw_prepare_block_causal(h3_gpu *gpu, qwcu_attn_args *args, h3_gpu_tensor *output,
                            const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                            const h3_gpu_tensor *value, const h3_gpu_tensor *kv_limit,
                            uint32_t batch, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                            uint32_t head_dim, const uint32_t *text_len, uint32_t text_pad,
                            float scale) {
    if (head_dim != 128 || !heads || !kv_heads || heads % kv_heads || !batch || batch > 8) {
        qw_set_error(gpu, "block-causal attention: unsupported geometry");
        return 0;
    }
    size_t q_count = (size_t)batch * rows * heads * head_dim;
    size_t kv_count = (size_t)batch * rows * kv_heads * head_dim;
    if (!rows ||
        !qw_require_dtype(gpu, query, q_count, H3_GPU_BF16, "block-causal attention query") ||
        !qw_require_dtype(gpu, key, kv_count, H3_GPU_BF16, "block-causal attention key") ||
        !qw_require_dtype(gpu, value, kv_count, H3_GPU_BF16, "block-causal attention value") ||
        (output &&
         !qw_require_dtype(gpu, output, q_count, H3_GPU_BF16, "block-causal attention output")))
        return 0;
    int per_batch = 0;
    if (kv_limit) {
        if (!qw_require_elements(gpu, kv_limit, rows, "block-causal attention limit") ||
            kv_limit->dtype != H3_GPU_U32)
            return 0;
        /* One table shared by the batch (`rows` entries) or one per item
         * (`batch * rows`): the size says which, so it must be one of the two. */
        if (batch > 1 && kv_limit->elements != rows &&
            kv_limit->elements != (size_t)batch * rows) {
            qw_set_error(gpu, "block-causal attention limit tensor must hold rows (%u) or "
                              "batch*rows (%zu) entries, not %zu",
                         rows, (size_t)batch * rows, kv_limit->elements);
            return 0;
        }
        per_batch = batch > 1 && kv_limit->elements == (size_t)batch * rows;
    }
    if (text_len && text_pad) {
        if (text_pad > rows) {
            qw_set_error(gpu, "block-causal attention: text_pad exceeds the row count");
            return 0;
        }
        for (uint32_t b = 0; b < batch; b++)
            if (text_len[b] > text_pad) {
                qw_set_error(gpu, "block-causal attention: text_len[%u] exceeds text_pad", b);
                return 0;
            }
    }
    if (!qw_require_command(gpu)) return 0;
    memset(args, 0, sizeof(*args));
    args->q = query->dev;
    args->k = key->dev;
    args->v = value->dev;
    args->out = output ? output->dev : NULL;
    args->kv_limit = kv_limit ? kv_limit->dev : NULL;
    args->per_batch_limits = per_batch;
    args->batch = batch;
    args->q_rows = rows;
    args->kv_rows = rows;
    args->heads = heads;
    args->kv_heads = kv_heads;
    if (text_len && text_pad) {
        for (uint32_t b = 0; b < batch; b++) args->text_len[b] = text_len[b];
        args->text_pad = text_pad;
    }
    args->scale = scale;
    return 1;
}

/* NEW: batched block-causal attention with key padding. */
int qw_gpu_attn_block_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                  const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                  const h3_gpu_tensor *value, const h3_gpu_tensor *kv_limit,
                                  uint32_t batch, uint32_t rows, uint32_t heads,
                                  uint32_t kv_heads, uint32_t head_dim,
                                  const uint32_t *text_len, uint32_t text_pad, float scale) {
    if (!gpu) return 0;
    if (!output) {
        qw_set_error(gpu, "block-causal attention output tensor is absent or too small");
        return 0;
    }
    qwcu_attn_args args;
    if (!qw_prepare_block_causal(gpu, &args, output, query, key, value, kv_limit, batch, rows,
                                 heads, kv_heads, head_dim, text_len, text_pad, scale))
        return 0;
    return qw_launch_attention(gpu, &args, "block-causal attention");
}

/* NEW: the same op for normed inputs.  score_bound (F32 tensor, two elements, as
 * left by qw_gpu_qk_norm_rope_bound_bf16) promises ||q row|| <= [0] and
 * ||k row|| <= [1]; the kernel then runs the softmax against one fixed reference
 * exponent instead of a running row maximum. */
int qw_gpu_attn_block_causal_bounded_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                          const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                          const h3_gpu_tensor *value,
                                          const h3_gpu_tensor *kv_limit,
                                          const h3_gpu_tensor *score_bound, uint32_t batch,
                                          uint32_t rows, uint32_t heads, uint32_t kv_heads,
                                          uint32_t head_dim, const uint32_t *text_len,
                                          uint32_t text_pad, float scale) {
    if (!gpu) return 0;
    if (!output) {
        qw_set_error(gpu, "block-causal attention output tensor is absent or too small");
        return 0;
    }
    if (!qw_require_dtype(gpu, score_bound, 2, H3_GPU_F32, "block-causal attention score bound"))
        return 0;
    qwcu_attn_args args;
    if (!qw_prepare_block_causal(gpu, &args, output, query, key, value, kv_limit, batch, rows,
                                 heads, kv_heads, head_dim, text_len, text_pad, scale))
        return 0;
    args.score_bound = (const float *)score_bound->dev;
    return qw_launch_attention(gpu, &args, "block-causal attention (bounded)");
}
