/* The linear layers either side of the attention path in the DiT block: the fused
 * q/k/v projection in front of it (reference qwen_dit.m:1270) and the output
 * projection behind it (qwen_dit.m:1446), on the tcgen05 GEMM of
 * cuda/qw_linear_sm100.cu.  Validation follows the reference's op wrappers. */
#include "qw_internal.h"

#include <string.h>

static int launch_linear(h3_gpu *gpu, qwcu_linear_args *args, const char *what) {
    if (!qw_bind(gpu)) return 0;
    args->status = gpu->status_dev;
    int rc = qwcu_linear_sm100_launch(args, qwcu_device_sm_count(gpu->device), gpu->stream);
    qw_count_launch(gpu, rc, what);
    return rc == 0;
}

/* reference h3_gpu.h:295-299, h3_gpu.m:2697-2812, h3_shaders.metal:788-822:
 * output[rows, output_dim] = bf16(bias + input[rows, input_dim] . weight[output_dim,
 * input_dim]^T), fp32 accumulation. */
int h3_gpu_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                       const h3_gpu_tensor *weight, const h3_gpu_tensor *bias, uint32_t rows,
                       uint32_t input_dim, uint32_t output_dim) {
    if (!gpu) return 0;
    size_t input_count = (size_t)rows * input_dim;
    size_t weight_count = (size_t)output_dim * input_dim;
    size_t output_count = (size_t)rows * output_dim;
    if (!qw_require_dtype(gpu, input, input_count, H3_GPU_BF16, "linear input") ||
        !qw_require_dtype(gpu, weight, weight_count, H3_GPU_BF16, "linear weight") ||
        !qw_require_dtype(gpu, output, output_count, H3_GPU_BF16, "linear output") ||
        (bias && !qw_require_dtype(gpu, bias, output_dim, H3_GPU_BF16, "linear bias")))
        return 0;
    if (!qw_require_command(gpu)) return 0;
    if (!rows || !input_dim || !output_dim || input_dim % 8 || output_dim % 8) {
        qw_set_error(gpu, "linear: unsupported geometry (dimensions must be non-zero multiples of 8)");
        return 0;
    }
    qwcu_linear_args args;
    memset(&args, 0, sizeof(args));
    args.a = input->dev;
    args.w[0] = weight->dev;
    args.c[0] = output->dev;
    args.bias[0] = bias ? bias->dev : NULL;
    args.n_outputs = 1;
    args.m = rows;
    args.k = input_dim;
    args.n = output_dim;
    return launch_linear(gpu, &args, "linear");
}

static int qkv(h3_gpu *gpu, h3_gpu_tensor *query_out, h3_gpu_tensor *key_out,
               h3_gpu_tensor *value_out, const h3_gpu_tensor *input,
               const h3_gpu_tensor *query_weight, const h3_gpu_tensor *key_weight,
               const h3_gpu_tensor *value_weight, uint32_t rows, uint32_t dim,
               qwcu_linear_args *args) {
    size_t count = (size_t)rows * dim;
    size_t weight_count = (size_t)dim * dim;
    if (!qw_require_dtype(gpu, input, count, H3_GPU_BF16, "Qwen QKV input") ||
        !qw_require_dtype(gpu, query_weight, weight_count, H3_GPU_BF16, "Qwen QKV query weight") ||
        !qw_require_dtype(gpu, key_weight, weight_count, H3_GPU_BF16, "Qwen QKV key weight") ||
        !qw_require_dtype(gpu, value_weight, weight_count, H3_GPU_BF16, "Qwen QKV value weight") ||
        !qw_require_dtype(gpu, query_out, count, H3_GPU_BF16, "Qwen QKV query output") ||
        !qw_require_dtype(gpu, key_out, count, H3_GPU_BF16, "Qwen QKV key output") ||
        !qw_require_dtype(gpu, value_out, count, H3_GPU_BF16, "Qwen QKV value output"))
        return 0;
    if (!qw_require_command(gpu)) return 0;
    if (!rows || !dim || dim % 8) {
        qw_set_error(gpu, "Qwen QKV: unsupported geometry (dim must be a non-zero multiple of 8)");
        return 0;
    }
    memset(args, 0, sizeof(*args));
    args->a = input->dev;
    args->w[0] = query_weight->dev;
    args->w[1] = key_weight->dev;
    args->w[2] = value_weight->dev;
    args->c[0] = query_out->dev;
    args->c[1] = key_out->dev;
    args->c[2] = value_out->dev;
    args->n_outputs = 3;
    args->m = rows;
    args->k = dim;
    args->n = dim;
    return 1;
}

/* reference qwen_gpu_ext.h:202-210, h3_gpu.m:2918-3018: q, k, v = input . W^T for the
 * three [dim, dim] weights, one launch. */
int qw_gpu_qkv_bf16(h3_gpu *gpu, h3_gpu_tensor *query_out, h3_gpu_tensor *key_out,
                    h3_gpu_tensor *value_out, const h3_gpu_tensor *input,
                    const h3_gpu_tensor *query_weight, const h3_gpu_tensor *key_weight,
                    const h3_gpu_tensor *value_weight, uint32_t rows, uint32_t dim) {
    if (!gpu) return 0;
    qwcu_linear_args args;
    if (!qkv(gpu, query_out, key_out, value_out, input, query_weight, key_weight, value_weight,
             rows, dim, &args))
        return 0;
    return launch_linear(gpu, &args, "Qwen QKV");
}

/* NEW: the q/k/v projection with the per-head QK RMSNorm and the interleaved RoPE
 * in its epilogue (the reference's sequence qwen_dit.m:1270-1278 in one launch):
 * q and k leave the GEMM already normed and rotated, v plain.  rows = batch *
 * sequence; row r uses table row r % sequence.  score_bound (optional F32 tensor,
 * two elements) receives the row-norm bounds for the fixed-exponent softmax. */
int qw_gpu_qkv_norm_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query_out, h3_gpu_tensor *key_out,
                              h3_gpu_tensor *value_out, const h3_gpu_tensor *input,
                              const h3_gpu_tensor *query_weight, const h3_gpu_tensor *key_weight,
                              const h3_gpu_tensor *value_weight,
                              const h3_gpu_tensor *norm_weight_q,
                              const h3_gpu_tensor *norm_weight_k, const h3_gpu_tensor *rope_cos,
                              const h3_gpu_tensor *rope_sin, h3_gpu_tensor *score_bound,
                              uint32_t batch, uint32_t sequence, uint32_t dim, float epsilon) {
    if (!gpu) return 0;
    if ((uint64_t)batch * sequence > UINT32_MAX) {
        qw_set_error(gpu, "Qwen QKV norm+rope: too many rows");
        return 0;
    }
    size_t rope_count = (size_t)sequence * 64;
    if (!qw_require_dtype(gpu, norm_weight_q, 128, H3_GPU_BF16, "Qwen QKV query norm weight") ||
        !qw_require_dtype(gpu, norm_weight_k, 128, H3_GPU_BF16, "Qwen QKV key norm weight") ||
        !qw_require_dtype(gpu, rope_cos, rope_count, H3_GPU_F32, "Qwen QKV cosine") ||
        !qw_require_dtype(gpu, rope_sin, rope_count, H3_GPU_F32, "Qwen QKV sine") ||
        (score_bound && !qw_require_dtype(gpu, score_bound, 2, H3_GPU_F32, "Qwen QKV score bound")))
        return 0;
    qwcu_linear_args args;
    if (!qkv(gpu, query_out, key_out, value_out, input, query_weight, key_weight, value_weight,
             batch * sequence, dim, &args))
        return 0;
    if (dim % 128 || !sequence || !(epsilon >= 0.0f)) {
        qw_set_error(gpu, "Qwen QKV norm+rope: unsupported geometry (dim must be a multiple of the "
                          "head size 128, epsilon >= 0)");
        return 0;
    }
    args.norm_weight[0] = norm_weight_q->dev;
    args.norm_weight[1] = norm_weight_k->dev;
    args.rope_cos = rope_cos->dev;
    args.rope_sin = rope_sin->dev;
    args.table_rows = sequence;
    args.epsilon = epsilon;
    args.bound_out = score_bound ? (float *)score_bound->dev : NULL;
    return launch_linear(gpu, &args, "Qwen QKV norm+rope");
}
