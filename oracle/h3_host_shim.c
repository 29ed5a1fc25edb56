/* Host-memory stand-in for the handful of h3_gpu entry points the reference's
 * tests/test_prefix_kernel.c uses (TEST INFRASTRUCTURE ONLY).
 *
 * It lets that test file be compiled unmodified with the CPU oracle behind
 * qw_gpu_flash_sdpa_prefix_bf16, so the reference's own inline CPU loop
 * (tests/test_prefix_kernel.c:72-97) and its own relL2 gate (:133-142) judge
 * the oracle.  Tensors are plain malloc'd host arrays; nothing here touches a
 * GPU and nothing in the shipped library links this file.
 */
#include "h3_gpu.h"
#include "qwen_gpu_ext.h"
#include "qw_oracle.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

struct h3_gpu {
    int open;
    char error[256];
};

struct h3_gpu_tensor {
    h3_gpu_dtype dtype;
    size_t elements;
    void *data;
};

static size_t dtype_size(h3_gpu_dtype dtype) {
    return dtype == H3_GPU_BF16 ? 2 : dtype == H3_GPU_I8 ? 1 : 4;
}

h3_gpu *h3_gpu_create(const char *path, char *error, size_t error_size) {
    (void)path;
    h3_gpu *gpu = calloc(1, sizeof(*gpu));
    if (!gpu && error && error_size) snprintf(error, error_size, "out of memory");
    return gpu;
}

void h3_gpu_free(h3_gpu *gpu) { free(gpu); }

const char *h3_gpu_error(const h3_gpu *gpu) {
    return gpu && gpu->error[0] ? gpu->error : "unknown error";
}

static h3_gpu_tensor *tensor_new(h3_gpu_dtype dtype, size_t elements, const void *values) {
    h3_gpu_tensor *t = calloc(1, sizeof(*t));
    if (!t) return NULL;
    t->dtype = dtype;
    t->elements = elements;
    t->data = calloc(elements ? elements : 1, dtype_size(dtype));
    if (!t->data) {
        free(t);
        return NULL;
    }
    if (values) memcpy(t->data, values, elements * dtype_size(dtype));
    return t;
}

h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t elements) {
    (void)gpu;
    return tensor_new(H3_GPU_BF16, elements, NULL);
}

h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *values, size_t elements) {
    (void)gpu;
    return tensor_new(H3_GPU_U32, elements, values);
}

void h3_gpu_tensor_free(h3_gpu_tensor *tensor) {
    if (!tensor) return;
    free(tensor->data);
    free(tensor);
}

int h3_gpu_tensor_write_bf16(h3_gpu_tensor *tensor, const uint16_t *values, size_t elements) {
    if (!tensor || !values || tensor->dtype != H3_GPU_BF16 || elements > tensor->elements)
        return 0;
    memcpy(tensor->data, values, elements * 2);
    return 1;
}

int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *tensor, uint16_t *values, size_t elements) {
    if (!tensor || !values || tensor->dtype != H3_GPU_BF16 || elements > tensor->elements)
        return 0;
    memcpy(values, tensor->data, elements * 2);
    return 1;
}

int h3_gpu_begin(h3_gpu *gpu) {
    if (!gpu || gpu->open) return 0;
    gpu->open = 1;
    return 1;
}

int h3_gpu_submit(h3_gpu *gpu) {
    if (!gpu || !gpu->open) return 0;
    gpu->open = 0;
    return 1;
}

int qw_gpu_flash_sdpa_prefix_bf16(h3_gpu *gpu, h3_gpu_tensor *output,
                                  const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                  const h3_gpu_tensor *value, const h3_gpu_tensor *kv_limit,
                                  uint32_t q_rows, uint32_t kv_rows, uint32_t heads,
                                  uint32_t kv_heads, uint32_t head_dim, float scale) {
    if (!gpu || !gpu->open) return 0;
    size_t count = (size_t)q_rows * heads * head_dim;
    float *out = malloc(sizeof(float) * count);
    if (!out) return 0;
    qwo_sdpa_prefix(out, query->data, key->data, value->data, kv_limit->data, 0, 1, q_rows,
                    kv_rows, heads, kv_heads, head_dim, scale, NULL, 0, NULL, 0);
    uint16_t *dst = output->data;
    for (size_t i = 0; i < count; i++) dst[i] = qwo_f32_to_bf16(out[i]);
    /* Also leave the fp32 result where a harness can pick it up. */
    const char *dump = getenv("QWO_SHIM_DUMP_F32");
    if (dump && *dump) {
        FILE *f = fopen(dump, "wb");
        if (f) {
            fwrite(out, sizeof(float), count, f);
            fclose(f);
        }
    }
    free(out);
    return 1;
}
