/* Internal definitions shared by the C11 host translation units. */
#ifndef QW_INTERNAL_H
#define QW_INTERNAL_H

#include <cuda_runtime_api.h>
#include <stdarg.h>
#include <stddef.h>
#include <stdint.h>

#include "h3_gpu.h"
#include "qw_cuda.h"
#include "qwen_attn_host.h"
#include "qwen_gpu_ext.h"

enum { QW_ATTN_SM100 = 0, QW_ATTN_SCALAR = 1, QW_ATTN_SM100_WHOLE = 2, QW_ATTN_SM100_ROW = 3 };

struct h3_gpu {
    int device;
    cudaStream_t stream;
    int chain_open;
    int chain_failed; /* a launch in the open chain failed: submit reports it */
    char error[512];
    h3_gpu_stats stats;
    uint64_t kernel_launches;
    cudaEvent_t chain_start, chain_stop;
    double chain_start_wall;
    uint32_t *status_dev;  /* QWCU_STATUS_WORDS words, zero when healthy */
    uint32_t *status_host; /* pinned mirror */
    int attn_kernel;
    long long attn_wait_cycles; /* tests: budget of the attention kernel's waits (0 = default) */
    int attn_withhold_tile;     /* tests: first key tile the producer leaves out (0 = none) */
    /* A multi-GPU group's communication stream; submit waits for it too. */
    cudaStream_t aux_stream;
    cudaEvent_t aux_joined;
    /* Stream capture into a replayable graph (qw_gpu_graph_*). */
    int capturing;
    uint32_t capture_seq;      /* identifies the capture an event was recorded in */
    uint64_t capture_launches; /* kernel launches counted since capture began */
    /* Copy lanes beside the compute stream (qw_gpu_fence, qw_gpu_tensor_*_lane):
     * lane 0 is `stream`, lanes 1.. are created on first use; submit joins them. */
    cudaStream_t lane[3];
    cudaEvent_t lane_event;
    /* Scratch for the pre-scaled query of the h3 causal variant; grows on demand. */
    void *scratch;
    size_t scratch_bytes;
};

struct qw_gpu_graph {
    h3_gpu *owner;
    cudaGraphExec_t exec;
    uint64_t kernel_launches;
};

struct h3_gpu_tensor {
    h3_gpu *owner;
    h3_gpu_dtype dtype;
    size_t elements;
    size_t bytes;
    void *dev;
};

void qw_set_error(h3_gpu *gpu, const char *format, ...);
int qw_cuda_ok(h3_gpu *gpu, cudaError_t code, const char *what);
int qw_bind(h3_gpu *gpu);
size_t qw_dtype_size(h3_gpu_dtype dtype);
int qw_require_command(h3_gpu *gpu);
int qw_require_elements(h3_gpu *gpu, const h3_gpu_tensor *tensor, size_t elements,
                        const char *label);
int qw_require_dtype(h3_gpu *gpu, const h3_gpu_tensor *tensor, size_t elements,
                     h3_gpu_dtype dtype, const char *label);
void *qw_scratch(h3_gpu *gpu, size_t bytes);
void qw_count_launch(h3_gpu *gpu, int rc, const char *what);
double qw_now(void);
int qw_launch_attention(h3_gpu *gpu, qwcu_attn_args *args, const char *what);
int qw_prepare_block_causal(h3_gpu *gpu, qwcu_attn_args *args, h3_gpu_tensor *output,
                            const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                            const h3_gpu_tensor *value, const h3_gpu_tensor *kv_limit,
                            uint32_t batch, uint32_t rows, uint32_t heads, uint32_t kv_heads,
                            uint32_t head_dim, const uint32_t *text_len, uint32_t text_pad,
                            float scale);

#endif
