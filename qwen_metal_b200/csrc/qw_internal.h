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

enum { QW_ATTN_SM100 = 0, QW_ATTN_SCALAR = 1 };

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
    /* Scratch for the pre-scaled query of the h3 causal variant; grows on demand. */
    void *scratch;
    size_t scratch_bytes;
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

#endif
