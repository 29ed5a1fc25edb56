/* CUDA implementation of the h3_gpu context, tensor and command-chain ABI
 * (reference h3_gpu.m:380-1074).  C11; CUDA is reached through the runtime's C
 * API only.  The reference's command buffer maps onto one CUDA stream:
 *   begin    = mark the chain open, record the start event
 *   op       = asynchronous launch on the stream
 *   continue = no-op flush (the stream already runs ahead of the host)
 *   submit   = record stop event, synchronise, check launch errors and the
 *              device status words
 */
#define _POSIX_C_SOURCE 200809L
#include "qw_internal.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

double qw_now(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + (double)ts.tv_nsec / 1e9;
}

void qw_set_error(h3_gpu *gpu, const char *format, ...) {
    if (!gpu) return;
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(gpu->error, sizeof(gpu->error), format, arguments);
    va_end(arguments);
}

int qw_cuda_ok(h3_gpu *gpu, cudaError_t code, const char *what) {
    if (code == cudaSuccess) return 1;
    qw_set_error(gpu, "%s: %s", what, cudaGetErrorString(code));
    return 0;
}

int qw_bind(h3_gpu *gpu) {
    return gpu && cudaSetDevice(gpu->device) == cudaSuccess;
}

size_t qw_dtype_size(h3_gpu_dtype dtype) {
    switch (dtype) {
        case H3_GPU_BF16: return 2;
        case H3_GPU_I8: return 1;
        default: return 4;
    }
}

/* reference h3_gpu.m:274-280 */
int qw_require_command(h3_gpu *gpu) {
    if (!gpu || !gpu->chain_open) {
        if (gpu) qw_set_error(gpu, "h3_gpu_begin() was not called");
        return 0;
    }
    return 1;
}

/* reference h3_gpu.m:282-289 */
int qw_require_elements(h3_gpu *gpu, const h3_gpu_tensor *tensor, size_t elements,
                        const char *label) {
    if (!tensor || tensor->elements < elements) {
        qw_set_error(gpu, "%s tensor is absent or too small", label);
        return 0;
    }
    return 1;
}

/* reference h3_gpu.m:2588-2616 */
int qw_require_dtype(h3_gpu *gpu, const h3_gpu_tensor *tensor, size_t elements,
                     h3_gpu_dtype dtype, const char *label) {
    static const char *const names[] = {"F32", "BF16", "int8", "U32"};
    if (!qw_require_elements(gpu, tensor, elements, label)) return 0;
    if (tensor->dtype != dtype) {
        qw_set_error(gpu, "%s tensor is not %s", label, names[dtype]);
        return 0;
    }
    return 1;
}

void qw_count_launch(h3_gpu *gpu, int rc, const char *what) {
    if (rc == 0) {
        if (gpu->capturing) {
            gpu->capture_launches++; /* credited on every replay of the graph */
            return;
        }
        gpu->stats.direct_dispatches++;
        gpu->kernel_launches++;
    } else {
        gpu->chain_failed = 1;
        qw_set_error(gpu, "%s launch failed: %s", what, cudaGetErrorString((cudaError_t)rc));
    }
}

/* Scratch of at least `bytes`, or NULL with the error set.  The block is cached in
 * the context, so it must never be a graph-owned allocation: while a capture is
 * active the block may be reused but neither created nor grown (an allocation
 * captured into a graph is only backed while that graph runs). */
void *qw_scratch(h3_gpu *gpu, size_t bytes) {
    if (gpu->scratch_bytes >= bytes) return gpu->scratch;
    if (gpu->capturing) {
        qw_set_error(gpu, "this op needs %zu bytes of scratch but only %zu are allocated: run it "
                          "once at this size before capturing it into a graph",
                     bytes, gpu->scratch_bytes);
        gpu->chain_failed = 1;
        return NULL;
    }
    if (gpu->scratch) {
        /* Earlier launches may still read the old block: stream-ordered free. */
        cudaFreeAsync(gpu->scratch, gpu->stream);
        gpu->scratch = NULL;
        gpu->scratch_bytes = 0;
    }
    void *block = NULL;
    if (cudaMallocAsync(&block, bytes, gpu->stream) != cudaSuccess) {
        cudaGetLastError();
        qw_set_error(gpu, "cannot allocate %zu bytes of scratch", bytes);
        return NULL;
    }
    gpu->scratch = block;
    gpu->scratch_bytes = bytes;
    return block;
}

static void fill_error(char *error, size_t error_size, const char *format, ...) {
    if (!error || !error_size) return;
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(error, error_size, format, arguments);
    va_end(arguments);
}

h3_gpu *qw_gpu_create_on_device(int device, char *error, size_t error_size) {
    int count = 0;
    cudaError_t code = cudaGetDeviceCount(&count);
    if (code != cudaSuccess || count <= 0) {
        fill_error(error, error_size, "no CUDA device: %s (this library has no CPU path)",
                   code == cudaSuccess ? "device count is 0" : cudaGetErrorString(code));
        cudaGetLastError();
        return NULL;
    }
    if (device < 0 || device >= count) {
        fill_error(error, error_size, "CUDA device %d out of range (0..%d)", device, count - 1);
        return NULL;
    }
    int cc = qwcu_device_cc(device);
    if (cc / 10 != 10) {
        fill_error(error, error_size,
                   "CUDA device %d has compute capability %d.%d; the kernels are built for "
                   "sm_100a only",
                   device, cc / 10, cc % 10);
        return NULL;
    }
    h3_gpu *gpu = calloc(1, sizeof(*gpu));
    if (!gpu) {
        fill_error(error, error_size, "out of host memory");
        return NULL;
    }
    gpu->device = device;
    const char *step = "cudaSetDevice";
    code = cudaSetDevice(device);
    if (code == cudaSuccess) {
        step = "cudaStreamCreate";
        code = cudaStreamCreateWithFlags(&gpu->stream, cudaStreamNonBlocking);
    }
    if (code == cudaSuccess) {
        step = "cudaEventCreate";
        code = cudaEventCreate(&gpu->chain_start);
        if (code == cudaSuccess) code = cudaEventCreate(&gpu->chain_stop);
    }
    if (code == cudaSuccess) {
        step = "status allocation";
        code = cudaMalloc((void **)&gpu->status_dev, QWCU_STATUS_WORDS * sizeof(uint32_t));
        if (code == cudaSuccess)
            code = cudaMemset(gpu->status_dev, 0, QWCU_STATUS_WORDS * sizeof(uint32_t));
        if (code == cudaSuccess)
            code = cudaMallocHost((void **)&gpu->status_host, QWCU_STATUS_WORDS * sizeof(uint32_t));
    }
    if (code != cudaSuccess) {
        fill_error(error, error_size, "%s: %s", step, cudaGetErrorString(code));
        h3_gpu_free(gpu);
        return NULL;
    }
    const char *kernel = getenv("QW_CUDA_ATTN");
    gpu->attn_kernel = kernel && !strcmp(kernel, "scalar") ? QW_ATTN_SCALAR : QW_ATTN_SM100;
    return gpu;
}

/* reference h3_gpu.m:380-576 */
h3_gpu *h3_gpu_create(const char *shader_source_path, char *error, size_t error_size) {
    (void)shader_source_path;
    int device = 0;
    const char *choice = getenv("QW_CUDA_DEVICE");
    if (choice && *choice) {
        device = atoi(choice);
    } else if (cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
        device = 0;
    }
    return qw_gpu_create_on_device(device, error, error_size);
}

/* reference h3_gpu.m:578-579 (NULL-safe) */
void h3_gpu_free(h3_gpu *gpu) {
    if (!gpu) return;
    cudaSetDevice(gpu->device);
    if (gpu->stream) cudaStreamSynchronize(gpu->stream);
    if (gpu->scratch) cudaFree(gpu->scratch);
    if (gpu->status_dev) cudaFree(gpu->status_dev);
    if (gpu->status_host) cudaFreeHost(gpu->status_host);
    if (gpu->chain_start) cudaEventDestroy(gpu->chain_start);
    if (gpu->chain_stop) cudaEventDestroy(gpu->chain_stop);
    if (gpu->aux_joined) cudaEventDestroy(gpu->aux_joined);
    if (gpu->lane_event) cudaEventDestroy(gpu->lane_event);
    for (int lane = 1; lane < 3; lane++)
        if (gpu->lane[lane]) cudaStreamDestroy(gpu->lane[lane]);
    if (gpu->stream) cudaStreamDestroy(gpu->stream);
    cudaGetLastError();
    free(gpu);
}

int qw_gpu_device(const h3_gpu *gpu) { return gpu ? gpu->device : -1; }
void *qw_gpu_stream(const h3_gpu *gpu) { return gpu ? (void *)gpu->stream : NULL; }
uint64_t qw_gpu_kernel_launches(const h3_gpu *gpu) { return gpu ? gpu->kernel_launches : 0; }

int qw_gpu_set_attention_kernel(h3_gpu *gpu, const char *name) {
    if (!gpu || !name) return 0;
    if (!strcmp(name, "sm100")) gpu->attn_kernel = QW_ATTN_SM100;
    else if (!strcmp(name, "sm100-whole")) gpu->attn_kernel = QW_ATTN_SM100_WHOLE;
    else if (!strcmp(name, "sm100-row")) gpu->attn_kernel = QW_ATTN_SM100_ROW;
    else if (!strcmp(name, "scalar")) gpu->attn_kernel = QW_ATTN_SCALAR;
    else {
        qw_set_error(gpu, "unknown attention kernel '%s'", name);
        return 0;
    }
    return 1;
}

int h3_gpu_is_m5(const h3_gpu *gpu) { (void)gpu; return 0; }
int h3_gpu_has_nax_mlp(const h3_gpu *gpu) { (void)gpu; return 0; }
int h3_gpu_has_int8_mlp(const h3_gpu *gpu) { (void)gpu; return 0; }
void h3_gpu_clear_graph_cache(h3_gpu *gpu) { (void)gpu; }
void h3_gpu_profile_set_label(h3_gpu *gpu, const char *label) { (void)gpu; (void)label; }
void h3_gpu_profile_mark(h3_gpu *gpu, const char *phase) { (void)gpu; (void)phase; }

/* ---- tensors (reference h3_gpu.m:621-647, 887-973) ---------------------- */

static h3_gpu_tensor *tensor_new(h3_gpu *gpu, h3_gpu_dtype dtype, size_t elements,
                                 const void *values) {
    if (!gpu || !elements || !qw_bind(gpu)) return NULL;
    size_t size = qw_dtype_size(dtype);
    if (elements > SIZE_MAX / size) return NULL;
    h3_gpu_tensor *tensor = calloc(1, sizeof(*tensor));
    if (!tensor) return NULL;
    tensor->owner = gpu;
    tensor->dtype = dtype;
    tensor->elements = elements;
    tensor->bytes = elements * size;
    if (cudaMalloc(&tensor->dev, tensor->bytes) != cudaSuccess) {
        qw_set_error(gpu, "cannot allocate %zu bytes of device memory", tensor->bytes);
        cudaGetLastError();
        free(tensor);
        return NULL;
    }
    cudaError_t code = values
        ? cudaMemcpyAsync(tensor->dev, values, tensor->bytes, cudaMemcpyHostToDevice, gpu->stream)
        : cudaMemsetAsync(tensor->dev, 0, tensor->bytes, gpu->stream);
    if (code != cudaSuccess) {
        cudaGetLastError();
        cudaFree(tensor->dev);
        free(tensor);
        return NULL;
    }
    gpu->stats.allocated_bytes += tensor->bytes;
    gpu->stats.live_bytes += tensor->bytes;
    if (gpu->stats.live_bytes > gpu->stats.peak_live_bytes)
        gpu->stats.peak_live_bytes = gpu->stats.live_bytes;
    gpu->stats.tensor_allocations++;
    return tensor;
}

h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *gpu, size_t elements) {
    return tensor_new(gpu, H3_GPU_F32, elements, NULL);
}
h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t elements) {
    return tensor_new(gpu, H3_GPU_BF16, elements, NULL);
}
h3_gpu_tensor *h3_gpu_tensor_new_i8(h3_gpu *gpu, size_t elements) {
    return tensor_new(gpu, H3_GPU_I8, elements, NULL);
}
h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *gpu, const float *values, size_t elements) {
    return values ? tensor_new(gpu, H3_GPU_F32, elements, values) : NULL;
}
h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *gpu, const uint16_t *values, size_t elements) {
    return values ? tensor_new(gpu, H3_GPU_BF16, elements, values) : NULL;
}
h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *values, size_t elements) {
    return values ? tensor_new(gpu, H3_GPU_U32, elements, values) : NULL;
}

void h3_gpu_tensor_free(h3_gpu_tensor *tensor) {
    if (!tensor) return;
    h3_gpu *gpu = tensor->owner;
    if (gpu) {
        qw_bind(gpu);
        gpu->stats.live_bytes =
            gpu->stats.live_bytes >= tensor->bytes ? gpu->stats.live_bytes - tensor->bytes : 0;
        /* Enqueued work may still use the buffer (the reference's command buffer
         * retains it): free in stream order. */
        if (cudaFreeAsync(tensor->dev, gpu->stream) != cudaSuccess) {
            cudaGetLastError();
            cudaStreamSynchronize(gpu->stream);
            cudaFree(tensor->dev);
        }
    }
    free(tensor);
}

size_t h3_gpu_tensor_elements(const h3_gpu_tensor *tensor) {
    return tensor ? tensor->elements : 0;
}

h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *tensor) {
    return tensor ? tensor->dtype : H3_GPU_F32;
}

void *qw_gpu_tensor_device_ptr(const h3_gpu_tensor *tensor) {
    return tensor ? tensor->dev : NULL;
}

static int tensor_read(const h3_gpu_tensor *tensor, h3_gpu_dtype dtype, size_t offset,
                       void *values, size_t elements) {
    if (!tensor || !values || tensor->dtype != dtype || offset > tensor->elements ||
        elements > tensor->elements - offset)
        return 0;
    h3_gpu *gpu = tensor->owner;
    if (!qw_bind(gpu)) return 0;
    size_t size = qw_dtype_size(dtype);
    if (!elements) return 1;
    if (cudaMemcpyAsync(values, (const char *)tensor->dev + offset * size, elements * size,
                        cudaMemcpyDeviceToHost, gpu->stream) != cudaSuccess ||
        cudaStreamSynchronize(gpu->stream) != cudaSuccess) {
        qw_set_error(gpu, "tensor read failed: %s", cudaGetErrorString(cudaGetLastError()));
        return 0;
    }
    return 1;
}

static int tensor_write(h3_gpu_tensor *tensor, h3_gpu_dtype dtype, size_t offset,
                        const void *values, size_t elements) {
    if (!tensor || !values || tensor->dtype != dtype || offset > tensor->elements ||
        elements > tensor->elements - offset)
        return 0;
    h3_gpu *gpu = tensor->owner;
    if (!qw_bind(gpu)) return 0;
    size_t size = qw_dtype_size(dtype);
    if (!elements) return 1;
    if (cudaMemcpyAsync((char *)tensor->dev + offset * size, values, elements * size,
                        cudaMemcpyHostToDevice, gpu->stream) != cudaSuccess) {
        qw_set_error(gpu, "tensor write failed: %s", cudaGetErrorString(cudaGetLastError()));
        return 0;
    }
    return 1;
}

int h3_gpu_tensor_read_f32(const h3_gpu_tensor *tensor, float *values, size_t elements) {
    return tensor_read(tensor, H3_GPU_F32, 0, values, elements);
}
int h3_gpu_tensor_read_f32_range(const h3_gpu_tensor *tensor, size_t source_offset,
                                 float *values, size_t elements) {
    return tensor_read(tensor, H3_GPU_F32, source_offset, values, elements);
}
int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *tensor, uint16_t *values, size_t elements) {
    return tensor_read(tensor, H3_GPU_BF16, 0, values, elements);
}
int h3_gpu_tensor_write_f32(h3_gpu_tensor *tensor, const float *values, size_t elements) {
    return tensor_write(tensor, H3_GPU_F32, 0, values, elements);
}
int h3_gpu_tensor_write_f32_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                  const float *values, size_t elements) {
    return tensor_write(tensor, H3_GPU_F32, destination_offset, values, elements);
}
int h3_gpu_tensor_write_bf16(h3_gpu_tensor *tensor, const uint16_t *values, size_t elements) {
    return tensor_write(tensor, H3_GPU_BF16, 0, values, elements);
}
int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                   const uint16_t *values, size_t elements) {
    return tensor_write(tensor, H3_GPU_BF16, destination_offset, values, elements);
}

int qw_gpu_tensor_read_async(h3_gpu *gpu, const h3_gpu_tensor *tensor, void *host,
                             size_t elements) {
    if (!gpu || !tensor || !host || elements > tensor->elements || !qw_bind(gpu)) return 0;
    return qw_cuda_ok(gpu,
                      cudaMemcpyAsync(host, tensor->dev, elements * qw_dtype_size(tensor->dtype),
                                      cudaMemcpyDeviceToHost, gpu->stream),
                      "asynchronous tensor read");
}

/* Exercise of the attention kernel's bounded waits (tests): the next launches
 * run with a wait budget of `wait_cycles` SM cycles and their producer leaves out
 * every key tile from visited tile `withhold_from_tile` (>= 1) on, so the waits
 * behind it run out: the kernel records where, exits cleanly and h3_gpu_submit
 * returns 0 with the message.  (0, 0) restores normal operation. */
int qw_gpu_debug_attention_waits(h3_gpu *gpu, long long wait_cycles, int withhold_from_tile) {
    if (!gpu || wait_cycles < 0 || withhold_from_tile < 0) return 0;
    gpu->attn_wait_cycles = wait_cycles;
    gpu->attn_withhold_tile = withhold_from_tile;
    return 1;
}

/* ---- copy lanes (no counterpart in the reference) -------------------------
 * A host program that streams inputs in and results out overlaps three things:
 * the upload of the next layer, the compute of this one, the read-back of the
 * last.  Lane 0 is the context's stream (every op runs there); lanes 1 and 2 are
 * two more streams that only carry copies.  qw_gpu_fence(from, to) orders
 * everything enqueued on `from` so far before whatever is enqueued on `to` next.
 * Host buffers must be pinned (qw_gpu_host_alloc) and stay valid until the next
 * h3_gpu_submit, which waits for all lanes. */
#define QW_LANES 3
static cudaStream_t lane_stream(h3_gpu *gpu, int lane) {
    if (lane < 0 || lane >= QW_LANES) return NULL;
    if (lane == 0) return gpu->stream;
    if (!gpu->lane[lane] &&
        cudaStreamCreateWithFlags(&gpu->lane[lane], cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        gpu->lane[lane] = NULL;
    }
    return gpu->lane[lane];
}

int qw_gpu_fence(h3_gpu *gpu, int from_lane, int to_lane) {
    if (!gpu || !qw_bind(gpu)) return 0;
    if (gpu->capturing) {
        qw_set_error(gpu, "copy lanes cannot be used inside a graph capture");
        return 0;
    }
    cudaStream_t from = lane_stream(gpu, from_lane), to = lane_stream(gpu, to_lane);
    if (!from || !to) {
        qw_set_error(gpu, "fence: no such lane (0..%d)", QW_LANES - 1);
        return 0;
    }
    if (from == to) return 1;
    /* One event per fence call would leak; a single event re-recorded is fine:
     * cudaStreamWaitEvent captures the record that is current when it is called. */
    if (!gpu->lane_event &&
        !qw_cuda_ok(gpu, cudaEventCreateWithFlags(&gpu->lane_event, cudaEventDisableTiming),
                    "fence event"))
        return 0;
    return qw_cuda_ok(gpu, cudaEventRecord(gpu->lane_event, from), "fence record") &&
           qw_cuda_ok(gpu, cudaStreamWaitEvent(to, gpu->lane_event, 0), "fence wait");
}

static int lane_copy(h3_gpu *gpu, const h3_gpu_tensor *tensor, void *host, size_t elements,
                     int lane, int to_device) {
    if (!gpu || !tensor || !host || tensor->owner != gpu || elements > tensor->elements ||
        !qw_bind(gpu))
        return 0;
    if (gpu->capturing) {
        qw_set_error(gpu, "copy lanes cannot be used inside a graph capture");
        return 0;
    }
    cudaStream_t stream = lane_stream(gpu, lane);
    if (!stream) {
        qw_set_error(gpu, "lane copy: no such lane (0..%d)", QW_LANES - 1);
        return 0;
    }
    size_t bytes = elements * qw_dtype_size(tensor->dtype);
    return qw_cuda_ok(gpu,
                      to_device ? cudaMemcpyAsync(tensor->dev, host, bytes, cudaMemcpyHostToDevice,
                                                  stream)
                                : cudaMemcpyAsync(host, tensor->dev, bytes, cudaMemcpyDeviceToHost,
                                                  stream),
                      to_device ? "lane upload" : "lane read-back");
}

int qw_gpu_tensor_write_lane(h3_gpu *gpu, h3_gpu_tensor *tensor, const void *host,
                             size_t elements, int lane) {
    return lane_copy(gpu, tensor, (void *)host, elements, lane, 1);
}

int qw_gpu_tensor_read_lane(h3_gpu *gpu, const h3_gpu_tensor *tensor, void *host,
                            size_t elements, int lane) {
    return lane_copy(gpu, tensor, host, elements, lane, 0);
}

void *qw_gpu_host_alloc(size_t bytes) {
    void *pointer = NULL;
    if (!bytes || cudaMallocHost(&pointer, bytes) != cudaSuccess) {
        cudaGetLastError();
        return NULL;
    }
    return pointer;
}

void qw_gpu_host_free(void *pointer) {
    if (pointer) cudaFreeHost(pointer);
}

/* ---- command chain (reference h3_gpu.m:975-1047) ------------------------ */

int h3_gpu_begin(h3_gpu *gpu) {
    if (!gpu || gpu->chain_open || !qw_bind(gpu)) return 0;
    gpu->error[0] = 0;
    gpu->chain_failed = 0;
    if (!qw_cuda_ok(gpu, cudaEventRecord(gpu->chain_start, gpu->stream), "begin")) return 0;
    gpu->chain_open = 1;
    gpu->chain_start_wall = qw_now();
    return 1;
}

int h3_gpu_continue(h3_gpu *gpu) {
    if (!gpu || !gpu->chain_open) return 0;
    gpu->stats.submissions++;
    return 1;
}

int h3_gpu_submit(h3_gpu *gpu) {
    if (!gpu || !gpu->chain_open || !qw_bind(gpu)) return 0;
    if (gpu->capturing) {
        qw_set_error(gpu, "h3_gpu_submit() inside a graph capture; call qw_gpu_graph_end() first");
        return 0;
    }
    gpu->chain_open = 0;
    double commit_time = qw_now();
    if (gpu->aux_stream) {
        /* Work a multi-GPU group put on its communication stream belongs to the
         * chain: join it before the stop event. */
        if (!gpu->aux_joined) cudaEventCreateWithFlags(&gpu->aux_joined, cudaEventDisableTiming);
        if (gpu->aux_joined && cudaEventRecord(gpu->aux_joined, gpu->aux_stream) == cudaSuccess)
            cudaStreamWaitEvent(gpu->stream, gpu->aux_joined, 0);
    }
    for (int lane = 1; lane < QW_LANES; lane++) /* copies on the other lanes belong to the chain */
        if (gpu->lane[lane]) qw_gpu_fence(gpu, lane, 0);
    cudaEventRecord(gpu->chain_stop, gpu->stream);
    cudaMemcpyAsync(gpu->status_host, gpu->status_dev, QWCU_STATUS_WORDS * sizeof(uint32_t),
                    cudaMemcpyDeviceToHost, gpu->stream);
    cudaError_t code = cudaStreamSynchronize(gpu->stream);
    if (code == cudaSuccess && gpu->aux_stream) code = cudaStreamSynchronize(gpu->aux_stream);
    double complete_time = qw_now();
    if (code != cudaSuccess) {
        qw_set_error(gpu, "CUDA command failed: %s", cudaGetErrorString(code));
        cudaGetLastError();
        return 0;
    }
    if (gpu->chain_failed) return 0; /* message already set by the failing launch */
    if (gpu->status_host[0] != QWCU_STATUS_OK) {
        if (gpu->status_host[0] == QWCU_STATUS_BAD_ARGUMENT)
            qw_set_error(gpu,
                         "CUDA kernel reported status %u (where 0x%x): row %u carries modulation "
                         "row index %u, outside the modulation tensor; block 0 was used instead",
                         gpu->status_host[0], gpu->status_host[1], gpu->status_host[2],
                         gpu->status_host[3]);
        else
            qw_set_error(gpu,
                         "CUDA kernel reported status %u (where 0x%x, tile %u, block 0x%x): a "
                         "bounded device-side wait ran out",
                         gpu->status_host[0], gpu->status_host[1], gpu->status_host[2],
                         gpu->status_host[3]);
        cudaMemsetAsync(gpu->status_dev, 0, QWCU_STATUS_WORDS * sizeof(uint32_t), gpu->stream);
        return 0;
    }
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, gpu->chain_start, gpu->chain_stop) == cudaSuccess)
        gpu->stats.gpu_seconds += (double)ms * 1e-3;
    else
        cudaGetLastError();
    gpu->stats.submissions++;
    gpu->stats.command_encode_seconds += commit_time - gpu->chain_start_wall;
    gpu->stats.command_wait_seconds += complete_time - commit_time;
    return 1;
}

/* ---- replayable graphs (no counterpart in the reference) ------------------
 * The ops enqueued between begin and end are captured instead of run; the graph
 * replays them with one launch, which takes the per-op host cost out of short
 * layers (at 8 GPUs a layer is ~70 us of device time). */
int qw_gpu_graph_begin(h3_gpu *gpu) {
    if (!qw_require_command(gpu) || !qw_bind(gpu)) return 0;
    if (gpu->capturing) {
        qw_set_error(gpu, "graph capture is already active");
        return 0;
    }
    if (!qw_cuda_ok(gpu, cudaStreamBeginCapture(gpu->stream, cudaStreamCaptureModeRelaxed),
                    "graph capture begin"))
        return 0;
    gpu->capturing = 1;
    gpu->capture_seq++;
    gpu->capture_launches = 0;
    return 1;
}

qw_gpu_graph *qw_gpu_graph_end(h3_gpu *gpu) {
    if (!gpu || !gpu->capturing || !qw_bind(gpu)) return NULL;
    /* Join the communication stream back into the capture, if this capture forked
     * into it at all (a capturing stream must not wait on an event of a stream that
     * is not part of the capture). */
    enum cudaStreamCaptureStatus aux_status = cudaStreamCaptureStatusNone;
    if (gpu->aux_stream && cudaStreamIsCapturing(gpu->aux_stream, &aux_status) == cudaSuccess &&
        aux_status == cudaStreamCaptureStatusActive) {
        if (!gpu->aux_joined) cudaEventCreateWithFlags(&gpu->aux_joined, cudaEventDisableTiming);
        if (gpu->aux_joined && cudaEventRecord(gpu->aux_joined, gpu->aux_stream) == cudaSuccess)
            cudaStreamWaitEvent(gpu->stream, gpu->aux_joined, 0);
    }
    cudaGraph_t graph = NULL;
    cudaError_t code = cudaStreamEndCapture(gpu->stream, &graph);
    gpu->capturing = 0;
    if (code != cudaSuccess || !graph) {
        qw_set_error(gpu, "graph capture end: %s", cudaGetErrorString(code));
        cudaGetLastError();
        return NULL;
    }
    qw_gpu_graph *handle = calloc(1, sizeof(*handle));
    if (handle) code = cudaGraphInstantiate(&handle->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (!handle || code != cudaSuccess) {
        qw_set_error(gpu, "graph instantiate: %s", cudaGetErrorString(code));
        cudaGetLastError();
        free(handle);
        return NULL;
    }
    handle->owner = gpu;
    handle->kernel_launches = gpu->capture_launches;
    return handle;
}

int qw_gpu_graph_launch(h3_gpu *gpu, qw_gpu_graph *graph) {
    if (!qw_require_command(gpu) || !qw_bind(gpu)) return 0;
    if (!graph || graph->owner != gpu || gpu->capturing) {
        qw_set_error(gpu, "graph launch: no graph of this context");
        return 0;
    }
    if (!qw_cuda_ok(gpu, cudaGraphLaunch(graph->exec, gpu->stream), "graph launch")) {
        gpu->chain_failed = 1;
        return 0;
    }
    gpu->stats.direct_dispatches += graph->kernel_launches;
    gpu->kernel_launches += graph->kernel_launches;
    return 1;
}

void qw_gpu_graph_free(qw_gpu_graph *graph) {
    if (!graph) return;
    if (graph->owner) qw_bind(graph->owner);
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    free(graph);
}

/* reference h3_gpu.m:1049-1053 */
const char *h3_gpu_error(const h3_gpu *gpu) {
    return gpu && gpu->error[0] ? gpu->error : "unknown CUDA error";
}

/* reference h3_gpu.m:1055-1059 */
int h3_gpu_get_stats(const h3_gpu *gpu, h3_gpu_stats *stats) {
    if (!gpu || !stats) return 0;
    *stats = gpu->stats;
    return 1;
}

/* ---- range copies (reference h3_gpu.m:1384-1444) ------------------------ */

static int copy_range(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                      const h3_gpu_tensor *source, size_t source_offset, size_t elements,
                      h3_gpu_dtype dtype, const char *name) {
    size_t size = qw_dtype_size(dtype);
    if (!qw_require_command(gpu)) return 0;
    if (!destination || !source || destination->dtype != dtype || source->dtype != dtype ||
        source_offset > source->elements || elements > source->elements - source_offset ||
        destination_offset > destination->elements ||
        elements > destination->elements - destination_offset || elements > SIZE_MAX / size) {
        qw_set_error(gpu, "invalid %s blit range", name);
        return 0;
    }
    if (!qw_bind(gpu)) return 0;
    if (elements &&
        !qw_cuda_ok(gpu,
                    cudaMemcpyAsync((char *)destination->dev + destination_offset * size,
                                    (const char *)source->dev + source_offset * size,
                                    elements * size, cudaMemcpyDeviceToDevice, gpu->stream),
                    "blit copy"))
        return 0;
    gpu->stats.blit_copies++;
    return 1;
}

int h3_gpu_copy_bf16(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                     const h3_gpu_tensor *source, size_t source_offset, size_t elements) {
    return copy_range(gpu, destination, destination_offset, source, source_offset, elements,
                      H3_GPU_BF16, "BF16");
}

int h3_gpu_copy_f32(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                    const h3_gpu_tensor *source, size_t source_offset, size_t elements) {
    return copy_range(gpu, destination, destination_offset, source, source_offset, elements,
                      H3_GPU_F32, "F32");
}
