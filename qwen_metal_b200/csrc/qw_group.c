/* Multi-GPU group: one process per GPU.  The ranks form batch_groups x
 * head_groups: a batch group owns some of the batch items (the two branches of
 * classifier-free guidance, which the reference runs as two separate forwards:
 * qwen_pipeline.m:376-381, :396-401), inside it the attention heads are sharded
 * and only the per-layer [rows, heads*128] output is gathered over NVLink, by
 * this library's own push kernel (cuda/qw_push.cu) or, for comparison, by NCCL.
 *
 * NCCL is bound at run time (dlopen of libnccl.so.2) so the library loads on a
 * machine without it and shares the copy a host program already loaded.  The
 * reference has no counterpart: it is a single-device engine.
 */
#define _GNU_SOURCE
#include "qw_internal.h"

#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct ncclComm *nccl_comm_t;
typedef struct { char internal[QW_GPU_GROUP_ID_BYTES]; } nccl_unique_id;
enum { NCCL_UINT8 = 1, NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9 }; /* ncclDataType_t values */
enum { NCCL_SUM = 0 };                                      /* ncclRedOp_t */

typedef int (*nccl_get_unique_id_fn)(nccl_unique_id *);
typedef int (*nccl_comm_init_rank_fn)(nccl_comm_t *, int, nccl_unique_id, int);
typedef int (*nccl_comm_destroy_fn)(nccl_comm_t);
typedef int (*nccl_all_gather_fn)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t);
typedef int (*nccl_all_reduce_fn)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t);
typedef const char *(*nccl_get_error_string_fn)(int);

static struct {
    void *handle;
    nccl_get_unique_id_fn get_unique_id;
    nccl_comm_init_rank_fn comm_init_rank;
    nccl_comm_destroy_fn comm_destroy;
    nccl_all_gather_fn all_gather;
    nccl_all_reduce_fn all_reduce;
    nccl_get_error_string_fn get_error_string;
} g_nccl;

static int nccl_bind(char *error, size_t error_size) {
    if (g_nccl.handle) return 1;
    const char *names[] = {getenv("QW_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    void *handle = NULL;
    for (size_t i = 0; i < sizeof(names) / sizeof(names[0]) && !handle; i++)
        if (names[i] && *names[i]) handle = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!handle) {
        if (error && error_size) snprintf(error, error_size, "cannot load NCCL: %s", dlerror());
        return 0;
    }
    g_nccl.get_unique_id = (nccl_get_unique_id_fn)dlsym(handle, "ncclGetUniqueId");
    g_nccl.comm_init_rank = (nccl_comm_init_rank_fn)dlsym(handle, "ncclCommInitRank");
    g_nccl.comm_destroy = (nccl_comm_destroy_fn)dlsym(handle, "ncclCommDestroy");
    g_nccl.all_gather = (nccl_all_gather_fn)dlsym(handle, "ncclAllGather");
    g_nccl.all_reduce = (nccl_all_reduce_fn)dlsym(handle, "ncclAllReduce");
    g_nccl.get_error_string = (nccl_get_error_string_fn)dlsym(handle, "ncclGetErrorString");
    if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.comm_destroy ||
        !g_nccl.all_gather || !g_nccl.all_reduce || !g_nccl.get_error_string) {
        if (error && error_size) snprintf(error, error_size, "NCCL library lacks a required symbol");
        dlclose(handle);
        memset(&g_nccl, 0, sizeof(g_nccl));
        return 0;
    }
    g_nccl.handle = handle;
    return 1;
}

#define QW_GROUP_MAX_WORLD 8
#define QW_IPC_HANDLE_BYTES 64
#define QW_GROUP_MAX_BOUND 4

/* Flag block of a rank (uint32 words, peer-mapped on every rank):
 *   [0, 4)    slot_use[slot]   epoch counter, incremented by the attention kernel
 *   [4, 8)    arrivals[slot]   CTA counter of the push kernel
 *   [8, 40)   freed[slot][r]   written by rank r: its slot may be stored into
 *   [40, 72)  ready[slot][r]   written by rank r: its columns have landed here */
#define QW_SYNC_WORDS 128
#define QW_SYNC_BLOCK_BYTES ((size_t)4 << 20)
#define QW_SYNC_USE(slot) (slot)
#define QW_SYNC_ARRIVALS(slot) (4 + (slot))
#define QW_SYNC_FREED(slot, r) (8 + (slot) * QW_GROUP_MAX_WORLD + (r))
#define QW_SYNC_READY(slot, r) (40 + (slot) * QW_GROUP_MAX_WORLD + (r))

struct qw_gpu_group {
    h3_gpu *gpu;
    nccl_comm_t comm;
    int rank, world;
    /* rank = batch_index * head_groups + head_index; peers = the other ranks of
     * this rank's batch group, the only ones it exchanges output columns with. */
    int batch_groups, head_groups, batch_index, head_index;
    int peers[QW_GROUP_MAX_WORLD], n_peers;
    void *staging; /* [world][rows][slice] landing zone of the NCCL collective */
    size_t staging_bytes;
    int sm_count;
    unsigned char *exchange; /* device: world * 64-byte IPC handles, then one float */
    uint32_t *sync_peer[QW_GROUP_MAX_WORLD]; /* every rank's flag block ([rank] = own) */
    /* Up to QW_GROUP_MAX_BOUND outputs can be bound at once; a layer's gather runs
     * under the next layer's compute, so consecutive layers alternate between two. */
    h3_gpu_tensor *bound[QW_GROUP_MAX_BOUND];
    void *peer_out[QW_GROUP_MAX_BOUND][QW_GROUP_MAX_WORLD];
    /* The push runs on its own stream; slot_done[b] marks the end of the last one
     * that covered bound output b (all ranks' columns present). */
    cudaStream_t comm_stream;
    cudaEvent_t kernel_done;
    cudaEvent_t slot_done[QW_GROUP_MAX_BOUND];
    int slot_pending[QW_GROUP_MAX_BOUND];
    uint32_t slot_capture[QW_GROUP_MAX_BOUND]; /* capture the slot's event belongs to (0 = none) */
    uint32_t push_blocks, wait_ms;
    int push_copy_engine; /* QW_CUDA_GROUP_PUSH=ce: copy engines move the bytes */
};

static void group_layout(qw_gpu_group *group, int batch_groups) {
    group->batch_groups = batch_groups;
    group->head_groups = group->world / batch_groups;
    group->batch_index = group->rank / group->head_groups;
    group->head_index = group->rank % group->head_groups;
    group->n_peers = 0;
    for (int k = 0; k < group->head_groups; k++)
        if (k != group->head_index)
            group->peers[group->n_peers++] = group->batch_index * group->head_groups + k;
}

/* Collective: every rank contributes the device allocation `mine`; on return
 * peers[r] is rank r's allocation mapped into this process (CUDA IPC over the
 * NVLink peer path), peers[rank] = mine.  The handles travel through the group's
 * NCCL communicator. */
static int exchange_and_open(qw_gpu_group *group, void *mine, void **peers, const char *what) {
    h3_gpu *gpu = group->gpu;
    cudaIpcMemHandle_t handle;
    if (!qw_cuda_ok(gpu, cudaIpcGetMemHandle(&handle, mine), "cudaIpcGetMemHandle")) return 0;
    unsigned char host[QW_GROUP_MAX_WORLD * QW_IPC_HANDLE_BYTES];
    unsigned char *slot = group->exchange + (size_t)group->rank * QW_IPC_HANDLE_BYTES;
    if (!qw_cuda_ok(gpu, cudaMemcpyAsync(slot, &handle, QW_IPC_HANDLE_BYTES, cudaMemcpyHostToDevice,
                                         gpu->stream), "handle upload"))
        return 0;
    int rc = g_nccl.all_gather(slot, group->exchange, QW_IPC_HANDLE_BYTES, NCCL_UINT8, group->comm,
                               gpu->stream);
    if (rc) {
        qw_set_error(gpu, "ncclAllGather (%s handles): %s", what, g_nccl.get_error_string(rc));
        return 0;
    }
    if (!qw_cuda_ok(gpu, cudaMemcpyAsync(host, group->exchange,
                                         (size_t)group->world * QW_IPC_HANDLE_BYTES,
                                         cudaMemcpyDeviceToHost, gpu->stream), "handle download") ||
        !qw_cuda_ok(gpu, cudaStreamSynchronize(gpu->stream), "handle exchange"))
        return 0;
    for (int r = 0; r < group->world; r++) {
        if (r == group->rank) {
            peers[r] = mine;
            continue;
        }
        cudaIpcMemHandle_t theirs;
        memcpy(&theirs, host + (size_t)r * QW_IPC_HANDLE_BYTES, QW_IPC_HANDLE_BYTES);
        if (!qw_cuda_ok(gpu, cudaIpcOpenMemHandle(&peers[r], theirs, cudaIpcMemLazyEnablePeerAccess),
                        "cudaIpcOpenMemHandle"))
            return 0;
    }
    return 1;
}

int qw_gpu_group_new_id(void *id_bytes, char *error, size_t error_size) {
    if (!id_bytes || !nccl_bind(error, error_size)) return 0;
    nccl_unique_id id;
    int rc = g_nccl.get_unique_id(&id);
    if (rc) {
        if (error && error_size)
            snprintf(error, error_size, "ncclGetUniqueId: %s", g_nccl.get_error_string(rc));
        return 0;
    }
    memcpy(id_bytes, &id, sizeof(id));
    return 1;
}

static uint32_t env_u32(const char *name, uint32_t fallback) {
    const char *text = getenv(name);
    if (!text || !*text) return fallback;
    long value = strtol(text, NULL, 10);
    return value > 0 && value < 1000000 ? (uint32_t)value : fallback;
}

qw_gpu_group *qw_gpu_group_join(h3_gpu *gpu, const void *id_bytes, int rank, int world,
                                char *error, size_t error_size) {
    if (!gpu || !id_bytes || world < 1 || world > QW_GROUP_MAX_WORLD || rank < 0 ||
        rank >= world) {
        if (error && error_size)
            snprintf(error, error_size, "group: bad arguments (1 to %d ranks)", QW_GROUP_MAX_WORLD);
        return NULL;
    }
    if (!nccl_bind(error, error_size) || !qw_bind(gpu)) return NULL;
    qw_gpu_group *group = calloc(1, sizeof(*group));
    if (!group) return NULL;
    group->gpu = gpu;
    group->rank = rank;
    group->world = world;
    group->sm_count = qwcu_device_sm_count(gpu->device);
    /* CTAs of the push kernel and the budget of its flag waits (tuning / tests). */
    group->push_blocks = env_u32("QW_CUDA_GROUP_PUSH_BLOCKS", 0); /* 0 = by the launch shape */
    group->wait_ms = env_u32("QW_CUDA_GROUP_WAIT_MS", 2000);
    {
        const char *mode = getenv("QW_CUDA_GROUP_PUSH");
        group->push_copy_engine = mode && !strcmp(mode, "ce");
    }
    group_layout(group, 1);
    nccl_unique_id id;
    memcpy(&id, id_bytes, sizeof(id));
    int rc = g_nccl.comm_init_rank(&group->comm, world, id, rank);
    if (rc) {
        if (error && error_size)
            snprintf(error, error_size, "ncclCommInitRank: %s", g_nccl.get_error_string(rc));
        free(group);
        return NULL;
    }
    uint32_t *sync_local = NULL;
    if (cudaMalloc((void **)&group->exchange, QW_GROUP_MAX_WORLD * QW_IPC_HANDLE_BYTES + 16) !=
            cudaSuccess ||
        /* (an allocation of its own: small ones share a block, and a block can be
         * opened through IPC only once per process) */
        cudaMalloc((void **)&sync_local, QW_SYNC_BLOCK_BYTES) != cudaSuccess) {
        if (error && error_size) snprintf(error, error_size, "group: exchange buffer allocation failed");
        qw_gpu_group_free(group);
        return NULL;
    }
    group->sync_peer[rank] = sync_local;
    cudaMemset(group->exchange, 0, QW_GROUP_MAX_WORLD * QW_IPC_HANDLE_BYTES + 16);
    cudaMemset(sync_local, 0, QW_SYNC_WORDS * sizeof(uint32_t));
    /* The communication stream gets the highest priority: when SMs free up between
     * the next layer's kernels, the few CTAs of the push are placed first and finish
     * early instead of queueing behind a full wave of attention CTAs. */
    int least = 0, greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) {
        cudaGetLastError();
        greatest = 0;
    }
    int ok = cudaStreamCreateWithPriority(&group->comm_stream, cudaStreamNonBlocking, greatest) ==
                 cudaSuccess &&
             cudaEventCreateWithFlags(&group->kernel_done, cudaEventDisableTiming) == cudaSuccess;
    for (int b = 0; ok && b < QW_GROUP_MAX_BOUND; b++)
        ok = cudaEventCreateWithFlags(&group->slot_done[b], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        if (error && error_size) snprintf(error, error_size, "group: stream/event creation failed");
        qw_gpu_group_free(group);
        return NULL;
    }
    /* Every rank's flag block, mapped everywhere (collective). */
    if (world > 1 &&
        !exchange_and_open(group, sync_local, (void **)group->sync_peer, "flag block")) {
        if (error && error_size) snprintf(error, error_size, "group: %s", h3_gpu_error(gpu));
        qw_gpu_group_free(group);
        return NULL;
    }
    gpu->aux_stream = group->comm_stream;
    return group;
}

/* Split the ranks into batch_groups x (world / batch_groups) head groups; call it
 * on every rank with the same value before the first sharded attention.  With 1
 * (the default) all ranks shard the heads of every batch item. */
int qw_gpu_group_set_batch_groups(qw_gpu_group *group, int batch_groups) {
    if (!group) return 0;
    if (batch_groups < 1 || group->world % batch_groups) {
        qw_set_error(group->gpu, "group: %d ranks do not split into %d batch groups", group->world,
                     batch_groups);
        return 0;
    }
    group_layout(group, batch_groups);
    return 1;
}

int qw_gpu_group_batch_index(const qw_gpu_group *group) { return group ? group->batch_index : -1; }
int qw_gpu_group_head_index(const qw_gpu_group *group) { return group ? group->head_index : -1; }
int qw_gpu_group_head_groups(const qw_gpu_group *group) { return group ? group->head_groups : 0; }

void qw_gpu_group_free(qw_gpu_group *group) {
    if (!group) return;
    if (group->gpu) {
        qw_bind(group->gpu);
        cudaStreamSynchronize(group->gpu->stream);
        if (group->comm_stream) cudaStreamSynchronize(group->comm_stream);
        if (group->gpu->aux_stream == group->comm_stream) group->gpu->aux_stream = NULL;
    }
    if (group->kernel_done) cudaEventDestroy(group->kernel_done);
    for (int b = 0; b < QW_GROUP_MAX_BOUND; b++)
        if (group->slot_done[b]) cudaEventDestroy(group->slot_done[b]);
    if (group->comm_stream) cudaStreamDestroy(group->comm_stream);
    for (int r = 0; r < group->world && r < QW_GROUP_MAX_WORLD; r++) {
        for (int b = 0; b < QW_GROUP_MAX_BOUND; b++)
            if (group->peer_out[b][r] && r != group->rank)
                cudaIpcCloseMemHandle(group->peer_out[b][r]);
        if (group->sync_peer[r] && r != group->rank) cudaIpcCloseMemHandle(group->sync_peer[r]);
    }
    if (group->sync_peer[group->rank]) cudaFree(group->sync_peer[group->rank]);
    if (group->staging) cudaFree(group->staging);
    if (group->exchange) cudaFree(group->exchange);
    if (group->comm) g_nccl.comm_destroy(group->comm);
    free(group);
}

int qw_gpu_group_rank(const qw_gpu_group *group) { return group ? group->rank : -1; }
int qw_gpu_group_world(const qw_gpu_group *group) { return group ? group->world : 0; }

int qw_gpu_group_all_gather_heads_bf16(qw_gpu_group *group, h3_gpu_tensor *full,
                                       const h3_gpu_tensor *local, uint32_t rows,
                                       uint32_t heads_local, uint32_t head_dim) {
    if (!group) return 0;
    h3_gpu *gpu = group->gpu;
    size_t slice = (size_t)heads_local * head_dim;
    size_t local_count = (size_t)rows * slice;
    size_t full_count = local_count * (size_t)group->world;
    if (!qw_require_dtype(gpu, local, local_count, H3_GPU_BF16, "head gather input") ||
        !qw_require_dtype(gpu, full, full_count, H3_GPU_BF16, "head gather output") ||
        !qw_require_command(gpu))
        return 0;
    if (!rows || !slice || slice % 8 || slice > UINT32_MAX) {
        qw_set_error(gpu, "head gather: unsupported geometry");
        return 0;
    }
    if (group->batch_groups != 1) {
        qw_set_error(gpu, "head gather: the NCCL gather spans all ranks; it needs one batch group");
        return 0;
    }
    if (!qw_bind(gpu)) return 0;
    if (group->world == 1)
        return qw_cuda_ok(gpu,
                          cudaMemcpyAsync(full->dev, local->dev, local_count * 2,
                                          cudaMemcpyDeviceToDevice, gpu->stream),
                          "head gather copy");
    if (group->staging_bytes < full_count * 2) {
        if (gpu->capturing) {
            qw_set_error(gpu, "head gather: the landing zone must grow to %zu bytes: run the "
                              "gather once at this size before capturing it into a graph",
                         full_count * 2);
            gpu->chain_failed = 1;
            return 0;
        }
        if (group->staging) {
            cudaStreamSynchronize(gpu->stream);
            cudaFree(group->staging);
            group->staging = NULL;
            group->staging_bytes = 0;
        }
        if (!qw_cuda_ok(gpu, cudaMalloc(&group->staging, full_count * 2), "head gather staging"))
            return 0;
        group->staging_bytes = full_count * 2;
    }
    int rc = g_nccl.all_gather(local->dev, group->staging, local_count, NCCL_BFLOAT16,
                               group->comm, gpu->stream);
    if (rc) {
        qw_set_error(gpu, "ncclAllGather: %s", g_nccl.get_error_string(rc));
        gpu->chain_failed = 1;
        return 0;
    }
    rc = qwcu_interleave_launch(full->dev, group->staging, rows, (uint32_t)slice,
                                (uint32_t)group->world, group->sm_count, gpu->stream);
    qw_count_launch(gpu, rc, "head interleave");
    return rc == 0;
}

/* Map every rank's `full` output buffer into this process (CUDA IPC over the
 * NVLink peer path) so the push kernel can store this rank's head columns
 * straight into all of them.  Collective: every rank calls it with its own tensor
 * of the same size. */
int qw_gpu_group_bind_output(qw_gpu_group *group, h3_gpu_tensor *full) {
    if (!group) return 0;
    h3_gpu *gpu = group->gpu;
    if (!full || full->dtype != H3_GPU_BF16 || full->owner != gpu) {
        qw_set_error(gpu, "group bind: output tensor is absent or not BF16");
        return 0;
    }
    if (gpu->capturing) {
        qw_set_error(gpu, "group bind: not inside a graph capture");
        return 0;
    }
    if (!qw_bind(gpu)) return 0;
    int slot_index = -1;
    for (int b = 0; b < QW_GROUP_MAX_BOUND && slot_index < 0; b++)
        if (!group->bound[b]) slot_index = b;
    if (slot_index < 0) {
        qw_set_error(gpu, "group bind: at most %d outputs can be bound", QW_GROUP_MAX_BOUND);
        return 0;
    }
    if (group->world > 1) {
        if (!exchange_and_open(group, full->dev, group->peer_out[slot_index], "output")) return 0;
    } else {
        group->peer_out[slot_index][0] = full->dev;
    }
    group->bound[slot_index] = full;
    return 1;
}

/* Cross-rank barrier on the context's stream: when it completes on a rank,
 * every rank has finished the work it enqueued before its own barrier. */
int qw_gpu_group_barrier(qw_gpu_group *group) {
    if (!group) return 0;
    h3_gpu *gpu = group->gpu;
    if (!qw_require_command(gpu) || !qw_bind(gpu)) return 0;
    if (group->world == 1) return 1;
    float *word = (float *)(group->exchange + QW_GROUP_MAX_WORLD * QW_IPC_HANDLE_BYTES);
    int rc = g_nccl.all_reduce(word, word, 1, NCCL_FLOAT32, NCCL_SUM, group->comm, gpu->stream);
    if (rc) {
        qw_set_error(gpu, "ncclAllReduce (barrier): %s", g_nccl.get_error_string(rc));
        gpu->chain_failed = 1;
        return 0;
    }
    return 1;
}

/* Sharded block-causal attention with the gather behind it.  This rank computes
 * its heads_local heads of its batch group's `batch` items into head columns
 * [head_index*heads_local, +heads_local) of its own bound `full` output
 * [batch*rows, head_groups*heads_local*128]; the push kernel then copies that
 * column slice into every peer's `full` on the communication stream, under
 * whatever the context's stream runs next.  When the event behind it has passed
 * (qw_gpu_group_wait_output, or h3_gpu_submit), `full` is complete on this rank.
 * score_bound may be NULL (running-maximum softmax). */
int qw_gpu_group_attn_block_causal_bf16(qw_gpu_group *group, h3_gpu_tensor *full,
                                        const h3_gpu_tensor *query, const h3_gpu_tensor *key,
                                        const h3_gpu_tensor *value,
                                        const h3_gpu_tensor *kv_limit,
                                        const h3_gpu_tensor *score_bound, uint32_t batch,
                                        uint32_t rows, uint32_t heads_local,
                                        uint32_t kv_heads_local, uint32_t head_dim,
                                        const uint32_t *text_len, uint32_t text_pad, float scale) {
    if (!group) return 0;
    h3_gpu *gpu = group->gpu;
    int slot_index = -1;
    for (int b = 0; b < QW_GROUP_MAX_BOUND; b++)
        if (full && group->bound[b] == full) slot_index = b;
    if (slot_index < 0) {
        qw_set_error(gpu, "group attention: output is not a tensor bound with "
                          "qw_gpu_group_bind_output");
        return 0;
    }
    const uint32_t heads_total = heads_local * (uint32_t)group->head_groups;
    size_t full_count = (size_t)batch * rows * heads_total * head_dim;
    if (!qw_require_dtype(gpu, full, full_count, H3_GPU_BF16, "group attention output")) return 0;
    if (score_bound &&
        !qw_require_dtype(gpu, score_bound, 2, H3_GPU_F32, "group attention score bound"))
        return 0;
    if ((uint64_t)batch * rows > UINT32_MAX || (uint64_t)heads_total * head_dim * 2 > UINT32_MAX) {
        qw_set_error(gpu, "group attention: output too large");
        return 0;
    }
    qwcu_attn_args args;
    if (!qw_prepare_block_causal(gpu, &args, NULL, query, key, value, kv_limit, batch, rows,
                                 heads_local, kv_heads_local, head_dim, text_len, text_pad, scale))
        return 0;
    args.out = full->dev;
    args.n_out_peers = 1;
    args.out_peers[0] = full->dev;
    args.out_heads_total = heads_total;
    args.out_head_offset = heads_local * (uint32_t)group->head_index;
    args.score_bound = score_bound ? (const float *)score_bound->dev : NULL;
    uint32_t *sync_local = group->sync_peer[group->rank];
    if (group->n_peers) {
        args.slot_use = sync_local + QW_SYNC_USE(slot_index);
        args.n_freed = (uint32_t)group->n_peers;
        for (int d = 0; d < group->n_peers; d++)
            args.freed_peer[d] =
                group->sync_peer[group->peers[d]] + QW_SYNC_FREED(slot_index, group->rank);
    }
    /* The previous push out of (and the peers' pushes into) this output must be
     * over before the kernel overwrites its columns.  (An event recorded outside
     * the current graph capture belongs to work that is complete before the graph
     * can run: nothing to wait for.) */
    const uint32_t capture_now = gpu->capturing ? gpu->capture_seq : 0;
    if (group->slot_pending[slot_index] && group->slot_capture[slot_index] == capture_now &&
        !qw_cuda_ok(gpu, cudaStreamWaitEvent(gpu->stream, group->slot_done[slot_index], 0),
                    "group attention (slot wait)"))
        return 0;
    if (!qw_launch_attention(gpu, &args, "group attention")) return 0;
    if (!group->n_peers) return 1;
    if (!qw_cuda_ok(gpu, cudaEventRecord(group->kernel_done, gpu->stream), "group attention") ||
        !qw_cuda_ok(gpu, cudaStreamWaitEvent(group->comm_stream, group->kernel_done, 0),
                    "group attention"))
        return 0;
    qwcu_push_args push;
    memset(&push, 0, sizeof(push));
    push.src = full->dev;
    push.n_peers = (uint32_t)group->n_peers;
    push.my_rank = (uint32_t)group->rank;
    for (int d = 0; d < group->n_peers; d++) {
        const int peer = group->peers[d];
        push.dst[d] = group->peer_out[slot_index][peer];
        push.peer_rank[d] = (uint32_t)peer;
        push.ready_peer[d] = group->sync_peer[peer] + QW_SYNC_READY(slot_index, group->rank);
    }
    push.rows = batch * rows;
    push.row_bytes = heads_total * head_dim * 2;
    push.col_byte0 = args.out_head_offset * head_dim * 2;
    push.slice_bytes = heads_local * head_dim * 2;
    push.slot_use = sync_local + QW_SYNC_USE(slot_index);
    push.freed_local = sync_local + QW_SYNC_FREED(slot_index, 0);
    push.ready_local = sync_local + QW_SYNC_READY(slot_index, 0);
    push.arrivals = sync_local + QW_SYNC_ARRIVALS(slot_index);
    push.status = gpu->status_dev;
    push.wait_ms = group->wait_ms;
    push.max_blocks = group->push_blocks;
    if (!push.max_blocks) {
        /* The push runs beside the NEXT layer's attention and should be done well
         * before it.  A CTA of the push moves about 5.6 MB/ms over NVLink (measured:
         * 32 CTAs, 180 GB/s); the attention takes roughly waves x key tiles x 1.7 us.
         * So: enough CTAs to finish in ~70 % of that time, at least 32 (a small grid
         * that slips in as attention CTAs retire disturbs a full device least: 32
         * CTAs expose 14 us per layer at 2 GPUs, 128 expose 40).  Where the attention
         * is a single, partly filled wave (few heads per GPU) the layer is short and
         * the small grid wins as well: at 8 GPUs 32 CTAs exposed 19 us per layer, two
         * CTAs per idle SM (92) exposed 34 us. */
        uint64_t units = (uint64_t)batch * heads_local * ((rows + 255) / 256);
        uint32_t sms = group->sm_count > 0 ? (uint32_t)group->sm_count : 148u;
        double waves = (double)units / sms;
        if (waves < 1.0) waves = 1.0;
        double attention_us = waves * ((double)rows / 128.0) * 1.7;
        double bytes_out = (double)push.rows * push.slice_bytes * group->n_peers;
        double want = 1.4 * bytes_out / (attention_us * 5600.0);
        uint32_t blocks = want > 128.0 ? 128u : want < 32.0 ? 32u : (uint32_t)want;
        if (units < sms) blocks = 32u;
        push.max_blocks = blocks;
    }
    push.copy_engine = group->push_copy_engine;
    int rc = qwcu_push_launch(&push, group->comm_stream);
    qw_count_launch(gpu, rc, "head push");
    if (!rc && push.copy_engine) qw_count_launch(gpu, 0, "head push"); /* two small kernels */
    if (rc) return 0;
    if (!qw_cuda_ok(gpu, cudaEventRecord(group->slot_done[slot_index], group->comm_stream),
                    "group attention"))
        return 0;
    group->slot_pending[slot_index] = 1;
    group->slot_capture[slot_index] = capture_now;
    return 1;
}

/* Make the context's stream wait until `full` (a bound output) is complete on
 * this rank, i.e. until the push behind the last sharded attention into it has
 * seen every peer's columns land.  Call it before enqueueing a consumer of
 * `full`; h3_gpu_submit waits for every outstanding push by itself. */
int qw_gpu_group_wait_output(qw_gpu_group *group, const h3_gpu_tensor *full) {
    if (!group) return 0;
    h3_gpu *gpu = group->gpu;
    for (int b = 0; b < QW_GROUP_MAX_BOUND; b++)
        if (full && group->bound[b] == full) {
            if (!group->slot_pending[b]) return 1;
            if (group->slot_capture[b] != (gpu->capturing ? gpu->capture_seq : 0)) return 1;
            return qw_bind(gpu) &&
                   qw_cuda_ok(gpu, cudaStreamWaitEvent(gpu->stream, group->slot_done[b], 0),
                              "group wait");
        }
    qw_set_error(gpu, "group wait: output is not a tensor bound with qw_gpu_group_bind_output");
    return 0;
}
