/* Multi-GPU group: one process per GPU, attention heads sharded across ranks,
 * the per-layer [rows, heads*128] output gathered over NVLink with NCCL.
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
enum { NCCL_BFLOAT16 = 9 }; /* ncclDataType_t value of ncclBfloat16 */

typedef int (*nccl_get_unique_id_fn)(nccl_unique_id *);
typedef int (*nccl_comm_init_rank_fn)(nccl_comm_t *, int, nccl_unique_id, int);
typedef int (*nccl_comm_destroy_fn)(nccl_comm_t);
typedef int (*nccl_all_gather_fn)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t);
typedef const char *(*nccl_get_error_string_fn)(int);

static struct {
    void *handle;
    nccl_get_unique_id_fn get_unique_id;
    nccl_comm_init_rank_fn comm_init_rank;
    nccl_comm_destroy_fn comm_destroy;
    nccl_all_gather_fn all_gather;
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
    g_nccl.get_error_string = (nccl_get_error_string_fn)dlsym(handle, "ncclGetErrorString");
    if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.comm_destroy ||
        !g_nccl.all_gather || !g_nccl.get_error_string) {
        if (error && error_size) snprintf(error, error_size, "NCCL library lacks a required symbol");
        dlclose(handle);
        memset(&g_nccl, 0, sizeof(g_nccl));
        return 0;
    }
    g_nccl.handle = handle;
    return 1;
}

struct qw_gpu_group {
    h3_gpu *gpu;
    nccl_comm_t comm;
    int rank, world;
    void *staging; /* [world][rows][slice] landing zone of the collective */
    size_t staging_bytes;
    int sm_count;
};

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

qw_gpu_group *qw_gpu_group_join(h3_gpu *gpu, const void *id_bytes, int rank, int world,
                                char *error, size_t error_size) {
    if (!gpu || !id_bytes || world < 1 || rank < 0 || rank >= world) {
        if (error && error_size) snprintf(error, error_size, "group: bad arguments");
        return NULL;
    }
    if (!nccl_bind(error, error_size) || !qw_bind(gpu)) return NULL;
    qw_gpu_group *group = calloc(1, sizeof(*group));
    if (!group) return NULL;
    group->gpu = gpu;
    group->rank = rank;
    group->world = world;
    group->sm_count = qwcu_device_sm_count(gpu->device);
    nccl_unique_id id;
    memcpy(&id, id_bytes, sizeof(id));
    int rc = g_nccl.comm_init_rank(&group->comm, world, id, rank);
    if (rc) {
        if (error && error_size)
            snprintf(error, error_size, "ncclCommInitRank: %s", g_nccl.get_error_string(rc));
        free(group);
        return NULL;
    }
    return group;
}

void qw_gpu_group_free(qw_gpu_group *group) {
    if (!group) return;
    if (group->gpu) {
        qw_bind(group->gpu);
        cudaStreamSynchronize(group->gpu->stream);
    }
    if (group->staging) cudaFree(group->staging);
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
    if (!qw_bind(gpu)) return 0;
    if (group->world == 1)
        return qw_cuda_ok(gpu,
                          cudaMemcpyAsync(full->dev, local->dev, local_count * 2,
                                          cudaMemcpyDeviceToDevice, gpu->stream),
                          "head gather copy");
    if (group->staging_bytes < full_count * 2) {
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
