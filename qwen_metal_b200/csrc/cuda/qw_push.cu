// Per-layer gather of the head-sharded attention output over NVLink, and the
// cross-GPU hand-shake that goes with it.
//
// Every rank of a head group computes its heads into its own columns of its own
// full [rows, heads_total*128] output.  This kernel then copies that column slice
// into the same place of every peer's output (plain 16-byte loads from local
// memory, plain 16-byte stores to peer-mapped memory) and exchanges two kinds of
// flag words with the peers, all epochs of one counter per output slot:
//
//   freed[slot][r]  written by rank r at the START of its attention kernel for
//                   this slot: "whatever read my slot's previous contents is done,
//                   you may store epoch e into it".  The push waits for it before
//                   the first store to r.
//   ready[slot][r]  written by rank r when all its stores of epoch e into my slot
//                   have been issued and fenced: "my columns are in your buffer".
//                   The last CTA of the push waits for every peer's before the
//                   kernel ends, so the stream's next consumer sees a full row.
//
// The epoch is a device counter (slot_use[slot]) that the attention kernel
// increments, so a captured graph replays with fresh epochs.  Every wait is
// bounded by a wall-clock budget; on expiry the status words are set, the stores
// to that peer are skipped and the kernel returns.
//
// The kernel runs on the group's communication stream under the NEXT layer's
// compute; a few dozen CTAs saturate what a layer needs of the NVLink bandwidth.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../qw_cuda.h"

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait until *flag has reached `epoch` (wrap-safe).  False when the budget ran out.
__device__ __forceinline__ bool wait_epoch(const uint32_t *flag, uint32_t epoch,
                                           unsigned long long budget_ns) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    const unsigned long long start = global_ns();
    for (;;) {
        for (int i = 0; i < 16; ++i) {
            if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
            __nanosleep(64);
        }
        if (global_ns() - start > budget_ns) return false;
    }
}

struct PushParams {
    const uint4 *src;        // this rank's full output
    uint4 *dst[8];           // the peers' full outputs, peer-mapped
    uint32_t peer_rank[8];   // their indices in the flag arrays
    uint32_t n_peers;
    uint32_t my_rank;
    uint32_t rows;           // batch * rows
    uint32_t row_vecs;       // 16-byte vectors per output row
    uint32_t col_vec0;       // first vector of this rank's column slice
    uint32_t slice_vecs;     // vectors in the slice
    const uint32_t *slot_use;     // epoch of this slot (set by the attention kernel)
    const uint32_t *freed_local;  // [8] this slot's freed flags, written by peers
    const uint32_t *ready_local;  // [8] this slot's ready flags, written by peers
    uint32_t *ready_peer[8];      // peer p's ready[slot][my_rank]
    uint32_t *arrivals;           // CTA arrival counter of this slot (self-resetting)
    uint32_t *status;
    unsigned long long budget_ns;
};

constexpr int kPushThreads = 256;
constexpr int kInFlight = 4;  // 16-byte loads per thread before the first store

__global__ void __launch_bounds__(kPushThreads) qw_push_kernel(const PushParams p) {
    __shared__ uint32_t s_epoch;
    __shared__ uint32_t s_open;  // bit d set: peer d freed its slot in time
    __shared__ uint32_t s_last;
    if (threadIdx.x == 0) {
        s_epoch = *reinterpret_cast<const volatile uint32_t *>(p.slot_use);
        s_open = 0;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch;
    if (threadIdx.x < p.n_peers) {
        const uint32_t d = threadIdx.x;
        if (wait_epoch(p.freed_local + p.peer_rank[d], epoch, p.budget_ns)) {
            atomicOr(&s_open, 1u << d);
        } else if (atomicCAS(p.status, 0u, (uint32_t)QWCU_STATUS_WAIT_TIMEOUT) == 0u) {
            p.status[1] = 0x50000u | p.peer_rank[d];  // where: push, waiting for a peer's slot
            p.status[2] = epoch;
            p.status[3] = blockIdx.x;
        }
    }
    __syncthreads();
    const uint32_t open = s_open;

    // Copy the slice: items are (row, vector) pairs, kInFlight loads in flight per
    // thread, each value stored to every peer whose slot is open.
    const unsigned long long items = (unsigned long long)p.rows * p.slice_vecs;
    const unsigned long long stride = (unsigned long long)gridDim.x * kPushThreads;
    for (unsigned long long i0 = (unsigned long long)blockIdx.x * kPushThreads + threadIdx.x;
         i0 < items; i0 += stride * kInFlight) {
        uint4 v[kInFlight];
        size_t at[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const unsigned long long i = i0 + (unsigned long long)u * stride;
            if (i < items) {
                const uint32_t row = (uint32_t)(i / p.slice_vecs);
                const uint32_t vec = (uint32_t)(i - (unsigned long long)row * p.slice_vecs);
                at[u] = (size_t)row * p.row_vecs + p.col_vec0 + vec;
                v[u] = __ldcg(p.src + at[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const unsigned long long i = i0 + (unsigned long long)u * stride;
            if (i < items)
                for (uint32_t d = 0; d < p.n_peers; ++d)
                    if (open >> d & 1u) p.dst[d][at[u]] = v[u];
        }
    }

    // All stores of this CTA are ordered before its arrival; the last CTA to arrive
    // publishes the ready flags and then waits for the peers' own.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t before = atomicAdd(p.arrivals, 1u);
        s_last = before == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) {
        *p.arrivals = 0;  // ready for the next launch on this slot
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x < p.n_peers) {
        const uint32_t d = threadIdx.x;
        if (open >> d & 1u) st_release_sys(p.ready_peer[d], epoch);
        if (!wait_epoch(p.ready_local + p.peer_rank[d], epoch, p.budget_ns) &&
            atomicCAS(p.status, 0u, (uint32_t)QWCU_STATUS_WAIT_TIMEOUT) == 0u) {
            p.status[1] = 0x60000u | p.peer_rank[d];  // where: push, waiting for a peer's columns
            p.status[2] = epoch;
            p.status[3] = blockIdx.x;
        }
    }
}

// Copy-engine form: the same hand-shake around plain strided device-to-device
// copies (one per peer), which need no SM at all.  One warp waits for the peers'
// `freed` flags before the copies; one warp publishes `ready` after them and
// waits for the peers' own.  (A wait that ran out is reported; the copies after
// it are part of the stream and still run.)
__global__ void __launch_bounds__(32) qw_push_open_kernel(const PushParams p) {
    if (threadIdx.x >= p.n_peers) return;
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t *>(p.slot_use);
    const uint32_t d = threadIdx.x;
    if (!wait_epoch(p.freed_local + p.peer_rank[d], epoch, p.budget_ns) &&
        atomicCAS(p.status, 0u, (uint32_t)QWCU_STATUS_WAIT_TIMEOUT) == 0u) {
        p.status[1] = 0x50000u | p.peer_rank[d];
        p.status[2] = epoch;
        p.status[3] = 0;
    }
}

__global__ void __launch_bounds__(32) qw_push_close_kernel(const PushParams p) {
    if (threadIdx.x >= p.n_peers) return;
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t *>(p.slot_use);
    const uint32_t d = threadIdx.x;
    __threadfence_system();
    st_release_sys(p.ready_peer[d], epoch);
    if (!wait_epoch(p.ready_local + p.peer_rank[d], epoch, p.budget_ns) &&
        atomicCAS(p.status, 0u, (uint32_t)QWCU_STATUS_WAIT_TIMEOUT) == 0u) {
        p.status[1] = 0x60000u | p.peer_rank[d];
        p.status[2] = epoch;
        p.status[3] = 0;
    }
}

}  // namespace

extern "C" int qwcu_push_launch(const qwcu_push_args *a, qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a->n_peers || a->n_peers > 8 || !a->rows || !a->slice_bytes || a->slice_bytes % 16 ||
        a->row_bytes % 16 || a->col_byte0 % 16 || a->col_byte0 + a->slice_bytes > a->row_bytes)
        return (int)cudaErrorInvalidValue;
    PushParams p;
    p.src = static_cast<const uint4 *>(a->src);
    for (uint32_t d = 0; d < 8; ++d) {
        p.dst[d] = d < a->n_peers ? static_cast<uint4 *>(a->dst[d]) : nullptr;
        p.peer_rank[d] = d < a->n_peers ? a->peer_rank[d] : 0;
        p.ready_peer[d] = d < a->n_peers ? a->ready_peer[d] : nullptr;
        if (d < a->n_peers && (!p.dst[d] || !p.ready_peer[d] || p.peer_rank[d] >= 8 ||
                               ((uintptr_t)p.dst[d] & 15u)))
            return (int)cudaErrorInvalidValue;
    }
    if (((uintptr_t)a->src & 15u) || !a->slot_use || !a->freed_local || !a->ready_local ||
        !a->arrivals || !a->status)
        return (int)cudaErrorInvalidValue;
    p.n_peers = a->n_peers;
    p.my_rank = a->my_rank;
    p.rows = a->rows;
    p.row_vecs = a->row_bytes / 16;
    p.col_vec0 = a->col_byte0 / 16;
    p.slice_vecs = a->slice_bytes / 16;
    p.slot_use = a->slot_use;
    p.freed_local = a->freed_local;
    p.ready_local = a->ready_local;
    p.arrivals = a->arrivals;
    p.status = a->status;
    p.budget_ns = (unsigned long long)(a->wait_ms ? a->wait_ms : 2000u) * 1000000ull;
    if (a->copy_engine) {
        qw_push_open_kernel<<<1, 32, 0, stream>>>(p);
        int rc = (int)cudaGetLastError();
        if (rc) return rc;
        const char *src = static_cast<const char *>(a->src) + a->col_byte0;
        for (uint32_t d = 0; d < a->n_peers; ++d) {
            char *dst = static_cast<char *>(a->dst[d]) + a->col_byte0;
            rc = (int)cudaMemcpy2DAsync(dst, a->row_bytes, src, a->row_bytes, a->slice_bytes, a->rows,
                                        cudaMemcpyDeviceToDevice, stream);
            if (rc) return rc;
        }
        qw_push_close_kernel<<<1, 32, 0, stream>>>(p);
        return (int)cudaGetLastError();
    }
    unsigned long long items = (unsigned long long)p.rows * p.slice_vecs;
    unsigned long long want = (items + (unsigned long long)kPushThreads * kInFlight - 1) /
                              ((unsigned long long)kPushThreads * kInFlight);
    unsigned blocks = a->max_blocks ? a->max_blocks : 32u;
    if (want < blocks) blocks = (unsigned)want;
    if (!blocks) blocks = 1;
    qw_push_kernel<<<blocks, kPushThreads, 0, stream>>>(p);
    return (int)cudaGetLastError();
}
