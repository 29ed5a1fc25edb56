// Block-causal (prefix-visible) flash-attention forward for sm_100a.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row sub-tiles that
// ping-pong on the tensor pipe.  Q/K/V tiles arrive through TMA (128B swizzle)
// into shared memory; S = Q K^T and O += P V run as tcgen05.mma with fp32
// accumulators in tensor memory (TMEM); the softmax is fp32 in the exp2 domain,
// one thread per query row, and writes P back to TMEM as bf16 over the S
// columns so P V reads its A operand straight from TMEM.
//
// Warp roles (384 threads = 3 warpgroups; registers are moved from the third
// warpgroup to the two softmax warpgroups with setmaxnreg):
//   warps 0-3   softmax + epilogue of sub-tile 0 (TMEM lanes 0..127)
//   warps 4-7   softmax + epilogue of sub-tile 1
//   warp  8     MMA issue (one elected lane), TMEM allocation
//   warp  9     TMA producer (one elected lane)
//   warps 10-11 idle (they only complete the third warpgroup)
//
// Mask: every row has an integer key limit (prefix) and the batch item may have
// a key-padding window.  Key tiles past the largest limit of a sub-tile are
// never issued, key tiles that lie completely inside the padding window are
// skipped by all roles, interior tiles run without a compare, boundary tiles
// apply the integer compare per element.
//
// Epilogue: O / l is rounded to bf16 into the (by then dead) Q tile in shared
// memory and leaves as TMA stores of the whole 128x128 tile.  When the heads
// are sharded over several GPUs the tile goes to this rank's head columns of a
// full-width output (the kernel can address several such destinations, peer-
// mapped ones included); the multi-GPU group writes the rank's own buffer here
// and carries the columns to the peers with a push kernel under the next layer,
// because with a single wave of CTAs all peer stores would leave at the kernel's
// end as one exposed burst.  At its start the kernel then opens the output slot's
// next epoch for the peers' pushes.
//
// Softmax.  Callers that promise bounded row norms (the DiT layer's QK-norm) get
// P = exp2(score*c - bound) against one fixed exponent: no row maximum, no
// rescaling, scores streamed out of TMEM in 32-column chunks; short launches pair
// both warpgroups on one sub-tile's keys at a time.  Other callers get the
// running maximum with lazy rescaling.
//
// Wave tail.  The grid is one CTA per (batch, head, 256-row block), heaviest
// blocks first, and rarely a multiple of the SM count.  The units that would
// form the last, partly filled wave are therefore run in split form, two CTAs per
// unit: a CTA takes 128 of the rows and gives each of its two sub-tiles half of
// the key tiles; at the end warpgroup 0 merges the two accumulators (both sit in
// the same TMEM lanes) with the usual exp2 reweighting.  Twice the CTAs of half
// the length fill the idle SMs, and nothing leaves the CTA unmerged.
//
// Every wait is bounded: when one runs out the CTA records where in the status
// words, raises a shared abort flag that all other waits poll, drains its TMA
// loads, frees its TMEM and returns.
//
// Semantics follow the reference prefix kernel (h3_shaders.metal:3061-3272):
// scale applied to fp32 scores, P rounded to bf16 before P V, fp32 accumulate,
// output acc / l rounded to bf16; rows without a visible key store zeros.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../qw_cuda.h"

namespace {

constexpr int kHeadDim = 128;
constexpr int kTileM = 128;  // query rows per sub-tile (= TMEM lanes)
constexpr int kTileN = 128;  // keys per tile
constexpr int kStages = 4;   // K/V ring slots
constexpr int kTileBytes = kTileN * kHeadDim * 2;  // 32 KiB
constexpr int kHalfTileBytes = kTileBytes / 2;     // one 64-column TMA box
constexpr int kThreads = 384;
// setmaxnreg only redistributes the registers the CTA got at launch
// (kThreads * 168 = 64512): 2 * 128 * 208 + 128 * 88 = 64512.  Asking for more
// would block the second softmax warpgroup forever.
constexpr int kLaunchRegs = 168;
constexpr int kSoftmaxRegs = 208;
constexpr int kOtherRegs = 88;
static_assert(2 * 128 * kSoftmaxRegs + 128 * kOtherRegs <= kThreads * kLaunchRegs,
              "setmaxnreg budget exceeds the launch allocation");
constexpr int kSoftmaxThreads = 256;
constexpr int kMmaWarp = 8;
constexpr int kTmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS0 = 0, kTmemS1 = 128, kTmemO0 = 256, kTmemO1 = 384;
// Lazy rescale threshold in the exp2 domain: P may grow to 2^8 before O and l
// are brought back to the running maximum.
constexpr float kRescaleThreshold = 8.0f;
// Wait budget in SM clock cycles (~0.2 s); a healthy wait is microseconds.
constexpr long long kWaitCycles = 400000000LL;

enum Barrier : int {
    kBarQFull = 0,                        // 2: Q sub-tile i landed
    kBarKvFull = 2,                       // kStages
    kBarKvEmpty = kBarKvFull + kStages,   // kStages
    kBarSFull = kBarKvEmpty + kStages,    // 2: S_i complete in TMEM
    kBarPFull = kBarSFull + 2,            // 2: P_i written (one arrival per warp)
    kBarOFinal = kBarPFull + 2,           // 2: last P V of sub-tile i complete
    kBarDebug = kBarOFinal + 2,           // trace builds: group completion probe
    kBarEpi = kBarDebug + 1,              // 2: output tile of sub-tile i staged in shared memory
    kBarMerge = kBarEpi + 2,              // split form: sub-tile 1 published its exponent and row sum
    kBarCount = kBarMerge + 1
};

struct __align__(16) SharedControl {
    unsigned long long bars[kBarCount];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
    long long wait_cycles;  // budget of every bounded wait of this CTA
    int n_tiles[2];      // key tiles each sub-tile needs (by its largest limit)
    int warp_max[8];     // per softmax warp: largest limit
    int skip_lo, skip_hi;  // key tiles [skip_lo, skip_hi) lie inside the padding window
    // Visited key tiles (the padding window taken out) are numbered 0, 1, ...;
    // sub-tile i walks tile_count[i] of them from tile_first[i].  Whole form: both
    // from 0.  Split form: the two halves of one list.
    int tile_first[2], tile_count[2];
    float merge_m[kTileM];  // split form: sub-tile 1's reference exponent and row sum
    float merge_l[kTileM];
    // Paired organisation: row sums of the two key halves, [key half][sub-tile][row].
    float pair_l[2][2][kTileM];
};

constexpr size_t kSmemData = (size_t)(2 + kStages) * kTileBytes;
constexpr size_t kSmemBytes = kSmemData + sizeof(SharedControl) + 1024;  // +1024: manual alignment

struct KernelParams {
    __nv_bfloat16 *out;
    const int32_t *kv_limit;
    uint32_t *status;
#ifdef QW_ATTN_TRACE
    unsigned long long *trace;  // event log of block (0,0,0), dumped to $QW_CUDA_ATTN_TRACE
#endif
    int per_batch_limits;
    int causal;
    uint32_t causal_offset;
    uint32_t batch, q_rows, kv_rows, heads, kv_heads;
    uint32_t text_len[8];
    uint32_t text_pad;
    float scale_log2;  // scale * log2(e)
    // Optional promise by the caller (two floats in device memory): every query row
    // has a 2-norm of at most score_bound[0] and every key row of at most
    // score_bound[1], so |q.k| <= their product and the softmax can use one fixed
    // reference exponent instead of a running row maximum.
    const float *score_bound;
    int pair_org;  // fixed-exponent softmax: both warpgroups share each sub-tile's keys
    int head_major_out;
    // Sharded runs: the rows are stored at this rank's head columns of n_out
    // full-width outputs (peer-mapped pointers allowed).  out_heads_total is the
    // head count of the destination rows and out_head_offset this rank's first head.
    __nv_bfloat16 *out_peers[8];
    uint32_t n_out, out_heads_total, out_head_offset;
    // Launch geometry: CTA c < total_units - tail_units runs unit c whole; the
    // last tail_units units run in split form, two CTAs each.
    uint32_t n_qblocks, total_units, tail_units;
    // Gather by a separate push: epoch counter of the output slot and the peers'
    // flag words that receive the new epoch when this kernel starts.
    uint32_t *slot_use;
    uint32_t *freed_peer[8];
    uint32_t n_freed;
    // Bounded-wait exercise (tests only): budget in SM cycles (0 = the default) and
    // the first visited key tile the producer does NOT load (< 0: loads everything),
    // so that the waits downstream of it run out and the CTA takes its clean exit.
    long long wait_cycles;
    int withhold_from;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// The P and staging barriers count one arrival per softmax warp of the CTA (8).
// Where only one warpgroup works on a sub-tile, each of its four warps arrives
// for two.
__device__ __forceinline__ void mbar_arrive_twice(unsigned long long *bar) {
    mbar_arrive(bar);
    mbar_arrive(bar);
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try(unsigned long long *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait.  Returns false when the budget ran out here (recorded) or
// another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait_slow(SharedControl *ctl, unsigned long long *bar,
                                            uint32_t parity, uint32_t *status, uint32_t where,
                                            uint32_t tile) {
    long long start = clock64();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if (mbar_try(bar, parity)) return true;
        if (ctl->abort_flag) return false;
        if (clock64() - start > ctl->wait_cycles) {
            ctl->abort_flag = 1;
            if (atomicCAS(status, 0u, (uint32_t)QWCU_STATUS_WAIT_TIMEOUT) == 0u) {
                status[1] = where;
                status[2] = tile;
                status[3] = blockIdx.x;
            }
            __threadfence();
            return false;
        }
    }
}

__device__ __forceinline__ bool mbar_wait(SharedControl *ctl, unsigned long long *bar,
                                          uint32_t parity, uint32_t *status, uint32_t where,
                                          uint32_t tile) {
    if (mbar_try(bar, parity)) return true;
    return mbar_wait_slow(ctl, bar, parity, status, where, tile);
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map,
                                            unsigned long long *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Output tensor maps, one per destination (one on a single GPU, one per rank
// when the heads are sharded and every rank receives the rows).
struct OutMaps {
    CUtensorMap m[8];
};

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *src, int c0, int c1,
                                             int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptors (sm_100 format) are built as two 32-bit words
// further down (desc_hi / desc_lo_fixed): start address >> 4 in bits 0-13, leading
// byte offset >> 4 in bits 16-29, stride byte offset >> 4 in bits 32-45, descriptor
// version 1 in bit 46, 128B swizzle = 2 in bits 61-63.

// Instruction descriptor, kind::f16: bf16 x bf16 -> fp32, M = 128, N = 128.
constexpr uint32_t make_idesc(bool b_mn_major) {
    return (1u << 4)                      // D format: f32
           | (1u << 7)                    // A format: bf16
           | (1u << 10)                   // B format: bf16
           | ((b_mn_major ? 1u : 0u) << 16)
           | ((uint32_t)(kTileN >> 3) << 17)
           | ((uint32_t)(kTileM >> 4) << 24);
}
constexpr uint32_t kIdescQK = make_idesc(false);
constexpr uint32_t kIdescPV = make_idesc(true);

// Descriptors travel as (low word, high word): stepping through a tile only
// changes the start-address field in the low word, so each MMA costs one
// integer add per operand on the issuing thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                       uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

#define QW_TMEM_LD32(taddr, r)                                                                  \
    asm volatile(                                                                               \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                               \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "              \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "    \
        "[%32];"                                                                                \
        : "=r"((r)[0]), "=r"((r)[1]), "=r"((r)[2]), "=r"((r)[3]), "=r"((r)[4]), "=r"((r)[5]),   \
          "=r"((r)[6]), "=r"((r)[7]), "=r"((r)[8]), "=r"((r)[9]), "=r"((r)[10]), "=r"((r)[11]), \
          "=r"((r)[12]), "=r"((r)[13]), "=r"((r)[14]), "=r"((r)[15]), "=r"((r)[16]),            \
          "=r"((r)[17]), "=r"((r)[18]), "=r"((r)[19]), "=r"((r)[20]), "=r"((r)[21]),            \
          "=r"((r)[22]), "=r"((r)[23]), "=r"((r)[24]), "=r"((r)[25]), "=r"((r)[26]),            \
          "=r"((r)[27]), "=r"((r)[28]), "=r"((r)[29]), "=r"((r)[30]), "=r"((r)[31])             \
        : "r"(taddr))

#define QW_TMEM_ST32(taddr, r)                                                                  \
    asm volatile(                                                                               \
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                         \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "             \
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"     \
        ::"r"(taddr), "r"((r)[0]), "r"((r)[1]), "r"((r)[2]), "r"((r)[3]), "r"((r)[4]),          \
          "r"((r)[5]), "r"((r)[6]), "r"((r)[7]), "r"((r)[8]), "r"((r)[9]), "r"((r)[10]),        \
          "r"((r)[11]), "r"((r)[12]), "r"((r)[13]), "r"((r)[14]), "r"((r)[15]), "r"((r)[16]),   \
          "r"((r)[17]), "r"((r)[18]), "r"((r)[19]), "r"((r)[20]), "r"((r)[21]), "r"((r)[22]),   \
          "r"((r)[23]), "r"((r)[24]), "r"((r)[25]), "r"((r)[26]), "r"((r)[27]), "r"((r)[28]),   \
          "r"((r)[29]), "r"((r)[30]), "r"((r)[31])                                              \
        : "memory")

#define QW_TMEM_ST16(taddr, r)                                                                  \
    asm volatile(                                                                               \
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                         \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"             \
        ::"r"(taddr), "r"((r)[0]), "r"((r)[1]), "r"((r)[2]), "r"((r)[3]), "r"((r)[4]),          \
          "r"((r)[5]), "r"((r)[6]), "r"((r)[7]), "r"((r)[8]), "r"((r)[9]), "r"((r)[10]),        \
          "r"((r)[11]), "r"((r)[12]), "r"((r)[13]), "r"((r)[14]), "r"((r)[15])                  \
        : "memory")

// tcgen05.wait::ld that names the 32 registers of an earlier load as read-write
// operands: no use of them can be scheduled ahead of the wait.
#define QW_TMEM_WAIT_LD32(r)                                                                    \
    asm volatile(                                                                               \
        "tcgen05.wait::ld.sync.aligned;"                                                        \
        : "+r"((r)[0]), "+r"((r)[1]), "+r"((r)[2]), "+r"((r)[3]), "+r"((r)[4]), "+r"((r)[5]),   \
          "+r"((r)[6]), "+r"((r)[7]), "+r"((r)[8]), "+r"((r)[9]), "+r"((r)[10]), "+r"((r)[11]), \
          "+r"((r)[12]), "+r"((r)[13]), "+r"((r)[14]), "+r"((r)[15]), "+r"((r)[16]),            \
          "+r"((r)[17]), "+r"((r)[18]), "+r"((r)[19]), "+r"((r)[20]), "+r"((r)[21]),            \
          "+r"((r)[22]), "+r"((r)[23]), "+r"((r)[24]), "+r"((r)[25]), "+r"((r)[26]),            \
          "+r"((r)[27]), "+r"((r)[28]), "+r"((r)[29]), "+r"((r)[30]), "+r"((r)[31])             \
        :                                                                                       \
        : "memory")

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Packed fp32 pairs (one issue slot for two lanes of work on sm_100).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for a pair on the FMA pipe instead of the special-function unit, which
// the exponentials of a 128x128 tile otherwise keep as busy as its MMAs keep the
// tensor pipe: n = round(x) by the 1.5*2^23 trick, r = x - n in [-0.5, 0.5], a
// cubic for 2^r (exact at r = 0, max relative error 1.2e-4, far below the bf16 rounding of P),
// then n is added into the exponent field.  x is clamped at -127 (result 0).
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    const float kMagic = 12582912.0f;  // 1.5 * 2^23
    x.x = fmaxf(x.x, -127.0f);
    x.y = fmaxf(x.y, -127.0f);
    const float2 t = fadd2(x, make_float2(kMagic, kMagic));
    const float2 n = fadd2(t, make_float2(-kMagic, -kMagic));
    const float2 r = ffma2(n, make_float2(-1.0f, -1.0f), x);
    float2 q = ffma2(r, make_float2(0.05541782081127167f, 0.05541782081127167f),
                     make_float2(0.24221134185791016f, 0.24221134185791016f));
    q = ffma2(q, r, make_float2(0.6931995153427124f, 0.6931995153427124f));
    q = ffma2(q, r, make_float2(1.0f, 1.0f));
    float2 out;
    out.x = __uint_as_float(__float_as_uint(q.x) + (__float_as_uint(t.x) << 23));
    out.y = __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(t.y) << 23));
    return out;
}

// Pipeline event log, compiled in only with -DQW_ATTN_TRACE (a debugging build).
#ifdef QW_ATTN_TRACE
// Event log for pipeline analysis: (role, event, tile) and the SM clock, written
// by one thread per role of block (0, 0, 0) when a trace buffer is attached.
constexpr int kTraceSlots = 4096;
__device__ __forceinline__ void trace_event(const KernelParams &p, int role, int event, int tile,
                                            uint32_t &cursor) {
    // One private region per role and a register cursor: a plain store, no
    // round trip, so the log barely perturbs what it measures.
    if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && cursor < 1000) {
        p.trace[1 + role * 1024 + cursor] =
            ((unsigned long long)(role << 20 | event << 12 | (tile & 0xfff)) << 40) |
            ((unsigned long long)clock64() & 0xffffffffffull);
        ++cursor;
    }
}
#define QW_TRACE(role, event, tile) trace_event(p, role, event, tile, trace_cursor)
#else
#define QW_TRACE(role, event, tile) ((void)0)
#endif

__device__ __forceinline__ int row_limit(const KernelParams &p, uint32_t b, uint32_t r) {
    if (r >= p.q_rows) return 0;
    if (p.text_pad && r >= p.text_len[b] && r < p.text_pad) return 0;  // padding query row
    int limit;
    if (p.kv_limit) {
        limit = p.kv_limit[p.per_batch_limits ? (size_t)b * p.q_rows + r : r];
        limit = max(limit, 0);
    } else if (p.causal) {
        unsigned long long c = (unsigned long long)r + 1ull + p.causal_offset;
        limit = (int)min(c, (unsigned long long)p.kv_rows);
    } else {
        limit = (int)p.kv_rows;
    }
    return min(limit, (int)p.kv_rows);
}

// Visited tile u -> key tile index, and how many of `tiles` key tiles are visited.
__device__ __forceinline__ int phys_tile(const SharedControl *ctl, int u) {
    return u < ctl->skip_lo ? u : u + (ctl->skip_hi - ctl->skip_lo);
}
__device__ __forceinline__ int visited_tiles(int tiles, int lo, int hi) {
    if (tiles <= lo) return tiles;
    if (tiles >= hi) return tiles - (hi - lo);
    return lo;
}

// ---------------------------------------------------------------------------
// Softmax + epilogue role: 128 threads per sub-tile, one query row each.
// ---------------------------------------------------------------------------
// kBounded: the caller promised |score * scale * log2(e)| <= bound (see
// KernelParams::score_bound), so P = exp2(score*c - bound) needs no row maximum:
// the scores stream out of TMEM 32 columns at a time, each chunk's exponentials
// run under the next chunk's load, and O is never rescaled.
template <int kPoly, bool kBounded>
__device__ __forceinline__ void softmax_role(const KernelParams &p, SharedControl *ctl,
                                             const OutMaps &maps_out, uint8_t *stage, int sub,
                                             int tid_in_group, int my_limit, uint32_t b, uint32_t h,
                                             uint32_t row, uint32_t tile_row0, bool split,
                                             float bound) {
    const int warp_in_group = tid_in_group >> 5;
    const uint32_t lane_base = (uint32_t)(warp_in_group * 32) << 16;
    const uint32_t tmem = ctl->tmem_base;
    const uint32_t tmem_s = tmem + lane_base + (sub ? kTmemS1 : kTmemS0);
    const uint32_t tmem_o = tmem + lane_base + (sub ? kTmemO1 : kTmemO0);
    unsigned long long *bar_s = &ctl->bars[kBarSFull + sub];
    unsigned long long *bar_p = &ctl->bars[kBarPFull + sub];
    const int pad_lo = p.text_pad ? (int)p.text_len[b] : 0;
    const int pad_hi = (int)p.text_pad;
    const float c = p.scale_log2;
    const bool neg = c < 0.0f;

    [[maybe_unused]] uint32_t trace_cursor = 0;
    float m_run = -INFINITY;  // running extreme of the raw scores (max, or min when c < 0)
    float m_ref = -INFINITY;  // extreme the stored exponents refer to
    float l_run = 0.0f;
    uint32_t phase = 0;
    bool ok = true;
    int processed = 0;

    const int u_first = ctl->tile_first[sub], u_end = u_first + ctl->tile_count[sub];
    if constexpr (kBounded) {
        const float2 cs2 = make_float2(c, c), bias2 = make_float2(-bound, -bound);
        float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
        for (int u = u_first; u < u_end && ok; ++u) {
            const int j = phys_tile(ctl, u);
            ok = mbar_wait(ctl, bar_s, phase, p.status, (1u << 16) | (uint32_t)(kBarSFull + sub),
                           (uint32_t)j);
            if (!ok) break;
            phase ^= 1u;
            tc_fence_after();
            if (tid_in_group == 0) QW_TRACE(sub, 0, j);
            const int key0 = j * kTileN;
            const bool pad_hit = pad_hi > pad_lo && key0 < pad_hi && key0 + kTileN > pad_lo;
            const bool boundary = __any_sync(0xffffffffu, key0 + kTileN > my_limit) || pad_hit;
            uint32_t sa[32], sb[32];
            QW_TMEM_LD32(tmem_s, sa);
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk) {
                uint32_t(&cur)[32] = (chunk & 1) ? sb : sa;
                uint32_t(&nxt)[32] = (chunk & 1) ? sa : sb;
                QW_TMEM_WAIT_LD32(cur);
                if (chunk == 0 && tid_in_group == 0) QW_TRACE(sub, 1, j);
                if (chunk < 3) QW_TMEM_LD32(tmem_s + 32 * (chunk + 1), nxt);
                if (boundary) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + chunk * 32 + i;
                        const bool visible = key < my_limit && !(key >= pad_lo && key < pad_hi);
                        cur[i] = visible ? cur[i] : __float_as_uint(-INFINITY);
                    }
                }
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 x = ffma2(make_float2(__uint_as_float(cur[2 * i]),
                                                 __uint_as_float(cur[2 * i + 1])),
                                     cs2, bias2);
                    float2 pr;
                    if ((i & 3) < kPoly) {
                        pr = exp2_poly2(x);
                    } else {
                        pr.x = fast_exp2(x.x);
                        pr.y = fast_exp2(x.y);
                    }
                    if (i & 1) sum_b = fadd2(sum_b, pr);
                    else sum_a = fadd2(sum_a, pr);
                    pk[i] = pack_bf16(pr.x, pr.y);
                }
                // P chunk c lands on columns [16c, 16c+16): scores already consumed.
                QW_TMEM_ST16(tmem_s + chunk * 16, pk);
                if (chunk == 1 && tid_in_group == 0) QW_TRACE(sub, 2, j);
            }
            if (tid_in_group == 0) QW_TRACE(sub, 3, j);
            tmem_wait_st();
            tc_fence_before();
            if ((tid_in_group & 31) == 0) mbar_arrive_twice(bar_p);
            if (tid_in_group == 0) QW_TRACE(sub, 4, j);
            ++processed;
        }
        sum_a = fadd2(sum_a, sum_b);
        l_run = sum_a.x + sum_a.y;
    } else
    for (int u = u_first; u < u_end && ok; ++u) {
        const int j = phys_tile(ctl, u);
        ok = mbar_wait(ctl, bar_s, phase, p.status, (1u << 16) | (uint32_t)(kBarSFull + sub),
                       (uint32_t)j);
        if (!ok) break;
        phase ^= 1u;
        tc_fence_after();
        if (tid_in_group == 0) QW_TRACE(sub, 0, j);

        uint32_t s[128];
        QW_TMEM_LD32(tmem_s + 0, s + 0);
        QW_TMEM_LD32(tmem_s + 32, s + 32);
        QW_TMEM_LD32(tmem_s + 64, s + 64);
        QW_TMEM_LD32(tmem_s + 96, s + 96);
        tmem_wait_ld();
        if (tid_in_group == 0) QW_TRACE(sub, 1, j);

        const int key0 = j * kTileN;
        const bool pad_hit = pad_hi > pad_lo && key0 < pad_hi && key0 + kTileN > pad_lo;
        const bool boundary = __any_sync(0xffffffffu, key0 + kTileN > my_limit) || pad_hit;
        const float sign = neg ? -1.0f : 1.0f;
        if (boundary) {
#pragma unroll
            for (int i = 0; i < 128; ++i) {
                int key = key0 + i;
                bool visible = key < my_limit && !(key >= pad_lo && key < pad_hi);
                s[i] = visible ? s[i] : __float_as_uint(neg ? INFINITY : -INFINITY);
            }
        }
        // Row extreme of sign*score (four independent chains).
        float e0 = -INFINITY, e1 = -INFINITY, e2 = -INFINITY, e3 = -INFINITY;
        if (!neg) {
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
                e0 = fmax3(e0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
                e1 = fmax3(e1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
                e2 = fmax3(e2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
                e3 = fmax3(e3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 128; i += 4) {
                e0 = fmaxf(e0, -__uint_as_float(s[i]));
                e1 = fmaxf(e1, -__uint_as_float(s[i + 1]));
                e2 = fmaxf(e2, -__uint_as_float(s[i + 2]));
                e3 = fmaxf(e3, -__uint_as_float(s[i + 3]));
            }
        }
        const float m_tile = fmaxf(fmaxf(e0, e1), fmaxf(e2, e3));  // in sign*score units
        const float m_new = fmaxf(m_run, m_tile);
        m_run = m_new;
        const float ac = fabsf(c);
        // Does the reference point have to move?  (first finite value, or drift > threshold)
        const bool move = (m_new != -INFINITY) &&
                          (m_ref == -INFINITY || (m_new - m_ref) * ac > kRescaleThreshold);
        const bool any_move = __any_sync(0xffffffffu, move && processed > 0 && m_ref != -INFINITY);
        float alpha = 1.0f;
        if (move) {
            alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2((m_ref - m_new) * ac);
            m_ref = m_new;
        }
        if (any_move) {
            // s_full of this tile was committed after the previous P V of this
            // sub-tile, so O is quiescent until P of this tile is published.
#pragma unroll 1
            for (int chunk = 0; chunk < 4; ++chunk) {
                uint32_t o[32];
                QW_TMEM_LD32(tmem_o + chunk * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                QW_TMEM_ST32(tmem_o + chunk * 32, o);
            }
            tmem_wait_st();
        }
        l_run *= alpha;
        if (tid_in_group == 0) QW_TRACE(sub, 2, j);

        // P = exp2(sign*score*|c| - m_ref*|c|) as bf16 pairs, written over S.
        const float bias = (m_ref == -INFINITY) ? 0.0f : -m_ref * ac;
        const float cs = sign * ac;
        // kPoly of every 4 pairs take the polynomial instead of the SFU.  P goes
        // back to TMEM 32 keys (16 packed columns) at a time.
        const float2 cs2 = make_float2(cs, cs), bias2 = make_float2(bias, bias);
        float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int chunk = 0; chunk < 4; ++chunk) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int e = chunk * 32 + 2 * i;
                float2 x = ffma2(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])),
                                 cs2, bias2);
                float2 pr;
                if ((i & 3) < kPoly) {
                    pr = exp2_poly2(x);
                } else {
                    pr.x = fast_exp2(x.x);
                    pr.y = fast_exp2(x.y);
                }
                if (i & 1) sum_b = fadd2(sum_b, pr);
                else sum_a = fadd2(sum_a, pr);
                pk[i] = pack_bf16(pr.x, pr.y);
            }
            QW_TMEM_ST16(tmem_s + chunk * 16, pk);
        }
        if (tid_in_group == 0) QW_TRACE(sub, 3, j);
        tmem_wait_st();  // warp-collective: every lane's stores have landed
        tc_fence_before();
        if ((tid_in_group & 31) == 0) mbar_arrive_twice(bar_p);  // stands for two warps
        if (tid_in_group == 0) QW_TRACE(sub, 4, j);
        sum_a = fadd2(sum_a, sum_b);
        l_run += sum_a.x + sum_a.y;
        ++processed;
    }

    // Epilogue: O / l -> bf16.  Token-major output goes through shared memory (the
    // dead Q tile of this sub-tile, same swizzled box layout) and leaves as TMA
    // stores of the whole 128x128 tile, one pair per destination: on a single
    // GPU that is one coalesced write, with sharded heads the same tile also
    // goes to every peer's output over NVLink in bulk instead of 64-byte pieces.
    if (!ok || tile_row0 >= p.q_rows) return;  // gave up, or this sub-tile holds no rows
    const bool has_row = row < p.q_rows;
    if (processed > 0) {
        ok = mbar_wait(ctl, &ctl->bars[kBarOFinal + sub], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarOFinal + sub), 0xffffu);
        if (!ok) return;
        tc_fence_after();
    }
    // Scale factors of the accumulators that make up the output rows: O_sub alone,
    // or in split form O_0 and O_1 brought to a common reference exponent.
    // out = (w_own * O_own + w_other * O_other) * inv: the weights are exactly 1 when
    // the reference exponents agree, so a split block of equal-score rows merges
    // exactly like the whole block would have summed.
    float w_own = 1.0f, w_other = 0.0f, inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    bool use_own = processed > 0, use_other = false;
    if (split) {
        const float m_own = kBounded ? (processed > 0 ? bound : -INFINITY)
                            : (processed > 0 && m_ref != -INFINITY) ? m_ref * fabsf(c)
                                                                    : -INFINITY;
        if (sub == 1) {
            // Publish exponent and row sum; warpgroup 0 reads O_1 itself (same lanes).
            ctl->merge_m[tid_in_group] = m_own;
            ctl->merge_l[tid_in_group] = l_run;
            __syncwarp();
            if ((tid_in_group & 31) == 0) mbar_arrive(&ctl->bars[kBarMerge]);
            return;
        }
        ok = mbar_wait(ctl, &ctl->bars[kBarMerge], 0, p.status, (1u << 16) | (uint32_t)kBarMerge,
                       0xfffbu);
        if (!ok) return;
        use_other = ctl->tile_count[1] > 0;
        if (use_other) {
            ok = mbar_wait(ctl, &ctl->bars[kBarOFinal + 1], 0, p.status,
                           (1u << 16) | (uint32_t)(kBarOFinal + 1), 0xfffeu);
            if (!ok) return;
            tc_fence_after();
        }
        const float m_other = ctl->merge_m[tid_in_group], l_other = ctl->merge_l[tid_in_group];
        const float m_all = fmaxf(m_own, m_other);
        const float a_own = m_own == -INFINITY ? 0.0f : fast_exp2(m_own - m_all);
        const float a_other = m_other == -INFINITY ? 0.0f : fast_exp2(m_other - m_all);
        const float l_all = a_own * l_run + a_other * l_other;
        inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
        w_own = a_own;
        w_other = a_other;
    } else if (processed == 0 && !p.head_major_out) {
        // Nothing was computed for this sub-tile (zeros go out), but its Q load may
        // still be in flight into the staging area: let it land first.
        ok = mbar_wait(ctl, &ctl->bars[kBarQFull + sub], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarQFull + sub), 0xfffdu);
        if (!ok) return;
    }
    if (split && !p.head_major_out && !use_own) {
        // (same reason: the shared Q tile is the staging area)
        ok = mbar_wait(ctl, &ctl->bars[kBarQFull + 0], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarQFull + 0), 0xfffdu);
        if (!ok) return;
    }
    const uint32_t tmem_other = tmem + lane_base + kTmemO1;
    // Row r of the tile in the staging area: two 128-byte lines (columns 0..63 and
    // 64..127, one half tile apart), 16-byte chunks XOR-swizzled by the row like TMA
    // does.  Head-major output is written directly.  (Every lane takes part in the
    // warp-collective TMEM loads; only the stores depend on the row being real.)
    uint8_t *line = stage + tid_in_group * 128;
    const int sw = tid_in_group & 7;
    __nv_bfloat16 *direct =
        p.out + (((size_t)b * p.heads + h) * p.q_rows + (has_row ? row : 0u)) * kHeadDim;
#pragma unroll 1
    for (int chunk = 0; chunk < 4; ++chunk) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        if (use_own) {
            uint32_t o[32];
            QW_TMEM_LD32(tmem_o + chunk * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]) * w_own;
        }
        if (use_other) {
            uint32_t o[32];
            QW_TMEM_LD32(tmem_other + chunk * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = fmaf(__uint_as_float(o[i]), w_other, v[i]);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            packed.x = pack_bf16(v[i] * inv, v[i + 1] * inv);
            packed.y = pack_bf16(v[i + 2] * inv, v[i + 3] * inv);
            packed.z = pack_bf16(v[i + 4] * inv, v[i + 5] * inv);
            packed.w = pack_bf16(v[i + 6] * inv, v[i + 7] * inv);
            if (p.head_major_out) {
                if (has_row) reinterpret_cast<uint4 *>(direct + chunk * 32)[i >> 3] = packed;
            } else {
                const int c16 = chunk * 4 + (i >> 3);  // 16-byte chunk of the 256-byte row
                *reinterpret_cast<uint4 *>(line + (c16 >> 3) * kHalfTileBytes +
                                           (((c16 & 7) ^ sw) << 4)) = packed;
            }
        }
    }
    if (p.head_major_out) return;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> TMA reads
    __syncwarp();
    if ((tid_in_group & 31) == 0) mbar_arrive_twice(&ctl->bars[kBarEpi + sub]);
    if (tid_in_group == 0) {
        if (!mbar_wait(ctl, &ctl->bars[kBarEpi + sub], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarEpi + sub), 0xfffcu))
            return;
        const int col = (int)((p.out_head_offset + h) * kHeadDim);
        for (uint32_t d = 0; d < p.n_out; ++d) {
            tma_store_3d(&maps_out.m[d], stage, col, (int)tile_row0, (int)b);
            tma_store_3d(&maps_out.m[d], stage + kHalfTileBytes, col + 64, (int)tile_row0, (int)b);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // Shared memory may be released once the stores have read it; the
        // writes themselves are complete when the grid completes, which is
        // what the barrier behind a sharded launch waits for.
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
}

// ---------------------------------------------------------------------------
// Paired softmax role (fixed reference exponent only): all 256 softmax threads
// work on one sub-tile's scores at a time, then on the other's.  TMEM lanes are
// tied to warp_id % 4, so warps w and w + 4 both reach rows 32w..32w+31 of either
// sub-tile: thread (half, r) takes keys [64*half, 64*half + 64) of row r.  Two
// warps per scheduler run the exponentials of one tile together, which halves
// the time a tile's S -> P step stays on the dependency chain S -> P -> P V; the
// other sub-tile's MMAs fill the tensor pipe meanwhile.  Without a row maximum
// the two threads of a row share nothing until the row sums meet at the end.
// ---------------------------------------------------------------------------
template <int kPoly>
__device__ __forceinline__ void softmax_pair_role(const KernelParams &p, SharedControl *ctl,
                                                  const OutMaps &maps_out, uint8_t *smem_q,
                                                  int tid, int limit0, int limit1, uint32_t b,
                                                  uint32_t h, uint32_t row0, bool split,
                                                  float bound) {
    const int half = tid >> 7, r = tid & 127;
    const uint32_t lane_base = (uint32_t)((r >> 5) * 32) << 16;
    const uint32_t tmem = ctl->tmem_base + lane_base;
    const uint32_t s_col[2] = {kTmemS0 + 64u * (uint32_t)half, kTmemS1 + 64u * (uint32_t)half};
    const int limits[2] = {limit0, limit1};
    const int pad_lo = p.text_pad ? (int)p.text_len[b] : 0;
    const int pad_hi = (int)p.text_pad;
    const float2 cs2 = make_float2(p.scale_log2, p.scale_log2);
    const float2 bias2 = make_float2(-bound, -bound);
    [[maybe_unused]] uint32_t trace_cursor = 0;

    float2 sums[2][2] = {{make_float2(0.f, 0.f), make_float2(0.f, 0.f)},
                         {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}};
    uint32_t phase[2] = {0, 0};
    const int first[2] = {ctl->tile_first[0], ctl->tile_first[1]};
    const int count[2] = {ctl->tile_count[0], ctl->tile_count[1]};
    const int steps = max(count[0], count[1]);
    bool ok = true;
    // The first 32 scores of the next tile (the other sub-tile's, as a rule complete
    // long before) are requested while this tile's last P chunk is still on its way
    // to TMEM, so a tile does not start with an exposed TMEM round trip.
    bool prefetched = false;
    uint32_t sa[32], sb[32];

    for (int s = 0; s < steps && ok; ++s) {
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            if (s >= count[sub] || !ok) continue;
            const int j = phys_tile(ctl, first[sub] + s);
            if (!prefetched) {
                ok = mbar_wait(ctl, &ctl->bars[kBarSFull + sub], phase[sub], p.status,
                               (1u << 16) | (uint32_t)(kBarSFull + sub), (uint32_t)j);
                if (!ok) continue;
                phase[sub] ^= 1u;
                tc_fence_after();
                QW_TMEM_LD32(tmem + s_col[sub], sa);
            }
            prefetched = false;
            if (tid == 0) QW_TRACE(sub, 0, j);
            const int key0 = j * kTileN + 64 * half;
            const int my_limit = limits[sub];
            const bool pad_hit = pad_hi > pad_lo && key0 < pad_hi && key0 + 64 > pad_lo;
            const bool boundary = __any_sync(0xffffffffu, key0 + 64 > my_limit) || pad_hit;
#pragma unroll
            for (int chunk = 0; chunk < 2; ++chunk) {
                uint32_t(&cur)[32] = chunk ? sb : sa;
                QW_TMEM_WAIT_LD32(cur);
                if (chunk == 0) QW_TMEM_LD32(tmem + s_col[sub] + 32, sb);
                if (chunk == 0 && tid == 0) QW_TRACE(sub, 1, j);
                if (boundary) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + chunk * 32 + i;
                        const bool visible = key < my_limit && !(key >= pad_lo && key < pad_hi);
                        cur[i] = visible ? cur[i] : __float_as_uint(-INFINITY);
                    }
                }
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 x = ffma2(make_float2(__uint_as_float(cur[2 * i]),
                                                 __uint_as_float(cur[2 * i + 1])),
                                     cs2, bias2);
                    float2 pr;
                    if ((i & 3) < kPoly) {
                        pr = exp2_poly2(x);
                    } else {
                        pr.x = fast_exp2(x.x);
                        pr.y = fast_exp2(x.y);
                    }
                    sums[sub][i & 1] = fadd2(sums[sub][i & 1], pr);
                    pk[i] = pack_bf16(pr.x, pr.y);
                }
                // P of this thread's keys lands over this thread's own scores.
                QW_TMEM_ST16(tmem + s_col[sub] + chunk * 16, pk);
                if (chunk == 0 && tid == 0) QW_TRACE(sub, 2, j);
            }
            if (tid == 0) QW_TRACE(sub, 3, j);
            {
                const int nsub = 1 - sub, ns = sub ? s + 1 : s;
                if (ns < count[nsub]) {
                    const bool ready = mbar_try(&ctl->bars[kBarSFull + nsub], phase[nsub]);
                    if (__all_sync(0xffffffffu, ready)) {
                        phase[nsub] ^= 1u;
                        tc_fence_after();
                        QW_TMEM_LD32(tmem + s_col[nsub], sa);
                        prefetched = true;
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before();
            if ((tid & 31) == 0) mbar_arrive(&ctl->bars[kBarPFull + sub]);
            if (tid == 0) QW_TRACE(sub, 4, j);
        }
    }
    // Row sums of the two key halves meet here.  Every softmax thread reaches this
    // barrier, also after a wait gave up (its rows are then simply not stored).
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
        const float2 t = fadd2(sums[sub][0], sums[sub][1]);
        ctl->pair_l[half][sub][r] = t.x + t.y;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
    if (!ok || ctl->abort_flag) return;

    // Epilogue.  Whole form: output tile t is sub-tile t, O_t / l_t.  Split form: one
    // tile whose keys were divided between the sub-tiles: (O_0 + O_1) / (l_0 + l_1);
    // both carry the same reference exponent, so the sum needs no reweighting.
    // Thread (half, r) converts columns [64*half, 64*half + 64) of row r: exactly one
    // 128-byte line of the swizzled staging box of its half.
    const int n_out_tiles = split ? 1 : 2;
#pragma unroll 1
    for (int t = 0; t < n_out_tiles; ++t) {
        const uint32_t tile_row0 = row0 + (uint32_t)t * kTileM;
        if (tile_row0 >= p.q_rows) continue;
        const uint32_t row = tile_row0 + (uint32_t)r;
        const bool has_row = row < p.q_rows;
        const bool use0 = split ? count[0] > 0 : count[t] > 0;
        const bool use1 = split && count[1] > 0;
        float l = ctl->pair_l[0][t][r] + ctl->pair_l[1][t][r];
        if (split) l += ctl->pair_l[0][1][r] + ctl->pair_l[1][1][r];
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        if (use0 &&
            !mbar_wait(ctl, &ctl->bars[kBarOFinal + t], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarOFinal + t), 0xffffu))
            return;
        if (use1 &&
            !mbar_wait(ctl, &ctl->bars[kBarOFinal + 1], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarOFinal + 1), 0xfffeu))
            return;
        if (!use0 && !p.head_major_out &&
            // nothing was computed (zeros go out), but the Q load may still be in
            // flight into what is now the staging area: let it land first
            !mbar_wait(ctl, &ctl->bars[kBarQFull + t], 0, p.status,
                       (1u << 16) | (uint32_t)(kBarQFull + t), 0xfffdu))
            return;
        tc_fence_after();
        const uint32_t o_own = tmem + (t ? kTmemO1 : kTmemO0) + 64u * (uint32_t)half;
        const uint32_t o_other = tmem + kTmemO1 + 64u * (uint32_t)half;
        uint8_t *line = smem_q + (size_t)t * kTileBytes + (size_t)half * kHalfTileBytes +
                        (size_t)r * 128;
        const int sw = r & 7;
        __nv_bfloat16 *direct =
            p.out + (((size_t)b * p.heads + h) * p.q_rows + (has_row ? row : 0u)) * kHeadDim +
            64 * half;
#pragma unroll 1
        for (int chunk = 0; chunk < 2; ++chunk) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.0f;
            if (use0) {
                uint32_t o[32];
                QW_TMEM_LD32(o_own + chunk * 32, o);
                QW_TMEM_WAIT_LD32(o);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]);
            }
            if (use1) {
                uint32_t o[32];
                QW_TMEM_LD32(o_other + chunk * 32, o);
                QW_TMEM_WAIT_LD32(o);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += __uint_as_float(o[i]);
            }
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                uint4 packed;
                packed.x = pack_bf16(v[i] * inv, v[i + 1] * inv);
                packed.y = pack_bf16(v[i + 2] * inv, v[i + 3] * inv);
                packed.z = pack_bf16(v[i + 4] * inv, v[i + 5] * inv);
                packed.w = pack_bf16(v[i + 6] * inv, v[i + 7] * inv);
                if (p.head_major_out) {
                    if (has_row) reinterpret_cast<uint4 *>(direct + chunk * 32)[i >> 3] = packed;
                } else {
                    const int c16 = chunk * 4 + (i >> 3);  // 16-byte piece of the 128-byte line
                    *reinterpret_cast<uint4 *>(line + ((c16 ^ sw) << 4)) = packed;
                }
            }
        }
        if (p.head_major_out) continue;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> TMA reads
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(&ctl->bars[kBarEpi + t]);
        if (tid == 0) {
            if (!mbar_wait(ctl, &ctl->bars[kBarEpi + t], 0, p.status,
                           (1u << 16) | (uint32_t)(kBarEpi + t), 0xfffcu))
                return;
            const uint8_t *stage = smem_q + (size_t)t * kTileBytes;
            const int col = (int)((p.out_head_offset + h) * kHeadDim);
            for (uint32_t d = 0; d < p.n_out; ++d) {
                tma_store_3d(&maps_out.m[d], stage, col, (int)tile_row0, (int)b);
                tma_store_3d(&maps_out.m[d], stage + kHalfTileBytes, col + 64, (int)tile_row0, (int)b);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
    // Shared memory may be released once the stores have read it.
    if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// MMA issue role (one thread).
// ---------------------------------------------------------------------------
// High words of the two descriptor kinds (everything but the start address).
constexpr uint32_t desc_hi(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // SBO, version 1, SWIZZLE_128B
}
constexpr uint32_t desc_lo_fixed(uint32_t lbo_bytes) { return ((lbo_bytes >> 4) & 0x3FFFu) << 16; }
constexpr uint32_t kDescHi = desc_hi(1024);
constexpr uint32_t kDescLoKMajor = desc_lo_fixed(16);               // LBO unused for K-major SW128
constexpr uint32_t kDescLoVMajor = desc_lo_fixed(kHalfTileBytes);   // next 64-column half

__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint32_t q_lo, uint32_t k_lo) {
    // K-major operands, 128B swizzle: 8-row groups 1024 B apart; the second
    // 64-column box sits one half tile further; 16 columns = 32 B per step.
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = ((uint32_t)(kk >> 2) * kHalfTileBytes + (uint32_t)(kk & 3) * 32u) >> 4;
        mma_ss(d_tmem, q_lo + off, kDescHi, k_lo + off, kDescHi, kIdescQK, kk > 0 ? 1u : 0u);
    }
}

__device__ __forceinline__ void issue_pv(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_lo,
                                         bool accumulate, bool paired) {
    // A = P from TMEM (16 keys = 8 packed columns per step).  B = V, MN-major:
    // 16 keys = 2 groups of 8 rows (1024 B apart), the two 64-wide column
    // halves one half tile apart.  P of keys 0..127 sits on columns 0..63 of the
    // score region; in the paired organisation each key half is written by its own
    // warp over its own scores, so keys 64..127 sit on columns 64..95.
    const uint32_t upper = paired ? 64u - 32u : 0u;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        const uint32_t col = (uint32_t)kk * 8u + (kk >= 4 ? upper : 0u);
        mma_ts(d_tmem, p_tmem + col, v_lo + (uint32_t)(kk * 2048 >> 4), kDescHi, kIdescPV,
               (accumulate || kk > 0) ? 1u : 0u);
    }
}

__device__ __forceinline__ void mma_role(const KernelParams &p, SharedControl *ctl,
                                         uint8_t *smem_q, uint8_t *smem_kv, bool paired) {
    // Whole form: both sub-tiles walk the visited tiles from 0; u counts them.
    const int n0 = ctl->tile_count[0], n1 = ctl->tile_count[1];
    const int n_max = max(n0, n1);
    int j = 0;
    if (j >= n_max) return;
    const uint32_t tmem = ctl->tmem_base;
    // Low descriptor words: start address in 16-byte units plus the fixed LBO field.
    const uint32_t q_lo[2] = {(smem_u32(smem_q) >> 4) | kDescLoKMajor,
                              (smem_u32(smem_q + kTileBytes) >> 4) | kDescLoKMajor};
    const uint32_t kv_lo = smem_u32(smem_kv) >> 4;  // slot s starts (s * kTileBytes) >> 4 further
    const uint32_t s_tmem[2] = {tmem + kTmemS0, tmem + kTmemS1};
    const uint32_t o_tmem[2] = {tmem + kTmemO0, tmem + kTmemO1};
    const int n_sub[2] = {n0, n1};
    uint32_t p_phase[2] = {0, 0};
    bool o_started[2] = {false, false};
    uint32_t t = 0;  // ring position (K and V tiles alternate)
    [[maybe_unused]] uint32_t trace_cursor = 0;
    [[maybe_unused]] uint32_t dbg_phase = 0;
    const uint32_t where = 2u << 16;

#pragma unroll
    for (int i = 0; i < 2; ++i)
        if (n_sub[i] > 0 &&
            !mbar_wait(ctl, &ctl->bars[kBarQFull + i], 0, p.status, where | (kBarQFull + i), 0))
            return;
    {
        uint32_t slot = t % kStages, par = (t / kStages) & 1u;
        ++t;
        if (!mbar_wait(ctl, &ctl->bars[kBarKvFull + slot], par, p.status,
                       where | (kBarKvFull + slot), (uint32_t)j))
            return;
        tc_fence_after();
        const uint32_t k_lo = (kv_lo + slot * (kTileBytes >> 4)) | kDescLoKMajor;
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (j < n_sub[i]) {
                issue_qk(s_tmem[i], q_lo[i], k_lo);
                tc_commit(&ctl->bars[kBarSFull + i]);
            }
        tc_commit(&ctl->bars[kBarKvEmpty + slot]);
    }
    while (j < n_max) {
        const int jn = j + 1;
        uint32_t v_slot = t % kStages, v_par = (t / kStages) & 1u;
        ++t;
        uint32_t k_slot = 0, k_par = 0;
        if (jn < n_max) {
            k_slot = t % kStages;
            k_par = (t / kStages) & 1u;
            ++t;
        }
        QW_TRACE(2, 6, j);
        if (!mbar_wait(ctl, &ctl->bars[kBarKvFull + v_slot], v_par, p.status,
                       where | (kBarKvFull + v_slot), (uint32_t)j))
            return;
        QW_TRACE(2, 7, j);
        const uint32_t v_lo = (kv_lo + v_slot * (kTileBytes >> 4)) | kDescLoVMajor;
        const uint32_t k_lo = (kv_lo + k_slot * (kTileBytes >> 4)) | kDescLoKMajor;
        bool k_ready = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (j < n_sub[i]) {
                if (!mbar_wait(ctl, &ctl->bars[kBarPFull + i], p_phase[i], p.status,
                               where | (kBarPFull + i), (uint32_t)j))
                    return;
                p_phase[i] ^= 1u;
                tc_fence_after();
                QW_TRACE(2, i, j);
                issue_pv(o_tmem[i], s_tmem[i], v_lo, o_started[i], paired);
                o_started[i] = true;
                QW_TRACE(2, 4 + i, j);
            }
            if (i == 1) tc_commit(&ctl->bars[kBarKvEmpty + v_slot]);
            if (jn < n_max && jn < n_sub[i]) {
                if (!k_ready) {
                    QW_TRACE(2, 8, jn);
                    if (!mbar_wait(ctl, &ctl->bars[kBarKvFull + k_slot], k_par, p.status,
                                   where | (kBarKvFull + k_slot), (uint32_t)jn))
                        return;
                    tc_fence_after();
                    k_ready = true;
                    QW_TRACE(2, 9, jn);
                }
                issue_qk(s_tmem[i], q_lo[i], k_lo);
                tc_commit(&ctl->bars[kBarSFull + i]);
                QW_TRACE(2, 2 + i, jn);
#ifdef QW_ATTN_TRACE_SERIAL
                // Probe: wait until the group just issued has executed.
                tc_commit(&ctl->bars[kBarDebug]);
                if (!mbar_wait(ctl, &ctl->bars[kBarDebug], dbg_phase, p.status, where | kBarDebug, 0))
                    return;
                dbg_phase ^= 1u;
                QW_TRACE(2, 10 + i, jn);
#endif
            }
        }
        if (jn < n_max) {
            if (!k_ready &&
                !mbar_wait(ctl, &ctl->bars[kBarKvFull + k_slot], k_par, p.status,
                           where | (kBarKvFull + k_slot), (uint32_t)jn))
                return;
            tc_commit(&ctl->bars[kBarKvEmpty + k_slot]);
        }
        j = jn;
    }
    tc_commit(&ctl->bars[kBarOFinal + 0]);
    tc_commit(&ctl->bars[kBarOFinal + 1]);
}

// Split form: sub-tile 0 walks visited tiles [0, la), sub-tile 1 [la, la + lb),
// both against the one Q tile.  K/V pairs are loaded in the order a0 b0 a1 b1 ...
// (pair = K then V, one ring slot each); slot_of() gives the ring position of a
// pair's K, its V follows.
__device__ __forceinline__ uint32_t pair_a(int s, int lb) { return 2u * (uint32_t)(s + min(s, lb)); }
__device__ __forceinline__ uint32_t pair_b(int s) { return 2u * (uint32_t)(2 * s + 1); }

__device__ __forceinline__ void mma_role_split(const KernelParams &p, SharedControl *ctl,
                                               uint8_t *smem_q, uint8_t *smem_kv, bool paired) {
    const int la = ctl->tile_count[0], lb = ctl->tile_count[1];
    if (la <= 0) return;
    const uint32_t tmem = ctl->tmem_base;
    const uint32_t q_lo = (smem_u32(smem_q) >> 4) | kDescLoKMajor;
    const uint32_t kv_lo = smem_u32(smem_kv) >> 4;
    const uint32_t s_tmem[2] = {tmem + kTmemS0, tmem + kTmemS1};
    const uint32_t o_tmem[2] = {tmem + kTmemO0, tmem + kTmemO1};
    const uint32_t where = 2u << 16;
    uint32_t p_phase[2] = {0, 0};

    // Waits for ring position t, returns the low descriptor word of its slot.
#define QW_RING_WAIT(t_, lo_fixed_, out_)                                                       \
    {                                                                                           \
        const uint32_t slot_ = (t_) % kStages, par_ = ((t_) / kStages) & 1u;                    \
        if (!mbar_wait(ctl, &ctl->bars[kBarKvFull + slot_], par_, p.status,                     \
                       where | (kBarKvFull + slot_), (uint32_t)(t_)))                           \
            return;                                                                             \
        tc_fence_after();                                                                       \
        out_ = (kv_lo + slot_ * (kTileBytes >> 4)) | (lo_fixed_);                               \
    }
#define QW_RING_FREE(t_) tc_commit(&ctl->bars[kBarKvEmpty + ((t_) % kStages)])

    if (!mbar_wait(ctl, &ctl->bars[kBarQFull + 0], 0, p.status, where | kBarQFull, 0)) return;
    uint32_t desc;
    QW_RING_WAIT(pair_a(0, lb), kDescLoKMajor, desc);
    issue_qk(s_tmem[0], q_lo, desc);
    tc_commit(&ctl->bars[kBarSFull + 0]);
    QW_RING_FREE(pair_a(0, lb));
    if (lb > 0) {
        QW_RING_WAIT(pair_b(0), kDescLoKMajor, desc);
        issue_qk(s_tmem[1], q_lo, desc);
        tc_commit(&ctl->bars[kBarSFull + 1]);
        QW_RING_FREE(pair_b(0));
    }
    for (int s = 0; s < la; ++s) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int count = i ? lb : la;
            if (s >= count) continue;
            const uint32_t t_now = i ? pair_b(s) : pair_a(s, lb);
            QW_RING_WAIT(t_now + 1, kDescLoVMajor, desc);
            if (!mbar_wait(ctl, &ctl->bars[kBarPFull + i], p_phase[i], p.status,
                           where | (kBarPFull + i), (uint32_t)s))
                return;
            p_phase[i] ^= 1u;
            tc_fence_after();
            issue_pv(o_tmem[i], s_tmem[i], desc, s > 0, paired);
            QW_RING_FREE(t_now + 1);
            if (s + 1 < count) {
                const uint32_t t_next = i ? pair_b(s + 1) : pair_a(s + 1, lb);
                QW_RING_WAIT(t_next, kDescLoKMajor, desc);
                issue_qk(s_tmem[i], q_lo, desc);
                tc_commit(&ctl->bars[kBarSFull + i]);
                QW_RING_FREE(t_next);
            }
        }
    }
#undef QW_RING_WAIT
#undef QW_RING_FREE
    tc_commit(&ctl->bars[kBarOFinal + 0]);
    tc_commit(&ctl->bars[kBarOFinal + 1]);
}

// ---------------------------------------------------------------------------
// TMA producer role (one thread).
// ---------------------------------------------------------------------------
__device__ void tma_role(const KernelParams &p, SharedControl *ctl, uint8_t *smem_kv,
                         const CUtensorMap *map_k, const CUtensorMap *map_v, uint32_t b,
                         uint32_t kvh, bool split) {
    const uint32_t where = 3u << 16;
    // K and V of the first visited tile are already on their way (ring slots 0, 1):
    // the kernel body issued them before the row limits were known.
    uint32_t t = 2;
    bool ok = true;
    const int col = (int)(kvh * kHeadDim);
    // One (K, V) pair of visited tile u into the next two ring slots.
    auto load_pair = [&](int u) {
        if (p.withhold_from >= 0 && u >= p.withhold_from) {
            ok = false;  // the tile stays away: nothing is issued, nothing is in flight
            return;
        }
        const int j = phys_tile(ctl, u);
        for (int which = 0; which < 2 && ok; ++which) {
            uint32_t slot = t % kStages, par = ((t / kStages) & 1u) ^ 1u;
            ok = mbar_wait(ctl, &ctl->bars[kBarKvEmpty + slot], par, p.status,
                           where | (kBarKvEmpty + slot), (uint32_t)j);
            if (!ok) break;
            ++t;
            uint8_t *dst = smem_kv + (size_t)slot * kTileBytes;
            unsigned long long *bar = &ctl->bars[kBarKvFull + slot];
            mbar_expect_tx(bar, kTileBytes);
            const CUtensorMap *map = which ? map_v : map_k;
            tma_load_3d(dst, map, bar, col, j * kTileN, (int)b);
            tma_load_3d(dst + kHalfTileBytes, map, bar, col + 64, j * kTileN, (int)b);
        }
    };
    if (!split) {
        const int n_max = max(ctl->tile_count[0], ctl->tile_count[1]);
        for (int u = 1; u < n_max && ok; ++u) load_pair(u);
    } else {
        // pairs in the order a0 (under way), b0, a1, b1, ...
        const int la = ctl->tile_count[0], lb = ctl->tile_count[1];
        for (int s = 0; s < la && ok; ++s) {
            if (s > 0) load_pair(s);
            if (s < lb && ok) load_pair(la + s);
        }
    }
    // Leave no copy in flight: every issued load must have landed before the
    // CTA may release its shared memory (bounded like every other wait).
    uint32_t first = t > (uint32_t)kStages ? t - kStages : 0;
    for (uint32_t u = first; u < t; ++u) {
        uint32_t slot = u % kStages, par = (u / kStages) & 1u;
        long long start = clock64();
        while (!mbar_try(&ctl->bars[kBarKvFull + slot], par))
            if (clock64() - start > ctl->wait_cycles) break;
    }
}

__device__ __forceinline__ void issue_q_loads(const KernelParams &p, SharedControl *ctl,
                                              uint8_t *smem_q, const CUtensorMap *map_q, uint32_t b,
                                              uint32_t h, uint32_t row0, int tiles) {
    for (int i = 0; i < tiles; ++i) {
        uint32_t r = row0 + (uint32_t)i * kTileM;
        if (r >= p.q_rows) continue;  // inactive sub-tile: n_tiles is 0, nobody waits
        unsigned long long *bar = &ctl->bars[kBarQFull + i];
        mbar_expect_tx(bar, kTileBytes);
        uint8_t *dst = smem_q + (size_t)i * kTileBytes;
        tma_load_3d(dst, map_q, bar, (int)(h * kHeadDim), (int)r, (int)b);
        tma_load_3d(dst + kHalfTileBytes, map_q, bar, (int)(h * kHeadDim) + 64, (int)r, (int)b);
    }
}

template <int kPoly, bool kMayBound>
__global__ void __launch_bounds__(kThreads, 1)
qw_attn_sm100_kernel(const __grid_constant__ CUtensorMap map_q,
                     const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v,
                     const __grid_constant__ OutMaps maps_out, const KernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_q = smem;
    uint8_t *smem_kv = smem + 2 * kTileBytes;
    SharedControl *ctl = reinterpret_cast<SharedControl *>(smem + kSmemData);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    // CTA -> unit.  Units are numbered batch-major, then head, then query block
    // with the heaviest blocks first (rows late in the joint sequence see the most
    // keys).  The last tail_units units run in split form, two CTAs each.
    const uint32_t whole_units = p.total_units - p.tail_units;
    const bool split = blockIdx.x >= whole_units;
    const uint32_t unit = split ? whole_units + ((blockIdx.x - whole_units) >> 1) : blockIdx.x;
    const uint32_t half = split ? (blockIdx.x - whole_units) & 1u : 0u;
    const uint32_t bh = unit / p.n_qblocks;
    const uint32_t b = bh / p.heads;
    const uint32_t h = bh - b * p.heads;
    const uint32_t kvh = (uint32_t)((unsigned long long)h * p.kv_heads / p.heads);
    const uint32_t qblock = p.n_qblocks - 1 - (unit - bh * p.n_qblocks);
    const uint32_t row0 = qblock * (2 * kTileM) + half * kTileM;

    // The producer thread sets the barriers up itself and starts Q and the first
    // K/V tile at once, under the row-limit loads of the softmax threads.
    if (warp == kTmaWarp && lane == 0) {
        for (int i = 0; i < 2; ++i) mbar_init(&ctl->bars[kBarQFull + i], 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&ctl->bars[kBarKvFull + i], 1);
            mbar_init(&ctl->bars[kBarKvEmpty + i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctl->bars[kBarSFull + i], 1);
            mbar_init(&ctl->bars[kBarPFull + i], kSoftmaxThreads / 32);
            mbar_init(&ctl->bars[kBarOFinal + i], 1);
            mbar_init(&ctl->bars[kBarEpi + i], kSoftmaxThreads / 32);
        }
        mbar_init(&ctl->bars[kBarMerge], kTileM / 32);
        mbar_init(&ctl->bars[kBarDebug], 1);
        ctl->abort_flag = 0;
        ctl->wait_cycles = p.wait_cycles > 0 ? p.wait_cycles : kWaitCycles;
        int lo = 0, hi = 0;
        if (p.text_pad && p.text_len[b] < p.text_pad) {
            lo = ((int)p.text_len[b] + kTileN - 1) / kTileN;
            hi = (int)p.text_pad / kTileN;
            if (hi < lo) hi = lo;
        }
        ctl->skip_lo = lo;
        ctl->skip_hi = hi;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        issue_q_loads(p, ctl, smem_q, &map_q, b, h, row0, split ? 1 : 2);
        // First visited key tile, assuming the unit has one (if it has none the
        // tile is simply never consumed; the producer drains it before exit).
        const int j0 = lo == 0 ? hi : 0;
        for (int which = 0; which < 2; ++which) {
            uint8_t *dst = smem_kv + (size_t)which * kTileBytes;
            unsigned long long *bar = &ctl->bars[kBarKvFull + which];
            mbar_expect_tx(bar, kTileBytes);
            const CUtensorMap *map = which ? &map_v : &map_k;
            const int col = (int)(kvh * kHeadDim);
            tma_load_3d(dst, map, bar, col, j0 * kTileN, (int)b);
            tma_load_3d(dst + kHalfTileBytes, map, bar, col + 64, j0 * kTileN, (int)b);
        }
    }
    if (blockIdx.x == 0 && warp == 10 && lane == 0 && p.slot_use) {
        // Sharded heads: whatever read this output slot's previous contents was
        // enqueued before this kernel, so the peers may store the new epoch now.
        const uint32_t epoch = *p.slot_use + 1u;
        *p.slot_use = epoch;
        __threadfence_system();
        for (uint32_t d = 0; d < p.n_freed; ++d)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.freed_peer[d]), "r"(epoch)
                         : "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctl->tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // Row limits: each softmax thread owns one row; the largest limit of a
    // sub-tile bounds its key-tile loop.
    int my_limit = 0;
    uint32_t my_row = 0;
    int sub = 0, tid_in_group = 0;
    // Fixed reference exponent (log2 units, an integer so that P is the exact
    // power-of-two multiple of what any other reference would give), or < 0 for
    // the running-maximum softmax: no promise given, or one too loose to keep
    // exp2(score*c - bound) >= 2^-2*bound inside the normal fp32 range.
    float bound = -1.0f;
    if (kMayBound && p.score_bound) {  // every role needs to know which softmax runs
        const float limit = ceilf(p.score_bound[0] * p.score_bound[1] * p.scale_log2);
        if (limit >= 0.0f && limit <= 60.0f) bound = limit;
    }
    // Paired organisation of the fixed-exponent softmax (both warpgroups on one
    // sub-tile at a time) unless the launch asks for one thread per row.
    const bool paired = kMayBound && bound >= 0.0f && p.pair_org;
    int other_limit = 0;
    if (tid < kSoftmaxThreads) {
        sub = tid >> 7;
        tid_in_group = tid & 127;
        // (split form: both warpgroups work on the same 128 rows)
        my_row = row0 + (split ? 0u : (uint32_t)sub * kTileM) + (uint32_t)tid_in_group;
        my_limit = row_limit(p, b, my_row);
        // (paired: this thread also works on the same row of the other sub-tile)
        if (paired)
            other_limit = split ? my_limit
                                : row_limit(p, b, row0 + (uint32_t)(1 - sub) * kTileM +
                                                      (uint32_t)tid_in_group);
        int warp_max = my_limit;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            warp_max = max(warp_max, __shfl_xor_sync(0xffffffffu, warp_max, off));
        if (lane == 0) ctl->warp_max[warp] = warp_max;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid < 2) {
        int m = 0;
        for (int w = 0; w < 4; ++w) m = max(m, ctl->warp_max[tid * 4 + w]);
        const int tiles = (m + kTileN - 1) / kTileN;
        ctl->n_tiles[tid] = tiles;
        const int visited = visited_tiles(tiles, ctl->skip_lo, ctl->skip_hi);
        if (!split) {
            ctl->tile_first[tid] = 0;
            ctl->tile_count[tid] = visited;
        } else {
            // both warpgroups saw the same rows: the first half (rounded up) and the rest
            const int first_half = (visited + 1) / 2;
            ctl->tile_first[tid] = tid ? first_half : 0;
            ctl->tile_count[tid] = tid ? visited - first_half : first_half;
        }
    }
    __syncthreads();

    if (tid < kSoftmaxThreads) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        uint8_t *stage = smem_q + (size_t)sub * kTileBytes;
        const uint32_t tile_row0 = split ? row0 : row0 + (uint32_t)sub * kTileM;
        if (paired)
            softmax_pair_role<kPoly>(p, ctl, maps_out, smem_q, tid, sub ? other_limit : my_limit,
                                     sub ? my_limit : other_limit, b, h, row0, split, bound);
        else if (kMayBound && bound >= 0.0f)
            softmax_role<kPoly, kMayBound>(p, ctl, maps_out, stage, sub, tid_in_group, my_limit, b,
                                           h, my_row, tile_row0, split, bound);
        else
            softmax_role<kPoly, false>(p, ctl, maps_out, stage, sub, tid_in_group, my_limit, b, h,
                                       my_row, tile_row0, split, 0.0f);
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    }
    if (tid < kSoftmaxThreads) {
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            if (split) mma_role_split(p, ctl, smem_q, smem_kv, paired);
            else mma_role(p, ctl, smem_q, smem_kv, paired);
        }
    } else if (warp == kTmaWarp && lane == 0) {
        tma_role(p, ctl, smem_kv, &map_k, &map_v, b, kvh, split);
        // Q loads of active sub-tiles must have landed as well.
        for (int i = 0; i < (split ? 1 : 2); ++i) {
            if (row0 + (uint32_t)i * kTileM >= p.q_rows) continue;
            long long start = clock64();
            while (!mbar_try(&ctl->bars[kBarQFull + i], 0))
                if (clock64() - start > ctl->wait_cycles) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(ctl->tmem_base),
                     "r"(kTmemCols)
                     : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [batch][rows][heads*128] bf16, boxes of 128 rows x 64 columns, 128B swizzle.
int make_map(CUtensorMap *map, const void *base, uint32_t batch, uint32_t rows, uint32_t heads) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[3] = {(cuuint64_t)heads * kHeadDim, rows, batch};
    cuuint64_t strides[2] = {(cuuint64_t)heads * kHeadDim * 2,
                             (cuuint64_t)rows * heads * kHeadDim * 2};
    cuuint32_t box[3] = {64, kTileN, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims,
                    strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

#ifdef QW_ATTN_TRACE
// QW_CUDA_ATTN_TRACE=<file>: attach an event log to every launch and dump it after
// each one (synchronous; a debugging aid, never set in production runs).
unsigned long long *trace_buffer() {
    static unsigned long long *buffer = nullptr;
    static bool looked = false;
    if (!looked) {
        looked = true;
        const char *path = getenv("QW_CUDA_ATTN_TRACE");
        if (path && *path) {
            if (cudaMalloc(&buffer, kTraceSlots * 8) != cudaSuccess) buffer = nullptr;
            else cudaMemset(buffer, 0, kTraceSlots * 8);
        }
    }
    return buffer;
}

void trace_dump(cudaStream_t stream) {
    unsigned long long *buffer = trace_buffer();
    if (!buffer) return;
    static unsigned long long host[kTraceSlots];
    cudaStreamSynchronize(stream);
    cudaMemcpy(host, buffer, sizeof(host), cudaMemcpyDeviceToHost);
    cudaMemset(buffer, 0, kTraceSlots * 8);
    FILE *f = fopen(getenv("QW_CUDA_ATTN_TRACE"), "a");
    if (!f) return;
    fprintf(f, "launch\n");
    for (int i = 1; i < kTraceSlots; ++i) {
        unsigned long long w = host[i];
        if (!w) continue;
        unsigned tag = (unsigned)(w >> 40);
        fprintf(f, "%u %u %u %llu\n", tag >> 20, (tag >> 12) & 0xff, tag & 0xfff,
                w & 0xffffffffffull);
    }
    fclose(f);
}
#endif

typedef void (*AttnKernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const OutMaps,
                           const KernelParams);

int sm_count_of_current_device() {
    static int sms[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        if (sms[dev] <= 0) sms[dev] = 148;
    }
    return sms[dev];
}

// QW_CUDA_ATTN_TAIL=whole: never split the last wave's units (comparison runs).
bool whole_units_forced() {
    static int forced = -1;
    if (forced < 0) {
        const char *env = getenv("QW_CUDA_ATTN_TAIL");
        forced = env && !strcmp(env, "whole") ? 1 : 0;
    }
    return forced != 0;
}

// QW_CUDA_SOFTMAX_ORG=row / pair: force the organisation of the fixed-exponent
// softmax (one thread per row, or both warpgroups on one sub-tile's keys at a time)
// instead of choosing by the length of the launch (comparison runs).  -1 = not set.
int softmax_org_forced() {
    static int forced = -2;
    if (forced == -2) {
        const char *env = getenv("QW_CUDA_SOFTMAX_ORG");
        forced = !env ? -1 : !strcmp(env, "row") ? 0 : !strcmp(env, "pair") ? 1 : -1;
    }
    return forced;
}

// The kernel variants: how many of every 4 score pairs take the polynomial exp2
// (QW_CUDA_EXP_POLY=0..2 overrides the default for tuning), with or without the
// fixed-exponent softmax for callers that pass a score bound.  The opt-in to
// ~197 KB of dynamic shared memory is a per-device attribute: it is set on first
// use on every device a process drives.
AttnKernel pick_kernel(bool may_bound) {
    static int poly = -1;
    static bool ready[64][2];
    if (poly < 0) {
        const char *env = getenv("QW_CUDA_EXP_POLY");
        poly = (env && env[0] >= '0' && env[0] <= '2' && !env[1]) ? env[0] - '0' : 0;
    }
    AttnKernel table[3][2] = {
        {qw_attn_sm100_kernel<0, false>, qw_attn_sm100_kernel<0, true>},
        {qw_attn_sm100_kernel<1, false>, qw_attn_sm100_kernel<1, true>},
        {qw_attn_sm100_kernel<2, false>, qw_attn_sm100_kernel<2, true>},
    };
    AttnKernel chosen = table[poly][may_bound ? 1 : 0];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    const bool tracked = dev >= 0 && dev < 64;
    if (!tracked || !ready[dev][may_bound ? 1 : 0]) {
        if (cudaFuncSetAttribute(chosen, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBytes) != cudaSuccess)
            return nullptr;
        if (tracked) ready[dev][may_bound ? 1 : 0] = true;
    }
    return chosen;
}

}  // namespace

// Units of the last, partly filled wave that run in split form: all of them when
// the doubled CTAs still fit the SMs (a sixteenth over is tolerated: block-causal
// layouts always have a few near-empty units that retire at once), none otherwise
// -- two half-length waves would take as long as the one they replace.
extern "C" uint32_t qwcu_attn_sm100_tail_units(uint32_t units, uint32_t sm_count) {
    if (!sm_count) return 0;
    const uint32_t rest = units % sm_count;
    return rest && 2 * rest <= sm_count + sm_count / 16 ? rest : 0u;
}

extern "C" int qwcu_attn_sm100_launch(const qwcu_attn_args *a, qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (a->batch == 0 || a->batch > 8 || !a->q_rows || !a->kv_rows || !a->heads || !a->kv_heads)
        return (int)cudaErrorInvalidValue;
    // TMA needs 16-byte aligned bases; cudaMalloc gives 256.
    if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->out) & 15u)
        return (int)cudaErrorMisalignedAddress;
    AttnKernel kernel = pick_kernel(a->score_bound != nullptr);
    if (!kernel) return (int)cudaGetLastError();
    CUtensorMap map_q, map_k, map_v;
    int rc;
    if ((rc = make_map(&map_q, a->q, a->batch, a->q_rows, a->heads))) return rc;
    if ((rc = make_map(&map_k, a->k, a->batch, a->kv_rows, a->kv_heads))) return rc;
    if ((rc = make_map(&map_v, a->v, a->batch, a->kv_rows, a->kv_heads))) return rc;
    KernelParams p;
    p.out = static_cast<__nv_bfloat16 *>(a->out);
    p.kv_limit = a->kv_limit;
    p.status = a->status;
#ifdef QW_ATTN_TRACE
    p.trace = trace_buffer();
#endif
    p.per_batch_limits = a->per_batch_limits;
    p.causal = a->causal;
    p.causal_offset = a->causal_offset;
    p.batch = a->batch;
    p.q_rows = a->q_rows;
    p.kv_rows = a->kv_rows;
    p.heads = a->heads;
    p.kv_heads = a->kv_heads;
    for (int i = 0; i < 8; ++i) p.text_len[i] = a->text_len[i];
    p.text_pad = a->text_pad;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.score_bound = a->score_bound;
    p.pair_org = -1;  // decided below, once the unit count is known
    p.head_major_out = a->head_major_out;
    if (a->n_out_peers > 0) {
        if (a->n_out_peers > 8 || a->head_major_out) return (int)cudaErrorInvalidValue;
        p.n_out = a->n_out_peers;
        for (uint32_t d = 0; d < p.n_out; ++d) {
            if ((uintptr_t)a->out_peers[d] & 15u) return (int)cudaErrorMisalignedAddress;
            p.out_peers[d] = static_cast<__nv_bfloat16 *>(a->out_peers[d]);
        }
        p.out_heads_total = a->out_heads_total;
        p.out_head_offset = a->out_head_offset;
    } else {
        p.n_out = 1;
        p.out_peers[0] = p.out;
        p.out_heads_total = a->heads;
        p.out_head_offset = 0;
    }
    p.wait_cycles = a->wait_cycles;
    p.withhold_from = a->withhold_from > 0 ? a->withhold_from : -1;
    p.slot_use = a->slot_use;
    p.n_freed = a->slot_use ? a->n_freed : 0;
    if (p.n_freed > 8) return (int)cudaErrorInvalidValue;
    for (uint32_t d = 0; d < 8; ++d) p.freed_peer[d] = d < p.n_freed ? a->freed_peer[d] : nullptr;
    OutMaps maps_out;
    memset(&maps_out, 0, sizeof(maps_out));
    if (!p.head_major_out)
        for (uint32_t d = 0; d < p.n_out; ++d)
            if ((rc = make_map(&maps_out.m[d], p.out_peers[d], a->batch, a->q_rows, p.out_heads_total)))
                return rc;
    // One CTA per unit; the units of the last, partly filled wave run split in two
    // (half the rows each, the key tiles divided between the sub-tiles) when the
    // doubled CTAs still fit the idle SMs, give or take a few light units.
    const unsigned long long units =
        (unsigned long long)((a->q_rows + 2 * kTileM - 1) / (2 * kTileM)) * a->heads * a->batch;
    if (units > 0x3fffffffull) return (int)cudaErrorInvalidValue;
    p.n_qblocks = (a->q_rows + 2 * kTileM - 1) / (2 * kTileM);
    p.total_units = (uint32_t)units;
    p.tail_units = (a->whole_units || whole_units_forced())
                       ? 0u
                       : qwcu_attn_sm100_tail_units(p.total_units,
                                                    (uint32_t)sm_count_of_current_device());
    // Fixed-exponent softmax: paired organisation where the launch is short (at most
    // two waves of CTAs: the per-tile latency chain is what bounds it), one thread per
    // row where it is long (many waves run at the board's power limit, where the
    // organisation with fewer instructions per score is the faster one).
    {
        const int forced = softmax_org_forced();
        const bool long_launch =
            p.total_units > 2u * (uint32_t)sm_count_of_current_device();
        p.pair_org = a->row_softmax ? 0 : forced >= 0 ? forced : long_launch ? 0 : 1;
    }
    const unsigned grid = p.total_units + p.tail_units;
    kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, maps_out, p);
    rc = (int)cudaGetLastError();
#ifdef QW_ATTN_TRACE
    if (p.trace && !rc) trace_dump(stream);
#endif
    return rc;
}
