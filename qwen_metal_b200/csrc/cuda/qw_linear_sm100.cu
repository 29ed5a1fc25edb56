// bf16 linear layers of the DiT block on the tensor cores of sm_100a:
//   C[M, N] = A[M, K] * W[N, K]^T (+ bias), fp32 accumulate, one rounding to bf16
// (reference h3_gpu_linear_bf16: h3_gpu.m:2697-2812, h3_shaders.metal:788-822), and
// the fused q/k/v projection, three such products sharing A in one launch
// (reference qw_gpu_qkv_bf16: h3_gpu.m:2918-3018, called qwen_dit.m:1270).  The
// weights keep the checkpoint's [out, in] layout, which is the K-major B operand.
//
// Persistent CTAs, one per SM; tile 128 (M) x 256 (N), K step 64 (one 128-byte
// swizzle row):
//   warp 0 lane 0 : TMA producer  (A tile 16 KB + W tile 32 KB per stage, 4 stages)
//   warp 1 lane 0 : MMA issuer    (tcgen05.mma cta_group::1 kind::f16, M128 N256 K16)
//   warps 2..5    : epilogue      (TMEM -> registers -> bf16 -> swizzled staging ->
//                                  TMA store), TMEM lane quarter = warp % 4
// Two TMEM accumulators (2 x 256 columns) let the epilogue of tile i run under the
// main loop of tile i + 1.  Shared memory: 192 KB ring + 2 x 16 KB staging.
//
// Optional fused epilogue (q and k of the DiT block): a 256-column tile is two whole
// heads of 128 and a thread owns one row of it, so the per-head RMSNorm needs no
// exchange between threads and follows the reference's serial fma order exactly;
// the interleaved RoPE follows with the row's cos/sin.  The bf16 roundings the
// reference has between its three kernels are reproduced, which makes the result
// the same as GEMM -> h3_gpu_head_rms_norm_bf16 -> qw_gpu_qk_rope_bf16 without the
// two extra passes over q and k.
//
// Every wait is bounded (status words, abort flag); the epilogue's group barrier is
// reached by all of its threads on every path.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../qw_cuda.h"

namespace {

constexpr int kTileM = 128, kTileN = 256, kTileK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kTileM * kTileK * 2;  // 16 KB
constexpr int kWBytes = kTileN * kTileK * 2;  // 32 KB
constexpr int kStageBytes = kABytes + kWBytes;
constexpr int kStagingBytes = kTileM * 64 * 2;  // 16 KB, one 64-column box
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr long long kWaitCycles = 400000000LL;

enum Barrier : int {
    kBarFull = 0,                     // kStages: stage landed
    kBarEmpty = kBarFull + kStages,   // kStages: stage consumed
    kBarAccFull = kBarEmpty + kStages,  // 2: accumulator complete
    kBarAccEmpty = kBarAccFull + 2,     // 2: accumulator drained (4 warp arrivals)
    kBarCount = kBarAccEmpty + 2
};

struct __align__(16) Control {
    unsigned long long bars[kBarCount];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
    volatile uint32_t epilogue_go;  // the epilogue's one waiting thread tells the other 127
};

constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 2 * kStagingBytes + sizeof(Control) + 1024;

constexpr int kMaxOutputs = 3;

struct Params {
    uint32_t m, k;
    uint32_t n_each;            // columns of every output
    uint32_t n_outputs;         // 1 (linear) or 3 (q, k, v)
    uint32_t tiles_per_output;  // ceil(n_each / kTileN)
    const uint16_t *bias[kMaxOutputs];  // bf16 [n_each] or null
    uint32_t *status;
    // Optional fused epilogue for outputs 0 and 1 (q and k of the DiT block): per-head
    // RMSNorm over 128 columns and interleaved RoPE, with the reference's bf16
    // roundings between the stages (GEMM result -> bf16 -> norm -> bf16 -> rotation).
    const uint16_t *norm_weight[2];  // bf16 [128] each, null = plain output
    const float *rope_cos, *rope_sin;  // f32 [table_rows][64]
    uint32_t table_rows;               // table row = output row % table_rows
    float epsilon;
    float *bound_out;  // optional: [0], [1] = bounds of the 2-norm of any q row, k row
};

struct Maps {
    CUtensorMap w[kMaxOutputs];
    CUtensorMap c[kMaxOutputs];
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long *bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait(Control *ctl, unsigned long long *bar, uint32_t parity,
                                          uint32_t *status, uint32_t where) {
    if (mbar_try(bar, parity)) return true;
    long long start = clock64();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if (mbar_try(bar, parity)) return true;
        if (ctl->abort_flag) return false;
        if (clock64() - start > kWaitCycles) {
            ctl->abort_flag = 1;
            if (atomicCAS(status, 0u, 1u) == 0u) { status[1] = where; status[3] = blockIdx.x; }
            __threadfence();
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, unsigned long long *bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// descriptor words as in the attention kernel: K-major, 128B swizzle, SBO = 1024
constexpr uint32_t kDescHi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescLo = ((16u >> 4) & 0x3FFFu) << 16;
// instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N = 256, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                 "setp.ne.b32 p, %6, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_lo), "r"(kDescHi), "r"(b_lo), "r"(kDescHi), "r"(kIdesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
#define TMEM_LD32(taddr, r)                                                                        \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                        \
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "       \
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];" \
                 : "=r"((r)[0]), "=r"((r)[1]), "=r"((r)[2]), "=r"((r)[3]), "=r"((r)[4]), "=r"((r)[5]),   \
                   "=r"((r)[6]), "=r"((r)[7]), "=r"((r)[8]), "=r"((r)[9]), "=r"((r)[10]), "=r"((r)[11]), \
                   "=r"((r)[12]), "=r"((r)[13]), "=r"((r)[14]), "=r"((r)[15]), "=r"((r)[16]),            \
                   "=r"((r)[17]), "=r"((r)[18]), "=r"((r)[19]), "=r"((r)[20]), "=r"((r)[21]),            \
                   "=r"((r)[22]), "=r"((r)[23]), "=r"((r)[24]), "=r"((r)[25]), "=r"((r)[26]),            \
                   "=r"((r)[27]), "=r"((r)[28]), "=r"((r)[29]), "=r"((r)[30]), "=r"((r)[31])             \
                 : "r"(taddr))

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Tile order: N tiles fastest inside a band of M tiles, so the CTAs running side by
// side share the A band and stream the weights through L2.
__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t n_tiles, uint32_t &tm,
                                            uint32_t &tn) {
    tm = tile / n_tiles;
    tn = tile - tm * n_tiles;
}

// One head (128 columns) of one row out of the accumulator, as 64 packed bf16 pairs:
// the GEMM result rounded to bf16 (plus bias), and for q / k the per-head RMSNorm
// and the rotation on top, each stage rounded to bf16 like the reference's kernels.
__device__ __forceinline__ void head_from_tmem(uint32_t (&pk)[64], uint32_t taddr,
                                               const uint16_t *bias, const float *norm_w,
                                               const float *cos_row, const float *sin_row,
                                               float epsilon) {
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        TMEM_LD32(taddr + (uint32_t)(c * 32), o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float lo = __uint_as_float(o[2 * i]), hi = __uint_as_float(o[2 * i + 1]);
            if (bias) {
                const uint32_t b2 = *reinterpret_cast<const uint32_t *>(bias + c * 32 + 2 * i);
                lo = __fadd_rn(lo, bf16_lo(b2));
                hi = __fadd_rn(hi, bf16_hi(b2));
            }
            const uint32_t w = pack_bf16(lo, hi);
            pk[c * 16 + i] = w;
            if (norm_w) {  // serial fma over the bf16 values, element order 0..127
                ss = fmaf(bf16_lo(w), bf16_lo(w), ss);
                ss = fmaf(bf16_hi(w), bf16_hi(w), ss);
            }
        }
    }
    if (!norm_w) return;
    const float inverse = 1.0f / sqrtf(__fadd_rn(ss / 128.0f, epsilon));
#pragma unroll
    for (int q4 = 0; q4 < 16; ++q4) {  // four rotation pairs at a time
        const float4 c4 = *reinterpret_cast<const float4 *>(cos_row + 4 * q4);
        const float4 s4 = *reinterpret_cast<const float4 *>(sin_row + 4 * q4);
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int pair = 4 * q4 + u;
            const uint32_t w = pk[pair];
            // n = bf16(x * inv * w), stored as bf16 between the norm and the rotation
            const uint32_t n = pack_bf16(__fmul_rn(__fmul_rn(bf16_lo(w), inverse), norm_w[2 * pair]),
                                         __fmul_rn(__fmul_rn(bf16_hi(w), inverse), norm_w[2 * pair + 1]));
            const float e = bf16_lo(n), o = bf16_hi(n);
            pk[pair] = pack_bf16(__fsub_rn(__fmul_rn(e, cc[u]), __fmul_rn(o, sn[u])),
                                 __fadd_rn(__fmul_rn(e, sn[u]), __fmul_rn(o, cc[u])));
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1)
qw_linear_sm100_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ Maps maps,
                       const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *ring = smem;
    uint8_t *staging = smem + (size_t)kStages * kStageBytes;
    Control *ctl = reinterpret_cast<Control *>(staging + 2 * kStagingBytes);
    __shared__ float norm_w[2][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (p.m + kTileM - 1) / kTileM;
    const uint32_t n_tiles = p.tiles_per_output * p.n_outputs;
    const uint32_t tiles = m_tiles * n_tiles, k_steps = (p.k + kTileK - 1) / kTileK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&ctl->bars[kBarFull + i], 1);
            mbar_init(&ctl->bars[kBarEmpty + i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctl->bars[kBarAccFull + i], 1);
            mbar_init(&ctl->bars[kBarAccEmpty + i], 4);
        }
        ctl->abort_flag = 0;
        ctl->epilogue_go = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctl->tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 2) {  // norm weights of q and k as floats, shared by all rows
        const int t = threadIdx.x - 64;
#pragma unroll
        for (int which = 0; which < 2; ++which)
            norm_w[which][t] =
                p.norm_weight[which] ? __uint_as_float((uint32_t)p.norm_weight[which][t] << 16) : 0.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (blockIdx.x == 0 && warp == 2 && p.bound_out) {
        // A normalised head has sum (x*inv)^2 <= 128, so after the weight its 2-norm
        // is at most sqrt(128) * max|w|; the rotation preserves it and the two bf16
        // roundings add well under 1 %.
        for (int which = 0; which < 2; ++which) {
            float wmax = 0.0f;
            for (int i = lane; i < 128; i += 32) wmax = fmaxf(wmax, fabsf(norm_w[which][i]));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));
            if (lane == 0) p.bound_out[which] = 11.313708499f * 1.01f * wmax;
        }
    }

    if (warp == 0 && lane == 0) {
        // ---- producer
        uint32_t t = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            uint32_t tm, tn;
            tile_coords(tile, n_tiles, tm, tn);
            const uint32_t which = tn / p.tiles_per_output;
            const uint32_t tnl = tn - which * p.tiles_per_output;
            for (uint32_t ks = 0; ks < k_steps && ok; ++ks, ++t) {
                const uint32_t slot = t % kStages, par = ((t / kStages) & 1u) ^ 1u;
                ok = mbar_wait(ctl, &ctl->bars[kBarEmpty + slot], par, p.status, (3u << 16) | slot);
                if (!ok) break;
                unsigned long long *bar = &ctl->bars[kBarFull + slot];
                mbar_expect_tx(bar, kStageBytes);
                uint8_t *dst = ring + (size_t)slot * kStageBytes;
                tma_load_2d(dst, &map_a, bar, (int)(ks * kTileK), (int)(tm * kTileM));
                tma_load_2d(dst + kABytes, &maps.w[which], bar, (int)(ks * kTileK),
                            (int)(tnl * kTileN));
            }
        }
        // drain: the last kStages loads must have landed before the CTA may exit
        const uint32_t first = t > (uint32_t)kStages ? t - kStages : 0;
        for (uint32_t u = first; u < t; ++u) {
            long long start = clock64();
            while (!mbar_try(&ctl->bars[kBarFull + u % kStages], (u / kStages) & 1u))
                if (clock64() - start > kWaitCycles) break;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        uint32_t t = 0, local = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const uint32_t acc = local & 1u;
            // the epilogue must have drained this accumulator (used two tiles ago)
            if (local >= 2 &&
                !mbar_wait(ctl, &ctl->bars[kBarAccEmpty + acc], ((local >> 1) - 1u) & 1u, p.status,
                           (2u << 16) | (kBarAccEmpty + acc)))
                break;
            tc_fence_after();
            const uint32_t d_tmem = tmem + acc * kTileN;
            bool ok = true;
            for (uint32_t ks = 0; ks < k_steps; ++ks, ++t) {
                const uint32_t slot = t % kStages, par = (t / kStages) & 1u;
                ok = mbar_wait(ctl, &ctl->bars[kBarFull + slot], par, p.status, (2u << 16) | slot);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = (smem_u32(ring + (size_t)slot * kStageBytes) >> 4) | kDescLo;
                const uint32_t b_lo =
                    (smem_u32(ring + (size_t)slot * kStageBytes + kABytes) >> 4) | kDescLo;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    mma_ss(d_tmem, a_lo + (uint32_t)(kk * 32 >> 4), b_lo + (uint32_t)(kk * 32 >> 4),
                           (ks | kk) ? 1u : 0u);
                tc_commit(&ctl->bars[kBarEmpty + slot]);
            }
            if (!ok) break;
            tc_commit(&ctl->bars[kBarAccFull + acc]);
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads TMEM lanes 32 * (w % 4) ..., thread = one row
        const uint32_t quarter = (uint32_t)(warp & 3);
        const uint32_t lane_base = (quarter * 32u) << 16;
        const uint32_t r = quarter * 32u + (uint32_t)lane;  // row of the tile
        uint32_t local = 0, store_count = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            uint32_t tm, tn;
            tile_coords(tile, n_tiles, tm, tn);
            const uint32_t which = tn / p.tiles_per_output;
            const uint32_t tnl = tn - which * p.tiles_per_output;
            const uint32_t acc = local & 1u;
            // One thread waits for the accumulator and tells the rest through shared
            // memory: all 128 reach the group barrier on every path, also when a
            // wait gave up.
            if (threadIdx.x == 64)
                ctl->epilogue_go = mbar_wait(ctl, &ctl->bars[kBarAccFull + acc], (local >> 1) & 1u,
                                             p.status, (1u << 16) | (kBarAccFull + acc))
                                       ? 1u : 0u;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const bool go = ctl->epilogue_go != 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");  // everyone has read the flag
            if (!go) break;
            tc_fence_after();
            const bool fused = which < 2 && p.norm_weight[which] != nullptr;
            const uint32_t row_global = tm * kTileM + r;
            const uint32_t table_row = (row_global < p.m ? row_global : 0u) % p.table_rows;
            for (int hh = 0; hh < kTileN / 128; ++hh) {
                uint32_t pk[64];
                const uint32_t col0 = tnl * kTileN + (uint32_t)hh * 128u;
                head_from_tmem(pk, tmem + lane_base + acc * kTileN + (uint32_t)hh * 128u,
                               p.bias[which] ? p.bias[which] + col0 : nullptr,
                               fused ? norm_w[which] : nullptr,
                               fused ? p.rope_cos + (size_t)table_row * 64 : nullptr,
                               fused ? p.rope_sin + (size_t)table_row * 64 : nullptr, p.epsilon);
                if (hh == kTileN / 128 - 1) {
                    // the accumulator has left TMEM
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->bars[kBarAccEmpty + acc]);
                }
#pragma unroll
                for (int bb = 0; bb < 2; ++bb, ++store_count) {
                    uint8_t *stage = staging + (size_t)(store_count & 1u) * kStagingBytes;
                    // the store that used this staging buffer two boxes ago must have read
                    // it: thread 64 issues all stores and waits for them
                    if (store_count >= 2) {
                        if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                    uint8_t *line = stage + r * 128;
                    const uint32_t sw = r & 7u;
#pragma unroll
                    for (int c16 = 0; c16 < 8; ++c16) {
                        const int w0 = bb * 32 + c16 * 4;
                        *reinterpret_cast<uint4 *>(line + (((uint32_t)c16 ^ sw) << 4)) =
                            make_uint4(pk[w0], pk[w0 + 1], pk[w0 + 2], pk[w0 + 3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (threadIdx.x == 64) {
                        tma_store_2d(&maps.c[which], stage, (int)(col0 + bb * 64), (int)(tm * kTileM));
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
        }
        if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
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

// Row-major [rows][cols] bf16, boxes of box_rows x 64 columns, 128B swizzle; reads
// past either extent deliver zeros, writes past them are dropped.
int make_map_2d(CUtensorMap *map, const void *base, uint32_t rows, uint32_t cols,
                uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                    strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// The opt-in to ~225 KB of dynamic shared memory is a per-device attribute.
bool kernel_ready() {
    static bool ready[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked && ready[dev]) return true;
    if (cudaFuncSetAttribute(qw_linear_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSmemBytes) != cudaSuccess)
        return false;
    if (tracked) ready[dev] = true;
    return true;
}

}  // namespace

extern "C" int qwcu_linear_sm100_launch(const qwcu_linear_args *a, int sm_count,
                                        qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a->m || !a->k || !a->n || !a->n_outputs || a->n_outputs > (uint32_t)kMaxOutputs ||
        a->k % 8 || a->n % 8 || !a->a || !a->status)
        return (int)cudaErrorInvalidValue;
    const bool fused = a->norm_weight[0] || a->norm_weight[1];
    if (fused && (a->n % 128 || !a->rope_cos || !a->rope_sin || !a->table_rows))
        return (int)cudaErrorInvalidValue;
    if (a->bound_out && !(a->norm_weight[0] && a->norm_weight[1])) return (int)cudaErrorInvalidValue;
    if (!kernel_ready()) return (int)cudaGetLastError();
    CUtensorMap map_a;
    Maps maps;
    memset(&maps, 0, sizeof(maps));
    int rc;
    if (((uintptr_t)a->a & 15u)) return (int)cudaErrorMisalignedAddress;
    if ((rc = make_map_2d(&map_a, a->a, a->m, a->k, kTileM))) return rc;
    Params p;
    memset(&p, 0, sizeof(p));
    for (uint32_t i = 0; i < a->n_outputs; ++i) {
        if (!a->w[i] || !a->c[i]) return (int)cudaErrorInvalidValue;
        if (((uintptr_t)a->w[i] | (uintptr_t)a->c[i]) & 15u) return (int)cudaErrorMisalignedAddress;
        if ((rc = make_map_2d(&maps.w[i], a->w[i], a->n, a->k, kTileN))) return rc;
        if ((rc = make_map_2d(&maps.c[i], a->c[i], a->m, a->n, kTileM))) return rc;
        p.bias[i] = static_cast<const uint16_t *>(a->bias[i]);
    }
    p.m = a->m;
    p.k = a->k;
    p.n_each = a->n;
    p.n_outputs = a->n_outputs;
    p.tiles_per_output = (a->n + kTileN - 1) / kTileN;
    p.status = a->status;
    p.norm_weight[0] = static_cast<const uint16_t *>(a->norm_weight[0]);
    p.norm_weight[1] = static_cast<const uint16_t *>(a->norm_weight[1]);
    p.rope_cos = a->rope_cos;
    p.rope_sin = a->rope_sin;
    p.table_rows = a->table_rows ? a->table_rows : 1;
    p.epsilon = a->epsilon;
    p.bound_out = a->bound_out;
    const unsigned long long tiles =
        (unsigned long long)((a->m + kTileM - 1) / kTileM) * p.tiles_per_output * p.n_outputs;
    if (tiles > 0x7fffffffull) return (int)cudaErrorInvalidValue;
    unsigned grid = (unsigned)(sm_count > 0 ? sm_count : 148);
    if (tiles < grid) grid = (unsigned)tiles;
    qw_linear_sm100_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, maps, p);
    return (int)cudaGetLastError();
}
