/* Thin extern-"C" CUDA layer under the C11 host code.
 *
 * The host side (h3_context.c, qw_ops.c) validates arguments the way the
 * reference's op wrappers do and then calls one of these launchers with raw
 * device pointers.  Every launcher only enqueues work on `stream` and returns
 * 0 on success or a CUDA error code; device-side failures (a bounded wait
 * that ran out) are recorded in the `status` words and surface at submit.
 */
#ifndef QW_CUDA_H
#define QW_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque here so C11 translation units need no CUDA headers. */
typedef void *qwcu_stream;

enum {
    QWCU_STATUS_OK = 0,
    QWCU_STATUS_WAIT_TIMEOUT = 1, /* status[1] = role<<16 | barrier id, status[2] = tile */
    QWCU_STATUS_BAD_ARGUMENT = 2
};
#define QWCU_STATUS_WORDS 8

/* Geometry + mask description shared by every attention kernel.
 *
 * Layouts (elements are bf16):
 *   q   [batch][q_rows ][heads   ][128]
 *   k,v [batch][kv_rows][kv_heads][128]
 *   out [batch][q_rows ][heads   ][128], or [batch][heads][q_rows][128] when
 *       head_major_out != 0.
 * Visible keys of (batch b, row r): s < limit(b,r), minus the key-padding
 * window text_len[b] <= s < text_pad when text_pad != 0.  limit(b,r) is
 *   kv_limit != NULL : clamp((int32)kv_limit[per_batch ? b*q_rows+r : r], 0, kv_rows)
 *   causal != 0      : min(r + 1 + causal_offset, kv_rows)
 *   otherwise        : kv_rows.
 * Query rows inside the padding window and rows with no visible key store zeros.
 */
typedef struct {
    const void *q;
    const void *k;
    const void *v;
    void *out;
    const int32_t *kv_limit;
    int per_batch_limits;
    int causal;
    uint32_t causal_offset;
    uint32_t batch;
    uint32_t q_rows;
    uint32_t kv_rows;
    uint32_t heads;
    uint32_t kv_heads;
    uint32_t text_len[8]; /* per batch item; used when text_pad != 0 (batch <= 8) */
    uint32_t text_pad;
    float scale;
    int scale_in_q; /* h3 causal variant: q' = bf16(q*scale), scores unscaled */
    /* Optional (sm100 kernel): two device floats, upper bounds of the 2-norm of
     * every query row and of every key row.  When their product times
     * scale*log2(e) is at most 60 the softmax uses that as one fixed reference
     * exponent (no row maximum, no rescaling); otherwise it is ignored. */
    const float *score_bound;
    int head_major_out;
    /* Sharded heads (n_out_peers > 0, sm100 kernel only): instead of `out`, the
     * rows are stored at head columns [out_head_offset, out_head_offset + heads)
     * of [batch][q_rows][out_heads_total][128] in each of the peer-mapped buffers. */
    void *out_peers[8];
    uint32_t n_out_peers;
    uint32_t out_heads_total;
    uint32_t out_head_offset;
    uint32_t *status; /* QWCU_STATUS_WORDS device words, zero when healthy */
    /* Sharded heads with the gather as a separate push (cuda/qw_push.cu): at its
     * start the kernel increments *slot_use and stores the new epoch into
     * freed_peer[0..n_freed) (peer-mapped flag words): the peers may now store
     * their columns of this epoch into this rank's output slot. */
    uint32_t *slot_use;
    uint32_t *freed_peer[8];
    uint32_t n_freed;
    /* sm100 kernel: never run the units of the last wave in split form (two CTAs
     * per 256-row block, key tiles divided between the sub-tiles). */
    int whole_units;
    /* sm100 kernel with a score bound: one thread per query row (one warpgroup per
     * sub-tile) instead of both warpgroups sharing each sub-tile's keys. */
    int row_softmax;
    /* Bounded-wait exercise (sm100 kernel, tests only): wait budget in SM cycles
     * (0 = default, about 0.2 s) and the first visited key tile (>= 1) that the TMA
     * producer does not load (0 = none withheld): the waits behind it run out, the
     * CTA records where, drains, frees its TMEM and returns. */
    long long wait_cycles;
    int withhold_from;
} qwcu_attn_args;

/* tcgen05/TMEM/TMA flash-attention forward (sm_100a). */
int qwcu_attn_sm100_launch(const qwcu_attn_args *args, qwcu_stream stream);
/* How many of `units` (batch x heads x 256-row blocks) the sm100 launch runs in
 * split form on a device with sm_count SMs (host-side arithmetic only). */
uint32_t qwcu_attn_sm100_tail_units(uint32_t units, uint32_t sm_count);
/* One-warp-per-(row, head) fp32 kernel; the diagnostic cross-check path. */
int qwcu_attn_scalar_launch(const qwcu_attn_args *args, qwcu_stream stream);

/* Fused per-head RMSNorm + interleaved RoPE over q and k, in place or out of
 * place.  Any of the stages can be switched off so the three legacy entry
 * points share the same device code:
 *   norm_weight_q/k == NULL -> no norm for that tensor
 *   rope_cos == NULL        -> no rotation
 *   k_in == NULL            -> only q is processed
 *   v_in != NULL            -> a third tensor of the same shape is copied to
 *                              v_out untouched (K/V cache update in one launch)
 * double_round selects bf16(bf16(x*inv)*w). */
typedef struct {
    const void *q_in;
    const void *k_in;
    void *q_out;
    void *k_out;
    const void *v_in;
    void *v_out;
    const void *norm_weight_q;
    const void *norm_weight_k;
    const float *rope_cos;
    const float *rope_sin;
    uint32_t rows; /* batch*sequence rows of [heads][128] */
    uint32_t table_rows; /* rope row = row % table_rows (batch items share tables) */
    uint32_t heads;
    float epsilon;
    int double_round;
    /* Optional (q and k both normed, no third tensor): two device floats that
     * receive upper bounds of the 2-norm of any output q row and k row,
     * sqrt(128) * max|weight| plus rounding slack. */
    float *bound_out;
} qwcu_prologue_args;

int qwcu_prologue_launch(const qwcu_prologue_args *args, qwcu_stream stream);

/* The element-wise neighbours of the attention path: rows of `width` bf16
 * values, a modulation tensor [maps][slots][width] and a per-row map index.
 *   layer_norm_mod: output = LayerNorm(input) * (1 + modulation[map][slot])
 *   gate          : output = input + branch * modulation[map][slot] */
typedef struct {
    const void *input;  /* norm input / gate residual */
    const void *branch; /* gate only */
    const void *modulation;
    const uint32_t *row_map;
    void *output;
    uint32_t rows;
    uint32_t width;
    uint32_t slots;
    uint32_t slot;
    float epsilon; /* norm only */
    uint32_t maps;    /* [maps][slots][width] blocks the modulation tensor holds (>= 1) */
    uint32_t *status; /* a row_map entry >= maps is reported here; block 0 is used */
} qwcu_rowwise_args;

int qwcu_layer_norm_mod_launch(const qwcu_rowwise_args *args, int sm_count, qwcu_stream stream);
int qwcu_gate_launch(const qwcu_rowwise_args *args, int sm_count, qwcu_stream stream);

/* h3 causal variant helper: out = bf16(in * scale), elementwise. */
int qwcu_scale_bf16_launch(void *out, const void *in, size_t elements, float scale,
                           qwcu_stream stream);

/* Sharded heads: copy this rank's column slice of its full output into the same
 * place of every peer's output (peer-mapped pointers) and hand-shake with the
 * peers through epoch flags; see cuda/qw_push.cu.  All flag pointers are device
 * addresses: *_local in this rank's memory, ready_peer[d] in peer d's. */
typedef struct {
    const void *src;       /* this rank's full output [rows][row_bytes] */
    void *dst[8];          /* the peers' full outputs */
    uint32_t peer_rank[8]; /* the peers' indices into the 8-entry flag rows */
    uint32_t n_peers;
    uint32_t my_rank;
    uint32_t rows;
    uint32_t row_bytes;   /* bytes per output row */
    uint32_t col_byte0;   /* first byte of this rank's column slice in a row */
    uint32_t slice_bytes; /* bytes of the slice */
    const uint32_t *slot_use;    /* epoch counter of the output slot */
    const uint32_t *freed_local; /* [8] peers' "your stores may start" flags */
    const uint32_t *ready_local; /* [8] peers' "my columns have landed" flags */
    uint32_t *ready_peer[8];     /* where this rank reports to peer d */
    uint32_t *arrivals;          /* zero-initialised CTA counter of the slot */
    uint32_t *status;
    uint32_t wait_ms;    /* budget of every flag wait (0 = 2000 ms) */
    uint32_t max_blocks; /* CTAs of 256 threads (0 = 32) */
    /* Move the bytes with strided device-to-device copies (copy engines, no SM)
     * between two one-warp hand-shake kernels, instead of the copy kernel. */
    int copy_engine;
} qwcu_push_args;

int qwcu_push_launch(const qwcu_push_args *args, qwcu_stream stream);

/* Multi-GPU gather epilogue: staged [world][rows][slice] -> full [rows][world*slice]
 * (bf16 elements; slice_elements must be a multiple of 8). */
int qwcu_interleave_launch(void *full, const void *staged, uint32_t rows,
                           uint32_t slice_elements, uint32_t world, int sm_count,
                           qwcu_stream stream);

/* bf16 linear layers on the tensor cores (cuda/qw_linear_sm100.cu):
 *   c[i][m][n] = a[m][k] * w[i][n][k]^T (+ bias[i][n]) for i < n_outputs (1 or 3),
 * fp32 accumulate, one rounding to bf16.  k and n must be multiples of 8.
 * With norm_weight[0] / [1] set (n a multiple of 128), outputs 0 / 1 additionally
 * get the per-head RMSNorm (bf16 [128] weight, epsilon) and the interleaved RoPE
 * with f32 tables [table_rows][64] (table row = output row % table_rows), each
 * stage rounded to bf16; bound_out (optional, both weights set) receives the two
 * row-norm bounds qwcu_prologue_launch would leave. */
typedef struct {
    const void *a;
    const void *w[3];
    void *c[3];
    const void *bias[3];
    uint32_t n_outputs;
    uint32_t m, k, n;
    const void *norm_weight[2];
    const float *rope_cos;
    const float *rope_sin;
    uint32_t table_rows;
    float epsilon;
    float *bound_out;
    uint32_t *status;
} qwcu_linear_args;

int qwcu_linear_sm100_launch(const qwcu_linear_args *args, int sm_count, qwcu_stream stream);

/* Device properties needed by the host side. */
int qwcu_device_sm_count(int device);
int qwcu_device_cc(int device); /* major*10 + minor */

#ifdef __cplusplus
}
#endif
#endif
