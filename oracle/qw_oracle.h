/* CPU oracle for the DiT attention hot path (TEST INFRASTRUCTURE ONLY).
 *
 * A plain-C restatement of the reference's arithmetic for per-head RMSNorm,
 * interleaved-pair RoPE, RoPE table construction, prefix limits and
 * prefix-visible scaled-dot-product attention.  Nothing in the shipped
 * library links or calls this file; only the test-suite, the smoke check and
 * the bench's CPU-baseline legs do, and only as the checker or the timed CPU
 * baseline.
 *
 * Every function names the reference file:line it follows (paths relative to
 * the reference project root).
 */
#ifndef QW_ORACLE_H
#define QW_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* bf16 <-> f32, round-to-nearest-even by the integer trick
 * (h3_shaders.metal:11-19, tests/test_prefix_kernel.c:22-34). */
uint16_t qwo_f32_to_bf16(float value);
float qwo_bf16_to_f32(uint16_t bits);

/* The reference known-answer test's input generator: 32-bit LCG
 * state = state*1664525 + 1013904223, value = (state>>8)/2^23 - 1, interleaved
 * q,k,v per element, all rounded to bf16 (tests/test_prefix_kernel.c:15-20,51-58).
 * `count` elements are written to each of q,k,v. */
void qwo_kat_fill(uint32_t seed, uint16_t *q, uint16_t *k, uint16_t *v, size_t count);

/* Limits of the reference known-answer test, 149 rows in four runs
 * (tests/test_prefix_kernel.c:65-70). `limits` holds 149 values. */
void qwo_kat_limits(uint32_t *limits);

/* Run descriptor, same fields as qw_dit_segment (qwen_dit.h:25-29). */
typedef struct {
    uint32_t rows;
    int is_image;
    uint32_t src_offset;
} qwo_segment;

/* limits[row]: image rows see up to their run's end, text rows are
 * token-causal inside the joint sequence (qwen_dit.m:1651-1665). */
void qwo_prefix_limits(const qwo_segment *segs, uint32_t seg_count, uint32_t *limits);

/* Dense boolean mask [batch][rows][kv_rows] (1 = visible) from a limit table
 * plus optional key padding: key s is visible to row r of batch b iff
 * s < min(max(limit,0),kv_rows) and not (text_len[b] <= s < text_pad).
 * Limits are read as int32 and clamped like the kernel does
 * (h3_shaders.metal:3067,3110,3122).  text_len may be NULL (no padding).
 * kv_limit holds batch*rows entries when per_batch_limits != 0, else rows. */
void qwo_dense_mask(uint8_t *mask, const uint32_t *kv_limit, int per_batch_limits,
                    uint32_t batch, uint32_t rows, uint32_t kv_rows,
                    const uint32_t *text_len, uint32_t text_pad);

/* Joint 3-axis RoPE tables [text_rows + gh*gw, 64] f32, axes 16/56/56,
 * theta 1e4; text row t rides position t on all axes, image tokens use frame
 * = text_rows and centred h/w (qwen_pipeline.m:212-252). Returns rows. */
uint32_t qwo_rope_tables(uint32_t text_rows, uint32_t gh, uint32_t gw,
                         float *cos_out, float *sin_out);

/* Multi-block variant: [text_before[b] rows][block_h[b]*block_w[b] rows]...,
 * a running position that advances by 1 per text row and by max(gh,gw) per
 * image block (qwen_pipeline.m:611-674). Returns rows. */
uint32_t qwo_rope_tables_blocks(const uint32_t *block_h, const uint32_t *block_w,
                                const uint32_t *text_before, uint32_t n_blocks,
                                float *cos_out, float *sin_out);

/* Released per-axis table entry: f32 frequency, f32 angle, cosf/sinf
 * (qwen_host.c:94-136); coordinate may be negative. */
void qwo_rope_released_entry(int axis_dim, int pair, int coordinate,
                             float *cos_out, float *sin_out);

/* In-place per-(row, head) RMSNorm over head_dim bf16 values: serial fp32 fma
 * sum, inv = 1/sqrt(sum/head_dim + eps), x <- bf16(x*inv*w)
 * (h3_shaders.metal:4309-4329).  double_round != 0 selects
 * bf16(bf16(x*inv)*w) (h3_shaders.metal:4975-4997). */
void qwo_head_rms_norm_bf16(uint16_t *tensor, const uint16_t *weight,
                            uint32_t sequence, uint32_t heads, uint32_t head_dim,
                            float epsilon, int double_round);

/* Interleaved-pair RoPE on q and k, tables f32 [row, head_dim/2]
 * (h3_shaders.metal:4864-4890).  In-place safe. */
void qwo_qk_rope_bf16(uint16_t *q_out, uint16_t *k_out, const uint16_t *q_in,
                      const uint16_t *k_in, const float *rope_cos,
                      const float *rope_sin, uint32_t sequence, uint32_t heads,
                      uint32_t head_dim);

/* Prefix-visible SDPA in fp32 on bf16 inputs (tests/test_prefix_kernel.c:72-97
 * for the arithmetic; GQA map kvh = h*kv_heads/heads from
 * h3_shaders.metal:3096).  The visible set of (batch b, row r) is
 * [0, limit) minus the key-padding window [text_len[b], text_pad); query rows
 * inside that window and rows with an empty visible set produce zeros.
 * kv_limit == NULL means every limit = kv_rows; text_len == NULL means no
 * padding.  q: [batch][q_rows][heads][D], k,v: [batch][kv_rows][kv_heads][D],
 * out f32 [batch][q_rows][heads][D].  row_index == NULL computes every row;
 * otherwise only the n_rows listed (b*q_rows + r entries) are computed and
 * written, the rest of `out` is left untouched.  Threads: OpenMP when built
 * with -fopenmp.  Returns the number of visible (q,k) pairs summed over the
 * computed rows (one head), the figure mask-aware FLOPs are built from. */
uint64_t qwo_sdpa_prefix(float *out, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, const uint32_t *kv_limit,
                         int per_batch_limits, uint32_t batch, uint32_t q_rows,
                         uint32_t kv_rows, uint32_t heads, uint32_t kv_heads,
                         uint32_t head_dim, float scale, const uint32_t *text_len,
                         uint32_t text_pad, const uint32_t *row_index,
                         size_t n_rows);

/* Σ visible pairs for one head over all (batch, row), integer exact. */
uint64_t qwo_visible_pairs(const uint32_t *kv_limit, int per_batch_limits,
                           uint32_t batch, uint32_t q_rows, uint32_t kv_rows,
                           const uint32_t *text_len, uint32_t text_pad);

/* Affine-free LayerNorm over `width` bf16 values per row, then the per-row
 * modulation scale: out = bf16((x - mean) * rsqrt(var + eps) * (1 + scale)),
 * scale = modulation[row_map[row]][scale_slot][column], two-pass variance with
 * an fma sum of squares, all fp32, summed in the order of the shader's 256-thread
 * threadgroup: strided partial sums per thread, then a halving tree
 * (h3_shaders.metal:4767-4813, dispatch h3_gpu.m:357-378). */
void qwo_layer_norm_mod_bf16(uint16_t *out, const uint16_t *in,
                             const uint16_t *modulation, const uint32_t *row_map,
                             uint32_t rows, uint32_t width, uint32_t slots,
                             uint32_t scale_slot, float epsilon);

/* out = bf16(residual + branch * gate), gate =
 * modulation[row_map[row]][gate_slot][column], fp32, unfused product and sum
 * (h3_shaders.metal:3583-3599). */
void qwo_gate_bf16(uint16_t *out, const uint16_t *residual, const uint16_t *branch,
                   const uint16_t *modulation, const uint32_t *row_map, uint32_t rows,
                   uint32_t width, uint32_t slots, uint32_t gate_slot);

/* bf16 linear layer: out[r][c] = bf16(bias[c] + sum_k in[r][k] * w[c][k]), fp32,
 * a serial fma chain over k that starts from the bias (h3_shaders.metal:788-822;
 * weight in its [out, in] layout).  bias may be NULL.  row_index == NULL computes
 * every row; otherwise only the n_rows listed rows are computed and written. */
void qwo_linear_bf16(uint16_t *out, const uint16_t *in, const uint16_t *weight,
                     const uint16_t *bias, uint32_t rows, uint32_t input_dim,
                     uint32_t output_dim, const uint32_t *row_index, size_t n_rows);

/* OpenMP threads the loops above use; qwo_set_threads overrides the environment
 * (a launcher may export OMP_NUM_THREADS=1 to every rank). */
void qwo_set_threads(int threads);
int qwo_threads(void);

#ifdef __cplusplus
}
#endif
#endif
