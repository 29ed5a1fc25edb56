/* CPU oracle for the DiT attention hot path (TEST INFRASTRUCTURE ONLY).
 *
 * Plain C restatement of the reference arithmetic; see qw_oracle.h for the
 * contract and the reference file:line each function follows.  Never linked
 * into the shipped library.
 */
#include "qw_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

void qwo_set_threads(int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}

int qwo_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* tests/test_prefix_kernel.c:22-27, h3_shaders.metal:15-19 */
uint16_t qwo_f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

/* tests/test_prefix_kernel.c:29-34 */
float qwo_bf16_to_f32(uint16_t bits) {
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, 4);
    return value;
}

/* tests/test_prefix_kernel.c:15-20 (generator), :51-58 (draw order q,k,v) */
void qwo_kat_fill(uint32_t seed, uint16_t *q, uint16_t *k, uint16_t *v, size_t count) {
    uint32_t state = seed;
    for (size_t i = 0; i < count; i++) {
        uint16_t *dst[3] = {q, k, v};
        for (int t = 0; t < 3; t++) {
            state = state * 1664525u + 1013904223u;
            float value = ((float)(state >> 8) / 8388608.0f) - 1.0f;
            dst[t][i] = qwo_f32_to_bf16(value);
        }
    }
}

/* tests/test_prefix_kernel.c:65-70 */
void qwo_kat_limits(uint32_t *limits) {
    for (uint32_t r = 0; r < 20; r++) limits[r] = r + 1;
    for (uint32_t r = 20; r < 68; r++) limits[r] = 68;
    for (uint32_t r = 68; r < 85; r++) limits[r] = 68 + (r - 68) + 1;
    for (uint32_t r = 85; r < 149; r++) limits[r] = 149;
}

/* qwen_dit.m:1651-1665 */
void qwo_prefix_limits(const qwo_segment *segs, uint32_t seg_count, uint32_t *limits) {
    uint32_t start = 0;
    for (uint32_t s = 0; s < seg_count; s++) {
        for (uint32_t r = 0; r < segs[s].rows; r++)
            limits[start + r] = segs[s].is_image ? start + segs[s].rows : start + r + 1;
        start += segs[s].rows;
    }
}

/* Effective key count of one row: int32 read, negatives -> 0, capped at
 * kv_rows (h3_shaders.metal:3067,3110,3122). */
static uint32_t effective_limit(const uint32_t *kv_limit, size_t index, uint32_t kv_rows) {
    if (!kv_limit) return kv_rows;
    int32_t raw = (int32_t)kv_limit[index];
    uint32_t limit = raw > 0 ? (uint32_t)raw : 0u;
    return limit < kv_rows ? limit : kv_rows;
}

static int key_visible(uint32_t s, uint32_t limit, const uint32_t *text_len, uint32_t b,
                       uint32_t text_pad) {
    if (s >= limit) return 0;
    if (text_len && s >= text_len[b] && s < text_pad) return 0;
    return 1;
}

void qwo_dense_mask(uint8_t *mask, const uint32_t *kv_limit, int per_batch_limits,
                    uint32_t batch, uint32_t rows, uint32_t kv_rows,
                    const uint32_t *text_len, uint32_t text_pad) {
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t r = 0; r < rows; r++) {
            size_t li = per_batch_limits ? (size_t)b * rows + r : r;
            uint32_t limit = effective_limit(kv_limit, li, kv_rows);
            int padded_query = text_len && r >= text_len[b] && r < text_pad;
            uint8_t *row = mask + ((size_t)b * rows + r) * kv_rows;
            for (uint32_t s = 0; s < kv_rows; s++)
                row[s] = (uint8_t)(!padded_query &&
                                   key_visible(s, limit, text_len, b, text_pad));
        }
}

uint64_t qwo_visible_pairs(const uint32_t *kv_limit, int per_batch_limits,
                           uint32_t batch, uint32_t q_rows, uint32_t kv_rows,
                           const uint32_t *text_len, uint32_t text_pad) {
    uint64_t total = 0;
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t r = 0; r < q_rows; r++) {
            if (text_len && r >= text_len[b] && r < text_pad) continue;
            size_t li = per_batch_limits ? (size_t)b * q_rows + r : r;
            uint32_t limit = effective_limit(kv_limit, li, kv_rows);
            uint64_t visible = limit;
            if (text_len && text_pad > text_len[b]) {
                uint32_t lo = text_len[b] < limit ? text_len[b] : limit;
                uint32_t hi = text_pad < limit ? text_pad : limit;
                visible -= hi - lo;
            }
            total += visible;
        }
    return total;
}

static const double k_axis_dim[3] = {16.0, 56.0, 56.0};

/* One table row from three positions: qwen_pipeline.m:243-252 */
static void rope_row(const double position[3], float *cos_row, float *sin_row) {
    size_t pair = 0;
    for (int axis = 0; axis < 3; axis++) {
        uint32_t pairs = (uint32_t)(k_axis_dim[axis] / 2.0);
        for (uint32_t p = 0; p < pairs; p++, pair++) {
            double frequency = pow(10000.0, -2.0 * (double)p / k_axis_dim[axis]);
            double angle = position[axis] * frequency;
            cos_row[pair] = (float)cos(angle);
            sin_row[pair] = (float)sin(angle);
        }
    }
}

/* qwen_pipeline.m:212-252 */
uint32_t qwo_rope_tables(uint32_t text_rows, uint32_t gh, uint32_t gw,
                         float *cos_out, float *sin_out) {
    uint32_t rows = text_rows + gh * gw;
    long half_h = (long)(gh - gh / 2);
    long half_w = (long)(gw - gw / 2);
    for (uint32_t t = 0; t < rows; t++) {
        double position[3];
        if (t < text_rows) {
            position[0] = position[1] = position[2] = (double)t;
        } else {
            uint32_t index = t - text_rows;
            position[0] = (double)text_rows;
            position[1] = (double)((long)(index / gw) - half_h);
            position[2] = (double)((long)(index % gw) - half_w);
        }
        rope_row(position, cos_out + (size_t)t * 64, sin_out + (size_t)t * 64);
    }
    return rows;
}

/* qwen_pipeline.m:611-674 */
uint32_t qwo_rope_tables_blocks(const uint32_t *block_h, const uint32_t *block_w,
                                const uint32_t *text_before, uint32_t n_blocks,
                                float *cos_out, float *sin_out) {
    double position = 0.0;
    uint32_t row = 0;
    for (uint32_t b = 0; b < n_blocks; b++) {
        for (uint32_t t = 0; t < text_before[b]; t++) {
            double pos[3] = {position, position, position};
            rope_row(pos, cos_out + (size_t)row * 64, sin_out + (size_t)row * 64);
            position += 1.0;
            row++;
        }
        uint32_t gh = block_h[b], gw = block_w[b];
        long half_h = (long)(gh - gh / 2);
        long half_w = (long)(gw - gw / 2);
        double frame = position;
        for (uint32_t y = 0; y < gh; y++)
            for (uint32_t x = 0; x < gw; x++) {
                double pos[3] = {frame, (double)((long)y - half_h),
                                 (double)((long)x - half_w)};
                rope_row(pos, cos_out + (size_t)row * 64, sin_out + (size_t)row * 64);
                row++;
            }
        position += (gh > gw ? gh : gw);
    }
    return row;
}

/* qwen_host.c:116-131 */
void qwo_rope_released_entry(int axis_dim, int pair, int coordinate,
                             float *cos_out, float *sin_out) {
    double exponent = -2.0 * (double)pair / (double)axis_dim;
    float frequency = (float)pow(10000.0, exponent);
    float angle = (float)coordinate * frequency;
    *cos_out = cosf(angle);
    *sin_out = sinf(angle);
}

/* h3_shaders.metal:4309-4329 (single rounding), :4975-4997 (double rounding) */
void qwo_head_rms_norm_bf16(uint16_t *tensor, const uint16_t *weight,
                            uint32_t sequence, uint32_t heads, uint32_t head_dim,
                            float epsilon, int double_round) {
#pragma omp parallel for schedule(static)
    for (int64_t rh = 0; rh < (int64_t)sequence * heads; rh++) {
        uint16_t *x = tensor + (size_t)rh * head_dim;
        float sum = 0.0f;
        for (uint32_t d = 0; d < head_dim; d++) {
            float value = qwo_bf16_to_f32(x[d]);
            sum = fmaf(value, value, sum);
        }
        float inverse = 1.0f / sqrtf(sum / (float)head_dim + epsilon);
        for (uint32_t d = 0; d < head_dim; d++) {
            float value = qwo_bf16_to_f32(x[d]);
            float w = qwo_bf16_to_f32(weight[d]);
            if (double_round) {
                float rounded = qwo_bf16_to_f32(qwo_f32_to_bf16(value * inverse));
                x[d] = qwo_f32_to_bf16(rounded * w);
            } else {
                x[d] = qwo_f32_to_bf16(value * inverse * w);
            }
        }
    }
}

/* h3_shaders.metal:4864-4890 */
void qwo_qk_rope_bf16(uint16_t *q_out, uint16_t *k_out, const uint16_t *q_in,
                      const uint16_t *k_in, const float *rope_cos,
                      const float *rope_sin, uint32_t sequence, uint32_t heads,
                      uint32_t head_dim) {
    uint32_t half = head_dim / 2;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)sequence; row++)
        for (uint32_t head = 0; head < heads; head++)
            for (uint32_t pair = 0; pair < half; pair++) {
                float c = rope_cos[(size_t)row * half + pair];
                float s = rope_sin[(size_t)row * half + pair];
                size_t even = ((size_t)row * heads + head) * head_dim + 2 * pair;
                size_t odd = even + 1;
                float q_even = qwo_bf16_to_f32(q_in[even]);
                float q_odd = qwo_bf16_to_f32(q_in[odd]);
                float k_even = qwo_bf16_to_f32(k_in[even]);
                float k_odd = qwo_bf16_to_f32(k_in[odd]);
                /* volatile-free: products and sums kept as separate fp32
                 * operations (the shader has no fused form here). */
                q_out[even] = qwo_f32_to_bf16(q_even * c - q_odd * s);
                q_out[odd] = qwo_f32_to_bf16(q_even * s + q_odd * c);
                k_out[even] = qwo_f32_to_bf16(k_even * c - k_odd * s);
                k_out[odd] = qwo_f32_to_bf16(k_even * s + k_odd * c);
            }
}

/* h3_shaders.metal:4767-4813 */
/* The shader's threadgroup reduction: lane t of QWO_NORM_LANES sums columns t,
 * t + lanes, ... serially, then the lanes are folded in halves (stride lanes/2,
 * lanes/4, ..., 1).  The reference dispatches one threadgroup of 256 threads per
 * row (h3_gpu.m:357-378: the largest power of two <= min(256, pipeline
 * maximum)). */
#define QWO_NORM_LANES 256

static float norm_tree(float *lanes) {
    for (uint32_t stride = QWO_NORM_LANES / 2; stride; stride >>= 1)
        for (uint32_t t = 0; t < stride; t++) lanes[t] += lanes[t + stride];
    return lanes[0];
}

void qwo_layer_norm_mod_bf16(uint16_t *out, const uint16_t *in,
                             const uint16_t *modulation, const uint32_t *row_map,
                             uint32_t rows, uint32_t width, uint32_t slots,
                             uint32_t scale_slot, float epsilon) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const uint16_t *x = in + (size_t)row * width;
        float lanes[QWO_NORM_LANES];
        for (uint32_t t = 0; t < QWO_NORM_LANES; t++) {
            float local_sum = 0.0f;
            for (uint32_t c = t; c < width; c += QWO_NORM_LANES) local_sum += qwo_bf16_to_f32(x[c]);
            lanes[t] = local_sum;
        }
        float mean = norm_tree(lanes) / (float)width;
        for (uint32_t t = 0; t < QWO_NORM_LANES; t++) {
            float local_square = 0.0f;
            for (uint32_t c = t; c < width; c += QWO_NORM_LANES) {
                float centered = qwo_bf16_to_f32(x[c]) - mean;
                local_square = fmaf(centered, centered, local_square);
            }
            lanes[t] = local_square;
        }
        float inverse = 1.0f / sqrtf(norm_tree(lanes) / (float)width + epsilon);
        const uint16_t *scale =
            modulation + ((size_t)row_map[row] * slots + scale_slot) * width;
        for (uint32_t c = 0; c < width; c++) {
            float normalized = (qwo_bf16_to_f32(x[c]) - mean) * inverse;
            out[(size_t)row * width + c] =
                qwo_f32_to_bf16(normalized * (1.0f + qwo_bf16_to_f32(scale[c])));
        }
    }
}

/* h3_shaders.metal:3583-3599 */
void qwo_gate_bf16(uint16_t *out, const uint16_t *residual, const uint16_t *branch,
                   const uint16_t *modulation, const uint32_t *row_map, uint32_t rows,
                   uint32_t width, uint32_t slots, uint32_t gate_slot) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const uint16_t *gate =
            modulation + ((size_t)row_map[row] * slots + gate_slot) * width;
        for (uint32_t c = 0; c < width; c++) {
            size_t index = (size_t)row * width + c;
            float product = qwo_bf16_to_f32(branch[index]) * qwo_bf16_to_f32(gate[c]);
            out[index] = qwo_f32_to_bf16(qwo_bf16_to_f32(residual[index]) + product);
        }
    }
}

/* h3_shaders.metal:788-822 */
void qwo_linear_bf16(uint16_t *out, const uint16_t *in, const uint16_t *weight,
                     const uint16_t *bias, uint32_t rows, uint32_t input_dim,
                     uint32_t output_dim, const uint32_t *row_index, size_t n_rows) {
    const int64_t count = row_index ? (int64_t)n_rows : (int64_t)rows;
    /* the weights as floats once: every row reuses them */
    float *wf = malloc((size_t)output_dim * input_dim * sizeof(float));
    if (!wf) return;
    for (size_t i = 0; i < (size_t)output_dim * input_dim; i++) wf[i] = qwo_bf16_to_f32(weight[i]);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t n = 0; n < count; n++) {
        const uint32_t row = row_index ? row_index[n] : (uint32_t)n;
        if (row >= rows) continue;
        float *x = malloc(input_dim * sizeof(float));
        if (!x) continue;
        for (uint32_t k = 0; k < input_dim; k++)
            x[k] = qwo_bf16_to_f32(in[(size_t)row * input_dim + k]);
        for (uint32_t c = 0; c < output_dim; c++) {
            float sum = bias ? qwo_bf16_to_f32(bias[c]) : 0.0f;
            const float *w = wf + (size_t)c * input_dim;
            for (uint32_t k = 0; k < input_dim; k++) sum = fmaf(x[k], w[k], sum);
            out[(size_t)row * output_dim + c] = qwo_f32_to_bf16(sum);
        }
        free(x);
    }
    free(wf);
}

/* tests/test_prefix_kernel.c:72-97, one (batch,row): all heads. */
static uint64_t sdpa_row(float *out, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, uint32_t b, uint32_t r, uint32_t limit,
                         uint32_t q_rows, uint32_t kv_rows, uint32_t heads,
                         uint32_t kv_heads, uint32_t D, float scale,
                         const uint32_t *text_len, uint32_t text_pad, float *scores,
                         const float *kf, const float *vf) {
    int padded_query = text_len && r >= text_len[b] && r < text_pad;
    uint64_t visible = 0;
    for (uint32_t h = 0; h < heads; h++) {
        uint32_t kvh = (uint32_t)((uint64_t)h * kv_heads / heads); /* h3_shaders.metal:3096 */
        float *o = out + (((size_t)b * q_rows + r) * heads + h) * D;
        for (uint32_t d = 0; d < D; d++) o[d] = 0.0f;
        if (padded_query) continue;
        const uint16_t *qv = q + (((size_t)b * q_rows + r) * heads + h) * D;
        float qf[256];
        for (uint32_t d = 0; d < D; d++) qf[d] = qwo_bf16_to_f32(qv[d]);
        float m = -3.402823466e+38f;
        uint32_t count = 0;
        for (uint32_t s = 0; s < limit; s++) {
            if (!key_visible(s, limit, text_len, b, text_pad)) {
                scores[s] = 0.0f;
                continue;
            }
            const size_t at = (((size_t)b * kv_rows + s) * kv_heads + kvh) * D;
            float dot = 0.0f;
            if (kf) { /* keys already widened to fp32, as the reference's arrays are */
                const float *kr = kf + at;
                for (uint32_t d = 0; d < D; d++) dot += qf[d] * kr[d];
            } else {
                const uint16_t *kv = k + at;
                for (uint32_t d = 0; d < D; d++) dot += qf[d] * qwo_bf16_to_f32(kv[d]);
            }
            scores[s] = dot * scale;
            if (scores[s] > m) m = scores[s];
            count++;
        }
        if (h == 0) visible = count;
        if (!count) continue;
        float denom = 0.0f;
        for (uint32_t s = 0; s < limit; s++) {
            if (!key_visible(s, limit, text_len, b, text_pad)) continue;
            scores[s] = expf(scores[s] - m);
            denom += scores[s];
        }
        for (uint32_t s = 0; s < limit; s++) {
            if (!key_visible(s, limit, text_len, b, text_pad)) continue;
            const size_t at = (((size_t)b * kv_rows + s) * kv_heads + kvh) * D;
            float p = scores[s] / denom;
            if (vf) {
                const float *vr = vf + at;
                for (uint32_t d = 0; d < D; d++) o[d] += p * vr[d];
            } else {
                const uint16_t *vv = v + at;
                for (uint32_t d = 0; d < D; d++) o[d] += p * qwo_bf16_to_f32(vv[d]);
            }
        }
    }
    return visible;
}

uint64_t qwo_sdpa_prefix(float *out, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, const uint32_t *kv_limit,
                         int per_batch_limits, uint32_t batch, uint32_t q_rows,
                         uint32_t kv_rows, uint32_t heads, uint32_t kv_heads,
                         uint32_t head_dim, float scale, const uint32_t *text_len,
                         uint32_t text_pad, const uint32_t *row_index,
                         size_t n_rows) {
    if (head_dim > 256 || !heads || !kv_heads) return 0;
    size_t total_rows = row_index ? n_rows : (size_t)batch * q_rows;
    uint64_t visible_total = 0;
    /* The reference's loop runs on fp32 copies of the bf16 inputs
     * (tests/test_prefix_kernel.c:51-63): widen K and V once instead of inside the
     * dot products (same values, same order of operations; falls back to widening
     * in place when the copies do not fit). */
    const size_t kv_count = (size_t)batch * kv_rows * kv_heads * head_dim;
    float *kf = NULL, *vf = NULL;
    if (total_rows >= 64) {
        kf = (float *)malloc(kv_count * sizeof(float));
        vf = (float *)malloc(kv_count * sizeof(float));
        if (kf && vf) {
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < (int64_t)kv_count; i++) {
                kf[i] = qwo_bf16_to_f32(k[i]);
                vf[i] = qwo_bf16_to_f32(v[i]);
            }
        } else {
            free(kf);
            free(vf);
            kf = vf = NULL;
        }
    }
#pragma omp parallel reduction(+ : visible_total)
    {
        float *scores = (float *)malloc(sizeof(float) * (kv_rows ? kv_rows : 1));
#pragma omp for schedule(dynamic, 4)
        for (int64_t i = 0; i < (int64_t)total_rows; i++) {
            size_t flat = row_index ? row_index[i] : (size_t)i;
            uint32_t b = (uint32_t)(flat / q_rows);
            uint32_t r = (uint32_t)(flat % q_rows);
            size_t li = per_batch_limits ? flat : r;
            uint32_t limit = effective_limit(kv_limit, li, kv_rows);
            if (scores)
                visible_total += sdpa_row(out, q, k, v, b, r, limit, q_rows, kv_rows,
                                          heads, kv_heads, head_dim, scale, text_len,
                                          text_pad, scores, kf, vf);
        }
        free(scores);
    }
    free(kf);
    free(vf);
    return visible_total;
}
