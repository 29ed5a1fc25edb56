/* Host-side constructors of the attention path's inputs: per-row key limits
 * from the run layout and the joint 3-axis RoPE tables.  Pure C11, no CUDA.
 */
#include "qw_internal.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>

/* reference qwen_dit.m:1651-1665 */
void qw_dit_prefix_limits(const qw_dit_segment *segs, uint32_t seg_count, uint32_t *limits) {
    uint32_t run_start = 0;
    for (uint32_t s = 0; s < seg_count; s++) {
        const uint32_t run_rows = segs[s].rows;
        const uint32_t run_end = run_start + run_rows;
        for (uint32_t r = 0; r < run_rows; r++)
            limits[run_start + r] = segs[s].is_image ? run_end : run_start + r + 1;
        run_start = run_end;
    }
}

/* Pair frequencies theta^(-2p/axis_dim) for the 64 pairs of a head: axes
 * 16/56/56 give 8 + 28 + 28 pairs (reference qwen_pipeline.m:226,243-247). */
#define QW_ROPE_PAIRS 64
static void rope_frequencies(double frequency[QW_ROPE_PAIRS], int axis_of[QW_ROPE_PAIRS]) {
    static const int axis_dim[3] = {16, 56, 56};
    int pair = 0;
    for (int axis = 0; axis < 3; axis++)
        for (int p = 0; p < axis_dim[axis] / 2; p++, pair++) {
            frequency[pair] = pow(10000.0, -2.0 * (double)p / (double)axis_dim[axis]);
            axis_of[pair] = axis;
        }
}

static void rope_fill_row(const double frequency[QW_ROPE_PAIRS], const int axis_of[QW_ROPE_PAIRS],
                          double frame, double y, double x, float *cos_row, float *sin_row) {
    const double position[3] = {frame, y, x};
    for (int pair = 0; pair < QW_ROPE_PAIRS; pair++) {
        double angle = position[axis_of[pair]] * frequency[pair];
        cos_row[pair] = (float)cos(angle);
        sin_row[pair] = (float)sin(angle);
    }
}

/* reference qwen_pipeline.m:611-674 (one block with text_before = text_rows is
 * exactly the single-image layout of :227-252). */
uint32_t qw_rope_tables_blocks_host(const uint32_t *block_h, const uint32_t *block_w,
                                    const uint32_t *text_before, uint32_t n_blocks,
                                    float *cos_out, float *sin_out) {
    double frequency[QW_ROPE_PAIRS];
    int axis_of[QW_ROPE_PAIRS];
    rope_frequencies(frequency, axis_of);
    double cursor = 0.0; /* running position shared by the three axes for text */
    uint32_t row = 0;
    for (uint32_t b = 0; b < n_blocks; b++) {
        for (uint32_t t = 0; t < text_before[b]; t++, row++, cursor += 1.0)
            rope_fill_row(frequency, axis_of, cursor, cursor, cursor,
                          cos_out + (size_t)row * QW_ROPE_PAIRS,
                          sin_out + (size_t)row * QW_ROPE_PAIRS);
        const uint32_t gh = block_h[b], gw = block_w[b];
        const long centre_h = (long)(gh - gh / 2), centre_w = (long)(gw - gw / 2);
        for (uint32_t y = 0; y < gh; y++)
            for (uint32_t x = 0; x < gw; x++, row++)
                rope_fill_row(frequency, axis_of, cursor, (double)((long)y - centre_h),
                              (double)((long)x - centre_w),
                              cos_out + (size_t)row * QW_ROPE_PAIRS,
                              sin_out + (size_t)row * QW_ROPE_PAIRS);
        cursor += (double)(gh > gw ? gh : gw);
    }
    return row;
}

/* reference qwen_pipeline.m:227-252 */
uint32_t qw_rope_tables_host(uint32_t text_rows, uint32_t gh, uint32_t gw, float *cos_out,
                             float *sin_out) {
    return qw_rope_tables_blocks_host(&gh, &gw, &text_rows, 1, cos_out, sin_out);
}

static int tables_to_device(h3_gpu *gpu, uint32_t rows, float *cos_host, float *sin_host,
                            h3_gpu_tensor **rope_cos, h3_gpu_tensor **rope_sin, char *error,
                            size_t error_size, const char *what) {
    h3_gpu_tensor *cos_t = NULL, *sin_t = NULL;
    if (cos_host && sin_host) {
        cos_t = h3_gpu_tensor_from_f32(gpu, cos_host, (size_t)rows * QW_ROPE_PAIRS);
        sin_t = h3_gpu_tensor_from_f32(gpu, sin_host, (size_t)rows * QW_ROPE_PAIRS);
    }
    free(cos_host);
    free(sin_host);
    if (!cos_t || !sin_t) {
        h3_gpu_tensor_free(cos_t);
        h3_gpu_tensor_free(sin_t);
        if (error && error_size) snprintf(error, error_size, "%s", what);
        return 0;
    }
    *rope_cos = cos_t;
    *rope_sin = sin_t;
    return 1;
}

/* reference qwen_pipeline.m:212-270 */
int qw_pipe_rope_tables(h3_gpu *gpu, uint32_t text_rows, uint32_t gh, uint32_t gw,
                        h3_gpu_tensor **rope_cos, h3_gpu_tensor **rope_sin, char *error,
                        size_t error_size) {
    if (!text_rows || !gh || !gw) {
        if (error && error_size) snprintf(error, error_size, "rope: bad arguments");
        return 0;
    }
    uint32_t rows = text_rows + gh * gw;
    float *cos_host = malloc(sizeof(float) * (size_t)rows * QW_ROPE_PAIRS);
    float *sin_host = malloc(sizeof(float) * (size_t)rows * QW_ROPE_PAIRS);
    if (cos_host && sin_host) qw_rope_tables_host(text_rows, gh, gw, cos_host, sin_host);
    return tables_to_device(gpu, rows, cos_host, sin_host, rope_cos, rope_sin, error, error_size,
                            "rope: table build failed");
}

/* reference qwen_pipeline.m:611-691 */
int qw_pipe_rope_tables_blocks(h3_gpu *gpu, const uint32_t *block_h, const uint32_t *block_w,
                               const uint32_t *text_before, uint32_t n_blocks,
                               h3_gpu_tensor **rope_cos, h3_gpu_tensor **rope_sin, char *error,
                               size_t error_size) {
    uint32_t rows = 0;
    for (uint32_t b = 0; b < n_blocks; b++) rows += text_before[b] + block_h[b] * block_w[b];
    if (!rows) {
        if (error && error_size) snprintf(error, error_size, "rope blocks: empty layout");
        return 0;
    }
    float *cos_host = malloc(sizeof(float) * (size_t)rows * QW_ROPE_PAIRS);
    float *sin_host = malloc(sizeof(float) * (size_t)rows * QW_ROPE_PAIRS);
    if (cos_host && sin_host)
        qw_rope_tables_blocks_host(block_h, block_w, text_before, n_blocks, cos_host, sin_host);
    return tables_to_device(gpu, rows, cos_host, sin_host, rope_cos, rope_sin, error, error_size,
                            "rope blocks: build failed");
}
