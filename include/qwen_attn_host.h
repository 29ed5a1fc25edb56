/* qwen_attn_host.h -- host-side constructors of the attention path's integer
 * and table inputs, with the reference's names and signatures.  Citations are
 * path:line inside the reference project.
 */
#ifndef QWEN_ATTN_HOST_H
#define QWEN_ATTN_HOST_H

#include "h3_gpu.h"

#ifdef __cplusplus
extern "C" {
#endif

/* reference qwen_dit.h:25-29: one run of the joint sequence
 * [text0][img0]...[textN][target]; the target image run is last. */
typedef struct {
    uint32_t rows;
    int is_image;
    uint32_t src_offset;
} qw_dit_segment;

/* reference qwen_dit.m:1651-1665: per-row key limits of the block-causal mask.
 * Image rows see up to the end of their own run, text rows are token-causal.
 * `limits` holds sum(rows) entries. */
void qw_dit_prefix_limits(const qw_dit_segment *segs, uint32_t seg_count, uint32_t *limits);

/* reference qwen_pipeline.h / qwen_pipeline.m:212-270: joint 3-axis RoPE tables
 * [text_rows + gh*gw, 64] f32 (axes 16/56/56, theta 1e4); text row t uses
 * position t on all three axes, image tokens use frame = text_rows and centred
 * height/width indices.  On success the two tensors are owned by the caller. */
int qw_pipe_rope_tables(h3_gpu *gpu, uint32_t text_rows, uint32_t gh, uint32_t gw,
                        h3_gpu_tensor **rope_cos, h3_gpu_tensor **rope_sin, char *error,
                        size_t error_size);

/* reference qwen_pipeline.m:611-691: multi-block tables for the edit path,
 * layout [text_before[b] rows][block_h[b]*block_w[b] rows] per block. */
int qw_pipe_rope_tables_blocks(h3_gpu *gpu, const uint32_t *block_h, const uint32_t *block_w,
                               const uint32_t *text_before, uint32_t n_blocks,
                               h3_gpu_tensor **rope_cos, h3_gpu_tensor **rope_sin, char *error,
                               size_t error_size);

/* NEW: the same tables into caller-provided host arrays of rows*64 floats
 * (no GPU needed); return the row count. */
uint32_t qw_rope_tables_host(uint32_t text_rows, uint32_t gh, uint32_t gw, float *cos_out,
                             float *sin_out);
uint32_t qw_rope_tables_blocks_host(const uint32_t *block_h, const uint32_t *block_w,
                                    const uint32_t *text_before, uint32_t n_blocks,
                                    float *cos_out, float *sin_out);

#ifdef __cplusplus
}
#endif
#endif
