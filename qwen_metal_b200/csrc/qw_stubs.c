/* Link-compatibility stubs for the entry points of the reference's h3_gpu.h /
 * qwen_gpu_ext.h that lie outside the DiT attention path (linear layers, MLP,
 * VAE, vision and text-tower ops, file loaders, ...).  An engine built against
 * the reference's headers links against this library unchanged; calling one of
 * these ops fails in the reference's own way (0 / NULL) and, where the first
 * argument is a context, leaves "<name> is not implemented in the CUDA
 * attention build" in h3_gpu_error().
 *
 * Only the symbol names matter to the linker.  Each stub is defined with the
 * context (or first argument) as its only named parameter; on the System V
 * x86-64 and AArch64 calling conventions the remaining arguments of the real
 * prototype are simply ignored.
 */
#include "qw_internal.h"

#define QW_STUB_OP(name)                                                        \
    int name(h3_gpu *gpu, ...) {                                                \
        if (gpu) qw_set_error(gpu, #name " is not implemented in the CUDA attention build"); \
        return 0;                                                               \
    }
#define QW_STUB_LOADER(name)                                                    \
    h3_gpu_tensor *name(h3_gpu *gpu, ...) {                                     \
        if (gpu) qw_set_error(gpu, #name " is not implemented in the CUDA attention build"); \
        return NULL;                                                            \
    }
#define QW_STUB_PLAIN(name)                                                     \
    int name(void *first, ...) {                                                \
        (void)first;                                                            \
        return 0;                                                               \
    }

QW_STUB_OP(h3_gpu_adaln_bf16)
QW_STUB_OP(h3_gpu_adaln_bf16_offset)
QW_STUB_OP(h3_gpu_adaln_f32)
QW_STUB_OP(h3_gpu_adaln_linear_bf16)
QW_STUB_OP(h3_gpu_add_bf16)
QW_STUB_OP(h3_gpu_add_scaled_f32)
QW_STUB_OP(h3_gpu_alias_free_snake_f32)
QW_STUB_OP(h3_gpu_audio_attention_pool_f32)
QW_STUB_OP(h3_gpu_audio_qkv_split_f32)
QW_STUB_OP(h3_gpu_cast_bf16_to_f32)
QW_STUB_OP(h3_gpu_cast_f32_to_bf16)
QW_STUB_OP(h3_gpu_clip_f32)
QW_STUB_OP(h3_gpu_conv1d_f32)
QW_STUB_OP(h3_gpu_conv1d_stride_f32)
QW_STUB_OP(h3_gpu_conv3d_f32)
QW_STUB_OP(h3_gpu_conv3d_pad_f32)
QW_STUB_OP(h3_gpu_conv_transpose1d_f32)
QW_STUB_OP(h3_gpu_embedding_bf16)
QW_STUB_OP(h3_gpu_euler_bf16)
QW_STUB_OP(h3_gpu_gate_adaln_bf16)
QW_STUB_OP(h3_gpu_gate_adaln_quantize_int8)
QW_STUB_OP(h3_gpu_gate_f32)
QW_STUB_OP(h3_gpu_geglu_f32)
QW_STUB_OP(h3_gpu_gelu_bf16)
QW_STUB_OP(h3_gpu_grouped_qkv_linear_rope_bf16)
QW_STUB_OP(h3_gpu_grouped_qkv_linear_rope_int8)
QW_STUB_OP(h3_gpu_grouped_qkv_rope_bf16)
QW_STUB_OP(h3_gpu_layer_norm_bf16)
QW_STUB_OP(h3_gpu_layer_norm_f32)
QW_STUB_OP(h3_gpu_linear_f32)
QW_STUB_OP(h3_gpu_linear_int8_bf16)
QW_STUB_OP(h3_gpu_linear_int8_head_major_bf16)
QW_STUB_OP(h3_gpu_mlp_bf16)
QW_STUB_OP(h3_gpu_mlp_int8_bf16)
QW_STUB_OP(h3_gpu_mlp_nax_bf16)
QW_STUB_OP(h3_gpu_patch_linear_bf16)
QW_STUB_OP(h3_gpu_patch_linear_bf16_map)
QW_STUB_OP(h3_gpu_patch_linear_bf16_offset)
QW_STUB_OP(h3_gpu_qkv_rope_bf16)
QW_STUB_OP(h3_gpu_qkv_rope_f32)
QW_STUB_OP(h3_gpu_quantize_weight_int8)
QW_STUB_OP(h3_gpu_rms_norm_bf16)
QW_STUB_OP(h3_gpu_rms_norm_f32)
QW_STUB_OP(h3_gpu_rope_text_bf16)
QW_STUB_OP(h3_gpu_scale_add_f32)
QW_STUB_OP(h3_gpu_sdpa_causal_f32)
QW_STUB_OP(h3_gpu_sdpa_f32)
QW_STUB_OP(h3_gpu_silu_bf16)
QW_STUB_OP(h3_gpu_silu_f32)
QW_STUB_OP(h3_gpu_silu_mul_bf16)
QW_STUB_OP(h3_gpu_snake1d_f32)
QW_STUB_OP(h3_gpu_sub_bf16)
QW_STUB_OP(h3_gpu_swiglu_bf16)
QW_STUB_OP(h3_gpu_swiglu_f32)
QW_STUB_LOADER(h3_gpu_tensor_load_bf16)
QW_STUB_LOADER(h3_gpu_tensor_load_f32)
QW_STUB_PLAIN(h3_gpu_tensor_read_file_bf16)
QW_STUB_PLAIN(h3_gpu_tensor_stream_file_bf16)
QW_STUB_OP(h3_gpu_text_qk_rope_bf16)
QW_STUB_OP(h3_gpu_token_expand_adaln_bf16)
QW_STUB_OP(h3_gpu_token_expand_delta_bf16)
QW_STUB_OP(h3_gpu_token_pool_adaln_bf16)
QW_STUB_OP(h3_gpu_token_pool_bf16)
QW_STUB_OP(h3_gpu_vae_encoder_group_norm_silu_f32)
QW_STUB_OP(h3_gpu_vae_encoder_pad_f32)
QW_STUB_OP(h3_gpu_video_qkv_rope_f32)
QW_STUB_OP(h3_gpu_vision_qkv_rope_bf16)
QW_STUB_OP(h3_gpu_weight_norm_f32)
QW_STUB_OP(qw_gpu_qk_rope_half_bf16)
QW_STUB_OP(qw_gpu_rms_norm_bf16)
QW_STUB_OP(qw_gpu_rms_norm_one_bf16)
QW_STUB_OP(qw_gpu_swiglu_bf16)
QW_STUB_OP(qw_gpu_tanh_bf16)
QW_STUB_OP(qw_gpu_vae_add_f32)
QW_STUB_OP(qw_gpu_vae_avgdown_f32)
QW_STUB_OP(qw_gpu_vae_chw_to_hwc_f32)
QW_STUB_OP(qw_gpu_vae_conv3x3_f32)
QW_STUB_OP(qw_gpu_vae_conv_mm_f32)
QW_STUB_OP(qw_gpu_vae_conv_repack_f32)
QW_STUB_OP(qw_gpu_vae_downsample_f32)
QW_STUB_OP(qw_gpu_vae_dupup_f32)
QW_STUB_OP(qw_gpu_vae_hwc_to_chw_f32)
QW_STUB_OP(qw_gpu_vae_linear_t_f32)
QW_STUB_OP(qw_gpu_vae_nearest2x_f32)
QW_STUB_OP(qw_gpu_vae_rms_norm_f32)
QW_STUB_OP(qw_gpu_vae_softmax_rows_f32)
QW_STUB_OP(qw_gpu_vae_split3_f32)
QW_STUB_OP(qw_gpu_vision_add_bf16)
QW_STUB_OP(qw_gpu_vision_gelu_bf16)
QW_STUB_OP(qw_gpu_vision_ln_bf16)
QW_STUB_OP(qw_gpu_vision_merge2x2_bf16)
QW_STUB_OP(qw_gpu_vision_rope_bf16)
QW_STUB_OP(qw_gpu_vision_split3_bf16)
