// Launch interface of the decode-step glue kernels (decoder_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kArgmaxParts = 128;

cudaError_t launch_embed(const int32_t* tokens, const int8_t* table, const float* row_scales, int batch, int d,
                         float embed_scale, float* h, const int32_t* positions, int32_t* attn_len, cudaStream_t s);
cudaError_t launch_add_norm_quant(float* h, const float* delta, const float* gain, int batch, int d, float eps,
                                  int m_alloc, int8_t* q_tiled, float* scales, int32_t* zps, cudaStream_t s);
cudaError_t launch_geglu_quant(const float* gate_up, int batch, int f, int m_alloc, int8_t* q_tiled, float* scales,
                               int32_t* zps, cudaStream_t s);
cudaError_t launch_rope_cache(const float* qkv, int batch, int heads, int kv_heads, int head_dim, float rope_base,
                              const int32_t* positions, int max_seq, float* q_out, void* k_cache, void* v_cache,
                              float* k_scale, float* v_scale, int kv_int8, cudaStream_t s);
cudaError_t launch_argmax(const float* logits, int batch, int n, float* part_val, int32_t* part_idx,
                          int32_t* next_tokens, int32_t* positions, int max_seq, cudaStream_t s);

}  // namespace b200
