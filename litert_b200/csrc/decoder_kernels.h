// Launch interface of the decode-step glue kernels (decoder_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kArgmaxParts = 128;
constexpr int kArgmaxSlots = 512;  // candidate slots per row: kArgmaxParts, or one per CTA of the fused LM-head pick
constexpr int kMaxTpRanks = 8;

// One cross-rank exchange of a tensor-parallel step, done inside the kernel that consumes the sum.
// Every rank keeps its partial result in its own exchange buffer; the consuming kernel tells each
// peer "my partial number `epoch` is complete" with a release store into the peer's flag array,
// waits (bounded) until every peer's flag in its own array has reached `epoch`, then reads the
// peers' partials straight from their memory over NVLink and adds them in rank order.
// epoch = *step_epoch * per_step + seq + 1: the step counter lives on the device and is advanced
// by the first kernel of each step, so that a captured graph can be replayed.
struct TpExchange {
  int tp_size = 1, tp_rank = 0;
  int seq = 0, per_step = 1;
  const float* partial[kMaxTpRanks] = {nullptr};        // rank j's partial of this exchange (own entry: local)
  unsigned long long* flag_out[kMaxTpRanks] = {nullptr};  // slot [tp_rank] of rank j's flag array
  const unsigned long long* flags_in = nullptr;          // this rank's flag array [kMaxTpRanks]
  const unsigned long long* step_epoch = nullptr;
  int* status = nullptr;
  // Decode-sized rows (at most kTpPushRows): the producing GEMV has already PUSHED its partial into every peer's
  // memory as 8-byte messages {value bits, low 32 bits of the epoch} (FcParams::push_out), so the consumer only
  // polls its own memory until every message carries this exchange's epoch: no flag, no fence, no remote read.
  // push_in: this rank's message area of the exchange, [tp_size][push_stride] messages (slot j from rank j).
  const uint2* push_in = nullptr;
  int push_stride = 0;
};
constexpr int kTpPushRows = 8;

// step_epoch (optional): device counter advanced by one, the clock of the cross-rank exchanges.
// positions / attn_len (optional): attn_len[b] = positions[b] + 1.
cudaError_t launch_embed(const int32_t* tokens, const int8_t* table, const float* row_scales, int batch, int vocab, int d,
                         float embed_scale, float* h, const int32_t* positions, int32_t* attn_len,
                         unsigned long long* step_epoch, cudaStream_t s);
// h += delta; x = rms_norm(h) * gain; quantize x. With xch (tp_size > 1) delta is the sum over ranks of
// xch->partial[j], fetched inside the kernel.
cudaError_t launch_add_norm_quant(float* h, const float* delta, const float* gain, int batch, int d, float eps,
                                  int m_alloc, int8_t* q_tiled, float* scales, int32_t* zps, const TpExchange* xch,
                                  cudaStream_t s);
cudaError_t launch_geglu_quant(const float* gate_up, int batch, int f, int m_alloc, int8_t* q_tiled, float* scales,
                               int32_t* zps, cudaStream_t s);
// one_sequence: the rows are consecutive tokens of ONE sequence (a prompt pass) and k_cache / v_cache /
// k_scale / v_scale point at that sequence's cache; otherwise row b belongs to sequence b.
// Host side of the rotary embedding: cs[(pos * (head_dim / 2) + i) * 2 + {0, 1}] = {cos, sin} of
// pos * base^(-2 i / head_dim) for pos < positions, in float with the C library's powf / cosf / sinf.
void fill_rope_table(float* cs, int positions, int head_dim, float base);
// rope_cs: {cos, sin} per (position, rotation pair), [max_seq + 1][head_dim / 2] (fill_rope_table).
cudaError_t launch_rope_cache(const float* qkv, int batch, int heads, int kv_heads, int head_dim, const float2* rope_cs,
                              const int32_t* positions, int max_seq, float* q_out, void* k_cache, void* v_cache,
                              float* k_scale, float* v_scale, int kv_int8, int one_sequence, cudaStream_t s);
// First-index argmax of each row; advances positions. idx_offset is added to the winning column.
// With pair_out the winner goes to pair_out[b] = {value, index as float} instead, and neither
// next_tokens nor positions change (launch_argmax_pick finishes the job across ranks).
// soft_cap > 0: the comparison runs on cap * tanh(logit / cap). positions may be null.
cudaError_t launch_argmax(const float* logits, int batch, int n, int idx_offset, float soft_cap, float* part_val,
                          int32_t* part_idx, int32_t* next_tokens, int32_t* positions, int max_seq, float2* pair_out,
                          cudaStream_t s);
// The last stage alone, over `parts` candidates per row that an earlier kernel left in part_val / part_idx
// (row-major [batch, parts]): the LM-head GEMV's fused pick writes one per CTA.
cudaError_t launch_argmax_final(const float* part_val, const int32_t* part_idx, int batch, int parts, int idx_offset,
                                int32_t* next_tokens, int32_t* positions, int max_seq, float2* pair_out, cudaStream_t s);
// Picks the best of tp_size candidate pairs per row. pairs[j] = rank j's float2[batch]; when xch is given
// they are peers' memory and the exchange handshake runs first, otherwise they are local.
cudaError_t launch_argmax_pick(const float2* const* pairs, int tp_size, int batch, int32_t* next_tokens,
                               int32_t* positions, int max_seq, const TpExchange* xch, cudaStream_t s);

}  // namespace b200
