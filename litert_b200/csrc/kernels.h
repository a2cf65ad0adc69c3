// Internal launch interface between the C-ABI shim and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

inline int tiles_n(int n) { return (n + 127) / 128; }
inline int tiles_k8(int k) { return (k + 127) / 128; }
inline int tiles_k4(int k) { return (k + 255) / 256; }

// Number of 8-row activation groups one launch carries (1, 2, 4 or 8).
inline int m_tiles_for(int m) {
  const int g = (m + 7) / 8;
  return g <= 1 ? 1 : (g <= 2 ? 2 : (g <= 4 ? 4 : 8));
}
// Rows allocated in the tiled activation buffer for m real rows: a multiple of the rows either
// GEMM path takes per pass (8..64 for the mma.sync path, 16..256 for the tcgen05 path).
inline int m_alloc_for(int m) {
  int nb = 16;
  while (nb < m && nb < 256) nb *= 2;
  return ((m + nb - 1) / nb) * nb;
}

cudaError_t launch_pack_w8(const int8_t* w, int n, int k, uint8_t* packed, int32_t* row_sums, cudaStream_t s);
cudaError_t launch_pack_w4(const uint8_t* w4, const void* scales_f16, int n, int k, int blocksize, uint8_t* packed,
                           float* kfsum, cudaStream_t s);
cudaError_t launch_quantize_rows(const float* x, int m, int k, int k_pad, int m_alloc, int asymmetric,
                                 int8_t* q_tiled, int8_t* q_rowmajor, float* scales, int32_t* zps, cudaStream_t s,
                                 void* h_tiled = nullptr);
cudaError_t launch_retile_x8(const int8_t* x, int m, int k, int k_pad, int m_alloc, int8_t* q_tiled,
                             int32_t* x_sums, cudaStream_t s);

// Epilogue selection for the streamed int8 GEMM.
enum FcEpilogue : int {
  kEpiHybridF32 = 0,  // float out: bias + (acc - row_sum*zp) * (in_scale*w_scale), activation
  kEpiRequantI8 = 1,  // int8 out: fixed-point requantization
  kEpiRawI32 = 2,     // int32 accumulators out (row-major [m,n])
  kEpiHybridPick = 3, // the hybrid epilogue plus the fused greedy pick (FcParams::argmax_val), at most 16 rows
};

struct FcParams {
  // operands
  const uint8_t* w_packed;   // tiles [n_tiles][k_tiles]
  const int8_t* q_tiled;     // activations, tiled, m_alloc rows
  int m, n, k;               // logical sizes
  int n_tiles, k_tiles, m_alloc;
  // hybrid epilogue
  const float* in_scales;    // [m]
  const int32_t* in_zps;     // [m] or null
  const float* w_scales;     // [n] or [1]
  int per_channel;
  const float* bias_f32;     // [n] or null
  const int32_t* row_sums;   // [n]
  int activation;
  int float_offset;          // hybrid: zero-point correction through float, as BATCH_MATMUL's reference kernel does
  // int8 epilogue
  const int32_t* bias_i32;
  const int32_t* multipliers;  // [n] or [1]
  const int32_t* shifts;
  const int32_t* x_sums;     // [m] or null (only with filter_offset != 0)
  int32_t input_offset, filter_offset, output_offset, act_min, act_max;
  // 4-bit
  const float* kfsum;        // [n]
  // outputs
  void* y;                   // [m,n] row-major float / int8 / int32
  // split-K workspace: kZeroWsSlots counters (zero between calls) and as many per-CTA partial slots
  // (no initial contents needed)
  int32_t* ws_part;
  int32_t* ws_count;
  int* status;
  // Fused input prologue (decode-sized m, see prologue.cuh): when `prologue` is 1 the activation rows
  // are built inside the kernel from the residual stream instead of being read from q_tiled:
  // v = pro_h_in + pro_delta (delta may be null), pro_h_out = v, x = rms_norm(v, pro_eps) * pro_gain,
  // x quantized per row. q_tiled, in_scales and in_zps are ignored; pro_scales_out / pro_zps_out
  // (optional) receive the rows' parameters.
  int prologue;
  const float* pro_h_in;
  const float* pro_delta;
  const float* pro_gain;
  float* pro_h_out;
  float pro_eps;
  float* pro_scales_out;
  int32_t* pro_zps_out;
  // Tensor-parallel push (hybrid float outputs of the cluster kernel, decode-sized m): besides y, every output
  // also goes to each peer j != push_rank as one 8-byte message {float bits, low 32 bits of the exchange's
  // epoch} at push_out[j][m * n + channel] (peer memory); epoch = *push_step_epoch * push_per_step + push_seq + 1.
  uint2* push_out[8];
  int push_ranks, push_rank, push_seq, push_per_step;
  const unsigned long long* push_step_epoch;
  // measurement only: four %globaltimer stamps per launch (first CTA: entry, dependency wait passed,
  // exit; any CTA: latest exit), or null
  unsigned long long* trace;
  // Weight tiles beyond its shared-memory ring that a CTA asks L2 for before it waits for its
  // activations (0 = none). Only worth it inside a chain of dependent kernels, where the wait is long.
  int l2_prefetch_tiles;
  int max_ctas;              // 0 = chosen per shape
  int whole_tiles;           // set by the launcher: CTAs own whole n tiles (no split-K)
  int force_whole_tiles;     // set by the launcher for prefill-sized passes
  int split_passes;       // several passes in one launch, each split over its share of the SMs (stream-K)
  // Fused greedy pick (hybrid epilogue, at most 16 rows, tcgen05 path): every CTA writes the best value
  // and column of each row among the channels it owns to argmax_val / argmax_idx[row * argmax_parts +
  // CTA] (first index of the maximum, NaN rule of the reference's sampler); soft_cap > 0 replaces a logit
  // by cap * tanh(logit / cap) first. y may then be null (no logits written). The caller pre-fills
  // unused slots of a row with {-inf, INT_MAX} or reduces over exactly argmax_ctas() slots.
  float* argmax_val;
  int32_t* argmax_idx;
  int argmax_parts;
  float soft_cap;
};
// Number of CTAs (= candidate slots per row) the fused pick uses for n output channels.
int fc_argmax_ctas(int n);

// Streamed-weights GEMM on the packed int8 tiles, tcgen05 / TMEM path (any m): activation rows are processed
// umma_rows_per_pass(m) at a time and the tiled activation buffer must hold a multiple of that many rows.
cudaError_t launch_fc_i8_umma(const FcParams& p, FcEpilogue epi, cudaStream_t s);
int umma_rows_per_pass(int m);
// Whether FcParams::prologue can be used for these sizes (the tcgen05 kernels only).
bool fc_prologue_supported(int m, int k);
// Whether a hybrid projection of at most 16 rows runs on the cluster split-K kernel on the current device (the
// kernel that can push its outputs to tensor-parallel peers, FcParams::push_out).
bool fc_cluster_planned(int m, int n, int k);
// Blockwise 4-bit weights, float out: the tcgen05 path (any m; q_tiled holds the quantized rows as
// fp16 in the tiled layout, w4_rows_per_pass(m) rows per pass) ...
cudaError_t launch_fc_w4(const FcParams& p, cudaStream_t s);
int w4_rows_per_pass(int m);
// ... and the one-launch path for up to 16 rows, which quantizes the float rows `x` itself.
bool w4_gemv_supported(int m, int k);
cudaError_t launch_fc_w4_gemv(const FcParams& p, const float* x, cudaStream_t s);

constexpr int kZeroWsSlots = 320;            // counters; >= 2 x CTAs per launch
constexpr int kZeroWsSlotInts = 128 * 256;   // tcgen05 path: 128 rows x up to 256 activation rows per partial slot
int device_sm_count();

// Layout of the zero workspace: [status word + padding: 256 B][slot counters][partial slots]. Only the
// first two parts must be zero between calls.
inline size_t zero_ws_counter_off() { return 256; }
inline size_t zero_ws_part_off() { return 256 + ((sizeof(int32_t) * kZeroWsSlots + 255) / 256) * 256; }
inline size_t zero_ws_total_bytes() { return zero_ws_part_off() + sizeof(int32_t) * (size_t)kZeroWsSlots * kZeroWsSlotInts; }

struct SdpaParams {
  const void* q;        // [b, t(=1), n, h] f16 or f32
  const void* k;        // [b, s_max, nkv, h] f16 / int8 / f32
  const void* v;
  const float* k_scale; // [b, s_max, nkv] for int8 kv
  const float* v_scale;
  const int32_t* lengths;  // [b] or null (= s_max)
  const float* mask;       // [b,1,1,s_max] additive or null
  void* out;               // same type/shape as q
  int b, n, nkv, h, s_max;
  int q_dtype;   // 0 = f16, 1 = f32
  int kv_dtype;  // 0 = f16, 1 = int8, 2 = f32
  float scale, logit_cap;
  float* ws;     // partials workspace
  // optional fused output quantization (decoder): the merged [b, n*h] rows are quantized per row
  // (asymmetric) and written tiled for the next GEMM instead of / in addition to `out`
  int8_t* q_tiled_out;
  float* out_scales;
  int32_t* out_zps;
  int m_alloc;
  size_t ws_bytes;
  int* status;
  // > 1: rows b * rows_per_kv .. + rows_per_kv - 1 are the query tokens of sequence b and attend over
  // that sequence's cache (the composite with several query tokens; q / out / mask are then indexed by row)
  int rows_per_kv;
  // 1: every row of the batch attends over the SAME cache (k / v / scales of one sequence, [s_max, nkv, h]),
  // row b up to lengths[b] tokens: a prompt pass, whose rows are consecutive tokens of one sequence
  int shared_kv;
};
// One decode step of a decoder layer's attention in one launch (multi-query attention, at most
// eight query heads): rotary embedding of q and of the new key, cache append, attention over the
// cached tokens, per-row asymmetric int8 quantization of the result in the tiled activation layout.
struct AttnStepParams {
  const float* qkv;           // [b][(n + 2) * h]: n query heads, the new key, the new value
  const int32_t* positions;   // [b]: tokens already cached = position of the new token
  void* k_cache;              // [b][s_max][h] fp16 or int8
  void* v_cache;
  float* k_scale;             // [b][s_max] (int8 caches)
  float* v_scale;
  int b, n, h, s_max;
  int kv_dtype;               // 0 fp16, 1 int8
  const float2* rope_cs;      // {cos, sin} per (position, rotation pair): [s_max + 1][h / 2]
  float scale;
  int8_t* q_tiled_out;        // tiled rows of width n * h
  float* out_scales;
  int32_t* out_zps;
  int m_alloc;
  int* status;                // device status word (bounded waits)
  unsigned long long* trace;  // measurement only: nine %globaltimer stamps of the first CTA, or null
};
bool attn_step_supported(int n, int nkv, int h, int kv_dtype);
cudaError_t launch_attn_step(const AttnStepParams& p, cudaStream_t s);
cudaError_t launch_sdpa_decode(const SdpaParams& p, cudaStream_t s);
size_t sdpa_workspace_bytes(int b, int n, int nkv, int h, int s_max, int shared_kv = 0);

}  // namespace b200
