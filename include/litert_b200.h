/*
 * litert_b200 -- C ABI of the B200 (sm_100a) kernels behind the LiteRT /
 * TFLite quantized-inference hot path: FULLY_CONNECTED and BATCH_MATMUL with
 * full-integer int8, dynamic-range (hybrid) int8 and blockwise int4 weights,
 * and the odml.scaled_dot_product_attention decode step.
 *
 * This is the boundary a host runtime binds: plain pointers and sizes, no C++
 * or torch types. Every pointer named d_* is a device pointer on the current
 * CUDA device; `stream` is a cudaStream_t passed as void* (NULL = default
 * stream). Calls enqueue work and return without synchronising. Return value:
 * B200_OK or an error code; b200_last_error() gives the message of the last
 * failure on the calling thread. Reference interfaces cited below are paths
 * inside the LiteRT source tree.
 *
 * Weights are repacked once (b200_pack_w8 / b200_pack_w4) into the tiled
 * device layout the kernels stream; activations stay in the reference's
 * row-major layouts at this boundary.
 */
#ifndef LITERT_B200_H_
#define LITERT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

enum {
  B200_OK = 0,
  B200_ERR_INVALID_ARGUMENT = 1,
  B200_ERR_CUDA = 2,
  B200_ERR_KERNEL_TIMEOUT = 3, /* a bounded device-side wait ran out */
  B200_ERR_UNSUPPORTED = 4
};

/* Fused activations, numbered like TfLiteFusedActivation
 * (tflite/converter/core/c/builtin_op_data.h). */
enum {
  B200_ACT_NONE = 0,
  B200_ACT_RELU = 1,
  B200_ACT_RELU_N1_TO_1 = 2,
  B200_ACT_RELU6 = 3,
  B200_ACT_TANH = 4,
  B200_ACT_SIGN_BIT = 5,
  B200_ACT_SIGMOID = 6
};

enum { B200_DTYPE_F16 = 0, B200_DTYPE_I8 = 1, B200_DTYPE_F32 = 2 };

B200_API int b200_abi_version(void);
B200_API const char* b200_last_error(void);

/* ---- workspaces ---------------------------------------------------------
 * Two device buffers, owned by the caller, may be shared by all ops that run
 * on one stream (ops on different streams need their own):
 *  - the "zero workspace": fixed size, cleared once with
 *    b200_zero_workspace_init; kernels leave it cleared after every call. Its
 *    first int is a status word (see b200_read_status).
 *  - the "scratch": sized per op shape, no initial contents required; takes
 *    the role of the temporary tensors the reference op allocates
 *    (tflite/kernels/fully_connected.cc:602-719: input_quantized,
 *    scaling_factors, input_offsets). */
B200_API size_t b200_zero_workspace_bytes(void);
B200_API int b200_zero_workspace_init(void* d_zero_ws, void* stream);
B200_API size_t b200_fc_scratch_bytes(int m, int k);
/* Copies the status word to the host (synchronises the stream). 0 = ok. */
B200_API int b200_read_status(void* d_zero_ws, void* stream, int* status_out);

/* ---- weight preparation (once per constant tensor) ----------------------
 * int8 weights [n,k] row-major, as a FULLY_CONNECTED filter tensor lies in
 * the model (tflite/kernels/fully_connected.cc:498-503). d_row_sums [n]
 * (optional) receives sum_k w[n,k], the reference's cached row_sums temporary
 * (tflite/kernels/fully_connected.cc:697-708). */
B200_API size_t b200_packed_w8_bytes(int n, int k);
B200_API int b200_pack_w8(const int8_t* d_w, int n, int k, void* d_packed, int32_t* d_row_sums, void* stream);

/* int4 weights: n rows of ((k+1)&~1)/2 bytes, element 2i in the low nibble
 * (tflite/kernels/fully_connected.cc:1053-1067), fp16 scales
 * [n, k/blocksize] (TfLiteBlockwiseQuantization, tflite/core/c/common.h:390-398).
 * d_kfsum [n] receives the activation-independent zero-point term. */
B200_API size_t b200_packed_w4_bytes(int n, int k);
B200_API int b200_pack_w4(const uint8_t* d_w4, const uint16_t* d_scales_f16, int n, int k, int blocksize,
                          void* d_packed, float* d_kfsum, void* stream);

/* ---- activation quantization --------------------------------------------
 * Replaces tensor_utils::BatchQuantizeFloats
 * (tflite/kernels/internal/portable_tensor_utils.h:158-176): per row of
 * x [m,k], int8 values (row-major d_q), scale and zero point. */
B200_API int b200_quantize_rows(const float* d_x, int m, int k, int asymmetric, int8_t* d_q, float* d_scales,
                                int32_t* d_zero_points, void* stream);

/* ---- FULLY_CONNECTED ------------------------------------------------------
 * Full-integer int8. Replaces FullyConnectedPerChannelInt8 / FullyConnectedInt8
 * (tflite/kernels/fully_connected.cc:1383-1421, 1255-1285) i.e.
 * reference_integer_ops::FullyConnected[PerChannel]
 * (tflite/kernels/internal/reference/integer_ops/fully_connected.h:33-77,
 * 134-180). y = clamp(MBQM(sum (w+filter_offset)(x+input_offset) + bias,
 * mult, shift) + output_offset). per_channel != 0: d_multipliers/d_shifts have
 * n entries and filter_offset must be 0; else one entry. */
B200_API int b200_fc_int8(const int8_t* d_x, int m, int k, const void* d_w_packed, int n,
                          const int32_t* d_row_sums, const int32_t* d_bias, int32_t input_offset,
                          int32_t filter_offset, int32_t output_offset, const int32_t* d_multipliers,
                          const int32_t* d_shifts, int per_channel, int32_t act_min, int32_t act_max,
                          int8_t* d_y, void* d_zero_ws, void* d_scratch, size_t scratch_bytes, void* stream);

/* Dynamic-range hybrid. Replaces EvalHybridDense
 * (tflite/kernels/fully_connected.cc:763-858): per-row input quantization,
 * int8 dot products, y = act(bias + (dot - row_sum*zp) * in_scale * w_scale).
 * d_w_scales has n entries (per_channel) or 1. */
B200_API int b200_fc_hybrid(const float* d_x, int m, int k, const void* d_w_packed, int n,
                            const int32_t* d_row_sums, const float* d_w_scales, int per_channel,
                            const float* d_bias, int asymmetric_inputs, int activation, float* d_y,
                            void* d_zero_ws, void* d_scratch, size_t scratch_bytes, void* stream);

/* Blockwise int4. Replaces EvalBlockwise4Bit
 * (tflite/kernels/fully_connected.cc:1014-1086): always asymmetric inputs, no
 * fused activation. blocksize must be a multiple of 32. */
B200_API int b200_fc_w4(const float* d_x, int m, int k, const void* d_w4_packed, int n, int blocksize,
                        const float* d_kfsum, const float* d_bias, float* d_y, void* d_zero_ws,
                        void* d_scratch, size_t scratch_bytes, void* stream);

/* ---- odml.scaled_dot_product_attention, one query token -------------------
 * Replaces ops::custom::llm::SDPAEval (tflite/experimental/genai/sdpa.cc:361-662)
 * for T = 1. q/out [b,1,n,h] (f16 or f32), k/v [b,s_max,nkv,h] (f16, int8 with
 * one f32 scale per cached token and kv head in d_k_scale/d_v_scale
 * [b,s_max,nkv], or f32). d_lengths [b] (optional) bounds the attended prefix
 * per sequence; d_mask [b,1,1,s_max] (optional) is the reference's additive
 * mask. scale <= 0 means 1/sqrt(h) (sdpa.cc:99-105). logit_cap > 0 applies
 * cap*tanh(x/cap) before the mask
 * (tflite/delegates/xnnpack/xnnpack_delegate.cc:6639-6678). */
B200_API size_t b200_sdpa_workspace_bytes(int b, int n, int nkv, int h, int s_max);
B200_API int b200_sdpa_decode(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                              const float* d_v_scale, const int32_t* d_lengths, const float* d_mask,
                              void* d_out, int b, int n, int nkv, int h, int s_max, int q_dtype, int kv_dtype,
                              float scale, float logit_cap, void* d_workspace, size_t workspace_bytes,
                              void* stream);

/* Prompt-shaped attention: `rows` query tokens of ONE sequence (q and out [rows, n, h]) over that
 * sequence's cache (k / v [s_max, nkv, h], scales [s_max, nkv] for int8), row r attending over the
 * first d_lengths[r] cached tokens. With d_lengths[r] = start + r + 1 this is the causal composite
 * with several query tokens (tflite/delegates/xnnpack/xnnpack_delegate.cc:6639-6678 with the
 * lower-triangular mask the converter emits). At most 8 query heads per KV head, head size 64, 128
 * or 256; no additive mask. Workspace: b200_sdpa_rows_workspace_bytes. */
B200_API size_t b200_sdpa_rows_workspace_bytes(int rows, int n, int nkv, int h, int s_max);
B200_API int b200_sdpa_rows(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                            const float* d_v_scale, const int32_t* d_lengths, void* d_out, int rows, int n,
                            int nkv, int h, int s_max, int q_dtype, int kv_dtype, float scale, float logit_cap,
                            void* d_workspace, size_t workspace_bytes, void* stream);

/* ---- attention decode step without any allocation --------------------------
 * No counterpart in the reference: this entry point exists for callers of THIS
 * library that are not allowed to allocate device memory (a serving loop that
 * has frozen its allocator after start-up, a plugin living inside someone
 * else's fixed memory budget, code being recorded for replay) and therefore
 * cannot supply the workspace b200_sdpa_decode asks for. Same arguments and
 * results as b200_sdpa_decode, minus the workspace: the split-K partials go to
 * a built-in device array of b200_sdpa_static_workspace_limit() bytes (8 MiB,
 * held by every GPU that loads the library until exit). Shapes that need more
 * are rejected with B200_ERR_UNSUPPORTED. The first call on a device looks up
 * the array's device address (set-up; make it before any stream capture).
 * Calls share the array: calls that overlap on the GPU race, serialise them.
 * Calls no cudaMalloc/cudaFree or allocating routine. */
B200_API size_t b200_sdpa_static_workspace_limit(void);
B200_API int b200_sdpa_decode_static(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                                     const float* d_v_scale, const int32_t* d_lengths, const float* d_mask,
                                     void* d_out, int b, int n, int nkv, int h, int s_max, int q_dtype, int kv_dtype,
                                     float scale, float logit_cap, void* stream);
B200_API const char* b200_sdpa_static_last_error(void);

/* ---- Gemma-shaped decoder, one decode step per call ---------------------------
 * A resident decoder for the decode benchmark: every projection is a dynamic-range
 * hybrid FULLY_CONNECTED (b200_fc_hybrid semantics: per-row asymmetric input
 * quantization, int8 per-channel weights), attention is b200_sdpa_decode over an
 * fp16 or int8 KV cache kept on the device, and the ops in between (RMS norm,
 * rotary embedding, GELU(tanh)*up, residual adds, hybrid embedding lookup, greedy
 * argmax) follow the graph tensor/examples/gemma3/gemma3_graph.cc authors, with
 * the Gemma-1 layout (no q/k norms, no post-norms). The whole step is one CUDA
 * graph. No counterpart exists in the reference as a single entry point: there
 * the same work is the Interpreter invoking the graph node by node
 * (tflite/core/subgraph.cc:1666-1811).
 *
 * Tensor parallelism (one process per GPU, tp_size <= 8): the config holds the
 * whole model's sizes; rank r keeps heads [r*n_heads/tp, ...), feed-forward units
 * [r*d_ff/tp, ...) and LM-head rows [r*vocab/tp, ...): q/gate/up are cut by output
 * rows, o/down by input columns, a KV head that several ranks share is replicated.
 * Each rank quantizes its own slice of an activation row, as a graph with one
 * FULLY_CONNECTED per shard would. The two partial sums per layer and the greedy
 * winner over the vocabulary shards cross the ranks in one of two ways:
 *  - b200_decoder_connect_peers: every rank exports its exchange buffer
 *    (b200_decoder_exchange_handle, a CUDA IPC handle), the host passes all handles
 *    to every rank, and the kernel that consumes a sum (residual add + RMS norm +
 *    quantization, or the final token pick) reads the peers' partials itself over
 *    NVLink after a flag handshake: no collective launch on the path;
 *  - b200_decoder_init_nccl / b200_decoder_set_allreduce: an all-reduce (NCCL
 *    loaded at run time, or the caller's own) enqueued between the kernels.
 * All ranks must make the same calls in the same order. A peer that never arrives
 * makes the waiting kernel give up after one second; the step then returns
 * B200_ERR_KERNEL_TIMEOUT. */
typedef struct b200_decoder b200_decoder;

typedef struct {
  int n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab;
  int max_seq, max_batch;
  float rms_eps, rope_base, embed_scale;
  int kv_dtype;          /* B200_DTYPE_F16 or B200_DTYPE_I8 */
  int tp_size, tp_rank;  /* 1, 0 for a single GPU */
} b200_decoder_config;

/* All weight pointers are DEVICE pointers to row-major int8 [n,k] with one f32
 * scale per output channel; they are repacked inside and may be freed after the
 * call. With tp_size > 1 pass this rank's shard. */
typedef struct {
  const int8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
  const float *sq, *sk, *sv, *so, *sgate, *sup, *sdown;
  const float *norm1, *norm2; /* [d_model] */
} b200_decoder_layer_weights;

/* Sum over ranks, in place, of `count` floats on `stream` (device buffer). */
typedef int (*b200_allreduce_fn)(void* user, float* d_buf, size_t count, void* stream);

B200_API int b200_decoder_create(const b200_decoder_config* config, void* stream, b200_decoder** out);
B200_API void b200_decoder_destroy(b200_decoder* dec);
B200_API int b200_decoder_set_layer(b200_decoder* dec, int layer, const b200_decoder_layer_weights* w);
/* Embedding table [vocab, d_model] (also the LM head; with tp_size > 1 the LM
 * head uses rows [rank*vocab/tp, (rank+1)*vocab/tp) and the logits are left
 * sharded), per-row scales [vocab], final norm gain [d_model]. */
B200_API int b200_decoder_set_embedding(b200_decoder* dec, const int8_t* d_table, const float* d_row_scales,
                                        const float* d_final_norm);
B200_API int b200_decoder_set_allreduce(b200_decoder* dec, b200_allreduce_fn fn, void* user);
/* 128-byte NCCL unique id, made on one rank and handed to all (ncclGetUniqueId). */
B200_API int b200_nccl_unique_id(void* out, size_t bytes);
/* Joins the communicator of tp_size ranks (ncclCommInitRank) and installs its all-reduce. */
B200_API int b200_decoder_init_nccl(b200_decoder* dec, const void* unique_id);
/* CUDA IPC handle (64 bytes) of this rank's exchange buffer. */
B200_API int b200_decoder_exchange_handle(b200_decoder* dec, void* handle_out, size_t bytes);
/* handles: tp_size handles, bytes_per_handle apart, in rank order (the own entry is ignored). */
B200_API int b200_decoder_connect_peers(b200_decoder* dec, const void* handles, size_t bytes_per_handle);
B200_API int b200_decoder_reset(b200_decoder* dec);
/* Declares h_positions[i] tokens already cached for sequence i (cache rows never written hold
 * zeros): lets a caller resume from a cache filled elsewhere, or time a step at a given depth. */
B200_API int b200_decoder_set_positions(b200_decoder* dec, const int32_t* h_positions, int batch);
/* One token per sequence. h_tokens / h_next_tokens are HOST arrays of `batch`
 * ints (pinned memory avoids a staging copy); d_logits (optional, device,
 * [batch, vocab]) receives the logits. Synchronises the stream before returning
 * when h_next_tokens is given. */
B200_API int b200_decoder_step(b200_decoder* dec, const int32_t* h_tokens, int batch, int32_t* h_next_tokens,
                               float* d_logits);
/* Prompt pass: runs the n_tokens prompt tokens (HOST array) of sequence `seq` through the layers in
 * chunks of up to 1024 rows, every projection as one GEMM over the chunk, appends their keys and
 * values to the sequence's cache behind the tokens already there, and predicts the first generated
 * token from the last prompt token (greedy; written to *h_next_token when given, and kept on the
 * device so that b200_decoder_run(dec, NULL, ...) continues from it). Results are those of
 * n_tokens single steps of that sequence. Other sequences are untouched. With tp_size > 1 the
 * partial sums go through the all-reduce (b200_decoder_init_nccl / b200_decoder_set_allreduce).
 * Synchronises the stream. */
B200_API int b200_decoder_prefill(b200_decoder* dec, int seq, const int32_t* h_tokens, int n_tokens,
                                  int32_t* h_next_token);
/* Device-resident variant: feeds the previous step's greedy tokens back without
 * touching the host (first call after a reset uses h_first_tokens). Runs `steps`
 * steps; the last tokens are copied to h_next_tokens when given. */
B200_API int b200_decoder_run(b200_decoder* dec, const int32_t* h_first_tokens, int batch, int steps,
                              int32_t* h_next_tokens);
/* Runs ONE step eagerly (no graph) with CUDA events around every launch and
 * returns the device time per kernel class: [0] the streamed GEMVs, [1]
 * attention, [2] the glue kernels (ms), and how many launches each class had.
 * Advances the sequence like a normal step. */
B200_API int b200_decoder_profile_step(b200_decoder* dec, const int32_t* h_tokens, int batch, float* ms_by_class,
                                       int* launches_by_class);
/* Message of the last b200_decoder_* failure on the calling thread. */
B200_API const char* b200_decoder_last_error(void);
/* Number of kernels one step launches (for reporting). */
B200_API int b200_decoder_launches_per_step(const b200_decoder* dec);
/* Times the projections of one step alone: the step's GEMV launches, in step order over the
 * current activation buffers, replayed `reps` times as one CUDA graph between two events on the
 * decoder's stream. ms_per_step = device time of one pass over all of them. */
B200_API int b200_decoder_time_gemv(b200_decoder* dec, int batch, int reps, float* ms_per_step, int* launches_per_step);

#ifdef __cplusplus
}
#endif
#endif /* LITERT_B200_H_ */
