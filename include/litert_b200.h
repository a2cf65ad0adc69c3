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
/* Every wait inside a kernel (on a pipeline stage, an accumulator, a tensor-
 * parallel peer) gives up after a budget, one second unless set here: the kernel
 * then records a status code, finishes without waiting and the host sees
 * B200_ERR_KERNEL_TIMEOUT. The status word is sticky (later waits give up at
 * once, so a broken step ends fast) and an aborted launch may leave split-K
 * counters behind: after a time-out call b200_clear_status before the workspace
 * is used again. b200_set_wait_budget synchronises the stream. */
B200_API int b200_set_wait_budget(void* d_zero_ws, unsigned long long nanoseconds, void* stream);
B200_API int b200_clear_status(void* d_zero_ws, void* stream);

/* Measurement aid: the device's int8 tensor-core peak (operations per second; a
 * multiply-add counts as two), from one CTA per SM issuing resident-operand
 * tcgen05.mma kind::i8 instructions back to back, `iters` x 4 each: the
 * denominator for the prefill GEMM's roofline fraction. Runs on the default
 * stream, allocates 256 bytes for its duration and synchronises. */
B200_API int b200_measure_int8_tensor_peak(int iters, double* ops_per_second, double* ms_out);

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

/* BATCH_MATMUL, hybrid, one [m,k] x [k,n] product over a packed right-hand side
 * ([n,k] as b200_pack_w8 takes it: the reference transposes the RHS to that form
 * once, tflite/kernels/batch_matmul.cc:791-798). Replaces the hybrid
 * reference_ops::BatchMatMul (tflite/kernels/internal/reference/batch_matmul.h:
 * 111-209), including its zero-point correction through float (:189,197), which
 * b200_fc_hybrid does in int32 as FULLY_CONNECTED's kernel does. */
B200_API int b200_bmm_hybrid(const float* d_x, int m, int k, const void* d_w_packed, int n,
                             const int32_t* d_row_sums, const float* d_w_scales, int per_channel,
                             int asymmetric_inputs, float* d_y, void* d_zero_ws, void* d_scratch,
                             size_t scratch_bytes, void* stream);

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

/* The composite with any number of query tokens: q / out [b,t,n,h], k / v
 * [b,s_max,nkv,h] (f16 or f32), d_mask [b,1,t,s_max] additive (optional): SDPAEval
 * as it stands (tflite/experimental/genai/sdpa.cc:361-662), every (sequence,
 * query token) pair treated as one attention row over its sequence's cache.
 * Workspace: b200_sdpa_workspace_bytes(b * t, n, nkv, h, s_max). A causal prompt
 * pass without a mask tensor is faster through b200_sdpa_rows. */
B200_API int b200_sdpa(const void* d_q, const void* d_k, const void* d_v, const float* d_mask, void* d_out, int b,
                       int t, int n, int nkv, int h, int s_max, int q_dtype, int kv_dtype, float scale,
                       float logit_cap, void* d_workspace, size_t workspace_bytes, void* stream);

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
 * The array is the current device's: make the stream's device current first (a
 * stream of another device is refused). Head layouts that the split-K kernels do
 * not take need no workspace and are not limited by the array's size.
 * Calls no cudaMalloc/cudaFree or allocating routine. */
B200_API size_t b200_sdpa_static_workspace_limit(void);
B200_API int b200_sdpa_decode_static(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                                     const float* d_v_scale, const int32_t* d_lengths, const float* d_mask,
                                     void* d_out, int b, int n, int nkv, int h, int s_max, int q_dtype, int kv_dtype,
                                     float scale, float logit_cap, void* stream);
B200_API const char* b200_sdpa_static_last_error(void);

/* ---- decoder glue ops -------------------------------------------------------
 * The ops a decoder-only graph has between its projections, as
 * tensor/examples/gemma3/gemma3_graph.cc authors them out of TFLite builtins and
 * composites, each fused with the per-row int8 quantization of the hybrid
 * FULLY_CONNECTED that consumes its result (tensor_utils::BatchQuantizeFloats,
 * tflite/kernels/internal/reference/portable_tensor_utils.cc:74-119, asymmetric).
 * Quantized rows are written in the tiled layout the GEMM kernels stream
 * ("tiled rows": b200_tiled_rows_bytes(m, k) bytes, 128-byte aligned, m rows of
 * k int8 values; b200_untile_rows gives the row-major view) and go straight into
 * b200_fc_hybrid_quantized, so that a float activation row is never written. */
B200_API const char* b200_glue_last_error(void);
B200_API size_t b200_tiled_rows_bytes(int m, int k);
B200_API int b200_untile_rows(const int8_t* d_q_tiled, int m, int k, int8_t* d_q_rowmajor, void* stream);

/* Transposes the two minor dimensions of `batches` row-major matrices [rows, cols]
 * of elem_bytes-byte elements (1 or 4): what TransposeRowsColumns does for
 * BATCH_MATMUL's adj_x / adj_y (tflite/kernels/batch_matmul.cc:789-808). */
B200_API int b200_transpose_matrices(const void* d_in, void* d_out, int batches, int rows, int cols, int elem_bytes,
                                     void* stream);

/* Hybrid EMBEDDING_LOOKUP (tflite/kernels/embedding_lookup.cc:EvalHybrid:
 * out[r,:] = table[ids[r],:] * row_scale[ids[r]]) followed by the graph's MUL by
 * a constant (out_scale; 1 for none). An id outside [0, vocab) reads row 0. */
B200_API int b200_embedding_lookup(const int32_t* d_ids, int rows, const int8_t* d_table, const float* d_row_scales,
                                   int vocab, int d, float out_scale, float* d_out, void* stream);

/* Residual ADD + RMS norm (odml.rms_norm / the MUL-MEAN-RSQRT-MUL chain,
 * gemma3_graph.cc RmsNorm) + row quantization: h += delta (delta may be NULL),
 * x = h * rsqrt(mean(h^2) + eps) * gain, x quantized per row. h [rows, d] is
 * updated in place; d <= 12288. */
B200_API int b200_add_rmsnorm_quantize(float* d_h, const float* d_delta, const float* d_gain, int rows, int d, float eps,
                                       int8_t* d_q_tiled, float* d_scales, int32_t* d_zero_points, void* stream);

/* GELU(approximate = tanh) * up (gemma3_graph.cc:118-146) + row quantization.
 * d_gate_up [rows, 2 f]: the gate then the up projection of each row. */
B200_API int b200_geglu_quantize(const float* d_gate_up, int rows, int f, int8_t* d_q_tiled, float* d_scales,
                                 int32_t* d_zero_points, void* stream);

/* Rotary embedding. In the reference graph cos and sin are INPUT tensors the host
 * side prepares (gemma3_graph.cc:150-176: x * cos + rotate_half(x) * sin);
 * b200_rope_table fills such a table on the host: h_cos_sin[(pos * head_dim / 2
 * + i) * 2 + {0, 1}] = {cos, sin}(pos * base^(-2 i / head_dim)), pos < positions.
 * b200_rope_kv_append rotates the query and key heads of d_qkv [rows, (heads + 2
 * kv_heads) * head_dim] (row r at d_positions[r]; the table must cover positions
 * 0..max_seq), writes the queries to d_q_out [rows, heads, head_dim] and appends
 * key and value to the caches [batch, max_seq, kv_heads, head_dim] at that
 * position: odml.update_kv_cache semantics
 * (tflite/experimental/genai/kvcache.cc:230-340) on a device-resident fp16 or
 * int8 cache (int8: one symmetric scale per token and KV head, max|row| / 127).
 * one_sequence != 0: all rows are consecutive tokens of the sequence whose cache
 * is passed. A position >= max_seq leaves the cache alone. */
B200_API int b200_rope_table(float* h_cos_sin, int positions, int head_dim, float base);
B200_API int b200_rope_kv_append(const float* d_qkv, int rows, int heads, int kv_heads, int head_dim,
                                 const float* d_cos_sin, const int32_t* d_positions, int max_seq, float* d_q_out,
                                 void* d_k_cache, void* d_v_cache, float* d_k_scale, float* d_v_scale, int kv_dtype,
                                 int one_sequence, void* stream);

/* Greedy pick per row of d_logits [rows, n]: the first index of the maximum, with
 * the NaN rule of litert/vendors/nvidia/dispatch/greedy_sampler_kernel.cu:31-50
 * (a NaN at index 0 wins, a NaN elsewhere never does). soft_cap > 0 compares
 * cap * tanh(logit / cap) (litert/vendors/nvidia/trtllm/head_kernels.cu:35-43). */
B200_API size_t b200_argmax_workspace_bytes(int rows);
B200_API int b200_argmax_rows(const float* d_logits, int rows, int n, float soft_cap, int32_t* d_out,
                              void* d_workspace, size_t workspace_bytes, void* stream);

/* The LM head with the greedy pick in its epilogue, for up to 16 rows: the vocabulary projection
 * (b200_fc_hybrid_quantized arithmetic, one scale per vocabulary row), the logits soft-cap of
 * litert/vendors/nvidia/trtllm/head_kernels.cu:35-43 and the first-index arg-max with the NaN rule
 * of litert/vendors/nvidia/dispatch/greedy_sampler_kernel.cu:31-94, so that one int32 per row
 * leaves the kernels. d_logits (optional, [m, n]) also receives the (capped) logits. */
B200_API size_t b200_lm_head_workspace_bytes(int m);
B200_API int b200_lm_head_greedy(const int8_t* d_q_tiled, const float* d_scales, const int32_t* d_zero_points, int m,
                                 int k, const void* d_w_packed, int n, const int32_t* d_row_sums,
                                 const float* d_w_scales, float soft_cap, float* d_logits, int32_t* d_tokens,
                                 void* d_workspace, size_t workspace_bytes, void* d_zero_ws, void* stream);

/* One decode step of a layer's attention in ONE launch, for multi-query
 * attention (one KV head, at most 8 query heads, head size 64/128/256, at most
 * 9 sequences): b200_rope_kv_append + b200_sdpa_decode over the first
 * d_positions[b] + 1 cached tokens + row quantization of the [batch, heads *
 * head_dim] result. d_qkv [batch, (heads + 2) * head_dim]. */
B200_API int b200_attention_step_supported(int heads, int kv_heads, int head_dim, int kv_dtype);
B200_API int b200_attention_step(const float* d_qkv, const int32_t* d_positions, const float* d_cos_sin,
                                 void* d_k_cache, void* d_v_cache, float* d_k_scale, float* d_v_scale, int batch,
                                 int heads, int head_dim, int max_seq, int kv_dtype, float scale, int8_t* d_q_tiled,
                                 float* d_scales, int32_t* d_zero_points, void* stream);

/* b200_sdpa_decode whose [b, n * h] result leaves as quantized tiled rows (the
 * attention-output projection's input) instead of floats. fp16 / int8 caches,
 * at most 8 query heads per KV head, head size 64/128/256. The _masked form
 * also takes float32 caches, the composite's additive mask [b, 1, 1, s_max]
 * (tflite/experimental/genai/sdpa.cc:376-386) and its logit cap. */
B200_API int b200_sdpa_decode_quantized(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                                        const float* d_v_scale, const int32_t* d_lengths, int b, int n, int nkv, int h,
                                        int s_max, int q_dtype, int kv_dtype, float scale, int8_t* d_q_tiled,
                                        float* d_scales, int32_t* d_zero_points, void* d_workspace,
                                        size_t workspace_bytes, void* stream);
B200_API int b200_sdpa_decode_quantized_masked(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                                               const float* d_v_scale, const int32_t* d_lengths, const float* d_mask,
                                               int b, int n, int nkv, int h, int s_max, int q_dtype, int kv_dtype,
                                               float scale, float logit_cap, int8_t* d_q_tiled, float* d_scales,
                                               int32_t* d_zero_points, void* d_workspace, size_t workspace_bytes,
                                               void* stream);

/* b200_fc_hybrid on rows that are already quantized (tiled rows + per-row scale
 * and zero point from one of the ops above): the second half of EvalHybridDense
 * (tflite/kernels/fully_connected.cc:797-858). */
B200_API int b200_fc_hybrid_quantized(const int8_t* d_q_tiled, const float* d_scales, const int32_t* d_zero_points,
                                      int m, int k, const void* d_w_packed, int n, const int32_t* d_row_sums,
                                      const float* d_w_scales, int per_channel, const float* d_bias, int activation,
                                      float* d_y, void* d_zero_ws, void* stream);

/* ---- float32 builtins around the projections ------------------------------------
 * What a decoder-only graph has between its quantized projections when it comes out
 * of the reference's converters (tensor/examples/gemma3/gemma3_graph.cc): so that a
 * delegate can keep the whole graph in one partition. Shapes are given as four
 * dimensions (pad with leading ones). */
B200_API const char* b200_elementwise_last_error(void);
/* op 0 = ADD, 1 = MUL, NumPy broadcasting (tflite/kernels/internal/reference/add.h,
 * mul.h: BroadcastAdd4DSlow / BroadcastMul4DSlow), no fused activation. */
B200_API int b200_binary_f32(int op, const float* d_a, const int* a_dims4, const float* d_b, const int* b_dims4,
                             float* d_out, const int* out_dims4, void* stream);
/* GELU (tflite/kernels/internal/reference/gelu.h:31-45), tanh approximation or erf. */
B200_API int b200_gelu_f32(const float* d_x, float* d_y, size_t n, int approximate, void* stream);
/* Copies the box box4 from src (at src_begin4) to dst (at dst_begin4): SLICE
 * (tflite/kernels/slice.cc) and the pieces of CONCATENATION; elements of 1 or 4 bytes. */
B200_API int b200_box_copy(const void* d_src, const int* src_dims4, const int* src_begin4, void* d_dst,
                           const int* dst_dims4, const int* dst_begin4, const int* box4, int elem_bytes, void* stream);
/* odml.rms_norm composite (ml_drift_delegate/tflite/convert/convert_rms_norm.cc:40-61):
 * y = x * rsqrt(mean(x^2) + eps) * gain per row of d elements (gain may be NULL). */
B200_API int b200_rms_norm_f32(const float* d_x, const float* d_gain, float* d_y, int rows, int d, float eps,
                               void* stream);
/* odml.update_kv_cache custom op (tflite/experimental/genai/kvcache.cc:230-340) on
 * device-resident float32 caches [max_entries, row_elems]: the t rows of d_k / d_v go
 * to slots *d_position .. + t - 1. The reference shifts the cache down when the
 * write runs past the last slot; here that raises status 201 in the zero workspace
 * (b200_read_status) and writes nothing. */
B200_API int b200_kv_cache_update_f32(const int64_t* d_position, const float* d_k, const float* d_v, int t,
                                      int row_elems, int max_entries, float* d_k_cache, float* d_v_cache,
                                      void* d_zero_ws, void* stream);
/* The rotary embedding of gemma3_graph.cc:150-176 as one kernel: out = x * cos + concat(-x2, x1) * sin,
 * x / out [tokens, heads, h], cos / sin [tokens, h] (host-prepared graph inputs, shared by the heads). */
B200_API int b200_rope_f32(const float* d_x, const float* d_cos, const float* d_sin, float* d_out, int tokens,
                           int heads, int h, void* stream);
/* b200_rope_f32 on the step's query rows [t, heads_q, h] and key rows [t, heads_kv, h] and
 * b200_kv_cache_update_f32 of the rotated keys and the value rows [t, heads_kv, h] as one launch
 * (same arithmetic, same status 201 rule): d_q_out = rope(q); rope(k) and v go to slots
 * *d_position .. + t - 1 of the caches [max_entries, heads_kv * h]. */
B200_API int b200_rope_kv_cache_update_f32(const int64_t* d_position, const float* d_q, const float* d_k,
                                           const float* d_v, const float* d_cos, const float* d_sin, float* d_q_out,
                                           int t, int heads_q, int heads_kv, int h, int max_entries,
                                           float* d_k_cache, float* d_v_cache, void* d_zero_ws, void* stream);
B200_API int b200_widen_i32_to_i64(const int32_t* d_in, int64_t* d_out, int n, void* stream);

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
/* The same for ranks that live in ONE process (one thread per GPU with peer access enabled, or a
 * test): d_exchange_buffers[j] is rank j's b200_decoder_exchange_buffer as addressable from this
 * rank's device (the own entry is ignored), each b200_decoder_exchange_bytes long. */
B200_API size_t b200_decoder_exchange_bytes(const b200_decoder* dec);
B200_API void* b200_decoder_exchange_buffer(b200_decoder* dec);
B200_API int b200_decoder_connect_peer_pointers(b200_decoder* dec, void* const* d_exchange_buffers);
/* Forgets every sequence (positions to zero) and clears the fault state below. */
B200_API int b200_decoder_reset(b200_decoder* dec);
/* Bounded waits: a kernel that waits longer than the budget (one second unless set here) for a
 * pipeline stage or for a tensor-parallel peer records a status code and finishes without waiting;
 * the step or prompt pass that notices it returns B200_ERR_KERNEL_TIMEOUT, its results are void, and
 * it has already cleared the fault state (status word, split-K counters) so that the next call
 * starts clean. b200_decoder_clear_fault does the same on demand (synchronises). After a peer
 * time-out the ranks' step counters may differ: reset every rank before going on. */
B200_API int b200_decoder_set_wait_budget(b200_decoder* dec, unsigned long long nanoseconds);
B200_API int b200_decoder_clear_fault(b200_decoder* dec);
/* Logits soft-cap applied before the greedy pick: cap * tanh(logit / cap)
 * (litert/vendors/nvidia/trtllm/head_kernels.cu:35-43); 0 = none (the default). The pick itself is the
 * first index of the maximum with the NaN rule of
 * litert/vendors/nvidia/dispatch/greedy_sampler_kernel.cu:31-50, computed inside the LM-head GEMV's
 * epilogue for up to 16 sequences on one GPU (no logits leave the kernel unless d_logits is given). */
B200_API int b200_decoder_set_logit_soft_cap(b200_decoder* dec, float cap);
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
