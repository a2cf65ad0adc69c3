/*
 * CPU oracle for the quantized-inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a scalar restatement, in plain C, of the
 * reference kernels under tflite/kernels (paths below are relative to the
 * reference project root). It is the parity arbiter for the CUDA kernels and
 * the timed CPU baseline of the benchmark; nothing in the shipped library or
 * in the Python package may link, import or call it.
 *
 * Parity status: pinned. Every function here is checked against the golden
 * vectors and known-answer tests the reference's own unit tests hold for it
 * (tests/golden/), and the requantization helpers are additionally checked
 * against the reference's own quantization_util.cc compiled from source
 * (oracle/_ref). The blockwise 4-bit path has no reference unit test; it is
 * pinned only by the code it restates and by an independent float
 * dequantize-then-matmul cross-check.
 *
 * All matrices are dense, C-contiguous, row-major.
 */
#ifndef LITERT_B200_ORACLE_H_
#define LITERT_B200_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same integer values as TfLiteFusedActivation
 * (tflite/converter/core/c/builtin_op_data.h). */
enum {
  ORC_ACT_NONE = 0,
  ORC_ACT_RELU = 1,
  ORC_ACT_RELU_N1_TO_1 = 2,
  ORC_ACT_RELU6 = 3,
  ORC_ACT_TANH = 4,
  ORC_ACT_SIGN_BIT = 5,
  ORC_ACT_SIGMOID = 6
};

/* Requantization flavours of the full-integer path. */
enum {
  ORC_REQUANT_MBQM = 0,     /* fixed point, double rounding (the arbiter) */
  ORC_REQUANT_FLOAT_REF = 1 /* round(double(acc) * eff_scale) */
};

/* ---- fixed-point requantization --------------------------------------- */

/* tflite/kernels/internal/quantization_util.cc:53-104 */
void orc_quantize_multiplier(double real_multiplier, int32_t* quantized_multiplier, int* shift);

/* The two primitives MultiplyByQuantizedMultiplier is built from, restated
 * from their arithmetic definition (tflite/kernels/internal/common.cc:81-90,
 * tflite/kernels/internal/common.h:397-445). */
int32_t orc_saturating_rounding_doubling_high_mul(int32_t a, int32_t b);
int32_t orc_rounding_divide_by_pot(int32_t x, int exponent);

/* tflite/kernels/internal/common.cc:81-90 (double rounding, the default). */
int32_t orc_multiply_by_quantized_multiplier(int32_t x, int32_t quantized_multiplier, int shift);
/* tflite/kernels/internal/common.cc:93-115 (int64 accumulator overload). */
int32_t orc_multiply_by_quantized_multiplier_i64(int64_t x, int32_t quantized_multiplier, int shift);

/* tflite/kernels/kernel_util.cc:354-410 for an int8 output tensor.
 * Returns 0 on success. */
int orc_activation_range_int8(int activation, float out_scale, int32_t out_zero_point,
                              int32_t* act_min, int32_t* act_max);

/* tflite/kernels/fully_connected.cc:552-564: per-channel (multiplier, shift). */
void orc_fc_per_channel_multipliers(float input_scale, float output_scale, const float* filter_scales,
                                    int n, int32_t* multipliers, int32_t* shifts);
/* tflite/kernels/kernel_util.cc:291-339 + fully_connected.cc:566-572:
 * per-tensor (multiplier, shift). Returns non-zero when the bias-scale sanity
 * check fails (has_bias != 0 enables it). */
int orc_fc_per_tensor_multiplier(float input_scale, float filter_scale, int has_bias, float bias_scale,
                                 float output_scale, int32_t* multiplier, int* shift);

/* ---- full-integer FULLY_CONNECTED ------------------------------------- */

/* tflite/kernels/internal/reference/integer_ops/fully_connected.h:33-77
 * (requant == ORC_REQUANT_MBQM) and :83-132 (ORC_REQUANT_FLOAT_REF).
 * x [m,k] int8, w [n,k] int8, bias [n] int32 or NULL, y [m,n] int8.
 * input_offset = -input_zero_point. */
void orc_fc_int8_per_channel(int requant, int m, int n, int k, const int8_t* x, const int8_t* w,
                             const int32_t* bias, int32_t input_offset, int32_t output_offset,
                             const int32_t* multipliers, const int32_t* shifts, float input_scale,
                             float output_scale, const float* filter_scales, int32_t act_min,
                             int32_t act_max, int8_t* y);

/* tflite/kernels/internal/reference/integer_ops/fully_connected.h:134-180:
 * per-tensor, weights_offset = -filter_zero_point still applied. */
void orc_fc_int8_per_tensor(int m, int n, int k, const int8_t* x, const int8_t* w, const int32_t* bias,
                            int32_t input_offset, int32_t filter_offset, int32_t output_offset,
                            int32_t multiplier, int shift, int32_t act_min, int32_t act_max, int8_t* y);

/* ---- hybrid (float activations, int8 weights) ------------------------- */

/* tflite/kernels/internal/reference/portable_tensor_utils.cc:41-71 */
void orc_symmetric_quantize_floats(const float* values, int size, int8_t* q, float* scale);
/* tflite/kernels/internal/reference/portable_tensor_utils.cc:74-119 */
void orc_asymmetric_quantize_floats(const float* values, int size, int8_t* q, float* scale,
                                    int32_t* zero_point);
/* tflite/kernels/internal/portable_tensor_utils.h:158-176 */
void orc_batch_quantize_floats(const float* x, int m, int k, int8_t* q, float* scales,
                               int32_t* zero_points, int asymmetric);

/* tflite/kernels/internal/reference/portable_tensor_utils.cc:165-206:
 * result[m,n] += (dot(w[n,:], q[m,:]) - row_sums[n]*zp[m]) * (scales[m] * per_channel_scale[n]).
 * row_sums is recomputed from w when compute_row_sums != 0. */
void orc_matrix_batch_vector_mac_hybrid(const int8_t* w, int n, int k, const int8_t* q,
                                        const float* scales, int m, float* result,
                                        const float* per_channel_scale, const int32_t* zero_points,
                                        int32_t* row_sums, int compute_row_sums);

/* tflite/kernels/internal/tensor_utils.h:58-80 */
void orc_apply_activation(float* v, size_t size, int activation);

/* tflite/kernels/fully_connected.cc:763-858 (EvalHybridDense) for int8 weights.
 * filter_scales has n entries when per_channel != 0, else one entry. */
void orc_fc_hybrid(int m, int n, int k, const float* x, const int8_t* w, const float* filter_scales,
                   int per_channel, const float* bias, int asymmetric_inputs, int activation, float* y);

/* tflite/kernels/fully_connected.cc:1014-1086 (EvalBlockwise4Bit).
 * w4: n rows of ((k+1)&~1)/2 bytes, element 2i in the low nibble;
 * scales_f16 [n, k/blocksize] as IEEE binary16 bit patterns. */
void orc_fc_blockwise4(int m, int n, int k, int blocksize, const float* x, const uint8_t* w4,
                       const uint16_t* scales_f16, const float* bias, float* y);

/* tflite/kernels/internal/portable_tensor_utils.cc:96-150, 4-bit signed case */
void orc_unpack_int4(const uint8_t* src, int num_elements, int8_t* dst);

float orc_half_to_float(uint16_t h);
uint16_t orc_float_to_half(float f);

/* ---- BATCH_MATMUL ------------------------------------------------------ */

/* The three overloads of tflite/kernels/internal/reference/batch_matmul.h
 * (55-109 float, 111-209 hybrid, 211-284 int8), with the operand naming of
 * that file: "lhs" [.., rows, depth] and "rhs" [.., cols, depth] are both
 * depth-contiguous, shapes are extended to 5-D, output is [.., cols, rows]
 * (lhs_rows * j + i). The op-level wrappers below do what
 * tflite/kernels/batch_matmul.cc:744-827 does before calling them. */
void orc_ref_bmm_float(const int* lhs_shape5, const float* lhs, const int* rhs_shape5, const float* rhs,
                       float* out);
void orc_ref_bmm_hybrid(const int* lhs_shape5, const int8_t* lhs, const int* rhs_shape5,
                        const int8_t* rhs, const float* scaling_factors, const int32_t* input_offset,
                        int32_t* row_sums, int compute_row_sums, const float* per_channel_scales,
                        float* out);
void orc_ref_bmm_int8(const int* lhs_shape5, const int8_t* lhs, const int* rhs_shape5, const int8_t* rhs,
                      int32_t input_offset, int32_t filter_offset, int32_t output_offset,
                      int32_t multiplier, int shift, int32_t act_min, int32_t act_max, int8_t* out);

/* Op-level BATCH_MATMUL: x [.., A, B] (or [.., B, A] when adj_x) times
 * y [.., B, C] (or [.., C, B] when adj_y), broadcasting up to three batch
 * dims; ranks 2..5. Output [.., A, C] row-major. */
void orc_batch_matmul_float(int x_rank, const int* x_dims, const float* x, int y_rank, const int* y_dims,
                            const float* y, int adj_x, int adj_y, float* out);
/* Hybrid: float x, int8 y with per-tensor scale (tflite/kernels/batch_matmul.cc:454-526). */
void orc_batch_matmul_hybrid(int x_rank, const int* x_dims, const float* x, int y_rank, const int* y_dims,
                             const int8_t* y, float y_scale, int adj_x, int adj_y, int asymmetric_inputs,
                             float* out);
/* Same with one scale per output column instead of y_scale when per_channel_scales is given. */
void orc_batch_matmul_hybrid_pc(int x_rank, const int* x_dims, const float* x, int y_rank, const int* y_dims,
                                const int8_t* y, float y_scale, const float* per_channel_scales, int adj_x, int adj_y,
                                int asymmetric_inputs, float* out);
/* int8 x int8 -> int8 (tflite/kernels/batch_matmul.cc:528-556). */
void orc_batch_matmul_int8(int x_rank, const int* x_dims, const int8_t* x, int32_t x_zero_point,
                           int y_rank, const int* y_dims, const int8_t* y, int32_t y_zero_point,
                           int adj_x, int adj_y, int32_t multiplier, int shift, int32_t out_zero_point,
                           int8_t* out);

/* ---- odml.scaled_dot_product_attention -------------------------------- */

/* tflite/experimental/genai/sdpa.cc:361-662 with
 * tflite/kernels/internal/reference/softmax.h:33-64. q [b,t,n,h], k/v
 * [b,s,nkv,h], mask [b,1,t,s] additive (may be NULL = zeros), out [b,t,n,h].
 * logit_cap > 0 applies cap*tanh(logits/cap) before the mask add
 * (tflite/delegates/xnnpack/xnnpack_delegate.cc:6639-6678). q is NOT modified
 * (the reference scales it in place; callers compare outputs only). */
void orc_sdpa_f32(int b, int t, int n, int nkv, int h, int s, const float* q, const float* k,
                  const float* v, const float* mask, float scale, float logit_cap, float* out);

#ifdef __cplusplus
}
#endif
#endif  /* LITERT_B200_ORACLE_H_ */
