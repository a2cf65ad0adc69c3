/*
 * CPU oracle: scalar restatement of the reference kernels. TEST
 * INFRASTRUCTURE ONLY -- see oracle.h for the rules and the parity status.
 * Loop orders and float evaluation orders follow the cited reference code so
 * that float results match it bit for bit when compiled with
 * -ffp-contract=off (the reference's default x86-64 build has no FMA
 * contraction either).
 */
#include "oracle.h"

#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* fixed-point requantization                                         */
/* ------------------------------------------------------------------ */

/* tflite/kernels/internal/quantization_util.cc:53-104. TfLiteRound is
 * std::round (tflite/kernels/internal/cppmath.h:36). */
void orc_quantize_multiplier(double real_multiplier, int32_t* quantized_multiplier, int* shift) {
  if (real_multiplier == 0.0) {
    *quantized_multiplier = 0;
    *shift = 0;
    return;
  }
  const double q = frexp(real_multiplier, shift);
  int64_t q_fixed = (int64_t)round(q * (double)(1LL << 31));
  if (q_fixed == (1LL << 31)) {
    q_fixed /= 2;
    ++*shift;
  }
  if (*shift < -31) {
    *shift = 0;
    q_fixed = 0;
  }
  *quantized_multiplier = (int32_t)q_fixed;
}

/* Nearest integer to a*b / 2^31, ties toward +infinity, saturating for
 * INT32_MIN * INT32_MIN. Same semantics as ARM SQRDMULH, which the
 * reference's NEON path uses for this step
 * (tflite/kernels/internal/common.h:414-445). */
int32_t orc_saturating_rounding_doubling_high_mul(int32_t a, int32_t b) {
  if (a == INT32_MIN && b == INT32_MIN) return INT32_MAX;
  const int64_t ab = (int64_t)a * (int64_t)b;
  /* floor((ab + 2^30) / 2^31): >> on a negative int64 is arithmetic in gcc. */
  return (int32_t)((ab + (1LL << 30)) >> 31);
}

/* x / 2^exponent rounded to nearest, ties away from zero. */
int32_t orc_rounding_divide_by_pot(int32_t x, int exponent) {
  if (exponent == 0) return x;
  const int64_t half = 1LL << (exponent - 1);
  const int64_t q = (int64_t)x >> exponent; /* floor */
  const int64_t r = (int64_t)x - q * (1LL << exponent);
  if (r > half || (r == half && x >= 0)) return (int32_t)(q + 1);
  return (int32_t)q;
}

/* tflite/kernels/internal/common.cc:81-90 */
int32_t orc_multiply_by_quantized_multiplier(int32_t x, int32_t quantized_multiplier, int shift) {
  const int left_shift = shift > 0 ? shift : 0;
  const int right_shift = shift > 0 ? 0 : -shift;
  /* x * (1 << left_shift) in wrapping int32 arithmetic, as the reference. */
  const int32_t shifted = (int32_t)((uint32_t)x * (1u << left_shift));
  return orc_rounding_divide_by_pot(
      orc_saturating_rounding_doubling_high_mul(shifted, quantized_multiplier), right_shift);
}

/* tflite/kernels/internal/common.cc:93-115 */
int32_t orc_multiply_by_quantized_multiplier_i64(int64_t x, int32_t quantized_multiplier, int shift) {
  const int32_t reduced =
      (quantized_multiplier < 0x7FFF0000) ? ((quantized_multiplier + (1 << 15)) >> 16) : 0x7FFF;
  const int total_shift = 15 - shift;
  x = (x * (int64_t)reduced) + ((int64_t)1 << (total_shift - 1));
  return (int32_t)(x >> total_shift);
}

/* tflite/kernels/kernel_util.cc:342-351 */
static int quantize_bound(float scale, int32_t zero_point, float f, int32_t* q) {
  const float tmp = roundf(f / scale);
  if (!(tmp >= (float)INT32_MIN && tmp <= (float)INT32_MAX)) return 1;
  *q = zero_point + (int32_t)tmp;
  return 0;
}

/* tflite/kernels/kernel_util.cc:354-410, int8 output. */
int orc_activation_range_int8(int activation, float out_scale, int32_t out_zero_point, int32_t* act_min,
                              int32_t* act_max) {
  const int32_t qmin = -128, qmax = 127;
  int32_t t;
  if (activation == ORC_ACT_RELU) {
    if (quantize_bound(out_scale, out_zero_point, 0.0f, &t)) return 1;
    *act_min = qmin > t ? qmin : t;
    *act_max = qmax;
  } else if (activation == ORC_ACT_RELU6) {
    if (quantize_bound(out_scale, out_zero_point, 0.0f, &t)) return 1;
    *act_min = qmin > t ? qmin : t;
    if (quantize_bound(out_scale, out_zero_point, 6.0f, &t)) return 1;
    *act_max = qmax < t ? qmax : t;
  } else if (activation == ORC_ACT_RELU_N1_TO_1) {
    if (quantize_bound(out_scale, out_zero_point, -1.0f, &t)) return 1;
    *act_min = qmin > t ? qmin : t;
    if (quantize_bound(out_scale, out_zero_point, 1.0f, &t)) return 1;
    *act_max = qmax < t ? qmax : t;
  } else {
    *act_min = qmin;
    *act_max = qmax;
  }
  return 0;
}

/* tflite/kernels/fully_connected.cc:552-564 */
void orc_fc_per_channel_multipliers(float input_scale, float output_scale, const float* filter_scales,
                                    int n, int32_t* multipliers, int32_t* shifts) {
  for (int i = 0; i < n; ++i) {
    const double filter_scale = (double)filter_scales[i];
    const double eff = (double)input_scale * filter_scale / (double)output_scale;
    int sh;
    orc_quantize_multiplier(eff, &multipliers[i], &sh);
    shifts[i] = sh;
  }
}

/* tflite/kernels/kernel_util.cc:291-339: note the float product in the
 * multiplier and the double product in the bias check. */
int orc_fc_per_tensor_multiplier(float input_scale, float filter_scale, int has_bias, float bias_scale,
                                 float output_scale, int32_t* multiplier, int* shift) {
  if (has_bias) {
    const double ips = (double)input_scale * (double)filter_scale;
    const double diff = fabs(ips - (double)bias_scale);
    if (!(diff / (double)output_scale <= 0.02)) return 1;
  }
  const double input_product_scale = (double)(input_scale * filter_scale);
  if (!(input_product_scale >= 0)) return 1;
  orc_quantize_multiplier(input_product_scale / (double)output_scale, multiplier, shift);
  return 0;
}

/* ------------------------------------------------------------------ */
/* full-integer FULLY_CONNECTED                                       */
/* ------------------------------------------------------------------ */

static inline int32_t clamp_i32(int32_t v, int32_t lo, int32_t hi) {
  v = v > lo ? v : lo;
  return v < hi ? v : hi;
}

/* tflite/kernels/internal/reference/integer_ops/fully_connected.h:33-132 */
void orc_fc_int8_per_channel(int requant, int m, int n, int k, const int8_t* x, const int8_t* w,
                             const int32_t* bias, int32_t input_offset, int32_t output_offset,
                             const int32_t* multipliers, const int32_t* shifts, float input_scale,
                             float output_scale, const float* filter_scales, int32_t act_min,
                             int32_t act_max, int8_t* y) {
  for (int b = 0; b < m; ++b) {
    for (int c = 0; c < n; ++c) {
      int32_t acc = 0;
      for (int d = 0; d < k; ++d) {
        const int32_t iv = x[(size_t)b * k + d];
        const int32_t fv = w[(size_t)c * k + d];
        acc += fv * (iv + input_offset);
      }
      if (bias) acc += bias[c];
      int32_t scaled;
      if (requant == ORC_REQUANT_MBQM) {
        scaled = orc_multiply_by_quantized_multiplier(acc, multipliers[c], shifts[c]);
      } else {
        const double fs = (double)filter_scales[c];
        const double eff = (double)input_scale * fs / (double)output_scale;
        scaled = (int32_t)round((double)acc * eff);
      }
      scaled += output_offset;
      y[(size_t)b * n + c] = (int8_t)clamp_i32(scaled, act_min, act_max);
    }
  }
}

/* tflite/kernels/internal/reference/integer_ops/fully_connected.h:134-180 */
void orc_fc_int8_per_tensor(int m, int n, int k, const int8_t* x, const int8_t* w, const int32_t* bias,
                            int32_t input_offset, int32_t filter_offset, int32_t output_offset,
                            int32_t multiplier, int shift, int32_t act_min, int32_t act_max, int8_t* y) {
  for (int b = 0; b < m; ++b) {
    for (int c = 0; c < n; ++c) {
      int32_t acc = 0;
      for (int d = 0; d < k; ++d) {
        const int32_t iv = x[(size_t)b * k + d];
        const int32_t fv = w[(size_t)c * k + d];
        acc += (fv + filter_offset) * (iv + input_offset);
      }
      if (bias) acc += bias[c];
      int32_t scaled = orc_multiply_by_quantized_multiplier(acc, multiplier, shift);
      scaled += output_offset;
      y[(size_t)b * n + c] = (int8_t)clamp_i32(scaled, act_min, act_max);
    }
  }
}

/* ------------------------------------------------------------------ */
/* hybrid                                                             */
/* ------------------------------------------------------------------ */

/* tflite/kernels/internal/reference/portable_tensor_utils.cc:41-71 */
void orc_symmetric_quantize_floats(const float* values, int size, int8_t* q, float* scale) {
  float mn = values[0], mx = values[0];
  for (int i = 1; i < size; ++i) {
    if (values[i] < mn) mn = values[i];
    if (values[i] > mx) mx = values[i];
  }
  const int32_t kScale = 127;
  const float range = fmaxf(fabsf(mn), fabsf(mx));
  if (range == 0) {
    memset(q, 0, (size_t)size);
    *scale = 1;
    return;
  }
  *scale = range / kScale;
  const float inv = kScale / range;
  for (int i = 0; i < size; ++i) {
    const int32_t v = (int32_t)roundf(values[i] * inv);
    q[i] = (int8_t)(v < -kScale ? -kScale : (v > kScale ? kScale : v));
  }
}

/* tflite/kernels/internal/reference/portable_tensor_utils.cc:74-119 */
void orc_asymmetric_quantize_floats(const float* values, int size, int8_t* q, float* scaling_factor,
                                    int32_t* offset) {
  const int32_t kMinScale = -128, kMaxScale = 127;
  const double qmin_double = kMinScale, qmax_double = kMaxScale;
  float mn = values[0], mx = values[0];
  for (int i = 1; i < size; ++i) {
    if (values[i] < mn) mn = values[i];
    if (values[i] > mx) mx = values[i];
  }
  const double rmin = (double)fminf(0.0f, mn);
  const double rmax = (double)fmaxf(0.0f, mx);
  if (rmin == rmax) {
    memset(q, 0, (size_t)size);
    *scaling_factor = 1;
    *offset = 0;
    return;
  } else {
    const double scale = (rmax - rmin) / (qmax_double - qmin_double);
    const double zp_from_min = qmin_double - rmin / scale;
    const double zp_from_max = qmax_double - rmax / scale;
    const double zp_from_min_error = fabs(qmin_double) + fabs(rmin / scale);
    const double zp_from_max_error = fabs(qmax_double) + fabs(rmax / scale);
    const double zp_double = zp_from_min_error < zp_from_max_error ? zp_from_min : zp_from_max;
    int8_t nudged = 0;
    if (zp_double <= qmin_double) {
      nudged = (int8_t)kMinScale;
    } else if (zp_double >= qmax_double) {
      nudged = (int8_t)kMaxScale;
    } else {
      nudged = (int8_t)round(zp_double);
    }
    *scaling_factor = (float)scale;
    *offset = nudged;
  }
  const float inv = 1.0f / *scaling_factor;
  for (int i = 0; i < size; ++i) {
    /* int32 + float*float evaluated in float, then std::round. */
    const int32_t v = (int32_t)roundf((float)*offset + values[i] * inv);
    q[i] = (int8_t)(v < kMinScale ? kMinScale : (v > kMaxScale ? kMaxScale : v));
  }
}

/* tflite/kernels/internal/portable_tensor_utils.h:158-176 */
void orc_batch_quantize_floats(const float* x, int m, int k, int8_t* q, float* scales,
                               int32_t* zero_points, int asymmetric) {
  for (int b = 0; b < m; ++b) {
    const size_t off = (size_t)b * k;
    if (asymmetric) {
      orc_asymmetric_quantize_floats(x + off, k, q + off, &scales[b], &zero_points[b]);
    } else {
      orc_symmetric_quantize_floats(x + off, k, q + off, &scales[b]);
      if (zero_points) zero_points[b] = 0;
    }
  }
}

/* tflite/kernels/internal/reference/portable_tensor_utils.cc:165-206 */
void orc_matrix_batch_vector_mac_hybrid(const int8_t* w, int n, int k, const int8_t* q,
                                        const float* scales, int m, float* result,
                                        const float* per_channel_scale, const int32_t* zero_points,
                                        int32_t* row_sums, int compute_row_sums) {
  if (compute_row_sums) {
    for (int r = 0; r < n; ++r) {
      int32_t s = 0;
      for (int c = 0; c < k; ++c) s += w[(size_t)r * k + c];
      row_sums[r] = s;
    }
  }
  for (int b = 0; b < m; ++b) {
    const float batch_scale = scales[b];
    const int32_t batch_offset = zero_points[b];
    const int8_t* vec = q + (size_t)b * k;
    for (int r = 0; r < n; ++r) {
      const int8_t* row = w + (size_t)r * k;
      int32_t dot = 0;
      float scale = batch_scale;
      if (per_channel_scale) scale *= per_channel_scale[r];
      for (int c = 0; c < k; ++c) dot += row[c] * vec[c];
      dot -= row_sums[r] * batch_offset;
      result[(size_t)b * n + r] += (float)dot * scale;
    }
  }
}

/* tflite/kernels/internal/tensor_utils.h:58-80 and
 * tflite/kernels/internal/reference/portable_tensor_utils.cc (Apply*ToVector).
 * tanh and sigmoid go through Eigen in the reference; libm here, which the
 * float tolerance of the hybrid tests covers. */
void orc_apply_activation(float* v, size_t size, int activation) {
  switch (activation) {
    case ORC_ACT_NONE:
      return;
    case ORC_ACT_RELU:
      for (size_t i = 0; i < size; ++i) v[i] = fmaxf(0.0f, v[i]);
      return;
    case ORC_ACT_RELU_N1_TO_1:
      for (size_t i = 0; i < size; ++i) v[i] = fmaxf(-1.0f, fminf(v[i], 1.0f));
      return;
    case ORC_ACT_RELU6:
      for (size_t i = 0; i < size; ++i) v[i] = fmaxf(0.0f, fminf(v[i], 6.0f));
      return;
    case ORC_ACT_TANH:
      for (size_t i = 0; i < size; ++i) v[i] = tanhf(v[i]);
      return;
    case ORC_ACT_SIGN_BIT:
      for (size_t i = 0; i < size; ++i) v[i] = signbit(v[i]) ? 1.0f : 0.0f;
      return;
    case ORC_ACT_SIGMOID:
      for (size_t i = 0; i < size; ++i) v[i] = 1.0f / (1.0f + expf(-v[i]));
      return;
    default:
      return;
  }
}

/* tflite/kernels/fully_connected.cc:763-858 */
void orc_fc_hybrid(int m, int n, int k, const float* x, const int8_t* w, const float* filter_scales,
                   int per_channel, const float* bias, int asymmetric_inputs, int activation, float* y) {
  const size_t out_size = (size_t)m * n;
  for (int b = 0; b < m; ++b)
    for (int c = 0; c < n; ++c) y[(size_t)b * n + c] = bias ? bias[c] : 0.0f;

  int all_zero = 1;
  for (size_t i = 0; i < (size_t)m * k; ++i) {
    if (x[i] != 0.0f) {
      all_zero = 0;
      break;
    }
  }
  if (all_zero) {
    orc_apply_activation(y, out_size, activation);
    return;
  }

  int8_t* q = (int8_t*)malloc((size_t)m * k);
  float* scales = (float*)malloc(sizeof(float) * (size_t)m);
  int32_t* zps = (int32_t*)malloc(sizeof(int32_t) * (size_t)m);
  int32_t* row_sums = (int32_t*)malloc(sizeof(int32_t) * (size_t)n);
  orc_batch_quantize_floats(x, m, k, q, scales, zps, asymmetric_inputs);
  if (!per_channel) {
    for (int b = 0; b < m; ++b) scales[b] *= filter_scales[0];
  }
  orc_matrix_batch_vector_mac_hybrid(w, n, k, q, scales, m, y, per_channel ? filter_scales : NULL, zps,
                                     row_sums, 1);
  orc_apply_activation(y, out_size, activation);
  free(q);
  free(scales);
  free(zps);
  free(row_sums);
}

/* IEEE binary16 <-> binary32. The reference converts block scales with
 * Eigen::half (tflite/kernels/fully_connected.cc:1030-1036), an exact
 * widening. */
float orc_half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  const uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      uint32_t mm = man;
      do {
        ++e;
        mm <<= 1;
      } while ((mm & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mm & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t orc_float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t hm = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (hm & 1))) ++hm;
    return (uint16_t)(sign | hm);
  }
  uint32_t hm = man >> 13;
  const uint32_t rem = man & 0x1FFFu;
  uint16_t out = (uint16_t)(sign | ((uint32_t)exp << 10) | hm);
  if (rem > 0x1000u || (rem == 0x1000u && (hm & 1))) ++out;
  return out;
}

/* tflite/kernels/fully_connected.cc:1012 */
static inline int8_t sign_extend_int4(int8_t v) { return (int8_t)((v ^ 0x8) - 8); }

/* tflite/kernels/internal/portable_tensor_utils.cc:96-126 */
void orc_unpack_int4(const uint8_t* src, int num_elements, int8_t* dst) {
  for (int i = 0; i < num_elements / 2; ++i) {
    const int8_t byte = (int8_t)src[i];
    dst[2 * i] = (int8_t)((int8_t)(byte << 4) >> 4);
    dst[2 * i + 1] = (int8_t)(byte >> 4);
  }
  if (num_elements % 2 != 0) {
    const int8_t byte = (int8_t)src[num_elements / 2];
    dst[num_elements - 1] = (int8_t)((int8_t)(byte << 4) >> 4);
  }
}

/* tflite/kernels/fully_connected.cc:1014-1086 */
void orc_fc_blockwise4(int m, int n, int k, int blocksize, const float* x, const uint8_t* w4,
                       const uint16_t* scales_f16, const float* bias, float* y) {
  const size_t num_blocks = (size_t)k / blocksize;
  const size_t num_scales = (size_t)n * num_blocks;
  float* dq_scale = (float*)malloc(sizeof(float) * num_scales);
  for (size_t i = 0; i < num_scales; ++i) dq_scale[i] = orc_half_to_float(scales_f16[i]);
  memset(y, 0, sizeof(float) * (size_t)m * n);
  int8_t* q = (int8_t*)malloc((size_t)m * k);
  float* in_scales = (float*)malloc(sizeof(float) * (size_t)m);
  int32_t* in_zps = (int32_t*)malloc(sizeof(int32_t) * (size_t)m);
  orc_batch_quantize_floats(x, m, k, q, in_scales, in_zps, /*asymmetric=*/1);

  const size_t k2 = ((size_t)k + 1) & ~(size_t)1;
  for (size_t mi = 0; mi < (size_t)m; ++mi) {
    for (size_t ni = 0; ni < (size_t)n; ++ni) {
      float kfsum = 0.0f;
      float* out = &y[mi * n + ni];
      for (size_t bi = 0; bi < num_blocks; ++bi) {
        int32_t ksum = 0;
        int32_t c_ref_acc = 0;
        for (size_t ki = 0; ki < (size_t)blocksize; ++ki) {
          const size_t k_index = bi * blocksize + ki;
          const size_t nb_index = (ni * k2 + k_index) / 2;
          const int8_t k_value =
              (int8_t)((k_index % 2 == 0) ? (w4[nb_index] & 0xF) : (w4[nb_index] >> 4));
          const int32_t kernel_value = sign_extend_int4(k_value);
          ksum += kernel_value;
          /* int32 += int32 * float in the reference: the sum goes through
           * float and is converted back. */
          c_ref_acc = (int32_t)((float)c_ref_acc + (float)(int32_t)q[mi * k + k_index] * (float)kernel_value);
        }
        const float scale = dq_scale[ni * num_blocks + bi];
        *out += (float)c_ref_acc * scale;
        kfsum += scale * (float)ksum;
      }
      *out -= (float)in_zps[mi] * kfsum;
      *out *= in_scales[mi];
      if (bias) *out += bias[ni];
    }
  }
  free(dq_scale);
  free(q);
  free(in_scales);
  free(in_zps);
}

/* ------------------------------------------------------------------ */
/* BATCH_MATMUL                                                       */
/* ------------------------------------------------------------------ */

/* tflite/kernels/internal/reference/batch_matmul.h:30-51 */
static int bmm_broadcast_dim(int l, int r) {
  if (l == r) return l;
  if (l == 1) return r;
  return l; /* r == 1 checked by Prepare */
}
static size_t bmm_extent(const int* s5, int x) {
  if (s5[x] == 1) return 0;
  size_t prod = 1;
  for (int i = x + 1; i < 5; ++i) prod *= (size_t)s5[i];
  return prod;
}

#define BMM_PROLOGUE                                                                  \
  const size_t bd0 = (size_t)bmm_broadcast_dim(lhs_shape5[0], rhs_shape5[0]);         \
  const size_t bd1 = (size_t)bmm_broadcast_dim(lhs_shape5[1], rhs_shape5[1]);         \
  const size_t bd2 = (size_t)bmm_broadcast_dim(lhs_shape5[2], rhs_shape5[2]);         \
  const size_t le0 = bmm_extent(lhs_shape5, 0), le1 = bmm_extent(lhs_shape5, 1),      \
               le2 = bmm_extent(lhs_shape5, 2);                                       \
  const size_t re0 = bmm_extent(rhs_shape5, 0), re1 = bmm_extent(rhs_shape5, 1),      \
               re2 = bmm_extent(rhs_shape5, 2);                                       \
  const size_t lhs_rows = (size_t)lhs_shape5[3];                                      \
  const size_t rhs_cols = (size_t)rhs_shape5[4];                                      \
  const size_t depth = (size_t)lhs_shape5[4];

/* tflite/kernels/internal/reference/batch_matmul.h:55-109. As there, "rhs"
 * is indexed [j * depth + k]: the caller has already made depth contiguous. */
void orc_ref_bmm_float(const int* lhs_shape5, const float* lhs, const int* rhs_shape5, const float* rhs,
                       float* out) {
  BMM_PROLOGUE
  for (size_t b0 = 0; b0 < bd0; ++b0)
    for (size_t b1 = 0; b1 < bd1; ++b1)
      for (size_t b2 = 0; b2 < bd2; ++b2) {
        const float* l = lhs + b0 * le0 + b1 * le1 + b2 * le2;
        const float* r = rhs + b0 * re0 + b1 * re1 + b2 * re2;
        float* o = out + ((b0 * bd1 * bd2) + b1 * bd2 + b2) * lhs_rows * rhs_cols;
        for (size_t j = 0; j < rhs_cols; ++j)
          for (size_t i = 0; i < lhs_rows; ++i) {
            float total = 0;
            for (size_t kk = 0; kk < depth; ++kk) total += l[depth * i + kk] * r[j * depth + kk];
            o[lhs_rows * j + i] = total;
          }
      }
}

/* tflite/kernels/internal/reference/batch_matmul.h:111-209 */
void orc_ref_bmm_hybrid(const int* lhs_shape5, const int8_t* lhs, const int* rhs_shape5,
                        const int8_t* rhs, const float* scaling_factors, const int32_t* input_offset,
                        int32_t* row_sums, int compute_row_sums, const float* per_channel_scales,
                        float* out) {
  BMM_PROLOGUE
  const size_t io0 = re0 == 0 ? 0 : rhs_cols, io1 = re1 == 0 ? 0 : rhs_cols,
               io2 = re2 == 0 ? 0 : rhs_cols;
  const size_t wo0 = le0 == 0 ? 0 : lhs_rows, wo1 = le1 == 0 ? 0 : lhs_rows,
               wo2 = le2 == 0 ? 0 : lhs_rows;
  if (compute_row_sums) {
    /* The reference multiplies dims 1..2 only (its loop starts at i = 1). */
    size_t num_w = 1;
    for (int i = 1; i < 3; ++i) num_w *= (size_t)lhs_shape5[i];
    for (size_t r = 0; r < num_w * lhs_rows; ++r) {
      int32_t s = 0;
      for (size_t c = 0; c < depth; ++c) s += lhs[r * depth + c];
      row_sums[r] = s;
    }
  }
  for (size_t b0 = 0; b0 < bd0; ++b0)
    for (size_t b1 = 0; b1 < bd1; ++b1)
      for (size_t b2 = 0; b2 < bd2; ++b2) {
        const int8_t* l = lhs + b0 * le0 + b1 * le1 + b2 * le2;
        const int8_t* r = rhs + b0 * re0 + b1 * re1 + b2 * re2;
        const int32_t* ioff = input_offset + b0 * io0 + b1 * io1 + b2 * io2;
        const float* sc = scaling_factors + b0 * io0 + b1 * io1 + b2 * io2;
        const int32_t* woff = row_sums + b0 * wo0 + b1 * wo1 + b2 * wo2;
        float* o = out + ((b0 * bd1 * bd2) + b1 * bd2 + b2) * lhs_rows * rhs_cols;
        for (size_t j = 0; j < rhs_cols; ++j) {
          const float batch_scaling_factor = sc[j];
          const float batch_offset = (float)ioff[j];
          for (size_t i = 0; i < lhs_rows; ++i) {
            int32_t total = 0;
            for (size_t kk = 0; kk < depth; ++kk) total += l[depth * i + kk] * r[j * depth + kk];
            const int32_t row_sum = woff[i];
            /* int32 -= int32 * float: through float, truncated back. */
            total = (int32_t)((float)total - (float)row_sum * batch_offset);
            float scale = batch_scaling_factor;
            if (per_channel_scales) scale *= per_channel_scales[i];
            o[lhs_rows * j + i] += scale * (float)total;
          }
        }
      }
}

/* tflite/kernels/internal/reference/batch_matmul.h:211-284 */
void orc_ref_bmm_int8(const int* lhs_shape5, const int8_t* lhs, const int* rhs_shape5, const int8_t* rhs,
                      int32_t input_offset, int32_t filter_offset, int32_t output_offset,
                      int32_t multiplier, int shift, int32_t act_min, int32_t act_max, int8_t* out) {
  BMM_PROLOGUE
  for (size_t b0 = 0; b0 < bd0; ++b0)
    for (size_t b1 = 0; b1 < bd1; ++b1)
      for (size_t b2 = 0; b2 < bd2; ++b2) {
        const int8_t* l = lhs + b0 * le0 + b1 * le1 + b2 * le2;
        const int8_t* r = rhs + b0 * re0 + b1 * re1 + b2 * re2;
        int8_t* o = out + ((b0 * bd1 * bd2) + b1 * bd2 + b2) * lhs_rows * rhs_cols;
        for (size_t j = 0; j < rhs_cols; ++j)
          for (size_t i = 0; i < lhs_rows; ++i) {
            int32_t total = 0;
            for (size_t kk = 0; kk < depth; ++kk) {
              const int32_t lv = l[depth * i + kk];
              const int32_t rv = r[depth * j + kk];
              total += (lv + filter_offset) * (rv + input_offset);
            }
            int32_t scaled = orc_multiply_by_quantized_multiplier(total, multiplier, shift);
            scaled += output_offset;
            o[lhs_rows * j + i] = (int8_t)clamp_i32(scaled, act_min, act_max);
          }
      }
}

/* ---- op level: what tflite/kernels/batch_matmul.cc:744-827 does ------- */

typedef struct {
  int rank;
  int dims[5];
} shape_t;

static size_t shape_size(const shape_t* s) {
  size_t n = 1;
  for (int i = 0; i < s->rank; ++i) n *= (size_t)s->dims[i];
  return n;
}
static void extend5(const shape_t* s, int* out5) {
  for (int i = 0; i < 5; ++i) out5[i] = 1;
  for (int i = 0; i < s->rank; ++i) out5[5 - s->rank + i] = s->dims[i];
}
static shape_t swap_rc(const shape_t* s) {
  shape_t r = *s;
  const int t = r.dims[r.rank - 1];
  r.dims[r.rank - 1] = r.dims[r.rank - 2];
  r.dims[r.rank - 2] = t;
  return r;
}
/* Transpose the two minor dims of every matrix in a batch (elem bytes). */
static void* transpose_rc(const void* src, const shape_t* s, size_t elem) {
  const size_t rows = (size_t)s->dims[s->rank - 2], cols = (size_t)s->dims[s->rank - 1];
  const size_t batches = shape_size(s) / (rows * cols);
  char* dst = (char*)malloc(shape_size(s) * elem + 1);
  const char* in = (const char*)src;
  for (size_t b = 0; b < batches; ++b)
    for (size_t r = 0; r < rows; ++r)
      for (size_t c = 0; c < cols; ++c)
        memcpy(dst + (b * rows * cols + c * rows + r) * elem, in + (b * rows * cols + r * cols + c) * elem,
               elem);
  return dst;
}

/* Shape compression of tflite/kernels/batch_matmul.cc:768-788 and the
 * transposes of :789-808. On return lhs/rhs hold the shapes the reference
 * passes on ("lhs_shape", "rhs_shape"), *lhs_buf / *rhs_buf the possibly
 * transposed data (to free when *own != 0). */
static void bmm_arrange(shape_t* xs, const void* x, shape_t* ys, const void* y, int adj_x, int adj_y,
                        size_t x_elem, size_t y_elem, const void** lhs_buf, int* own_l,
                        const void** rhs_buf, int* own_r) {
  if (!adj_x && ys->rank > 2 && xs->rank > 2 && ys->dims[ys->rank - 3] == 1) {
    shape_t tl;
    tl.rank = xs->rank - 1;
    for (int i = 0; i < tl.rank; ++i) tl.dims[i] = xs->dims[i];
    tl.dims[xs->rank - 3] = xs->dims[xs->rank - 3] * xs->dims[xs->rank - 2];
    tl.dims[xs->rank - 2] = xs->dims[xs->rank - 1];
    shape_t tr;
    tr.rank = ys->rank - 1;
    for (int i = 0; i < tr.rank; ++i) tr.dims[i] = ys->dims[i];
    tr.dims[ys->rank - 3] = ys->dims[ys->rank - 2];
    tr.dims[ys->rank - 2] = ys->dims[ys->rank - 1];
    *xs = tl;
    *ys = tr;
  }
  /* rhs: wanted as [.., C, B]; transpose unless adj_y. */
  if (adj_y) {
    *rhs_buf = y;
    *own_r = 0;
  } else {
    *rhs_buf = transpose_rc(y, ys, y_elem);
    *own_r = 1;
    *ys = swap_rc(ys); /* data is now [.., C, B] */
  }
  /* lhs: wanted as [.., A, B]; transpose when adj_x. */
  if (adj_x) {
    *lhs_buf = transpose_rc(x, xs, x_elem);
    *own_l = 1;
    *xs = swap_rc(xs);
  } else {
    *lhs_buf = x;
    *own_l = 0;
  }
  /* The reference then hands "SwapRowColumnDims" shapes to the kernels, whose
   * meaning is [.., depth, rows]; the 5-D shapes below are written in the
   * kernels' own convention instead: dims[3] = rows, dims[4] = depth. */
}

/* Kernel-convention 5-D shapes: first operand ("lhs" of the reference
 * kernel) is the op's RHS as [.., C, B] -> rows = C, depth = B; second is
 * the op's LHS as [.., A, B] -> "rhs_cols" = A. The reference encodes the
 * second as [.., B, A] (Dims(4) = cols); do the same. */
static void kernel_shapes(const shape_t* xs, const shape_t* ys, int* k_lhs5, int* k_rhs5) {
  extend5(ys, k_lhs5); /* [.., C, B] */
  int tmp[5];
  extend5(xs, tmp); /* [.., A, B] */
  for (int i = 0; i < 3; ++i) k_rhs5[i] = tmp[i];
  k_rhs5[3] = tmp[4];
  k_rhs5[4] = tmp[3];
}

void orc_batch_matmul_float(int x_rank, const int* x_dims, const float* x, int y_rank, const int* y_dims,
                            const float* y, int adj_x, int adj_y, float* out) {
  shape_t xs, ys;
  xs.rank = x_rank;
  ys.rank = y_rank;
  memcpy(xs.dims, x_dims, sizeof(int) * (size_t)x_rank);
  memcpy(ys.dims, y_dims, sizeof(int) * (size_t)y_rank);
  const void *lb, *rb;
  int ol, orr;
  bmm_arrange(&xs, x, &ys, y, adj_x, adj_y, sizeof(float), sizeof(float), &lb, &ol, &rb, &orr);
  int kl[5], kr[5];
  kernel_shapes(&xs, &ys, kl, kr);
  orc_ref_bmm_float(kl, (const float*)rb, kr, (const float*)lb, out);
  if (ol) free((void*)lb);
  if (orr) free((void*)rb);
}

/* per_channel_scales (optional): one scale per output column of the op (the RHS's quantized dimension
 * after the transposition of tflite/kernels/batch_matmul.cc:701-708); then y_scale is not used
 * (:487-503). */
void orc_batch_matmul_hybrid_pc(int x_rank, const int* x_dims, const float* x, int y_rank, const int* y_dims,
                                const int8_t* y, float y_scale, const float* per_channel_scales, int adj_x, int adj_y,
                                int asymmetric_inputs, float* out) {
  shape_t xs, ys;
  xs.rank = x_rank;
  ys.rank = y_rank;
  memcpy(xs.dims, x_dims, sizeof(int) * (size_t)x_rank);
  memcpy(ys.dims, y_dims, sizeof(int) * (size_t)y_rank);
  const void *lb, *rb;
  int ol, orr;
  bmm_arrange(&xs, x, &ys, y, adj_x, adj_y, sizeof(float), sizeof(int8_t), &lb, &ol, &rb, &orr);
  int kl[5], kr[5];
  kernel_shapes(&xs, &ys, kl, kr);
  /* tflite/kernels/batch_matmul.cc:454-526: every [B]-vector of the LHS is a
   * "batch" to quantize. */
  const size_t depth = (size_t)xs.dims[xs.rank - 1];
  const size_t num_vec = shape_size(&xs) / depth;
  int8_t* q = (int8_t*)malloc(shape_size(&xs) + 1);
  float* sf = (float*)malloc(sizeof(float) * num_vec);
  int32_t* zp = (int32_t*)malloc(sizeof(int32_t) * num_vec);
  orc_batch_quantize_floats((const float*)lb, (int)num_vec, (int)depth, q, sf, zp, asymmetric_inputs);
  if (!asymmetric_inputs) memset(zp, 0, sizeof(int32_t) * num_vec);
  if (!per_channel_scales)
    for (size_t i = 0; i < num_vec; ++i) sf[i] *= y_scale;
  /* output size */
  const size_t bd = (size_t)bmm_broadcast_dim(kl[0], kr[0]) * bmm_broadcast_dim(kl[1], kr[1]) *
                    bmm_broadcast_dim(kl[2], kr[2]);
  const size_t out_size = bd * (size_t)kl[3] * (size_t)kr[4];
  for (size_t i = 0; i < out_size; ++i) out[i] = 0.0f;
  const size_t n_rows = (size_t)kl[1] * kl[2] * kl[3] * (size_t)kl[0];
  int32_t* row_sums = (int32_t*)calloc(n_rows + 1, sizeof(int32_t));
  orc_ref_bmm_hybrid(kl, (const int8_t*)rb, kr, q, sf, zp, row_sums, 1, per_channel_scales, out);
  free(q);
  free(sf);
  free(zp);
  free(row_sums);
  if (ol) free((void*)lb);
  if (orr) free((void*)rb);
}

void orc_batch_matmul_hybrid(int x_rank, const int* x_dims, const float* x, int y_rank, const int* y_dims,
                             const int8_t* y, float y_scale, int adj_x, int adj_y, int asymmetric_inputs,
                             float* out) {
  orc_batch_matmul_hybrid_pc(x_rank, x_dims, x, y_rank, y_dims, y, y_scale, NULL, adj_x, adj_y, asymmetric_inputs, out);
}

void orc_batch_matmul_int8(int x_rank, const int* x_dims, const int8_t* x, int32_t x_zero_point,
                           int y_rank, const int* y_dims, const int8_t* y, int32_t y_zero_point,
                           int adj_x, int adj_y, int32_t multiplier, int shift, int32_t out_zero_point,
                           int8_t* out) {
  shape_t xs, ys;
  xs.rank = x_rank;
  ys.rank = y_rank;
  memcpy(xs.dims, x_dims, sizeof(int) * (size_t)x_rank);
  memcpy(ys.dims, y_dims, sizeof(int) * (size_t)y_rank);
  const void *lb, *rb;
  int ol, orr;
  bmm_arrange(&xs, x, &ys, y, adj_x, adj_y, 1, 1, &lb, &ol, &rb, &orr);
  int kl[5], kr[5];
  kernel_shapes(&xs, &ys, kl, kr);
  /* tflite/kernels/batch_matmul.cc:528-556: input_offset = -lhs zp, applied to
   * the kernel's second operand; filter_offset = -rhs zp on its first. */
  orc_ref_bmm_int8(kl, (const int8_t*)rb, kr, (const int8_t*)lb, -x_zero_point, -y_zero_point,
                   out_zero_point, multiplier, shift, -128, 127, out);
  if (ol) free((void*)lb);
  if (orr) free((void*)rb);
}

/* ------------------------------------------------------------------ */
/* odml.scaled_dot_product_attention                                  */
/* ------------------------------------------------------------------ */

/* tflite/experimental/genai/sdpa.cc:361-662. The transposes, reshapes and
 * GQA replication there only move data; the arithmetic per (batch, head,
 * query token) is: logits[s] = sum_h (q*scale)[h] * k[s,h] (h ascending),
 * + mask, softmax (softmax.h:33-64), out[h] = sum_s p[s] * v[s,h]
 * (s ascending). */
void orc_sdpa_f32(int b, int t, int n, int nkv, int h, int s, const float* q, const float* k,
                  const float* v, const float* mask, float scale, float logit_cap, float* out) {
  const int group = n / nkv;
  float* logits = (float*)malloc(sizeof(float) * (size_t)s);
  float* qs = (float*)malloc(sizeof(float) * (size_t)h);
  for (int bi = 0; bi < b; ++bi)
    for (int ti = 0; ti < t; ++ti)
      for (int ni = 0; ni < n; ++ni) {
        const int kv = ni / group; /* repeat-interleave, sdpa.cc:506-525 */
        const float* qp = q + (((size_t)bi * t + ti) * n + ni) * h;
        for (int hi = 0; hi < h; ++hi) qs[hi] = qp[hi] * scale;
        for (int si = 0; si < s; ++si) {
          const float* kp = k + (((size_t)bi * s + si) * nkv + kv) * h;
          float acc = 0.0f;
          for (int hi = 0; hi < h; ++hi) acc += qs[hi] * kp[hi];
          if (logit_cap > 0.0f) acc = logit_cap * tanhf(acc / logit_cap);
          if (mask) acc += mask[((size_t)bi * t + ti) * s + si];
          logits[si] = acc;
        }
        float mx = -3.402823466e+38f;
        for (int si = 0; si < s; ++si) mx = logits[si] > mx ? logits[si] : mx;
        float sum = 0.0f;
        for (int si = 0; si < s; ++si) {
          const float e = expf((logits[si] - mx) * 1.0f);
          logits[si] = e;
          sum += e;
        }
        for (int si = 0; si < s; ++si) logits[si] = logits[si] / sum;
        float* op = out + (((size_t)bi * t + ti) * n + ni) * h;
        for (int hi = 0; hi < h; ++hi) {
          float acc = 0.0f;
          for (int si = 0; si < s; ++si)
            acc += logits[si] * v[(((size_t)bi * s + si) * nkv + kv) * h + hi];
          op[hi] = acc;
        }
      }
  free(logits);
  free(qs);
}
