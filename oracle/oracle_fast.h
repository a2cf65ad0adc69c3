/*
 * Vectorised, multi-threaded twin of the CPU oracle. TEST INFRASTRUCTURE
 * ONLY: it exists to give the benchmark a fair CPU baseline (the reference's
 * x86 path for hybrid FULLY_CONNECTED is an AVX2 loop,
 * tflite/kernels/internal/optimized/sse_tensor_utils.cc:201-292, and its int8
 * GEMM is a third-party SIMD library that is not available offline). Same
 * formulas as oracle.c; the integer parts are exact, so results are
 * bit-identical to the scalar oracle, which the tests assert.
 * Weight-stationary and spread over all host threads with OpenMP: at least as
 * fast as the reference's own single-threaded, batch-outer loop.
 */
#ifndef LITERT_B200_ORACLE_FAST_H_
#define LITERT_B200_ORACLE_FAST_H_
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
int orcf_num_threads(void);
void orcf_set_num_threads(int n);
void orcf_fc_int8_per_channel(int m, int n, int k, const int8_t* x, const int8_t* w, const int32_t* bias,
                              int32_t input_offset, int32_t output_offset, const int32_t* multipliers,
                              const int32_t* shifts, int32_t act_min, int32_t act_max, int8_t* y);
void orcf_fc_hybrid(int m, int n, int k, const float* x, const int8_t* w, const float* filter_scales,
                    int per_channel, const float* bias, int asymmetric_inputs, int activation,
                    const int32_t* row_sums, float* y);
void orcf_row_sums(int n, int k, const int8_t* w, int32_t* row_sums);
void orcf_fc_blockwise4(int m, int n, int k, int blocksize, const float* x, const uint8_t* w4,
                        const uint16_t* scales_f16, const float* bias, float* y);
void orcf_sdpa_f32(int b, int t, int n, int nkv, int h, int s, const float* q, const float* k,
                   const float* v, const float* mask, const int32_t* lengths, float scale, float* out);
#ifdef __cplusplus
}
#endif
#endif
