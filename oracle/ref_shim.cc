// Thin C wrapper around the pieces of the reference that compile from their
// own source files (no third-party dependency): QuantizeMultiplier,
// CalculateActivationRangeQuantized and GetQuantizedConvolutionMultipler.
// TEST INFRASTRUCTURE ONLY: built into oracle/_ref/ by the Makefile beside
// this file, from the reference sources where they lie, and used by the tests
// to validate the restatement in oracle.c. Never linked into the product.
#include <cstdint>
#include <cstring>

#include "tflite/core/c/builtin_op_data.h"
#include "tflite/core/c/common.h"
#include "tflite/kernels/internal/quantization_util.h"
#include "tflite/kernels/kernel_util.h"

extern "C" {

void ref_quantize_multiplier(double m, int32_t* q, int* shift) { tflite::QuantizeMultiplier(m, q, shift); }

static void noop_report(TfLiteContext*, const char*, ...) {}

int ref_activation_range_int8(int activation, float scale, int32_t zero_point, int32_t* act_min,
                              int32_t* act_max) {
  TfLiteContext ctx;
  std::memset(&ctx, 0, sizeof(ctx));
  ctx.ReportError = noop_report;
  TfLiteTensor out;
  std::memset(&out, 0, sizeof(out));
  out.type = kTfLiteInt8;
  out.params.scale = scale;
  out.params.zero_point = zero_point;
  return tflite::CalculateActivationRangeQuantized(&ctx, static_cast<TfLiteFusedActivation>(activation), &out,
                                                   act_min, act_max);
}

int ref_conv_multiplier(float in_scale, float w_scale, int has_bias, float bias_scale, float out_scale,
                        double* multiplier) {
  TfLiteContext ctx;
  std::memset(&ctx, 0, sizeof(ctx));
  ctx.ReportError = noop_report;
  TfLiteTensor in, w, b, out;
  std::memset(&in, 0, sizeof(in));
  std::memset(&w, 0, sizeof(w));
  std::memset(&b, 0, sizeof(b));
  std::memset(&out, 0, sizeof(out));
  in.params.scale = in_scale;
  w.params.scale = w_scale;
  b.params.scale = bias_scale;
  out.params.scale = out_scale;
  if (has_bias) return tflite::GetQuantizedConvolutionMultipler(&ctx, &in, &w, &b, &out, multiplier);
  return tflite::GetQuantizedConvolutionMultipler(&ctx, &in, &w, &out, multiplier);
}
}

// The reference's greedy gap search, tflite/simple_memory_arena.cc:370-434,
// driven with a caller-chosen allocation order: offsets[i] for request
// order[i]. Returns the high-water mark. Used to validate the delegate's
// device-arena planner.
#include "tflite/simple_memory_arena.h"
extern "C" size_t ref_arena_offsets(int n, const size_t* sizes, const int* first, const int* last, const int* order,
                                    size_t alignment, size_t* offsets) {
  TfLiteContext ctx;
  std::memset(&ctx, 0, sizeof(ctx));
  ctx.ReportError = noop_report;
  tflite::SimpleMemoryArena arena(alignment);
  size_t high = 0;
  for (int i = 0; i < n; ++i) {
    const int r = order[i];
    tflite::ArenaAllocWithUsageInterval alloc;
    if (arena.Allocate(&ctx, alignment, sizes[r], r, first[r], last[r], &alloc) != kTfLiteOk) return (size_t)-1;
    offsets[r] = alloc.offset;
    if (alloc.offset + alloc.size > high) high = alloc.offset + alloc.size;
  }
  return high;
}
