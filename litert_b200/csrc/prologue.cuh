// Input prologue fused into the GEMV kernels for decode-sized batches: instead of streaming
// activation rows that an earlier kernel quantized, the kernel's (otherwise idle) epilogue warps
// build them: residual add, RMS norm with gain, per-row asymmetric int8 quantization
// (tflite/kernels/internal/reference/portable_tensor_utils.cc:74-108 through row_quant_params),
// written straight into the shared-memory operand the MMAs read. Every CTA redoes the whole row
// (a few KB from L2) because scale and zero point depend on all of it; only the k tiles the CTA
// multiplies are stored.
#pragma once

#include "common.cuh"
#include "kernels.h"
#include "quant.cuh"

namespace b200 {

constexpr int kPrologueMaxK = 2048;   // one 16-byte chunk of the row per epilogue thread
constexpr int kPrologueMaxM = 4;
constexpr int kPrologueThreads = 128;

struct PrologueShared {  // the kernels keep two of these (rows alternate)
  float red[8];
  float2 mm[4];
};

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Called by the kPrologueThreads epilogue threads (etid 0..127) after the dependency wait.
//   bbuf: operand rows for k tiles [kt_begin, kt_end): per k tile nb_rows/8 row groups of 1 KiB in
//         the tiled activation layout (128-byte-swizzled K-major groups, see common.cuh).
//   in_scale / in_aux: per-row scale and zero point for the kernel's own epilogue.
//   writer: this CTA stores the updated residual stream (exactly one CTA per launch does).
// Uses named barrier `bar_id` among the 128 threads.
__device__ __forceinline__ void prologue_norm_quant(const FcParams& p, uint8_t* bbuf, int nb_rows, int kt_begin,
                                                    int kt_end, float* in_scale, int32_t* in_aux, PrologueShared* ps,
                                                    int etid, bool writer, int bar_id) {
  const int d = p.k;
  const int lane = etid & 31, w = etid >> 5;
  const int q_bytes = nb_rows * kTileK8;
  const int k0 = etid * 16;  // this thread's 16-byte chunk of every row
  const int kt = k0 / kTileK8;
  const bool in_range = kt >= kt_begin && kt < kt_end;  // chunk belongs to a k tile this CTA multiplies
  const bool have = k0 < d;
  const bool vec = have && k0 + 16 <= d && (d & 3) == 0;  // whole chunk inside the row: 128-bit accesses
  uint8_t* tile = bbuf + (size_t)(kt - kt_begin) * q_bytes;  // this chunk's k tile
  const int cc = (k0 % kTileK8) / 16;                         // its 16-byte chunk inside the tile's rows
  // rows beyond m, and chunks in the zero padding of the last k tile, multiply as zeros
  if (in_range)
    for (int m = have ? p.m : 0; m < nb_rows; ++m)
      *reinterpret_cast<uint4*>(tile + (m / 8) * 1024 + swz_chunk_offset(m % 8, cc)) = make_uint4(0, 0, 0, 0);
  float g[16];
  if (vec) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 t = *reinterpret_cast<const float4*>(p.pro_gain + k0 + q * 4);
      g[q * 4] = t.x, g[q * 4 + 1] = t.y, g[q * 4 + 2] = t.z, g[q * 4 + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) g[j] = (have && k0 + j < d) ? p.pro_gain[k0 + j] : 0.0f;
  }
  for (int m = 0; m < p.m; ++m) {
    PrologueShared* cur = ps + (m & 1);  // two sets: a row never waits for the previous one's readers
    float v[16];
    const float* hin = p.pro_h_in + (size_t)m * d + k0;
    const float* din = p.pro_delta ? p.pro_delta + (size_t)m * d + k0 : nullptr;
    // every load of the row is issued before the first store (the buffers may not alias, but the
    // compiler cannot know)
    if (vec) {
      float4 a[4], e[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) a[q] = *reinterpret_cast<const float4*>(hin + q * 4);
      if (din) {
#pragma unroll
        for (int q = 0; q < 4; ++q) e[q] = *reinterpret_cast<const float4*>(din + q * 4);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        v[q * 4] = a[q].x, v[q * 4 + 1] = a[q].y, v[q * 4 + 2] = a[q].z, v[q * 4 + 3] = a[q].w;
        if (din) {
          v[q * 4] = __fadd_rn(v[q * 4], e[q].x);
          v[q * 4 + 1] = __fadd_rn(v[q * 4 + 1], e[q].y);
          v[q * 4 + 2] = __fadd_rn(v[q * 4 + 2], e[q].z);
          v[q * 4 + 3] = __fadd_rn(v[q * 4 + 3], e[q].w);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float t = 0.0f;
        if (have && k0 + j < d) {
          t = hin[j];
          if (din) t = __fadd_rn(t, din[j]);
        }
        v[j] = t;
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) ss += v[j] * v[j];
    if (writer && have) {
      float* hout = p.pro_h_out + (size_t)m * d + k0;
      if (vec) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<float4*>(hout + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (k0 + j < d) hout[j] = v[j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) cur->red[w] = ss;
    named_barrier(bar_id, kPrologueThreads);
    ss = (cur->red[0] + cur->red[1]) + (cur->red[2] + cur->red[3]);
    const float inv_rms = 1.0f / sqrtf(ss / (float)d + p.pro_eps);
    float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (have && k0 + j < d) {
        v[j] = __fmul_rn(__fmul_rn(v[j], inv_rms), g[j]);
        mn = fminf(mn, v[j]);
        mx = fmaxf(mx, v[j]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) cur->mm[w] = make_float2(mn, mx);
    named_barrier(bar_id, kPrologueThreads);
    // every thread derives the row's parameters itself (same inputs, same arithmetic)
    float lo = cur->mm[0].x, hi = cur->mm[0].y;
#pragma unroll
    for (int i = 1; i < 4; ++i) {
      lo = fminf(lo, cur->mm[i].x);
      hi = fmaxf(hi, cur->mm[i].y);
    }
    float sf, inv;
    int zp, zero_row;
    row_quant_params(lo, hi, true, &sf, &inv, &zp, &zero_row);
    if (etid == 0) {
      in_scale[m] = sf;
      in_aux[m] = zp;
      if (writer && p.pro_scales_out) {
        p.pro_scales_out[m] = sf;
        p.pro_zps_out[m] = zp;
      }
    }
    if (have && in_range) {
      const float zpf = (float)zp;
      uint32_t word[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        word[q] = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (!zero_row && k0 + q * 4 + e < d) word[q] |= quantize_value(v[q * 4 + e], inv, zpf, true) << (8 * e);
      }
      *reinterpret_cast<uint4*>(tile + (m / 8) * 1024 + swz_chunk_offset(m % 8, cc)) =
          make_uint4(word[0], word[1], word[2], word[3]);
    }
  }
  for (int m = p.m + etid; m < nb_rows; m += kPrologueThreads) {
    in_scale[m] = 0.0f;
    in_aux[m] = 0;
  }
  fence_proxy_async_smem();  // the MMAs read the operand through the async proxy
  named_barrier(bar_id, kPrologueThreads);
}

}  // namespace b200
