// Device helpers shared by every kernel that quantizes activation rows to int8
// and writes them in the tiled layout the GEMM kernels stream.
#pragma once

#include "common.cuh"

namespace b200 {

// Tiled activation layout shared by all MMA kernels: [k tile][row group of 8][1 KiB group in the
// 128-byte-swizzled K-major layout of common.cuh]; m_alloc rows are allocated.
__device__ __forceinline__ size_t q_tiled_offset(int m, int kk, int m_alloc) {
  const int kt = kk / kTileK8, c = (kk % kTileK8) / 16, b = kk % 16;
  return ((size_t)kt * (m_alloc / 8) + (m / 8)) * 1024 + swz_chunk_offset(m % 8, c) + b;
}

// The same rows as fp16 (operands of the kind::f16 MMA): k tiles of 64 elements, 128-byte rows.
__device__ __forceinline__ size_t h_tiled_offset(int m, int kk, int m_alloc) {
  const int kt = kk / 64, c = (kk % 64) / 8, b = kk % 8;
  return ((size_t)kt * (m_alloc / 8) + (m / 8)) * 1024 + swz_chunk_offset(m % 8, c) + b * 2;
}

template <typename T, typename Op>
__device__ __forceinline__ T block_reduce(T v, Op op, T identity, T* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  v = lane < nw ? scratch[lane] : identity;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  return v;
}


// Block-wide minimum and maximum in one pass (one barrier); every thread gets both.
// `scratch` holds one float2 per warp and must not be reused before the next barrier.
__device__ __forceinline__ void block_minmax(float& mn, float& mx, float2* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) scratch[warp] = make_float2(mn, mx);
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  const float2 v = scratch[lane < nw ? lane : 0];
  mn = v.x;
  mx = v.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
}

// Scale, reciprocal scale and zero point of one activation row from its min
// and max. Asymmetric: tflite/kernels/internal/reference/portable_tensor_utils.cc:74-108
// (range widened to include 0, scale and the two zero-point candidates in
// double, the candidate with the smaller error, nudged into [-128,127] and
// rounded half away from zero); symmetric: :41-61. zero_row: every element
// quantizes to 0 and the scale is 1.
__device__ __forceinline__ void row_quant_params(float mn, float mx, bool asymmetric, float* scale, float* inv,
                                                 int* zp, int* zero_row) {
  *zp = 0;
  *zero_row = 0;
  *inv = 0.0f;
  if (asymmetric) {
    const double rmin = (double)fminf(0.0f, mn);
    const double rmax = (double)fmaxf(0.0f, mx);
    if (rmin == rmax) {
      *zero_row = 1;
      *scale = 1.0f;
      return;
    }
    const double qmin = -128.0, qmax = 127.0;
    const double s = (rmax - rmin) / (qmax - qmin);
    const double zp_from_min = qmin - rmin / s;
    const double zp_from_max = qmax - rmax / s;
    const double err_min = fabs(qmin) + fabs(rmin / s);
    const double err_max = fabs(qmax) + fabs(rmax / s);
    const double zp_d = err_min < err_max ? zp_from_min : zp_from_max;
    if (zp_d <= qmin) {
      *zp = -128;
    } else if (zp_d >= qmax) {
      *zp = 127;
    } else {
      *zp = (int)(int8_t)round(zp_d);
    }
    *scale = (float)s;
    *inv = __fdiv_rn(1.0f, *scale);
  } else {
    const float range = fmaxf(fabsf(mn), fabsf(mx));
    if (range == 0.0f) {
      *zero_row = 1;
      *scale = 1.0f;
      return;
    }
    *inv = __fdiv_rn(127.0f, range);
    *scale = __fdiv_rn(range, 127.0f);
  }
}

// One element: float multiply, float add of the zero point, round half away
// from zero (the fraction t - trunc(t) is exact), clamp -- no fused
// multiply-add, as on the reference's x86 build.
__device__ __forceinline__ uint32_t quantize_value(float v, float inv, float zpf, bool asymmetric) {
  const float t = asymmetric ? __fadd_rn(zpf, __fmul_rn(v, inv)) : __fmul_rn(v, inv);
  float r = truncf(t);
  if (fabsf(t - r) >= 0.5f) r += copysignf(1.0f, t);
  int qv = (int)fmaxf(-129.0f, fminf(128.0f, r));
  qv = max(asymmetric ? -128 : -127, min(127, qv));
  return (uint32_t)(uint8_t)(int8_t)qv;
}

// Quantizes the row held in shared memory `xs[0..k)` (asymmetric, per row) and
// writes it tiled; thread 0 publishes scale and zero point.
// `live` false: same work, nothing stored (a dry run that pulls the code into the instruction caches).
__device__ __forceinline__ void quantize_smem_row(const float* xs, int k, int k_pad, int row, int m_alloc, float mn, float mx,
                                  int8_t* q_tiled, float* scales, int32_t* zps, float* red, bool live = true) {
  __shared__ float2 s_mm[32];
  __shared__ float s_inv;
  __shared__ int s_zp, s_zero;
  (void)red;
  block_minmax(mn, mx, s_mm);
  // One thread derives the row's parameters: the reference computes them in double precision (three
  // divisions), which every warp of a wide block would pay for in issue slots (1024 threads: 1.2 us,
  // measured on B200) while one thread's latency plus a barrier is 0.4 us.
  if (threadIdx.x == 0) {
    float sf, inv;
    int zp, zero_row;
    row_quant_params(mn, mx, true, &sf, &inv, &zp, &zero_row);
    s_zero = zero_row;
    s_inv = inv;
    s_zp = zp;
    if (live) {
      scales[row] = sf;
      zps[row] = zp;
    }
  }
  __syncthreads();
  const bool zero = s_zero != 0;
  const float inv = s_inv, zpf = (float)s_zp;
  for (int k4 = threadIdx.x * 4; k4 < k_pad; k4 += blockDim.x * 4) {
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if (k4 + b < k && !zero) word |= quantize_value(xs[k4 + b], inv, zpf, true) << (8 * b);
    if (live) *reinterpret_cast<uint32_t*>(q_tiled + q_tiled_offset(row, k4, m_alloc)) = word;
  }
}


}  // namespace b200
