// One-time weight repacking (run at delegate-kernel init) and the per-call
// activation preparation kernels: row quantization and int8 re-tiling.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "quant.cuh"

namespace b200 {

bool pdl_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = tuning_env("B200_PDL");
    cached = (e && e[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

// ---- int8 weights: row-major [n,k] -> tiles --------------------------------
// One thread per 16-byte chunk of the packed buffer.
__global__ void pack_w8_kernel(const int8_t* __restrict__ w, int n, int k, int n_tiles, int k_tiles,
                               uint8_t* __restrict__ packed) {
  const long long total = (long long)n_tiles * k_tiles * (kTileBytes / 16);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(idx & 7);
    const int c = (int)((idx >> 3) & 7);
    const int rg = (int)((idx >> 6) & 15);
    const long long tile = idx >> 10;
    const int kt = (int)(tile % k_tiles);
    const int nt = (int)(tile / k_tiles);
    const int row = nt * kTileN + rg * 8 + r;
    const int k0 = kt * kTileK8 + c * 16;
    uint32_t v[4] = {0, 0, 0, 0};
    if (row < n) {
      const int8_t* src = w + (size_t)row * k + k0;
#pragma unroll
      for (int b = 0; b < 16; ++b) {
        if (k0 + b < k) v[b >> 2] |= (uint32_t)(uint8_t)src[b] << (8 * (b & 3));
      }
    }
    uint8_t* dst = packed + (size_t)tile * kTileBytes + rg * 1024 + swz_chunk_offset(r, c);
    *reinterpret_cast<uint4*>(dst) = make_uint4(v[0], v[1], v[2], v[3]);
  }
}

// row_sums[r] = sum_k w[r,k]; one warp per row.
__global__ void row_sums_kernel(const int8_t* __restrict__ w, int n, int k, int32_t* __restrict__ row_sums) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n) return;
  const int8_t* row = w + (size_t)warp * k;
  int32_t s = 0;
  for (int i = lane; i < k; i += 32) s += row[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) row_sums[warp] = s;
}

// ---- int4 blockwise weights -------------------------------------------------
// Source: n rows of k2/2 bytes (k2 = k rounded up to even), element 2i in the
// low nibble of byte i (tflite/kernels/fully_connected.cc:1053-1067); fp16
// scales [n, k/blocksize]. Destination: tiles of kTileN rows x 256 reduction
// elements, 18 KiB each, in (n tile, k tile) order. A tile is four sub-tiles of
// 64 reduction elements (the K extent of one 128-byte-swizzled fp16 operand
// tile), each [2 blocks of 32][128 rows][4 words] of nibbles (one 16-byte load
// per row and block, conflict-free across a warp of consecutive rows) followed
// by [2 blocks][128 rows] fp16 scales. Word j (0..7) of a row holds its elements 8j .. 8j+7 as
// offset-binary nibbles (value + 8): element 2p in bits 4p .. 4p+3 and element
// 2p+1 in bits 16+4p .. 16+4p+3, so that `(word >> 4p) & 0x000F000F` is a pair
// of neighbouring elements, one per 16-bit half. A scale is stored once per
// block of 32 whatever the tensor's block size (a multiple of 32): blocks of 64
// or more repeat theirs.
__device__ __forceinline__ uint32_t nibble_at(const uint8_t* __restrict__ w4, size_t row_bytes, int row, int kk,
                                              int n, int k) {
  if (row >= n || kk >= k) return 0u;
  const uint8_t byte = w4[(size_t)row * row_bytes + (kk >> 1)];
  return (kk & 1) ? (byte >> 4) : (byte & 0xF);
}

__global__ void pack_w4_kernel(const uint8_t* __restrict__ w4, const __half* __restrict__ scales, int n, int k,
                               int blocksize, int n_tiles, int k_tiles, uint8_t* __restrict__ packed) {
  const size_t row_bytes = ((size_t)k + 1) / 2;
  const int num_blocks = k / blocksize;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // words of nibbles: 4 sub-tiles x 8 words x 128 rows per tile
  const long long total_words = (long long)n_tiles * k_tiles * (kTileBytes / 4);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_words; idx += stride) {
    const int r = (int)(idx & 127);
    const int j = (int)((idx >> 7) & 7);
    const int sub = (int)((idx >> 10) & 3);
    const long long tile = idx >> 12;
    const int kt = (int)(tile % k_tiles);
    const int nt = (int)(tile / k_tiles);
    const int row = nt * kTileN + r;
    const int k0 = kt * kTileK4 + sub * 64 + j * 8;
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      // two's complement nibble -> offset binary; padding (rows >= n, k >= the tensor's) holds the value 0
      const uint32_t u = (row < n && k0 + e < k) ? (nibble_at(w4, row_bytes, row, k0 + e, n, k) ^ 8u) : 8u;
      word |= u << ((e & 1) * 16 + (e >> 1) * 4);
    }
    *reinterpret_cast<uint32_t*>(packed + (size_t)tile * kTile4Bytes + (size_t)sub * kTile4SubBytes +
                                 (size_t)(((j >> 2) * 128 + r) * 4 + (j & 3)) * 4) = word;
  }
  // scales: 4 sub-tiles x 2 blocks x 128 rows per tile
  const long long scales_per_tile = kTileN * kSubBlocks4;
  const long long total_scales = (long long)n_tiles * k_tiles * scales_per_tile;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_scales; idx += stride) {
    const int r = (int)(idx & 127);
    const int blk = (int)((idx >> 7) & 1);
    const int sub = (int)((idx >> 8) & 3);
    const long long tile = idx >> 10;
    const int kt = (int)(tile % k_tiles);
    const int nt = (int)(tile / k_tiles);
    const int row = nt * kTileN + r;
    const int k0 = kt * kTileK4 + sub * 64 + blk * 32;
    __half s = __float2half(0.0f);
    if (row < n && k0 < k && k0 / blocksize < num_blocks) s = scales[(size_t)row * num_blocks + k0 / blocksize];
    reinterpret_cast<__half*>(packed + (size_t)tile * kTile4Bytes + (size_t)sub * kTile4SubBytes + kTile4SubWordBytes)
        [blk * 128 + r] = s;
  }
}

// kfsum[row] = sum over blocks, in increasing block order, of
// scale[row,b] * (sum of the block's weights)  -- the zero-point correction
// term of tflite/kernels/fully_connected.cc:1057-1078, which does not depend
// on the activations. One thread per row; float operations are kept
// unfused and in the reference's order.
__global__ void w4_kfsum_kernel(const uint8_t* __restrict__ w4, const __half* __restrict__ scales, int n, int k,
                                int blocksize, float* __restrict__ kfsum) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  const size_t row_bytes = ((size_t)k + 1) / 2;
  const int num_blocks = k / blocksize;
  float acc = 0.0f;
  for (int b = 0; b < num_blocks; ++b) {
    int32_t ksum = 0;
    for (int i = 0; i < blocksize; ++i) {
      const int v = (int)nibble_at(w4, row_bytes, row, b * blocksize + i, n, k);
      ksum += (v ^ 8) - 8;
    }
    const float s = __half2float(scales[(size_t)row * num_blocks + b]);
    acc = __fadd_rn(acc, __fmul_rn(s, (float)ksum));
  }
  kfsum[row] = acc;
}

// ---- activations ------------------------------------------------------------
// Per-row quantization of float activations to int8, one CTA per row.
// Asymmetric: tflite/kernels/internal/reference/portable_tensor_utils.cc:74-119;
// symmetric: :41-71. The scale and zero point are derived in double exactly as
// there; the element loop is float multiply, float add, round half away from
// zero, clamp -- with no fused multiply-add, as on the reference's x86 build.
__global__ void __launch_bounds__(1024) quantize_rows_kernel(const float* __restrict__ x, int m, int k, int k_pad,
                                                            int m_alloc, int asymmetric,
                                                            int8_t* __restrict__ q_tiled,
                                                            int8_t* __restrict__ q_rowmajor,
                                                            float* __restrict__ scales,
                                                            int32_t* __restrict__ zero_points,
                                                            __half* __restrict__ h_tiled) {
  __shared__ float2 s_mm[32];
  __shared__ float s_inv;
  __shared__ int s_zp;
  __shared__ int s_zero;
  pdl_enter();
  const int row = blockIdx.x;
  const float* xr = x + (size_t)row * k;
  float mn = xr[0], mx = xr[0];
  if ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
    const int k4 = k & ~3;
    for (int i = threadIdx.x * 4; i < k4; i += blockDim.x * 4) {
      const float4 f = *reinterpret_cast<const float4*>(xr + i);
      mn = fminf(fminf(mn, f.x), fminf(f.y, fminf(f.z, f.w)));
      mx = fmaxf(fmaxf(mx, f.x), fmaxf(f.y, fmaxf(f.z, f.w)));
    }
    for (int i = k4 + threadIdx.x; i < k; i += blockDim.x) {
      mn = fminf(mn, xr[i]);
      mx = fmaxf(mx, xr[i]);
    }
  } else {
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
      const float v = xr[i];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  block_minmax(mn, mx, s_mm);
  if (threadIdx.x == 0) {
    float sf, inv;
    int zp, zero_row;
    row_quant_params(mn, mx, asymmetric != 0, &sf, &inv, &zp, &zero_row);
    s_zero = zero_row;
    s_inv = inv;
    s_zp = zp;
    scales[row] = sf;
    if (zero_points) zero_points[row] = zp;
  }
  __syncthreads();
  const bool zero = s_zero != 0;
  const float inv = s_inv;
  const float zpf = (float)s_zp;
  auto quant = [&](float v) -> uint32_t { return zero ? 0u : quantize_value(v, inv, zpf, asymmetric != 0); };
  const bool vec = ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
  // four consecutive elements per thread and step: one float4 in, one 32-bit word out
  for (int k4 = threadIdx.x * 4; k4 < k_pad; k4 += blockDim.x * 4) {
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (vec && k4 + 3 < k) {
      const float4 f = *reinterpret_cast<const float4*>(xr + k4);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (k4 + b < k) v[b] = xr[k4 + b];
    }
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if (k4 + b < k) word |= quant(v[b]) << (8 * b);
    if (q_tiled) *reinterpret_cast<uint32_t*>(q_tiled + q_tiled_offset(row, k4, m_alloc)) = word;
    if (h_tiled) {
      // the same integers as fp16 (exact), for the kind::f16 MMA of the 4-bit path
      const __half2 lo = __floats2half2_rn((float)(int8_t)(word & 0xFF), (float)(int8_t)((word >> 8) & 0xFF));
      const __half2 hi = __floats2half2_rn((float)(int8_t)((word >> 16) & 0xFF), (float)(int8_t)(word >> 24));
      uint2 v;
      v.x = *reinterpret_cast<const uint32_t*>(&lo);
      v.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(h_tiled) + h_tiled_offset(row, k4, m_alloc)) = v;
    }
    if (q_rowmajor) {
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (k4 + b < k) q_rowmajor[(size_t)row * k + k4 + b] = (int8_t)(word >> (8 * b));
    }
  }
}

// int8 activations [m,k] row-major -> tiled layout, plus optional row sums
// (needed only when the weights have a non-zero zero point).
__global__ void __launch_bounds__(256) retile_x8_kernel(const int8_t* __restrict__ x, int m, int k, int k_pad,
                                                        int m_alloc, int8_t* __restrict__ q_tiled,
                                                        int32_t* __restrict__ x_sums) {
  __shared__ int red[32];
  const int row = blockIdx.x;
  const int8_t* xr = x + (size_t)row * k;
  int sum = 0;
  for (int c = threadIdx.x; c < k_pad / 16; c += blockDim.x) {
    uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      const int kk = c * 16 + b;
      if (kk < k) {
        const int8_t e = xr[kk];
        sum += e;
        v[b >> 2] |= (uint32_t)(uint8_t)e << (8 * (b & 3));
      }
    }
    *reinterpret_cast<uint4*>(q_tiled + q_tiled_offset(row, c * 16, m_alloc)) = make_uint4(v[0], v[1], v[2], v[3]);
  }
  if (x_sums) {
    sum = block_reduce(sum, [](int a, int b) { return a + b; }, 0, red);
    if (threadIdx.x == 0) x_sums[row] = sum;
  }
}

// ---- launchers ---------------------------------------------------------------
static inline int grid_for(long long work, int block, int cap = 148 * 16) {
  long long g = (work + block - 1) / block;
  if (g < 1) g = 1;
  return (int)(g > cap ? cap : g);
}

cudaError_t launch_pack_w8(const int8_t* w, int n, int k, uint8_t* packed, int32_t* row_sums, cudaStream_t s) {
  const int n_tiles = tiles_n(n), k_tiles = tiles_k8(k);
  const long long chunks = (long long)n_tiles * k_tiles * (kTileBytes / 16);
  pack_w8_kernel<<<grid_for(chunks, 256), 256, 0, s>>>(w, n, k, n_tiles, k_tiles, packed);
  if (row_sums) row_sums_kernel<<<(n * 32 + 255) / 256, 256, 0, s>>>(w, n, k, row_sums);
  return cudaGetLastError();
}

cudaError_t launch_pack_w4(const uint8_t* w4, const void* scales_f16, int n, int k, int blocksize, uint8_t* packed,
                           float* kfsum, cudaStream_t s) {
  const int n_tiles = tiles_n(n), k_tiles = tiles_k4(k);
  const long long words = (long long)n_tiles * k_tiles * (kTileBytes / 4);
  pack_w4_kernel<<<grid_for(words, 256), 256, 0, s>>>(w4, (const __half*)scales_f16, n, k, blocksize, n_tiles,
                                                      k_tiles, packed);
  w4_kfsum_kernel<<<(n + 127) / 128, 128, 0, s>>>(w4, (const __half*)scales_f16, n, k, blocksize, kfsum);
  return cudaGetLastError();
}

cudaError_t launch_quantize_rows(const float* x, int m, int k, int k_pad, int m_alloc, int asymmetric,
                                 int8_t* q_tiled, int8_t* q_rowmajor, float* scales, int32_t* zps,
                                 cudaStream_t s, void* h_tiled) {
  if (m <= 0) return cudaSuccess;
  // few long rows (decode): one large CTA per row hides more latency; many rows: more CTAs per SM
  const int threads = (m <= 32 && k >= 2048) ? 1024 : 256;
  return launch_chained(quantize_rows_kernel, dim3(m), dim3(threads), 0, s, x, m, k, k_pad, m_alloc, asymmetric, q_tiled,
                        q_rowmajor, scales, zps, static_cast<__half*>(h_tiled));
}

cudaError_t launch_retile_x8(const int8_t* x, int m, int k, int k_pad, int m_alloc, int8_t* q_tiled,
                             int32_t* x_sums, cudaStream_t s) {
  if (m <= 0) return cudaSuccess;
  retile_x8_kernel<<<m, 256, 0, s>>>(x, m, k, k_pad, m_alloc, q_tiled, x_sums);
  return cudaGetLastError();
}

}  // namespace b200
