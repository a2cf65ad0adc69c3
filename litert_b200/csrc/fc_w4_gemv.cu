// Blockwise 4-bit weights, decode-sized batches (up to 8 activation rows): one launch that quantizes
// the rows itself and streams the packed weights once, on the integer dot-product units.
//
//   Y[m,n] = (sum_b float(sum_{k in block b} W4[n,k] * Q[m,k]) * scale[n,b] - zp[m] * kfsum[n]) * in_scale[m] + bias[n]
//
// is the reference's arithmetic (tflite/kernels/fully_connected.cc:1014-1086): an exact integer sum
// per block of 32, one float multiply-add per block. Here the integer block sums are exact as
// well; four threads share an output channel (each takes one 64-element quarter of every 256-element
// tile, so that sixteen warps hide each other's latencies) and their four float sums are added in a
// fixed order at the end, so only the order of the float additions differs from the reference's
// (differences of a few 1e-7 of the result's magnitude, identical from run to run).
//
// The kernel is bound by the single pass over the weights in HBM (4.5 bits per weight with the
// block scales), so it is built around that stream: a producer lane keeps a ring of 18 KiB packed
// tiles (128 channels x 256 reduction elements) filled with bulk copies, starting before the
// kernel's dependencies have resolved (the weights are constants); meanwhile the other warps
// quantize the activation rows (per-row asymmetric int8, as BatchQuantizeFloats) into shared
// memory, in the byte order the packed nibbles come apart in. A packed word holds 8 weights as
// offset-binary nibbles; `w & 0x0F0F0F0F` and `w & 0xF0F0F0F0` are two unsigned dp4a operands (the
// second one carries 16 x its nibbles: its block sum is shifted back, exactly), and the +8 offset
// leaves as -8 * (sum of the block's activations), precomputed per block and row. Every wait is bounded.
#include <cuda_fp16.h>
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"
#include "quant.cuh"

namespace b200 {

namespace {

constexpr int kGemvMaxSmem = 227 * 1024;
constexpr int kGemvTpr = 4;  // threads per output channel
// Beyond eight rows the dot-product units cost more than the HBM stream (the work per weight byte
// grows with the rows) and the tensor-core path is faster.
constexpr int kGemvMaxRows = 8;

struct W4GemvShared {
  int abort_flag;
  int last;
  int pad[2];
  float2 mm[16][16];  // per activation row and compute warp: min, max
  float scale[16]; // per activation row
  float inv[16];
  float zpf[16];
  int zero[16];
};

template <int MR, int TPR>
struct W4GemvCfg {
  static constexpr int kComputeThreads = 128 * TPR;
  static constexpr int kComputeWarps = kComputeThreads / 32;
  static constexpr int kThreads = kComputeThreads + 32;  // + the producer warp
};

// Bytes of dynamic shared memory besides the weight ring.
__host__ __device__ inline size_t w4_gemv_fixed_bytes(int mr, int tpr, int k_tiles) {
  const size_t kblocks = (size_t)k_tiles * 8;
  return kblocks * mr * 32        // quantized rows, 8 words per (block, row)
         + kblocks * mr * 4       // -8 * block sums
         + (size_t)(tpr - 1) * mr * 128 * 4  // the other threads' partial sums
         + 2 * 16 * 8             // barriers (up to 16 stages)
         + sizeof(W4GemvShared) + 128;
}

// d = c + sum_i a.u8[i] * b.s8[i]
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <int MR, int TPR>
__global__ void __launch_bounds__(W4GemvCfg<MR, TPR>::kThreads, MR <= 2 ? 2 : 1)
    fc_w4_gemv_kernel(const FcParams p, const float* __restrict__ x, const int stages) {
  using C = W4GemvCfg<MR, TPR>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int kblocks = p.k_tiles * 8;
  uint8_t* ring = smem;
  uint32_t* qs = reinterpret_cast<uint32_t*>(ring + (size_t)stages * kTile4Bytes);
  int32_t* corr = reinterpret_cast<int32_t*>(qs + (size_t)kblocks * MR * 8);
  float* part = reinterpret_cast<float*>(corr + (size_t)kblocks * MR);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(part + (TPR - 1) * MR * 128);
  uint64_t* empty_bar = full_bar + 16;
  W4GemvShared* sh = reinterpret_cast<W4GemvShared*>(empty_bar + 16);
  volatile int* abort_flag = &sh->abort_flag;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], C::kComputeWarps);
    }
    sh->abort_flag = 0;
    sh->last = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // The flat (n tile, k tile) sequence of packed tiles is cut into equal contiguous ranges, one per
  // CTA: every SM streams the same number of bytes whatever the shape.
  const int total = p.n_tiles * p.k_tiles;  // (the launcher refuses shapes beyond 2^31 tiles)
  int t_begin, t_end;
  if (p.whole_tiles) {  // CTA c owns n tile c (CTAs beyond the tiles have nothing to do)
    t_begin = (int)blockIdx.x * p.k_tiles;
    t_end = (int)blockIdx.x < p.n_tiles ? t_begin + p.k_tiles : t_begin;
  } else {
    t_begin = (int)((long long)total * blockIdx.x / gridDim.x);
    t_end = (int)((long long)total * (blockIdx.x + 1) / gridDim.x);
  }

  if (warp == C::kComputeWarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      pdl_launch_dependents();
      const uint64_t stream_policy = l2_policy_evict_first();
      uint32_t it = 0;
      for (int t = t_begin; t < t_end; ++t, ++it) {
        const int s = it % stages;
        mbar_wait_bounded(&empty_bar[s], ((it / stages) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
        mbar_arrive_expect_tx(&full_bar[s], (uint32_t)kTile4Bytes);
        bulk_g2s_hint(ring + (size_t)s * kTile4Bytes, p.w_packed + (size_t)t * kTile4Bytes, kTile4Bytes, &full_bar[s],
                      stream_policy);
      }
      for (uint32_t back = 0; back < (uint32_t)stages && back < it; ++back) {  // no copies in flight at exit
        const uint32_t j = it - 1 - back;
        mbar_wait_bounded(&full_bar[j % stages], (j / stages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
      }
    }
    return;
  }

  // ---------------- activation rows: per-row asymmetric int8 (BatchQuantizeFloats) ----------------
  // All rows at once: one round of loads for the minima and maxima, one barrier, the rows' parameters
  // by one thread per row, one barrier, then every (row, group of 8 elements) pair by one thread.
  pdl_wait();
  const int groups = kblocks * 4;  // groups of 8 reduction elements = one packed word's worth
  // byte order of the two dp4a operands of a packed word: elements (0, 4, 1, 5) and (2, 6, 3, 7)
  auto store_group = [&](int m, int g, const uint32_t (&q)[8], int sum) {
    uint32_t* dst = qs + ((size_t)(g >> 2) * MR + m) * 8 + (g & 3) * 2;
    dst[0] = q[0] | (q[4] << 8) | (q[1] << 16) | (q[5] << 24);
    dst[1] = q[2] | (q[6] << 8) | (q[3] << 16) | (q[7] << 24);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((g & 3) == 0) corr[(g >> 2) * MR + m] = -8 * sum;
  };
  if (MR * groups <= C::kComputeThreads) {
    // Few enough elements for one (row, group of 8) pair per thread: the values stay in registers between
    // the min/max pass and the quantization. (groups is a multiple of 32: a warp's pairs share a row.)
    const bool active = tid < MR * groups;
    const int m0 = active ? tid / groups : 0, g0 = active ? tid - m0 * groups : 0;
    const bool row_ok = active && m0 < p.m;
    float v[8];
    float mn = CUDART_INF_F, mx = -CUDART_INF_F;
    if (row_ok) {
      const float* xr = x + (size_t)m0 * p.k;
      if (g0 * 8 + 7 < p.k && ((reinterpret_cast<uintptr_t>(xr + g0 * 8) & 15) == 0)) {
        const float4 a = *reinterpret_cast<const float4*>(xr + g0 * 8);
        const float4 b = *reinterpret_cast<const float4*>(xr + g0 * 8 + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = xr[min(g0 * 8 + e, p.k - 1)];  // padding repeats a real element
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        mn = fminf(mn, v[e]);
        mx = fmaxf(mx, v[e]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0 && row_ok) sh->mm[m0][g0 >> 5] = make_float2(mn, mx);
    named_barrier(1, C::kComputeThreads);
    if (tid < MR && tid < p.m) {
      float rmn = sh->mm[tid][0].x, rmx = sh->mm[tid][0].y;
      for (int w = 1; w < groups / 32; ++w) {
        rmn = fminf(rmn, sh->mm[tid][w].x);
        rmx = fmaxf(rmx, sh->mm[tid][w].y);
      }
      float sf, inv;
      int zp, zero_row;
      row_quant_params(rmn, rmx, true, &sf, &inv, &zp, &zero_row);
      sh->scale[tid] = sf;
      sh->inv[tid] = inv;
      sh->zpf[tid] = (float)zp;
      sh->zero[tid] = zero_row;
    }
    named_barrier(1, C::kComputeThreads);
    if (active) {  // (warp-uniform)
      uint32_t q[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      int sum = 0;
      if (row_ok && !sh->zero[m0]) {
        const float inv = sh->inv[m0], zpf = sh->zpf[m0];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (g0 * 8 + e < p.k) q[e] = quantize_value(v[e], inv, zpf, true);
          sum += (int)(int8_t)q[e];
        }
      }
      store_group(m0, g0, q, sum);
    }
  } else {
    float mn[MR], mx[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      const float* xr = x + (size_t)(m < p.m ? m : 0) * p.k;
      mn[m] = mx[m] = xr[0];
    }
    for (int i = tid; i < p.k; i += C::kComputeThreads) {
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        if (m < p.m) {
          const float v = x[(size_t)m * p.k + i];
          mn[m] = fminf(mn[m], v);
          mx[m] = fmaxf(mx[m], v);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn[m] = fminf(mn[m], __shfl_xor_sync(0xffffffffu, mn[m], o));
        mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xffffffffu, mx[m], o));
      }
      if (lane == 0) sh->mm[m][warp] = make_float2(mn[m], mx[m]);
    }
  named_barrier(1, C::kComputeThreads);
  if (tid < MR && tid < p.m) {
    float mn = sh->mm[tid][0].x, mx = sh->mm[tid][0].y;
    for (int w = 1; w < C::kComputeWarps; ++w) {
      mn = fminf(mn, sh->mm[tid][w].x);
      mx = fmaxf(mx, sh->mm[tid][w].y);
    }
    float sf, inv;
    int zp, zero_row;
    row_quant_params(mn, mx, true, &sf, &inv, &zp, &zero_row);
    sh->scale[tid] = sf;
    sh->inv[tid] = inv;
    sh->zpf[tid] = (float)zp;
    sh->zero[tid] = zero_row;
  }
  named_barrier(1, C::kComputeThreads);
  for (int idx = tid; idx < MR * groups; idx += C::kComputeThreads) {  // (groups is a multiple of 32: warp-uniform)
    const int m = idx / groups, g = idx - m * groups;
    uint32_t q[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    int sum = 0;
    if (m < p.m && !sh->zero[m]) {
      const float inv = sh->inv[m], zpf = sh->zpf[m];
      const float* xr = x + (size_t)m * p.k;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int kk = g * 8 + e;
        if (kk < p.k) q[e] = quantize_value(xr[kk], inv, zpf, true);
        sum += (int)(int8_t)q[e];
      }
    }
    store_group(m, g, q, sum);
  }
  }
  named_barrier(1, C::kComputeThreads);

  // ---------------- the weight stream ----------------
  const int row = tid & 127;
  const int half = tid >> 7;                 // which of a tile's four sub-tiles (TPR == 4), or which two
  constexpr int kSubs = 4 / TPR;
  float* y = static_cast<float*>(p.y);
  uint32_t it = 0;
  int t = t_begin;
  // ring slot, its phase, and the k tile within the n tile: carried along instead of divided out per stage
  int slot = 0;
  uint32_t phase = 0;
  int kt = (int)(t_begin % p.k_tiles);
  while (t < t_end) {
    const int nt = t / p.k_tiles;
    const int seg_end = (nt + 1) * p.k_tiles < t_end ? (nt + 1) * p.k_tiles : t_end;
    const int seg_tiles = seg_end - t;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.0f;
    for (; t < seg_end; ++t, ++it, ++kt) {
      const int s = slot;
      mbar_wait_bounded(&full_bar[s], phase, abort_flag, p.status, kStatusWaitTimeoutFull);
      if (++slot == stages) {
        slot = 0;
        phase ^= 1u;
      }
      
      const uint8_t* raw = ring + (size_t)s * kTile4Bytes;
#pragma unroll
      for (int si = 0; si < kSubs; ++si) {
        const int sub = half * kSubs + si;
        const uint32_t* wsub = reinterpret_cast<const uint32_t*>(raw + sub * kTile4SubBytes);
        const __half* ssub = reinterpret_cast<const __half*>(raw + sub * kTile4SubBytes + kTile4SubWordBytes);
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          uint32_t lo[4], hi[4];
          const uint4 w4 = reinterpret_cast<const uint4*>(wsub)[blk * 128 + row];
          const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w = wv[j];
            lo[j] = w & 0x0F0F0F0Fu;
            hi[j] = w & 0xF0F0F0F0u;  // 16 x the high nibbles: their sums are shifted back once per block
          }
          const float sc = __half2float(ssub[blk * 128 + row]);
          const int b = kt * 8 + sub * 2 + blk;
          const uint4* qp = reinterpret_cast<const uint4*>(qs + (size_t)b * MR * 8);
          const int32_t* cp = corr + b * MR;
#pragma unroll
          for (int m = 0; m < MR; ++m) {
            const uint4 q0 = qp[2 * m], q1 = qp[2 * m + 1];
            int ca = cp[m], cb = 0;
            ca = dp4a_us(lo[0], q0.x, ca);
            cb = dp4a_us(hi[0], q0.y, cb);
            ca = dp4a_us(lo[1], q0.z, ca);
            cb = dp4a_us(hi[1], q0.w, cb);
            ca = dp4a_us(lo[2], q1.x, ca);
            cb = dp4a_us(hi[2], q1.y, cb);
            ca = dp4a_us(lo[3], q1.z, ca);
            cb = dp4a_us(hi[3], q1.w, cb);
            const int c = ca + (cb >> 4);  // cb is an exact multiple of 16
            acc[m] = __fadd_rn(acc[m], __fmul_rn((float)c, sc));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    kt = 0;  // the next segment starts a new n tile
    if (half > 0) {
#pragma unroll
      for (int m = 0; m < MR; ++m) part[((half - 1) * MR + m) * 128 + row] = acc[m];
    }
    named_barrier(1, C::kComputeThreads);
    if (half == 0) {
#pragma unroll
      for (int m = 0; m < MR; ++m) {
#pragma unroll
        for (int h = 1; h < TPR; ++h) acc[m] = __fadd_rn(acc[m], part[((h - 1) * MR + m) * 128 + row]);
      }
    }
    const int n = nt * kTileN + row;
    // tflite/kernels/fully_connected.cc:1077-1082: subtract zp * kfsum, scale by the row, add the bias
    auto finish = [&](const float (&sum)[MR]) {
      if (n >= p.n) return;
      const float kf = p.kfsum[n];
      const float bias = p.bias_f32 ? p.bias_f32[n] : 0.0f;
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        if (m < p.m) {
          float out = __fsub_rn(sum[m], __fmul_rn(sh->zpf[m], kf));
          out = __fmul_rn(out, sh->scale[m]);
          if (p.bias_f32) out = __fadd_rn(out, bias);
          y[(size_t)m * p.n + n] = out;
        }
      }
    };
    if (seg_tiles == p.k_tiles) {
      if (half == 0) finish(acc);
      named_barrier(1, C::kComputeThreads);  // `part` is rewritten by the next tile
    } else {
      // A tile shared with other CTAs: this CTA's float sums go to a scratch slot of its own (two per
      // CTA: one for a tile begun by an earlier CTA, one for a tile that goes on in the next), its k
      // tile count to the tile's counter; whoever completes the count adds the contributors' slots in
      // CTA order and finishes the outputs, so the result does not depend on who came last.
      const long long tile_first = (long long)nt * p.k_tiles, tile_last = tile_first + p.k_tiles - 1;
      const long long g = gridDim.x;
      const int c_first = (int)(((tile_first + 1) * g - 1) / total);
      const int c_last = (int)(((tile_last + 1) * g - 1) / total);
      const int which = (t_begin <= tile_first) ? 1 : 0;
      float* slots = reinterpret_cast<float*>(p.ws_part);
      if (half == 0) {
        float* mine = slots + (size_t)(blockIdx.x * 2 + which) * kZeroWsSlotInts;
#pragma unroll
        for (int m = 0; m < MR; ++m) __stcg(&mine[m * 128 + row], acc[m]);
      }
      named_barrier(1, C::kComputeThreads);
      if (tid == 0) {
        __threadfence();
        const int old = atomicAdd(&p.ws_count[c_first], seg_tiles);
        sh->last = (old + seg_tiles == p.k_tiles) ? 1 : 0;
      }
      named_barrier(1, C::kComputeThreads);
      if (sh->last && half == 0) {
        __threadfence();
        float sum[MR];
#pragma unroll
        for (int m = 0; m < MR; ++m) sum[m] = 0.0f;
        for (int c = c_first; c <= c_last; ++c) {
          const float* slot = slots + (size_t)(c * 2 + (c == c_first ? 1 : 0)) * kZeroWsSlotInts + row;
#pragma unroll
          for (int m = 0; m < MR; ++m) sum[m] = __fadd_rn(sum[m], __ldcg(slot + m * 128));
        }
        finish(sum);
        if (tid == 0) p.ws_count[c_first] = 0;
      }
      named_barrier(1, C::kComputeThreads);  // sh->last and `part` are rewritten by the next tile
    }
  }
}

template <int MR, int TPR>
cudaError_t launch_gemv(const FcParams& p, const float* x, cudaStream_t s) {
  using C = W4GemvCfg<MR, TPR>;
  static bool configured[64] = {false};
  auto kernel = fc_w4_gemv_kernel<MR, TPR>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvMaxSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const size_t fixed = w4_gemv_fixed_bytes(MR, TPR, p.k_tiles);
  // A deep ring: with a reduction of up to 2560 elements a CTA's whole share of the weights is requested
  // at once, before the kernel's dependencies have resolved. (Measured on B200, [16384, 2048] weights, one
  // row, launches chained back to back: 10 stages and one CTA per SM 5.9 us per launch; 5 stages, so that
  // two CTAs fit an SM and the next launch's ring fills early, 7.6 us: its CTAs then land unevenly.)
  int stages = (int)((kGemvMaxSmem - fixed) / kTile4Bytes);
  if (stages > 10) stages = 10;
  const int sms = device_sm_count();
  const long long total = (long long)p.n_tiles * p.k_tiles;
  FcParams q = p;
  int ctas;
  // With at least half as many n tiles as SMs (and no more than SMs) a CTA owns one whole n tile: no
  // merge across CTAs, which costs three L2 round trips (measured: 11.1 us against 6.3 us per launch
  // for 128 n tiles on 148 SMs). Otherwise the flat tile sequence is cut into equal ranges.
  q.whole_tiles = (p.n_tiles * 2 >= sms && p.n_tiles <= sms) ? 1 : 0;
  if (q.whole_tiles) {
    ctas = p.n_tiles;
  } else {
    ctas = total < sms ? (int)total : sms;
    if (ctas > kZeroWsSlots / 2) ctas = kZeroWsSlots / 2;  // two scratch slots per CTA
  }
  return launch_chained(kernel, dim3(ctas), dim3(C::kThreads), fixed + (size_t)stages * kTile4Bytes, s, q, x, stages);
}

int gemv_rows(int m) { return m <= 1 ? 1 : (m <= 2 ? 2 : (m <= 4 ? 4 : 8)); }

}  // namespace

bool w4_gemv_supported(int m, int k) {
  if (m < 1 || m > kGemvMaxRows) return false;
  const int mr = gemv_rows(m);
  const size_t fixed = w4_gemv_fixed_bytes(mr, kGemvTpr, tiles_k4(k));
  return fixed + 4 * (size_t)kTile4Bytes <= (size_t)kGemvMaxSmem;  // a ring of four stages at least
}

cudaError_t launch_fc_w4_gemv(const FcParams& p, const float* x, cudaStream_t s) {
  if ((long long)p.n_tiles * p.k_tiles > 0x7fffffffLL) return cudaErrorInvalidValue;  // tile indices are 32-bit
  switch (gemv_rows(p.m)) {
    case 1: return launch_gemv<1, kGemvTpr>(p, x, s);
    case 2: return launch_gemv<2, kGemvTpr>(p, x, s);
    case 4: return launch_gemv<4, kGemvTpr>(p, x, s);
    default: return launch_gemv<8, kGemvTpr>(p, x, s);
  }
}

}  // namespace b200
