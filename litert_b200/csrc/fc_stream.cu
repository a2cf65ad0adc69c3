// Streamed-weights GEMM for small and medium batch (decode-shaped GEMV up to
// 64 activation rows per pass): Y[m,n] = epilogue(sum_k W[n,k] * Q[m,k]).
//
// The kernel is bound by the one pass over the packed weights in HBM, so it is
// organised around that stream:
//  * the packed weight tiles of a GEMM are one contiguous buffer; the grid
//    (one CTA per SM) cuts the flat (n tile, k tile) sequence into equal,
//    contiguous ranges ("stream-K"), so every SM pulls the same number of
//    bytes whatever the shape -- no wave quantisation on 148 SMs;
//  * one producer lane keeps a ring of stages filled with linear bulk copies
//    (16 KiB weight tile + the matching activation tile) signalled through
//    mbarriers; eight consumer warps read MMA fragments from shared memory
//    with conflict-free 32-bit loads (thread (g, t) reads word t of chunk c
//    of row g at swizzled chunk position c ^ g) and issue m16n8k32 int8 MMAs, weights as
//    the 16-row operand, activation rows as the 8 columns;
//  * a CTA that owns only part of an n tile's reduction adds its int32
//    partials into a global accumulator with coalesced reductions and bumps a
//    per-tile counter; whichever CTA completes the count reloads the totals,
//    runs the epilogue once and re-zeroes the scratch. Integer sums make this
//    exact and order-independent, so results are deterministic and bit-equal
//    to a serial sum.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;

template <int MT>
struct StageLayout {
  static constexpr int kWBytes = kTileBytes;
  static constexpr int kQBytes = MT * 1024;  // MT groups x 128 k bytes
  static constexpr int kStageBytes = kWBytes + kQBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * kStages * 8 + 64;
};

struct Flags {
  int abort_flag;
  int last;
};

template <int MT>
__device__ __forceinline__ void epilogue_hybrid(const FcParams& p, int nt, int m_base, const int (&acc)[MT][4],
                                                int warp, int lane) {
  const int g = lane >> 2, t4 = lane & 3;
  float* y = static_cast<float*>(p.y);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int n = nt * kTileN + warp * 16 + g + half * 8;
    if (n >= p.n) continue;
    const int32_t rs = p.row_sums ? p.row_sums[n] : 0;
    const float ws = p.per_channel ? p.w_scales[n] : p.w_scales[0];
    const float bias = p.bias_f32 ? p.bias_f32[n] : 0.0f;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = m_base + j * 8 + t4 * 2 + e;
        if (m >= p.m) continue;
        int32_t dot = acc[j][half * 2 + e];
        if (p.float_offset) {
          // BATCH_MATMUL's reference kernel subtracts through float (tflite/kernels/internal/reference/batch_matmul.h:189,197)
          const float off = p.in_zps ? (float)p.in_zps[m] : 0.0f;
          dot = __float2int_rz(__fsub_rn((float)dot, __fmul_rn((float)rs, off)));
        } else if (p.in_zps) {
          dot -= rs * p.in_zps[m];
        }
        // reference order: scale = in_scale * w_scale; out = bias + dot*scale
        const float scale = __fmul_rn(p.in_scales[m], ws);
        float out = __fadd_rn(bias, __fmul_rn((float)dot, scale));
        out = apply_activation(out, p.activation);
        y[(size_t)m * p.n + n] = out;
      }
    }
  }
}

template <int MT>
__device__ __forceinline__ void epilogue_requant(const FcParams& p, int nt, int m_base, const int (&acc)[MT][4],
                                                 int warp, int lane, bool raw) {
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int n = nt * kTileN + warp * 16 + g + half * 8;
    if (n >= p.n) continue;
    const int32_t rs = p.row_sums ? p.row_sums[n] : 0;
    const int32_t bias = p.bias_i32 ? p.bias_i32[n] : 0;
    const int32_t mult = p.multipliers ? p.multipliers[p.per_channel ? n : 0] : 0;
    const int32_t shift = p.shifts ? p.shifts[p.per_channel ? n : 0] : 0;
    // sum (w+fo)(x+io) = sum w x + io sum w + fo sum x + k fo io
    const int32_t base = p.input_offset * rs + p.k * p.filter_offset * p.input_offset + bias;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = m_base + j * 8 + t4 * 2 + e;
        if (m >= p.m) continue;
        int32_t total = acc[j][half * 2 + e] + base;
        if (p.x_sums) total += p.filter_offset * p.x_sums[m];
        if (raw) {
          static_cast<int32_t*>(p.y)[(size_t)m * p.n + n] = total;
        } else {
          int32_t v = requantize_mbqm(total, mult, shift) + p.output_offset;
          v = max(p.act_min, min(p.act_max, v));
          static_cast<int8_t*>(p.y)[(size_t)m * p.n + n] = (int8_t)v;
        }
      }
    }
  }
}

template <int MT, int EPI>
__global__ void __launch_bounds__(kThreads, 1) fc_stream_kernel(const FcParams p, const int m_base) {
  using L = StageLayout<MT>;
  using AccT = int;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  Flags* flags = reinterpret_cast<Flags*>(empty_bar + L::kStages);
  volatile int* abort_flag = &flags->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    flags->abort_flag = 0;
    flags->last = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // whole n tiles per CTA (no cross-CTA reduction) or equal ranges of the flat (n tile, k tile) sequence
  const long long total = (long long)p.n_tiles * p.k_tiles;
  const long long t_begin = p.whole_tiles ? ((long long)p.n_tiles * blockIdx.x / gridDim.x) * p.k_tiles
                                          : total * blockIdx.x / gridDim.x;
  const long long t_end = p.whole_tiles ? ((long long)p.n_tiles * (blockIdx.x + 1) / gridDim.x) * p.k_tiles
                                        : total * (blockIdx.x + 1) / gridDim.x;
  const int m_groups_alloc = p.m_alloc / 8;
  const int mg_base = m_base / 8;

  if (warp == kConsumerWarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (long long t = t_begin; t < t_end; ++t, ++it) {
        const int s = it % L::kStages;
        const uint32_t ph = (it / L::kStages) & 1u;
        mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
        uint8_t* dst = smem + (size_t)s * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], L::kStageBytes);
        bulk_g2s(dst, p.w_packed + (size_t)t * L::kWBytes, L::kWBytes, &full_bar[s]);
        const int kt = (int)(t % p.k_tiles);
        const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
        bulk_g2s(dst + L::kWBytes, p.q_tiled + off, MT * 1024, &full_bar[s]);
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  AccT acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0;

  uint32_t it = 0;
  long long seg_begin = t_begin;
  for (long long t = t_begin; t < t_end; ++t, ++it) {
    const int s = it % L::kStages;
    const uint32_t ph = (it / L::kStages) & 1u;
    mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.status, kStatusWaitTimeoutFull);
    const uint8_t* sw = smem + (size_t)s * L::kStageBytes;
    const uint8_t* sq = sw + L::kWBytes;
    {
      // weight rows 16*warp .. +15 = row groups 2*warp, 2*warp+1; thread (g, t) reads word t of the
      // 16-byte chunk `c` of row g, which the swizzled layout keeps at chunk position c ^ g
      const int g = lane >> 2, t4 = lane & 3;
      const uint32_t* wg0 = reinterpret_cast<const uint32_t*>(sw + (size_t)(2 * warp) * 1024) + g * 32 + t4;
      const uint32_t* wg1 = wg0 + 256;
      const uint32_t* qg = reinterpret_cast<const uint32_t*>(sq) + g * 32 + t4;
#pragma unroll
      for (int ks = 0; ks < kTileK8 / 32; ++ks) {
        const int c0 = ((2 * ks) ^ g) * 4, c1 = ((2 * ks + 1) ^ g) * 4;
        const uint32_t a0 = wg0[c0];
        const uint32_t a1 = wg1[c0];
        const uint32_t a2 = wg0[c1];
        const uint32_t a3 = wg1[c1];
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint32_t b0 = qg[j * 256 + c0];
          const uint32_t b1 = qg[j * 256 + c1];
          mma_s8(reinterpret_cast<int(&)[4]>(acc[j]), a0, a1, a2, a3, b0, b1);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);

    const bool tile_row_done = ((t + 1) % p.k_tiles) == 0;
    if (tile_row_done || t + 1 == t_end) {
      const int nt = (int)(t / p.k_tiles);
      const int seg_tiles = (int)(t + 1 - seg_begin);
      seg_begin = t + 1;
      bool run_epilogue = true;
      if (seg_tiles != p.k_tiles) {
        // partial reduction: merge through global scratch
        // Scratch slot = index of the CTA holding this tile's first k tile: tiles
        // that are split have distinct first CTAs, so gridDim.x slots suffice.
        const int slot = (int)((((long long)nt * p.k_tiles + 1) * gridDim.x - 1) / total);
        AccT* ws = reinterpret_cast<AccT*>(p.ws_acc) + (size_t)slot * kAccSlotInts;
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) atomicAdd(&ws[(j * 4 + c) * kConsumerThreads + tid], acc[j][c]);
        __threadfence();
        named_barrier(1, kConsumerThreads);
        if (tid == 0) {
          const int old = atomicAdd(&p.ws_count[slot], seg_tiles);
          flags->last = (old + seg_tiles == p.k_tiles) ? 1 : 0;
        }
        named_barrier(1, kConsumerThreads);
        run_epilogue = flags->last != 0;
        if (run_epilogue) {
          __threadfence();
#pragma unroll
          for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              AccT* slot = &ws[(j * 4 + c) * kConsumerThreads + tid];
              acc[j][c] = __ldcg(slot);
              __stcg(slot, (AccT)0);
            }
          if (tid == 0) p.ws_count[slot] = 0;
        }
        named_barrier(1, kConsumerThreads);  // flags->last may be rewritten next time
      }
      if (run_epilogue) {
        if constexpr (EPI == kEpiHybridF32) {
          epilogue_hybrid<MT>(p, nt, m_base, acc, warp, lane);
        } else {
          epilogue_requant<MT>(p, nt, m_base, acc, warp, lane, EPI == kEpiRawI32);
        }
      }
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0;
    }
  }
}

template <int MT, int EPI>
cudaError_t launch_one(const FcParams& p, int m_base, cudaStream_t s) {
  using L = StageLayout<MT>;
  static bool configured[64] = {false};
  auto kernel = fc_stream_kernel<MT, EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const long long total = (long long)p.n_tiles * p.k_tiles;
  const int sms = device_sm_count();
  int ctas = p.max_ctas > 0 ? p.max_ctas : sms;
  if (const char* e = tuning_env("B200_FC_MAX_CTAS")) {  // tuning knob
    const int v = atoi(e);
    if (v > 0) ctas = v;
  }
  FcParams q = p;
  // with at least half as many n tiles as SMs, whole tiles per CTA: nothing to merge across CTAs
  q.whole_tiles = (p.n_tiles * 2 >= sms && p.max_ctas <= 0 && !tuning_env("B200_FC_MAX_CTAS")) ? 1 : 0;
  if (const char* e = tuning_env("B200_FC_SPLIT")) q.whole_tiles = atoi(e) ? 0 : 1;  // measurement knob
  if (q.whole_tiles && ctas > p.n_tiles) ctas = p.n_tiles;
  if (ctas > kAccSlots) ctas = kAccSlots;
  if (ctas > total) ctas = (int)total;
  if (ctas < 1) ctas = 1;
  kernel<<<ctas, kThreads, L::kSmemBytes, s>>>(q, m_base);
  return cudaGetLastError();
}

template <int EPI>
cudaError_t launch_by_mt(const FcParams& p, int m_base, int mt, cudaStream_t s) {
  switch (mt) {
    case 1: return launch_one<1, EPI>(p, m_base, s);
    case 2: return launch_one<2, EPI>(p, m_base, s);
    case 4: return launch_one<4, EPI>(p, m_base, s);
    default: return launch_one<8, EPI>(p, m_base, s);
  }
}

cudaError_t launch_chunks(const FcParams& p, int epi, cudaStream_t s) {
  // up to 64 activation rows per pass over the weights
  for (int m_base = 0; m_base < p.m; m_base += 64) {
    const int rows = p.m - m_base < 64 ? p.m - m_base : 64;
    const int mt = p.m > 64 ? 8 : m_tiles_for(rows);
    cudaError_t e;
    if (epi == kEpiHybridF32) {
      e = launch_by_mt<kEpiHybridF32>(p, m_base, mt, s);
    } else if (epi == kEpiRequantI8) {
      e = launch_by_mt<kEpiRequantI8>(p, m_base, mt, s);
    } else {
      e = launch_by_mt<kEpiRawI32>(p, m_base, mt, s);
    }
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}


cudaError_t launch_fc_i8(const FcParams& p, FcEpilogue epi, cudaStream_t s) { return launch_chunks(p, epi, s); }

}  // namespace b200
