// Streamed-weights int8 GEMM on the 5th-generation tensor cores:
// Y[m,n] = epilogue(sum_k W[n,k] * Q[m,k]) with the accumulators in TMEM.
//
// Roles inside a CTA (one CTA per SM, 192 threads):
//   warp 0, one lane   producer: linear bulk copies (TMA engine) of one packed
//                      16 KiB weight tile and the matching activation tile per
//                      stage, completion counted on an mbarrier;
//   warp 1, one lane   MMA issuer: four tcgen05.mma (kind::i8, M = 128 weight
//                      rows, N = NB activation rows, K = 32) per stage, operands
//                      read straight from shared memory through matrix
//                      descriptors (the packed tile IS the canonical K-major
//                      core-matrix layout); tcgen05.commit releases the stage
//                      and, at the end of an n tile, publishes the accumulator;
//   warps 2..5         epilogue: tcgen05.ld brings 32 TMEM lanes (weight rows)
//                      per warp into registers, frees the accumulator at once
//                      (two accumulators alternate, so the next tile's MMAs run
//                      meanwhile), then requantizes / dequantizes and stores
//                      coalesced along n.
// The (n tile, k tile) sequence is cut into equal contiguous ranges, one per
// CTA (stream-K): every SM streams the same number of weight bytes. A CTA that
// holds only part of an n tile's reduction parks its int32 partials in a scratch
// slot of its own (plain stores); the CTA whose arrival completes the tile's k
// count sums the contributors' slots and runs the epilogue. Integer addition
// makes the result bit-equal to a serial sum.
// Every wait is bounded (see mbar_wait_bounded); TMEM is always freed.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

namespace {

constexpr int kUmmaThreads = 192;
constexpr int kEpiThreads = 128;

template <int NB>
struct UmmaLayout {
  static constexpr int kQBytes = NB * kTileK8;  // NB/8 row groups x 1 KiB
  static constexpr int kStageBytes = kTileBytes + kQBytes;
  static constexpr int kStagesRaw = 200 * 1024 / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr int kBarriers = 2 * kStages + 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarriers * 8 + 64;
  static constexpr int kTmemCols = 2 * NB < 32 ? 32 : 2 * NB;
};

struct UmmaShared {
  uint32_t tmem_base;
  int abort_flag;
  int last;
  int pad;
};

// Epilogue for one output element; `total` is the exact int32 dot product.
template <int EPI>
__device__ __forceinline__ void store_output(const FcParams& p, int m, int n, int32_t total, int32_t rs, float ws,
                                             float bias_f, int32_t base_i, int32_t mult, int32_t shift) {
  if constexpr (EPI == kEpiHybridF32) {
    int32_t dot = total;
    if (p.in_zps) dot -= rs * p.in_zps[m];
    // reference order: scale = in_scale * w_scale; out = bias + dot * scale (no fused multiply-add)
    const float scale = __fmul_rn(p.in_scales[m], ws);
    float out = __fadd_rn(bias_f, __fmul_rn((float)dot, scale));
    out = apply_activation(out, p.activation);
    static_cast<float*>(p.y)[(size_t)m * p.n + n] = out;
  } else {
    int32_t t = total + base_i;
    if (p.x_sums) t += p.filter_offset * p.x_sums[m];
    if constexpr (EPI == kEpiRawI32) {
      static_cast<int32_t*>(p.y)[(size_t)m * p.n + n] = t;
    } else {
      int32_t v = requantize_mbqm(t, mult, shift) + p.output_offset;
      v = max(p.act_min, min(p.act_max, v));
      static_cast<int8_t*>(p.y)[(size_t)m * p.n + n] = (int8_t)v;
    }
  }
}


template <int NB, int EPI>
__global__ void __launch_bounds__(kUmmaThreads, 1) fc_umma_kernel(const FcParams p, const int m_base) {
  using L = UmmaLayout<NB>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* acc_full = empty_bar + L::kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  UmmaShared* sh = reinterpret_cast<UmmaShared*>(acc_empty + 2);
  volatile int* abort_flag = &sh->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    sh->abort_flag = 0;
    sh->last = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&sh->tmem_base, L::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  // Work split over the CTAs: either whole n tiles (no cross-CTA reduction) or equal contiguous
  // ranges of the flat (n tile, k tile) sequence (stream-K), chosen on the host per shape.
  const long long total = (long long)p.n_tiles * p.k_tiles;
  const long long t_begin = p.whole_tiles ? ((long long)p.n_tiles * blockIdx.x / gridDim.x) * p.k_tiles
                                          : total * blockIdx.x / gridDim.x;
  const long long t_end = p.whole_tiles ? ((long long)p.n_tiles * (blockIdx.x + 1) / gridDim.x) * p.k_tiles
                                        : total * (blockIdx.x + 1) / gridDim.x;
  const int m_groups_alloc = p.m_alloc / 8;
  const int mg_base = m_base / 8;

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      // The weights are constants: start streaming them before the kernel that produces the
      // activations has finished (programmatic dependent launch), one ring's worth at most.
      pdl_launch_dependents();
      uint32_t pre = 0;
      for (long long t = t_begin; t < t_end && pre < (uint32_t)L::kStages; ++t, ++pre) {
        uint8_t* dst = smem + (size_t)pre * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[pre], L::kStageBytes);
        bulk_g2s(dst, p.w_packed + (size_t)t * kTileBytes, kTileBytes, &full_bar[pre]);
      }
      pdl_wait();               // activations (and the split-K scratch) are now safe to touch
      for (uint32_t i = 0; i < pre; ++i) {
        const int kt = (int)((t_begin + i) % p.k_tiles);
        const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
        bulk_g2s(smem + (size_t)i * L::kStageBytes + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[i]);
      }
      uint32_t it = pre;
      for (long long t = t_begin + pre; t < t_end; ++t, ++it) {
        const int s = it % L::kStages;
        const uint32_t ph = (it / L::kStages) & 1u;
        mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
        uint8_t* dst = smem + (size_t)s * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], L::kStageBytes);
        bulk_g2s(dst, p.w_packed + (size_t)t * kTileBytes, kTileBytes, &full_bar[s]);
        const int kt = (int)(t % p.k_tiles);
        const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
        bulk_g2s(dst + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[s]);
      }
      // never leave with copies in flight (only possible after an abort)
      const uint32_t issued = it;
      for (uint32_t back = 0; back < (uint32_t)L::kStages && back < issued; ++back) {
        const uint32_t j = issued - 1 - back;
        mbar_wait_bounded(&full_bar[j % L::kStages], (j / L::kStages) & 1u, abort_flag, p.status,
                          kStatusWaitTimeoutFull);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_s8(NB);
      uint32_t it = 0, seg = 0;
      long long t = t_begin;
      while (t < t_end) {
        const long long nt = t / p.k_tiles;
        const long long seg_end = (nt + 1) * p.k_tiles < t_end ? (nt + 1) * p.k_tiles : t_end;
        const uint32_t ab = seg & 1u;
        mbar_wait_bounded(&acc_empty[ab], ((seg >> 1) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * NB;
        bool first = true;
        for (; t < seg_end; ++t, ++it) {
          const int s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.status, kStatusWaitTimeoutFull);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * L::kStageBytes);
          const uint32_t b_addr = a_addr + kTileBytes;
#pragma unroll
          for (int ks = 0; ks < kTileK8 / 32; ++ks) {
            // two 16-byte K chunks per MMA: 128 B apart; 8-row groups 1 KiB apart
            const uint64_t a_desc = umma_smem_desc(a_addr + ks * 256, 128, 1024);
            const uint64_t b_desc = umma_smem_desc(b_addr + ks * 256, 128, 1024);
            if (!(p.debug_flags & 1)) umma_s8(d_tmem, a_desc, b_desc, idesc, (first && ks == 0) ? 0u : 1u);
          }
          first = false;
          umma_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
        }
        umma_commit(&acc_full[ab]);
        ++seg;
      }
      // wait for the last accumulator to be complete before the CTA tears TMEM down
      if (seg > 0) {
        const uint32_t lastseg = seg - 1;
        mbar_wait_bounded(&acc_full[lastseg & 1u], (lastseg >> 1) & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;  // TMEM lanes this warp may touch: 32*quarter .. +31
    const int row_in_tile = quarter * 32 + lane;
    const int etid = tid - 64;
    const int m_valid = p.m - m_base < NB ? p.m - m_base : NB;
    pdl_wait();  // the epilogue reads activation scales written by the previous kernel
    uint32_t seg = 0;
    long long t = t_begin;
    while (t < t_end) {
      const long long nt = t / p.k_tiles;
      const long long seg_end = (nt + 1) * p.k_tiles < t_end ? (nt + 1) * p.k_tiles : t_end;
      const int seg_tiles = (int)(seg_end - t);
      t = seg_end;
      const uint32_t ab = seg & 1u;
      const uint32_t taddr = tmem_base + ab * NB + ((uint32_t)(quarter * 32) << 16);

      const int n = (int)nt * kTileN + row_in_tile;
      const bool row_ok = n < p.n;
      int32_t rs = 0, base_i = 0, mult = 0, shift = 0;
      float wsc = 0.0f, bias_f = 0.0f;
      if (row_ok) {
        rs = p.row_sums ? p.row_sums[n] : 0;
        if constexpr (EPI == kEpiHybridF32) {
          wsc = p.per_channel ? p.w_scales[n] : p.w_scales[0];
          bias_f = p.bias_f32 ? p.bias_f32[n] : 0.0f;
        } else {
          // sum (w+fo)(x+io) = sum w x + io sum w + fo sum x + k fo io
          base_i = p.input_offset * rs + p.k * p.filter_offset * p.input_offset + (p.bias_i32 ? p.bias_i32[n] : 0);
          if (p.multipliers) {
            mult = p.multipliers[p.per_channel ? n : 0];
            shift = p.shifts[p.per_channel ? n : 0];
          }
        }
      }

      // the per-channel constants above are in flight while the MMAs of this segment finish
      mbar_wait_bounded(&acc_full[ab], (seg >> 1) & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      tc_fence_after();

      const bool partial = seg_tiles != p.k_tiles;
      if (p.debug_flags & 2) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      } else if (!partial) {
#pragma unroll 1
        for (int c = 0; c < NB / 16; ++c) {
          if (c * 16 >= m_valid) break;
          int r[16];
          tmem_ld16(taddr + c * 16, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = c * 16 + j;
              if (m < m_valid) store_output<EPI>(p, m_base + m, n, r[j], rs, wsc, bias_f, base_i, mult, shift);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      } else {
        // Split tile: every contributing CTA parks its int32 partials in a scratch slot of its own
        // (two per CTA: one for a tile continued from an earlier CTA, one for a tile that goes on in
        // the next) with plain coalesced stores, then adds its k-tile count to the tile's counter.
        // Whoever completes the count sums the contributors' slots in CTA order and runs the
        // epilogue. No accumulator ever needs clearing; only the counter is reset.
        const long long tile_first = nt * p.k_tiles, tile_last = tile_first + p.k_tiles - 1;
        const int g = gridDim.x;
        const int c_first = (int)(((tile_first + 1) * g - 1) / total);
        const int c_last = (int)(((tile_last + 1) * g - 1) / total);
        const int which = (t_begin <= tile_first) ? 1 : 0;
        int32_t* mine = p.ws_part + (size_t)(blockIdx.x * 2 + which) * kZeroWsSlotInts;
#pragma unroll 1
        for (int c = 0; c < NB / 16; ++c) {
          if (c * 16 >= m_valid) break;
          int r[16];
          tmem_ld16(taddr + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c * 16 + j;
            if (m < m_valid) __stcg(&mine[m * kTileN + row_in_tile], r[j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
        named_barrier(1, kEpiThreads);
        if (etid == 0) {
          __threadfence();
          const int old = atomicAdd(&p.ws_count[c_first], seg_tiles);
          sh->last = (old + seg_tiles == p.k_tiles) ? 1 : 0;
        }
        named_barrier(1, kEpiThreads);
        const bool last = sh->last != 0;
        if (last) {
          __threadfence();
          for (int m = 0; m < m_valid; ++m) {
            int32_t v = 0;
            for (int c = c_first; c <= c_last; ++c) {
              const int w = (c == c_first) ? 1 : 0;
              v += __ldcg(p.ws_part + (size_t)(c * 2 + w) * kZeroWsSlotInts + m * kTileN + row_in_tile);
            }
            if (row_ok) store_output<EPI>(p, m_base + m, n, v, rs, wsc, bias_f, base_i, mult, shift);
          }
          if (etid == 0) p.ws_count[c_first] = 0;
        }
        named_barrier(1, kEpiThreads);  // sh->last is rewritten by the next split tile
      }
      ++seg;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::kTmemCols);
}

// Chooses the number of CTAs and the split for one launch (measured on B200, batch 1, graph
// replays): with at least half as many n tiles as SMs, whole n tiles per CTA win (no cross-CTA
// reduction; CTAs with one tile fewer finish early and the kernel stays HBM-bound); with fewer,
// one SM per n tile cannot pull more than ~80 GB/s, so the flat (n tile, k tile) sequence is cut
// into equal ranges over all SMs (stream-K) and the partials are merged by the last arriver.
int plan_ctas(FcParams* p) {
  const int sms = device_sm_count();
  const long long total = (long long)p->n_tiles * p->k_tiles;
  int mode = -1;  // -1 auto, 0 stream-K, 1 whole tiles
  if (const char* e = getenv("B200_FC_SPLIT")) mode = atoi(e) ? 0 : 1;  // measurement knob
  int ctas;
  if (mode == 1 || (mode < 0 && p->n_tiles * 2 >= sms)) {
    p->whole_tiles = 1;
    ctas = p->n_tiles < sms ? p->n_tiles : sms;
  } else {
    p->whole_tiles = 0;
    ctas = sms;
  }
  if (p->max_ctas > 0) ctas = p->max_ctas;
  if (const char* e = getenv("B200_FC_MAX_CTAS")) {  // measurement knob
    const int v = atoi(e);
    if (v > 0) ctas = v;
  }
  if (ctas > kZeroWsSlots / 2) ctas = kZeroWsSlots / 2;  // two scratch slots per CTA
  if (p->whole_tiles && ctas > p->n_tiles) ctas = p->n_tiles;
  if (ctas > total) ctas = (int)total;
  if (ctas < 1) ctas = 1;
  return ctas;
}

template <int NB, int EPI>
cudaError_t launch_umma_one(const FcParams& p, int m_base, cudaStream_t s) {
  using L = UmmaLayout<NB>;
  static bool configured[64] = {false};
  auto kernel = fc_umma_kernel<NB, EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  FcParams q = p;
  const int ctas = plan_ctas(&q);
  return launch_chained(kernel, dim3(ctas), dim3(kUmmaThreads), (size_t)L::kSmemBytes, s, q, m_base);
}

template <int EPI>
cudaError_t launch_umma_nb(const FcParams& p_in, int m_base, int nb, cudaStream_t s) {
  FcParams p = p_in;
  if (const char* e = getenv("B200_FC_DEBUG")) p.debug_flags = atoi(e);
  switch (nb) {
    case 16: return launch_umma_one<16, EPI>(p, m_base, s);
    case 32: return launch_umma_one<32, EPI>(p, m_base, s);
    case 64: return launch_umma_one<64, EPI>(p, m_base, s);
    case 128: return launch_umma_one<128, EPI>(p, m_base, s);
    default: return launch_umma_one<256, EPI>(p, m_base, s);
  }
}

}  // namespace

int umma_rows_per_pass(int m) {
  int nb = 16;
  while (nb < m && nb < 256) nb *= 2;
  return nb;
}

cudaError_t launch_fc_i8_umma(const FcParams& p, FcEpilogue epi, cudaStream_t s) {
  const int nb = umma_rows_per_pass(p.m);
  for (int m_base = 0; m_base < p.m; m_base += nb) {
    cudaError_t e;
    if (epi == kEpiHybridF32) {
      e = launch_umma_nb<kEpiHybridF32>(p, m_base, nb, s);
    } else if (epi == kEpiRequantI8) {
      e = launch_umma_nb<kEpiRequantI8>(p, m_base, nb, s);
    } else {
      e = launch_umma_nb<kEpiRawI32>(p, m_base, nb, s);
    }
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace b200
