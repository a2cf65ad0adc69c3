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
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <math_constants.h>

#include "argmax.cuh"
#include "common.cuh"
#include "kernels.h"
#include "prologue.cuh"

namespace b200 {

namespace {

constexpr int kUmmaThreads = 192;
constexpr int kMaxDynamicSmem = 227 * 1024;  // opt-in limit per CTA
constexpr int kEpiThreads = 128;

struct UmmaShared {
  uint32_t tmem_base;
  int abort_flag;
  int last;
  int pad;
  // per activation row of this launch's pass: input scale, zero point (hybrid) or row sum (int8)
  float in_scale[256];
  int32_t in_aux[256];
};

// Shared-memory budget of a GEMV CTA, by activation rows per pass. For up to 16 rows (NB = 16) a CTA
// keeps a short ring (4 stages of 18 KB) and two CTAs per SM are launched: three fit, so the next
// kernel of a programmatically chained sequence gets a CTA onto every SM and fills its ring while
// this kernel's CTAs are still streaming. Measured on B200 on the batch-1 decode step (18 layers +
// LM head, 1024-token context): one 180 KB CTA per SM 1.100 ms, one 108 KB CTA 1.070 ms, two 72 KB
// CTAs 0.97-1.00 ms, three 54 KB CTAs 1.022 ms. With more rows per pass the stages are larger and
// the deep ring of a single CTA per SM does better (batch 32: 1.667 ms against 1.70 ms).
#ifndef B200_UMMA_KB16
#define B200_UMMA_KB16 72
#endif
#ifndef B200_CLUSTER_KB16
#define B200_CLUSTER_KB16 72
#endif
#ifndef B200_PER_SM16
#define B200_PER_SM16 2
#endif
template <int NB>
struct UmmaBudget {
  static constexpr int kUmmaKB = NB <= 16 ? B200_UMMA_KB16 : (NB >= 64 ? 206 : 200);
  static constexpr int kClusterKB = NB <= 16 ? B200_CLUSTER_KB16 : 200;
  static constexpr int kCtasPerSm = NB <= 16 ? B200_PER_SM16 : 1;
};

template <int NB>
struct UmmaLayout {
  static constexpr int kQBytes = NB * kTileK8;  // NB/8 row groups x 1 KiB
  static constexpr int kStageBytes = kTileBytes + kQBytes;
  static constexpr int kStagesRaw = UmmaBudget<NB>::kUmmaKB * 1024 / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static_assert(kStages >= 2, "the ring needs two stages");
  static constexpr int kBarriers = 2 * kStages + 5;
  // without the fused prologue's operand buffer, which the launcher adds (k tiles x kQBytes)
  static constexpr int kOutStageBytes = NB >= 64 ? 2 * 16 * kTileN * 4 : 0;  // two 16-row output blocks
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarriers * 8 + (int)sizeof(UmmaShared) +
                                    2 * (int)sizeof(PrologueShared) + 1024 + 16 + kOutStageBytes + 16;
  static constexpr int kTmemCols = 2 * NB < 32 ? 32 : 2 * NB;
};

// The zero-point correction of the hybrid path. FULLY_CONNECTED subtracts in int32
// (tflite/kernels/internal/reference/portable_tensor_utils.cc:165-206). BATCH_MATMUL's hybrid kernel
// writes `total -= row_sum * batch_offset` with a FLOAT batch_offset
// (tflite/kernels/internal/reference/batch_matmul.h:189,197): the int32 total goes through float, the
// product is rounded, the difference is rounded and truncated back to int32. Identical until a term
// passes 2^24; reproduced here bit for bit when the op is a BATCH_MATMUL.
__device__ __forceinline__ int32_t hybrid_dot(const FcParams& p, int32_t total, int32_t rs, int32_t zp) {
  if (!p.float_offset) return total - rs * zp;
  return __float2int_rz(__fsub_rn((float)total, __fmul_rn((float)rs, (float)zp)));
}

// Value of one output element from its exact int32 dot product: the float's bits (hybrid), the
// int32 (raw) or the requantized int8 (sign-extended).
// PLAIN (see plain_epilogue): no fused activation and the integer zero-point term, as straight-line code.
// An epilogue warp is alone, or nearly, on its scheduler and pays every branch's latency in full: with
// the activation switch and the zero-point form tested per output, 128 x 256 outputs took 20 us; hoisted
// out of the loops, 3.6 us (measured on B200).
template <int EPI, bool PLAIN = false>
__device__ __forceinline__ int32_t compute_output(const FcParams& p, int32_t total, int32_t rs, float ws, float bias_f,
                                                  int32_t base_i, int32_t mult, int32_t shift, float in_scale,
                                                  int32_t in_aux) {
  if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
    const int32_t dot = PLAIN ? total - rs * in_aux : hybrid_dot(p, total, rs, in_aux);  // in_aux: the row's zero point
    // reference order: scale = in_scale * w_scale; out = bias + dot * scale (no fused multiply-add)
    const float scale = __fmul_rn(in_scale, ws);
    float out = __fadd_rn(bias_f, __fmul_rn((float)dot, scale));
    if constexpr (!PLAIN) out = apply_activation(out, p.activation);
    return __float_as_int(out);
  } else {
    const int32_t t = total + base_i + p.filter_offset * in_aux;  // in_aux: the row's sum
    if constexpr (EPI == kEpiRawI32) {
      return t;
    } else {
      int32_t v = requantize_mbqm(t, mult, shift) + p.output_offset;
      return max(p.act_min, min(p.act_max, v));
    }
  }
}

// Whether the PLAIN form of compute_output applies to this launch (uniform over the grid).
template <int EPI>
__device__ __forceinline__ bool plain_epilogue(const FcParams& p) {
  if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) return p.activation == 0 && !p.float_offset;
  return EPI == kEpiRawI32;
}

// Epilogue for one output element; `total` is the exact int32 dot product.
template <int EPI>
__device__ __forceinline__ void store_output(const FcParams& p, int m, int n, int32_t total, int32_t rs, float ws,
                                             float bias_f, int32_t base_i, int32_t mult, int32_t shift,
                                             float in_scale, int32_t in_aux) {
  if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
    const int32_t dot = hybrid_dot(p, total, rs, in_aux);  // in_aux: the row's zero point
    // reference order: scale = in_scale * w_scale; out = bias + dot * scale (no fused multiply-add)
    const float scale = __fmul_rn(in_scale, ws);
    float out = __fadd_rn(bias_f, __fmul_rn((float)dot, scale));
    out = apply_activation(out, p.activation);
    static_cast<float*>(p.y)[(size_t)m * p.n + n] = out;
  } else {
    const int32_t t = total + base_i + p.filter_offset * in_aux;  // in_aux: the row's sum
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
__global__ void __launch_bounds__(kUmmaThreads, 1) fc_umma_kernel(const FcParams p, const int m_base_first) {
  // grid.y = passes of NB activation rows; the stream-K scratch (slots, counters) is numbered over
  // the whole grid, so every pass merges its own split tiles
  const int m_base = m_base_first + (int)blockIdx.y * NB;
  const int cta_base = (int)(blockIdx.y * gridDim.x);
  using L = UmmaLayout<NB>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* acc_full = empty_bar + L::kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint64_t* b_ready = acc_empty + 2;            // fused prologue: the operand rows are in place
  UmmaShared* sh = reinterpret_cast<UmmaShared*>(b_ready + 1);
  PrologueShared* ps = reinterpret_cast<PrologueShared*>(sh + 1);
  uint8_t* bbuf = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ps + 2) + 1023) & ~uintptr_t(1023));
  // output staging of the many-row epilogue (never together with the fused prologue's operand buffer)
  uint8_t* out_stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ps + 2) + 15) & ~uintptr_t(15));
  volatile int* abort_flag = &sh->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  if (p.trace && blockIdx.x == 0 && tid == 0) p.trace[0] = global_timer_ns();

  if (tid == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    mbar_init(b_ready, 1);
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
      const uint32_t stage_tx = p.prologue ? (uint32_t)kTileBytes : (uint32_t)L::kStageBytes;
      const uint64_t stream_policy = l2_policy_evict_first();  // weights are read once per launch
      uint32_t pre = 0;
      for (long long t = t_begin; t < t_end && pre < (uint32_t)L::kStages; ++t, ++pre) {
        uint8_t* dst = smem + (size_t)pre * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[pre], stage_tx);
        bulk_g2s_hint(dst, p.w_packed + (size_t)t * kTileBytes, kTileBytes, &full_bar[pre], stream_policy);
      }
      // ... and the tiles behind the ring go to L2 meanwhile (the row kernels between two projections
      // leave HBM idle otherwise)
      {
        const long long pf_end = t_begin + pre + p.l2_prefetch_tiles < t_end ? t_begin + pre + p.l2_prefetch_tiles : t_end;
        for (long long t = t_begin + pre; t < pf_end; ++t) prefetch_l2_bulk(p.w_packed + (size_t)t * kTileBytes, kTileBytes);
      }
      pdl_wait();               // activations (and the split-K scratch) are now safe to touch
      if (p.trace && blockIdx.x == 0) p.trace[1] = global_timer_ns();
      if (!p.prologue) {
        for (uint32_t i = 0; i < pre; ++i) {
          const int kt = (int)((t_begin + i) % p.k_tiles);
          const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
          bulk_g2s(smem + (size_t)i * L::kStageBytes + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[i]);
        }
      }
      uint32_t it = pre;
      for (long long t = t_begin + pre; t < t_end; ++t, ++it) {
        const int s = it % L::kStages;
        const uint32_t ph = (it / L::kStages) & 1u;
        mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
        uint8_t* dst = smem + (size_t)s * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], stage_tx);
        bulk_g2s_hint(dst, p.w_packed + (size_t)t * kTileBytes, kTileBytes, &full_bar[s], stream_policy);
        if (!p.prologue) {
          const int kt = (int)(t % p.k_tiles);
          const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
          bulk_g2s(dst + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[s]);
        }
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
      if (p.prologue) {
        mbar_wait_bounded(b_ready, 0, abort_flag, p.status, kStatusWaitTimeoutFull);
        tc_fence_after();
      }
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
          const uint32_t b_addr =
              p.prologue ? smem_u32(bbuf) + (uint32_t)(t % p.k_tiles) * (uint32_t)L::kQBytes : a_addr + kTileBytes;
#pragma unroll
          for (int ks = 0; ks < kTileK8 / 32; ++ks) {
            // 32 reduction bytes per MMA: 32 B further along the swizzled rows; 8-row groups 1 KiB apart
            const uint64_t a_desc = umma_smem_desc(a_addr + ks * 32);
            const uint64_t b_desc = umma_smem_desc(b_addr + ks * 32);
            umma_s8(d_tmem, a_desc, b_desc, idesc, (first && ks == 0) ? 0u : 1u);
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
    // Per-output-channel constants of a segment (weights-side data, never written by other kernels).
    int32_t rs = 0, base_i = 0, mult = 0, shift = 0;
    float wsc = 0.0f, bias_f = 0.0f;
    auto load_channel_constants = [&](int n) {
      rs = 0, base_i = 0, mult = 0, shift = 0, wsc = 0.0f, bias_f = 0.0f;
      if (n >= p.n) return;
      rs = p.row_sums ? p.row_sums[n] : 0;
      if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
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
    };
    // those of the first segment are fetched while the predecessor kernel is still running
    if (t_begin < t_end) load_channel_constants((int)(t_begin / p.k_tiles) * kTileN + row_in_tile);
    pdl_wait();  // the activation rows' scales are written by the previous kernel
    if (p.prologue) {
      prologue_norm_quant(p, bbuf, NB, 0, p.k_tiles, sh->in_scale, sh->in_aux, ps, etid, blockIdx.x == 0, 1);
      if (etid == 0) mbar_arrive(b_ready);
    } else {
      for (int i = etid; i < NB; i += kEpiThreads) {
        const int m = m_base + i;
        const bool ok = m < p.m;
        sh->in_scale[i] = (ok && p.in_scales) ? p.in_scales[m] : 0.0f;
        if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
          sh->in_aux[i] = (ok && p.in_zps) ? p.in_zps[m] : 0;
        } else {
          sh->in_aux[i] = (ok && p.x_sums) ? p.x_sums[m] : 0;
        }
      }
      named_barrier(1, kEpiThreads);
    }
    // fused greedy pick (one pass of up to 16 rows): this thread's best value and column per row
    BestPick best[EPI == kEpiHybridPick ? 16 : 1];
#pragma unroll
    for (int j = 0; j < (EPI == kEpiHybridPick ? 16 : 1); ++j) best[j] = BestPick{-CUDART_INF_F, 0x7fffffff};
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
      if (seg > 0) load_channel_constants(n);

      // the per-channel constants above are in flight while the MMAs of this segment finish
      mbar_wait_bounded(&acc_full[ab], (seg >> 1) & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      tc_fence_after();

      const bool partial = seg_tiles != p.k_tiles;
      const bool plain = plain_epilogue<EPI>(p);
      if (!partial) {
#pragma unroll 1
        for (int c = 0; c < NB / 16; ++c) {
          if (c * 16 >= m_valid) break;
          int r[16];
          tmem_ld16(taddr + c * 16, r);
          tmem_ld_wait();
          if constexpr (NB >= 64) {
            // Many activation rows: a thread storing its own output channel writes 4 bytes (1 for int8)
            // per row and a warp 128 (32) bytes per store instruction, 57 KB apart from the next; at
            // 256 rows that costs more than the MMAs. The 16 x 128 block goes through shared memory
            // instead and leaves as whole 512-byte (128-byte) row segments, 16 bytes per thread.
            {
              constexpr int kElem = EPI == kEpiRequantI8 ? 1 : 4;
              uint8_t* st = out_stage + (c & 1) * (16 * kTileN * 4);
              float sc[16];  // the rows' parameters first: behind the staging stores they would be reloaded one by one
              int32_t ax[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                sc[j] = sh->in_scale[c * 16 + j];
                ax[j] = sh->in_aux[c * 16 + j];
              }
              if (plain) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  reinterpret_cast<int32_t*>(st)[j * kTileN + row_in_tile] =
                      compute_output<EPI, true>(p, r[j], rs, wsc, bias_f, base_i, mult, shift, sc[j], ax[j]);
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const int32_t v = compute_output<EPI>(p, r[j], rs, wsc, bias_f, base_i, mult, shift, sc[j], ax[j]);
                  if constexpr (kElem == 4) {
                    reinterpret_cast<int32_t*>(st)[j * kTileN + row_in_tile] = v;
                  } else {
                    reinterpret_cast<int8_t*>(st)[j * kTileN + row_in_tile] = (int8_t)v;
                  }
                }
              }
              named_barrier(2, kEpiThreads);  // the block is complete (and the other buffer's readers are done)
              const int n0 = (int)nt * kTileN;
              constexpr int kChunksPerRow = kTileN * kElem / 16;        // 16-byte pieces per output row segment
              constexpr int kPieces = 16 * kChunksPerRow;
              const bool vec_ok = (((size_t)p.n * kElem) % 16 == 0) && (n0 + kTileN <= p.n) &&
                                  ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
              for (int idx = etid; idx < kPieces; idx += kEpiThreads) {
                const int rr = idx / kChunksPerRow, cc = idx % kChunksPerRow;
                const int m = c * 16 + rr;
                if (m >= m_valid) continue;
                const size_t off = ((size_t)(m_base + m) * p.n + n0) * kElem + cc * 16;
                uint8_t* dst = static_cast<uint8_t*>(p.y) + off;
                const uint8_t* src = st + (size_t)rr * kTileN * kElem + cc * 16;
                if (vec_ok) {
                  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
                } else {
                  for (int b = 0; b < 16; ++b)
                    if (n0 + (cc * 16 + b) / kElem < p.n) dst[b] = src[b];
                }
              }
            }
          } else if (row_ok) {
            float sc[16];  // parameters of the 16 rows, read before the first output store
            int32_t ax[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              sc[j] = sh->in_scale[c * 16 + j];
              ax[j] = sh->in_aux[c * 16 + j];
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = c * 16 + j;
              if (m >= m_valid) continue;
              if constexpr (NB == 16 && EPI == kEpiHybridPick) {
                {
                  // fused greedy pick: the value takes part in this thread's running best of row m; the
                  // logit itself is stored only when the caller wants the logits
                  float v = __int_as_float(compute_output<EPI>(p, r[j], rs, wsc, bias_f, base_i, mult, shift, sc[j], ax[j]));
                  v = soft_capped(v, p.soft_cap);
                  if (p.y) static_cast<float*>(p.y)[(size_t)(m_base + m) * p.n + n] = v;
                  best[j] = better_pick(best[j], BestPick{v, n});
                  continue;
                }
              }
              store_output<EPI>(p, m_base + m, n, r[j], rs, wsc, bias_f, base_i, mult, shift, sc[j], ax[j]);
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
        int32_t* mine = p.ws_part + (size_t)((cta_base + blockIdx.x) * 2 + which) * kZeroWsSlotInts;
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
          const int old = atomicAdd(&p.ws_count[cta_base + c_first], seg_tiles);
          sh->last = (old + seg_tiles == p.k_tiles) ? 1 : 0;
        }
        named_barrier(1, kEpiThreads);
        const bool last = sh->last != 0;
        if (last) {
          __threadfence();
          // eight activation rows at a time: all their loads are issued before the first store,
          // so the L2 round trips overlap instead of queueing behind one another
          for (int m0 = 0; m0 < m_valid; m0 += 8) {
            int32_t v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int c = c_first; c <= c_last; ++c) {
              const int w = (c == c_first) ? 1 : 0;
              const int32_t* slot = p.ws_part + (size_t)((cta_base + c) * 2 + w) * kZeroWsSlotInts + row_in_tile;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (m0 + j < m_valid) v[j] += __ldcg(slot + (m0 + j) * kTileN);
            }
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (m0 + j < m_valid)
                  store_output<EPI>(p, m_base + m0 + j, n, v[j], rs, wsc, bias_f, base_i, mult, shift, sh->in_scale[m0 + j],
                                    sh->in_aux[m0 + j]);
            }
          }
          if (etid == 0) p.ws_count[cta_base + c_first] = 0;
        }
        named_barrier(1, kEpiThreads);  // sh->last is rewritten by the next split tile
      }
      ++seg;
    }
    if constexpr (NB == 16 && EPI == kEpiHybridPick) {
      {
        // this CTA's candidate per row: over the lanes, then over the four epilogue warps; the rows'
        // candidates of all CTAs are compared by a small kernel afterwards
        BestPick* cand = reinterpret_cast<BestPick*>(sh->in_aux);  // the rows' zero points are no longer needed
        named_barrier(1, kEpiThreads);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j < m_valid) {  // uniform over the CTA: rows that do not exist cost nothing at the kernel's tail
            BestPick b = best[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
              b = better_pick(b, BestPick{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)});
            if (lane == 0) cand[quarter * 16 + j] = b;
          }
        }
        named_barrier(1, kEpiThreads);
        if (etid < m_valid) {
          BestPick b = cand[etid];
          for (int w = 1; w < 4; ++w) b = better_pick(b, cand[w * 16 + etid]);
          const size_t slot = (size_t)(m_base + etid) * p.argmax_parts + blockIdx.x;
          p.argmax_val[slot] = b.v;
          p.argmax_idx[slot] = b.i;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::kTmemCols);
  if (p.trace && tid == 0) {
    const unsigned long long now = global_timer_ns();
    if (blockIdx.x == 0) p.trace[2] = now;
    atomicMax(p.trace + 3, now);
  }
}

// ---- cluster split-K variant ---------------------------------------------------------------------
// For layers with few n tiles (attention and down projections at decode time) the reduction over K
// must be split across SMs to pull the weights fast enough, and merging the pieces through global
// memory costs more than streaming them. Here the `split` CTAs that share an n tile form one
// thread-block cluster: each accumulates its k range in TMEM, then sends every ceil(128/split)-row
// slice of its int32 accumulator to the CTA that owns those rows through distributed shared memory
// (reduce-scatter); after one cluster barrier each CTA adds the `split` pieces of its own rows and
// runs the epilogue on them. No global scratch, no counters, no fences; integer addition keeps the
// result bit-equal to a serial sum.
template <int NB>
struct ClusterLayout {
  static constexpr int kQBytes = NB * kTileK8;
  static constexpr int kStageBytes = kTileBytes + kQBytes;
  static constexpr int kRedBytes = (kTileN + 8) * NB * 4;  // split x ceil(128 / split) rows x NB columns of int32
  static constexpr int kStagesRaw = (UmmaBudget<NB>::kClusterKB * 1024 - kRedBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static_assert(kStages >= 2, "the ring needs two stages");
  static constexpr int kBarriers = 2 * kStages + 3;
  // without the fused prologue's operand buffer, which the launcher adds
  static constexpr int kSmemBytes = kStages * kStageBytes + kRedBytes + kBarriers * 8 + (int)sizeof(UmmaShared) +
                                    2 * (int)sizeof(PrologueShared) + 1024 + 16;
  static constexpr int kTmemCols = NB < 32 ? 32 : NB;
};

template <int NB, int EPI>
__global__ void __launch_bounds__(kUmmaThreads, 1) fc_cluster_kernel(const FcParams p, const int m_base, const int split) {
  using L = ClusterLayout<NB>;
  extern __shared__ __align__(1024) uint8_t smem[];
  int32_t* red = reinterpret_cast<int32_t*>(smem + L::kStages * L::kStageBytes);  // [source][column][row in slice]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes + L::kRedBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* acc_full = empty_bar + L::kStages;
  uint64_t* b_ready = acc_full + 1;  // fused prologue: the operand rows are in place
  uint64_t* red_full = b_ready + 1;  // the cluster's pieces of this CTA's rows have all arrived
  UmmaShared* sh = reinterpret_cast<UmmaShared*>(red_full + 1);
  PrologueShared* ps = reinterpret_cast<PrologueShared*>(sh + 1);
  uint8_t* bbuf = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ps + 2) + 1023) & ~uintptr_t(1023));
  volatile int* abort_flag = &sh->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int rank = (int)cluster_ctarank();
  const int nt = blockIdx.x / split;
  if (p.trace && blockIdx.x == 0 && tid == 0) p.trace[0] = global_timer_ns();
  const int kt_begin = (int)((long long)p.k_tiles * rank / split);
  const int kt_end = (int)((long long)p.k_tiles * (rank + 1) / split);
  const int rows_per_owner = (kTileN + split - 1) / split;  // the last owner may hold fewer

  if (tid == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(b_ready, 1);
    mbar_init(red_full, 1);
    sh->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&sh->tmem_base, L::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  cluster_arrive();  // phase 0: "this CTA is running, its barriers exist" (waited for before the first remote store)

  const int m_groups_alloc = p.m_alloc / 8;
  const int mg_base = m_base / 8;
  const uint8_t* w_tiles = p.w_packed + (size_t)nt * p.k_tiles * kTileBytes;

  if (warp == 0) {
    if (lane == 0) {
      pdl_launch_dependents();
      const uint32_t stage_tx = p.prologue ? (uint32_t)kTileBytes : (uint32_t)L::kStageBytes;
      const uint64_t stream_policy = l2_policy_evict_first();  // weights are read once per launch
      uint32_t pre = 0;
      for (int kt = kt_begin; kt < kt_end && pre < (uint32_t)L::kStages; ++kt, ++pre) {
        mbar_arrive_expect_tx(&full_bar[pre], stage_tx);
        bulk_g2s_hint(smem + (size_t)pre * L::kStageBytes, w_tiles + (size_t)kt * kTileBytes, kTileBytes, &full_bar[pre],
                      stream_policy);
      }
      {  // the tiles behind the ring go to L2 while this CTA waits for its activations
        const int pf_end = kt_begin + (int)pre + p.l2_prefetch_tiles < kt_end ? kt_begin + (int)pre + p.l2_prefetch_tiles : kt_end;
        for (int kt = kt_begin + (int)pre; kt < pf_end; ++kt) prefetch_l2_bulk(w_tiles + (size_t)kt * kTileBytes, kTileBytes);
      }
      pdl_wait();
      if (p.trace && blockIdx.x == 0) p.trace[1] = global_timer_ns();
      if (!p.prologue) {
        for (uint32_t i = 0; i < pre; ++i) {
          const size_t off = (((size_t)(kt_begin + i) * m_groups_alloc) + mg_base) * 1024;
          bulk_g2s(smem + (size_t)i * L::kStageBytes + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[i]);
        }
      }
      uint32_t it = pre;
      for (int kt = kt_begin + (int)pre; kt < kt_end; ++kt, ++it) {
        const int s = it % L::kStages;
        const uint32_t ph = (it / L::kStages) & 1u;
        mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
        uint8_t* dst = smem + (size_t)s * L::kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], stage_tx);
        bulk_g2s_hint(dst, w_tiles + (size_t)kt * kTileBytes, kTileBytes, &full_bar[s], stream_policy);
        if (!p.prologue) {
          const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
          bulk_g2s(dst + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[s]);
        }
      }
      const uint32_t issued = it;  // never leave with copies in flight (only possible after an abort)
      for (uint32_t back = 0; back < (uint32_t)L::kStages && back < issued; ++back) {
        const uint32_t j = issued - 1 - back;
        mbar_wait_bounded(&full_bar[j % L::kStages], (j / L::kStages) & 1u, abort_flag, p.status,
                          kStatusWaitTimeoutFull);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && kt_begin < kt_end) {
      constexpr uint32_t idesc = umma_idesc_s8(NB);
      uint32_t it = 0;
      if (p.prologue) {
        mbar_wait_bounded(b_ready, 0, abort_flag, p.status, kStatusWaitTimeoutFull);
        tc_fence_after();
      }
      for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
        const int s = it % L::kStages;
        const uint32_t ph = (it / L::kStages) & 1u;
        mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.status, kStatusWaitTimeoutFull);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * L::kStageBytes);
        const uint32_t b_addr =
            p.prologue ? smem_u32(bbuf) + (uint32_t)(kt - kt_begin) * (uint32_t)L::kQBytes : a_addr + kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kTileK8 / 32; ++ks) {
          const uint64_t a_desc = umma_smem_desc(a_addr + ks * 32);
          const uint64_t b_desc = umma_smem_desc(b_addr + ks * 32);
          umma_s8(tmem_base, a_desc, b_desc, idesc, (kt == kt_begin && ks == 0) ? 0u : 1u);
        }
        umma_commit(&empty_bar[s]);
      }
      umma_commit(acc_full);
      mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kStatusWaitTimeoutTmem);  // before TMEM goes away
    }
    __syncwarp();
  }

  // Rows this thread finishes after the exchange: row r_own of this CTA's slice, columns col0,
  // col0 + col_step, ... (threads beyond the last whole group of rows_per_owner stay idle).
  const int etid = tid - 64;
  const int col_step = kEpiThreads / rows_per_owner;
  const int r_own = etid >= 0 ? etid % rows_per_owner : 0;
  const int col0 = etid >= 0 ? etid / rows_per_owner : 0;
  const int row_own = rank * rows_per_owner + r_own;  // row of the n tile
  const bool owns = etid >= 0 && col0 < col_step && row_own < kTileN;
  const int n_own = owns ? nt * kTileN + row_own : p.n;
  int32_t rs = 0, base_i = 0, mult = 0, shift = 0;
  float wsc = 0.0f, bias_f = 0.0f;
  const int m_valid = p.m - m_base < NB ? p.m - m_base : NB;

  if (warp >= 2) {
    // weights-side constants of the owned row: fetched while the predecessor kernel still runs
    if (n_own < p.n) {
      rs = p.row_sums ? p.row_sums[n_own] : 0;
      if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
        wsc = p.per_channel ? p.w_scales[n_own] : p.w_scales[0];
        bias_f = p.bias_f32 ? p.bias_f32[n_own] : 0.0f;
      } else {
        base_i = p.input_offset * rs + p.k * p.filter_offset * p.input_offset + (p.bias_i32 ? p.bias_i32[n_own] : 0);
        if (p.multipliers) {
          mult = p.multipliers[p.per_channel ? n_own : 0];
          shift = p.shifts[p.per_channel ? n_own : 0];
        }
      }
    }
    pdl_wait();
    if (p.prologue) {
      prologue_norm_quant(p, bbuf, NB, kt_begin, kt_end, sh->in_scale, sh->in_aux, ps, etid, blockIdx.x == 0, 1);
      if (etid == 0) mbar_arrive(b_ready);
    } else {
      for (int i = etid; i < NB; i += kEpiThreads) {
        const int m = m_base + i;
        const bool ok = m < p.m;
        sh->in_scale[i] = (ok && p.in_scales) ? p.in_scales[m] : 0.0f;
        if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
          sh->in_aux[i] = (ok && p.in_zps) ? p.in_zps[m] : 0;
        } else {
          sh->in_aux[i] = (ok && p.x_sums) ? p.x_sums[m] : 0;
        }
      }
    }
    // this CTA's accumulator row (zero when its k range is empty)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool have = kt_begin < kt_end;
    if (have) {
      mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kStatusWaitTimeoutTmem);
      tc_fence_after();
    }
    cluster_wait();  // phase 0: every CTA of the cluster is running, remote stores are legal
    // Every int32 sent to an owner also counts as four transaction bytes on the owner's `red_full`
    // barrier (st.async): an owner knows its pieces are in without a second cluster-wide barrier, which
    // cost 0.4 us per launch (measured on B200 against the same exchange with barrier.cluster).
    if (etid == 0) {
      const int owned = min(rows_per_owner, kTileN - rank * rows_per_owner);
      mbar_arrive_expect_tx(red_full, (uint32_t)(owned > 0 ? split * owned * m_valid * 4 : 0));
    }
    const uint32_t owner = (uint32_t)(row / rows_per_owner);
    const uint32_t owner_bar = map_to_rank(smem_u32(red_full), owner);
    const uint32_t slot = map_to_rank(smem_u32(red), owner) +
                          4u * (uint32_t)((rank * NB) * rows_per_owner + row % rows_per_owner);
#pragma unroll 1
    for (int c = 0; c < NB / 16; ++c) {
      if (c * 16 >= m_valid) break;
      int r[16];
      if (have) {
        tmem_ld16(taddr + c * 16, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (c * 16 + j < m_valid) st_async_cluster_u32(slot + 4u * (uint32_t)((c * 16 + j) * rows_per_owner), r[j], owner_bar);
    }
    tc_fence_before();
    mbar_wait_bounded(red_full, 0, abort_flag, p.status, kStatusWaitTimeoutTmem);  // everyone's pieces of this CTA's rows
  } else {
    cluster_wait();  // phase 0
  }
  if (warp >= 2 && n_own < p.n) {
    uint32_t epoch32 = 0;
    if constexpr (EPI == kEpiHybridF32) {
      if (p.push_ranks > 1)
        epoch32 = (uint32_t)(*p.push_step_epoch * (unsigned long long)p.push_per_step + (unsigned long long)p.push_seq + 1ull);
    }
    for (int col = col0; col < m_valid; col += col_step) {
      int32_t v = 0;
      for (int src = 0; src < split; ++src) v += red[(src * NB + col) * rows_per_owner + r_own];
      if constexpr (EPI == kEpiHybridF32) {
        if (p.push_ranks > 1) {
          // the partial sum goes to every peer as a self-validating message (value and epoch in one 8-byte store)
          const int32_t bits = compute_output<EPI>(p, v, rs, wsc, bias_f, base_i, mult, shift, sh->in_scale[col], sh->in_aux[col]);
          const size_t at = (size_t)(m_base + col) * p.n + n_own;
          static_cast<float*>(p.y)[at] = __int_as_float(bits);
          for (int j = 0; j < p.push_ranks; ++j)
            if (j != p.push_rank)
              asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p.push_out[j] + at), "r"((uint32_t)bits), "r"(epoch32)
                           : "memory");
          continue;
        }
      }
      store_output<EPI>(p, m_base + col, n_own, v, rs, wsc, bias_f, base_i, mult, shift, sh->in_scale[col], sh->in_aux[col]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::kTmemCols);
  if (p.trace && tid == 0) {
    const unsigned long long now = global_timer_ns();
    if (blockIdx.x == 0) p.trace[2] = now;
    atomicMax(p.trace + 3, now);
  }
}

// ---- prefill-sized variant ------------------------------------------------------------------------
// 256 activation rows per pass, whole work units per CTA, persistent CTAs: a unit is (n tile, pass of
// 256 rows, k range) and a CTA takes units blockIdx.x, blockIdx.x + gridDim.x, ... One 16 KiB weight
// tile + the 32 KiB activation tile per stage; the two 256-column accumulators alternate, so the
// epilogue of a unit runs under the MMAs of the CTA's next unit. Eight epilogue warps, two per TMEM
// lane quarter, each pair splitting the unit's activation rows. 4-byte outputs leave straight from
// the registers (for one activation row a warp holds 32 consecutive output channels: one full
// 128-byte line per store instruction); int8 outputs go through shared-memory staging blocks and
// leave as whole 128-byte row segments.
// With few units and a long reduction (the down projection of a prompt pass: 16 n tiles x 4 passes,
// 128 k tiles) the reduction is cut into `ksplit` ranges: every unit parks its raw int32 accumulator
// in a scratch slot, adds one to the (n tile, pass) counter, and whoever completes the count sums the
// slots and runs the epilogue. Integer sums: the result does not depend on the order.
// Measured on B200, config 2 at M = 512: 86 us one unit per CTA -> 68 persistent -> 63 row parameters
// preloaded -> 43 with eight epilogue warps -> 35 with the per-output branches hoisted (plain_epilogue).
struct PrefillLayout {
  static constexpr int kNB = 256;
  static constexpr int kQBytes = kNB * kTileK8;                      // 32 KiB
  static constexpr int kStageBytes = kTileBytes + kQBytes;
  static constexpr int kStages = 206 * 1024 / kStageBytes;
  static constexpr int kEpiWarps = 8;                                 // two per TMEM lane quarter
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static constexpr int kOutStageBytes = 2 * 2 * 16 * kTileN * 4;      // two blocks per half of the epilogue warps
  static constexpr int kBarriers = 2 * kStages + 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarriers * 8 + (int)sizeof(UmmaShared) + 32 + kOutStageBytes;
  static constexpr int kTmemCols = 512;
  static_assert(kSmemBytes <= kMaxDynamicSmem, "prefill kernel: shared memory over the per-CTA limit");
};

struct PrefillUnit {
  int nt, pass, kt_begin, kt_end, tile_id;
};
__device__ __forceinline__ PrefillUnit prefill_unit(const FcParams& p, int u, int ksplit) {
  PrefillUnit w;
  const int ks = u % ksplit;
  w.tile_id = u / ksplit;
  w.pass = w.tile_id / p.n_tiles;
  w.nt = w.tile_id % p.n_tiles;
  w.kt_begin = (int)((long long)p.k_tiles * ks / ksplit);
  w.kt_end = (int)((long long)p.k_tiles * (ks + 1) / ksplit);
  return w;
}

template <int EPI>
__global__ void __launch_bounds__(PrefillLayout::kThreads, 1) fc_prefill_kernel(const FcParams p, const int units, const int ksplit) {
  using L = PrefillLayout;
  constexpr int NB = L::kNB;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kStages * L::kStageBytes);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* acc_full = empty_bar + L::kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  UmmaShared* sh = reinterpret_cast<UmmaShared*>(acc_empty + 2);
  uint8_t* out_stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sh + 1) + 15) & ~uintptr_t(15));
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
      mbar_init(&acc_empty[a], L::kEpiWarps);  // one arrival per epilogue warp
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
  const int m_groups_alloc = p.m_alloc / 8;

  if (warp == 0) {
    if (lane == 0) {
      pdl_launch_dependents();
      const uint64_t stream_policy = l2_policy_evict_first();
      pdl_wait();
      uint32_t it = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const PrefillUnit w = prefill_unit(p, u, ksplit);
        const int mg_base = w.pass * (NB / 8);
        for (int kt = w.kt_begin; kt < w.kt_end; ++kt, ++it) {
          const int s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
          uint8_t* dst = smem + (size_t)s * L::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[s], (uint32_t)L::kStageBytes);
          bulk_g2s_hint(dst, p.w_packed + ((size_t)w.nt * p.k_tiles + kt) * kTileBytes, kTileBytes, &full_bar[s], stream_policy);
          const size_t off = (((size_t)kt * m_groups_alloc) + mg_base) * 1024;
          bulk_g2s(dst + kTileBytes, p.q_tiled + off, L::kQBytes, &full_bar[s]);
        }
      }
      const uint32_t issued = it;  // never leave with copies in flight (only possible after an abort)
      for (uint32_t back = 0; back < (uint32_t)L::kStages && back < issued; ++back) {
        const uint32_t j = issued - 1 - back;
        mbar_wait_bounded(&full_bar[j % L::kStages], (j / L::kStages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_s8(NB);
      uint32_t it = 0, done = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x, ++done) {
        const PrefillUnit w = prefill_unit(p, u, ksplit);
        const uint32_t ab = done & 1u, use = done >> 1;
        // the accumulator is free once the epilogue has drained the unit before the previous one
        mbar_wait_bounded(&acc_empty[ab], (use & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * NB;
        for (int kt = w.kt_begin; kt < w.kt_end; ++kt, ++it) {
          const int s = it % L::kStages;
          const uint32_t ph = (it / L::kStages) & 1u;
          mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.status, kStatusWaitTimeoutFull);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * L::kStageBytes);
          const uint32_t b_addr = a_addr + kTileBytes;
#pragma unroll
          for (int ks = 0; ks < kTileK8 / 32; ++ks) {
            umma_s8(d_tmem, umma_smem_desc(a_addr + ks * 32), umma_smem_desc(b_addr + ks * 32), idesc,
                    (kt == w.kt_begin && ks == 0) ? 0u : 1u);
          }
          umma_commit(&empty_bar[s]);
        }
        umma_commit(&acc_full[ab]);
      }
      // wait for the last accumulators to be complete before the CTA tears TMEM down
      for (uint32_t back = 0; back < 2 && back < done; ++back) {
        const uint32_t i = done - 1 - back;
        mbar_wait_bounded(&acc_full[i & 1u], (i >> 1) & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      }
    }
  } else {
    // eight epilogue warps: the TMEM lane quarter is warp % 4; the two warps of a quarter split the rows
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int half = (warp - 2) >> 2;
    const int etid = (tid - 64) & 127;   // thread index within the half
    const int etid_all = tid - 64;
    constexpr int kHalfThreads = 128;
    constexpr int kAllEpi = L::kEpiWarps * 32;
    constexpr int kElem = EPI == kEpiRequantI8 ? 1 : 4;
    const bool plain = plain_epilogue<EPI>(p);
    pdl_wait();
    uint32_t done = 0;
    int staged_pass = -1;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++done) {
      const PrefillUnit w = prefill_unit(p, u, ksplit);
      const int m_base = w.pass * NB;
      const int m_valid = p.m - m_base < NB ? p.m - m_base : NB;
      const uint32_t ab = done & 1u, use = done >> 1;
      if (w.pass != staged_pass) {  // per-row scale and zero point (or row sum) of this pass
        named_barrier(1, kAllEpi);
        for (int i = etid_all; i < NB; i += kAllEpi) {
          const int m = m_base + i;
          const bool ok = m < p.m;
          sh->in_scale[i] = (ok && p.in_scales) ? p.in_scales[m] : 0.0f;
          if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
            sh->in_aux[i] = (ok && p.in_zps) ? p.in_zps[m] : 0;
          } else {
            sh->in_aux[i] = (ok && p.x_sums) ? p.x_sums[m] : 0;
          }
        }
        named_barrier(1, kAllEpi);
        staged_pass = w.pass;
      }
      int32_t rs = 0, base_i = 0, mult = 0, shift = 0;
      float wsc = 0.0f, bias_f = 0.0f;
      const int n0 = w.nt * kTileN;
      const int n = n0 + row_in_tile;
      const bool n_ok = n < p.n;
      if (n_ok) {
        rs = p.row_sums ? p.row_sums[n] : 0;
        if constexpr (EPI == kEpiHybridF32 || EPI == kEpiHybridPick) {
          wsc = p.per_channel ? p.w_scales[n] : p.w_scales[0];
          bias_f = p.bias_f32 ? p.bias_f32[n] : 0.0f;
        } else {
          base_i = p.input_offset * rs + p.k * p.filter_offset * p.input_offset + (p.bias_i32 ? p.bias_i32[n] : 0);
          if (p.multipliers) {
            mult = p.multipliers[p.per_channel ? n : 0];
            shift = p.shifts[p.per_channel ? n : 0];
          }
        }
      }
      // sixteen outputs of this thread's channel, activation rows m0 .. m0 + 15, from their exact dot products
      auto finish16 = [&](const int (&r)[16], int m0, uint8_t* st) {
        float sc[16];
        int32_t ax[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          sc[e] = sh->in_scale[m0 + e];
          ax[e] = sh->in_aux[m0 + e];
        }
        if constexpr (kElem == 4) {
          int32_t* ycol = static_cast<int32_t*>(p.y) + (size_t)m_base * p.n + n;
          if (plain) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int32_t v = compute_output<EPI, true>(p, r[e], rs, wsc, bias_f, base_i, mult, shift, sc[e], ax[e]);
              if (n_ok && m0 + e < m_valid) ycol[(size_t)(m0 + e) * p.n] = v;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int32_t v = compute_output<EPI>(p, r[e], rs, wsc, bias_f, base_i, mult, shift, sc[e], ax[e]);
              if (n_ok && m0 + e < m_valid) ycol[(size_t)(m0 + e) * p.n] = v;
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            reinterpret_cast<int8_t*>(st)[e * kTileN + row_in_tile] =
                (int8_t)compute_output<EPI>(p, r[e], rs, wsc, bias_f, base_i, mult, shift, sc[e], ax[e]);
        }
      };
      // int8 outputs: the staged 16 x 128 block leaves as whole 128-byte row segments, 16 bytes per thread
      auto flush_block = [&](const uint8_t* st, int m0) {
        constexpr int kChunksPerRow = kTileN * kElem / 16;
        constexpr int kPieces = 16 * kChunksPerRow;
        const bool vec_ok = (((size_t)p.n * kElem) % 16 == 0) && (n0 + kTileN <= p.n) &&
                            ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
        for (int i = etid; i < kPieces; i += kHalfThreads) {
          const int rr = i / kChunksPerRow, cc = i % kChunksPerRow;
          const int m = m0 + rr;
          if (m >= m_valid) continue;
          uint8_t* dst = static_cast<uint8_t*>(p.y) + ((size_t)(m_base + m) * p.n + n0) * kElem + cc * 16;
          const uint8_t* src = st + (size_t)rr * kTileN * kElem + cc * 16;
          if (vec_ok) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
          } else {
            for (int bb = 0; bb < 16; ++bb)
              if (n0 + (cc * 16 + bb) / kElem < p.n) dst[bb] = src[bb];
          }
        }
      };
      mbar_wait_bounded(&acc_full[ab], use & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      tc_fence_after();
      const uint32_t taddr = tmem_base + ab * NB + ((uint32_t)(quarter * 32) << 16);
      const int c_begin = half * (NB / 2), c_end = min((half + 1) * (NB / 2), m_valid);
      if (ksplit == 1) {
#pragma unroll 1
        for (int m0 = c_begin; m0 < c_end; m0 += 32) {
          int ra[16], rb[16];
          tmem_ld16(taddr + m0, ra);  // both loads in flight before the first wait
          tmem_ld16(taddr + m0 + 16, rb);
          tmem_ld_wait();
          uint8_t* st = out_stage + (half * 2 + ((m0 >> 5) & 1)) * (16 * kTileN * 4);
          finish16(ra, m0, st);
          if constexpr (kElem != 4) {
            named_barrier(2 + half, kHalfThreads);  // the block is complete
            flush_block(st, m0);
            named_barrier(2 + half, kHalfThreads);  // ... and read, before it is rewritten
          }
          if (m0 + 16 < c_end) {
            finish16(rb, m0 + 16, st);
            if constexpr (kElem != 4) {
              named_barrier(2 + half, kHalfThreads);
              flush_block(st, m0 + 16);
              named_barrier(2 + half, kHalfThreads);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      } else {
        // this unit's raw sums to its scratch slot (coalesced: a warp writes 32 consecutive channels of a row)
        int32_t* mine = p.ws_part + (size_t)u * kZeroWsSlotInts;
#pragma unroll 1
        for (int m0 = c_begin; m0 < c_end; m0 += 32) {
          int ra[16], rb[16];
          tmem_ld16(taddr + m0, ra);
          tmem_ld16(taddr + m0 + 16, rb);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            __stcg(&mine[(m0 + e) * kTileN + row_in_tile], ra[e]);
            __stcg(&mine[(m0 + 16 + e) * kTileN + row_in_tile], rb[e]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
        named_barrier(1, kAllEpi);
        if (etid_all == 0) {
          __threadfence();
          const int old = atomicAdd(&p.ws_count[w.tile_id], 1);
          sh->last = (old + 1 == ksplit) ? 1 : 0;
        }
        named_barrier(1, kAllEpi);
        if (sh->last) {
          __threadfence();
          const int32_t* first = p.ws_part + (size_t)w.tile_id * ksplit * kZeroWsSlotInts + row_in_tile;
#pragma unroll 1
          for (int m0 = c_begin; m0 < c_end; m0 += 16) {
            int r[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) r[e] = 0;
            for (int ks = 0; ks < ksplit; ++ks) {
#pragma unroll
              for (int e = 0; e < 16; ++e) r[e] += __ldcg(first + (size_t)ks * kZeroWsSlotInts + (m0 + e) * kTileN);
            }
            uint8_t* st = out_stage + (half * 2) * (16 * kTileN * 4);
            finish16(r, m0, st);
            if constexpr (kElem != 4) {
              named_barrier(2 + half, kHalfThreads);
              flush_block(st, m0);
              named_barrier(2 + half, kHalfThreads);
            }
          }
          if (etid_all == 0) p.ws_count[w.tile_id] = 0;
        }
        named_barrier(1, kAllEpi);  // sh->last is rewritten by the next unit
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::kTmemCols);
}

template <int EPI>
cudaError_t launch_prefill(const FcParams& p, cudaStream_t s) {
  using L = PrefillLayout;
  static bool configured[64] = {false};
  auto kernel = fc_prefill_kernel<EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int passes = (p.m + L::kNB - 1) / L::kNB;
  const int sms = device_sm_count();
  const int tiles = p.n_tiles * passes;
  // few tiles, a long reduction: cut it so that most SMs get a unit (at least 16 k tiles per range)
  int ksplit = 1;
  if (tiles * 2 <= sms && p.k_tiles >= 32) {
    ksplit = sms / tiles;
    if (ksplit > p.k_tiles / 16) ksplit = p.k_tiles / 16;
    while (ksplit > 1 && tiles * ksplit > kZeroWsSlots) --ksplit;
    if (ksplit < 1) ksplit = 1;
  }
  if (const char* e = tuning_env("B200_FC_KSPLIT")) ksplit = atoi(e) > 0 ? atoi(e) : ksplit;  // measurement knob
  const int units = tiles * ksplit;
  const int ctas = units < sms ? units : sms;
  return launch_chained(kernel, dim3(ctas), dim3(L::kThreads), (size_t)L::kSmemBytes, s, p, units, ksplit);
}

// Chooses the number of CTAs and the split for one launch (measured on B200, batch 1, graph
// replays): with at least half as many n tiles as SMs, whole n tiles per CTA win (no cross-CTA
// reduction; CTAs with one tile fewer finish early and the kernel stays HBM-bound); with fewer,
// one SM per n tile cannot pull more than ~80 GB/s, so the flat (n tile, k tile) sequence is cut
// into equal ranges over all SMs (stream-K) and the partials are merged by the last arriver.
int plan_ctas(FcParams* p, int passes, int ctas_per_sm) {
  const int sms = device_sm_count();
  const long long total = (long long)p->n_tiles * p->k_tiles;
  int mode = -1;  // -1 auto, 0 stream-K, 1 whole tiles
  if (const char* e = tuning_env("B200_FC_SPLIT")) mode = atoi(e) ? 0 : 1;  // measurement knob
  int ctas;
  if (p->split_passes && passes > 1 && mode != 1) {
    // few n tiles, a long reduction, several passes of activation rows: the SMs are shared out
    // among the passes and each pass cuts its (n tile, k tile) sequence into equal ranges
    p->whole_tiles = 0;
    ctas = (sms < kZeroWsSlots / 2 ? sms : kZeroWsSlots / 2) / passes;
  } else if (mode == 1 || passes > 1 || p->force_whole_tiles || (mode < 0 && p->n_tiles * 2 >= sms)) {
    // (several passes otherwise share one launch as whole n tiles: no cross-CTA reduction)
    p->whole_tiles = 1;
    const int cap = passes > 1 ? sms : sms * ctas_per_sm;
    ctas = p->n_tiles < cap ? p->n_tiles : cap;
  } else {
    p->whole_tiles = 0;
    ctas = sms * ctas_per_sm;
  }
  if (p->max_ctas > 0) ctas = p->max_ctas;
  if (const char* e = tuning_env("B200_FC_MAX_CTAS")) {  // measurement knob
    const int v = atoi(e);
    if (v > 0) ctas = v;
  }
  if (!p->whole_tiles && ctas * passes > kZeroWsSlots / 2) ctas = kZeroWsSlots / 2 / passes;  // two scratch slots per CTA
  if (p->whole_tiles && ctas > p->n_tiles) ctas = p->n_tiles;
  if (ctas > total) ctas = (int)total;
  if (ctas < 1) ctas = 1;
  return ctas;
}

template <int NB, int EPI>
cudaError_t launch_umma_one(const FcParams& p, int m_base, int passes, cudaStream_t s) {
  using L = UmmaLayout<NB>;
  static bool configured[64] = {false};
  auto kernel = fc_umma_kernel<NB, EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  FcParams q = p;
  const int ctas = plan_ctas(&q, passes, UmmaBudget<NB>::kCtasPerSm);
  size_t smem = (size_t)L::kSmemBytes;
  if (p.prologue) {
    if (!fc_prologue_supported(p.m, p.k) || NB != 16 || m_base != 0) return cudaErrorInvalidValue;
    smem += (size_t)p.k_tiles * L::kQBytes;
  }
  return launch_chained(kernel, dim3(ctas, passes), dim3(kUmmaThreads), smem, s, q, m_base);
}

template <int EPI>
cudaError_t launch_umma_nb(const FcParams& p, int m_base, int nb, int passes, cudaStream_t s) {
  switch (nb) {
    case 16: return launch_umma_one<16, EPI>(p, m_base, passes, s);
    case 32: return launch_umma_one<32, EPI>(p, m_base, passes, s);
    case 64: return launch_umma_one<64, EPI>(p, m_base, passes, s);
    case 128: return launch_umma_one<128, EPI>(p, m_base, passes, s);
    default: return launch_umma_one<256, EPI>(p, m_base, passes, s);
  }
}

// Largest split of {8, 4, 2} whose clusters all fit on the device at once, 0 when the shape is
// better served by the kernels above (many n tiles, or a single k tile).
template <int NB, int EPI>
int plan_cluster_split(const FcParams& p) {
  if (const char* e = tuning_env("B200_FC_CLUSTER"))  // measurement knob: 0 turns the cluster kernel off
    if (e[0] == '0') return 0;
  const int sms = device_sm_count();
  if (p.n_tiles * 2 >= sms || p.k_tiles < 2) return 0;
  using L = ClusterLayout<NB>;
  auto kernel = fc_cluster_kernel<NB, EPI>;
  static int capacity[64][17] = {{0}};  // [device][split]: co-resident clusters, -1 = query failed
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    configured[dev] = true;
  }
  if (const char* e = tuning_env("B200_FC_CLUSTER")) {  // measurement knob: force a split
    const int v = atoi(e);
    if (v >= 2 && v <= 16 && v <= p.k_tiles) {
      // beyond 8 the cluster size is "non-portable": the kernel has to opt in
      static bool opted[64] = {false};
      if (v > 8 && !opted[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
          cudaGetLastError();
          return 0;
        }
        opted[dev] = true;
      }
      return v;
    }
  }
  // co-resident clusters of `split` CTAs (one CTA per SM counted), -1 = the query failed
  auto clusters_resident = [&](int split) {
    if (capacity[dev][split] == 0) {
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(split * 16);
      cfg.blockDim = dim3(kUmmaThreads);
      cfg.dynamicSmemBytes = L::kSmemBytes + 4 * L::kQBytes;  // as with the fused prologue's operand buffer
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = split;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = -1;
      }
      capacity[dev][split] = n;
      if (tuning_env("B200_FC_VERBOSE")) fprintf(stderr, "[b200] cluster size %d: %d clusters resident (NB=%d)\n", split, n, NB);
    }
    return capacity[dev][split];
  };
  // A long reduction over few n tiles (a decoder's down projection: 16 n tiles x 128 k tiles) does better
  // with more CTAs than SMs: clusters of 12 (beyond the portable 8: the kernel opts in), two CTAs on some
  // SMs, more copies in flight per SM. Measured on B200, n = 2048, k = 16384, one row, inside the decode
  // step: 8.3 us with clusters of 8 (128 CTAs), 7.9 / 7.1 / 6.7 / 6.2 / 6.9 us with 9 / 10 / 11 / 12 / 13,
  // 12 us with 14 to 16.
  {
    int big = 12;
    if (const char* e = tuning_env("B200_FC_CLUSTER_BIG")) big = atoi(e);  // measurement knob (0 = off)
    if (big > 8 && big <= 16 && p.k_tiles >= 8 * big && p.n_tiles * big <= 2 * sms && UmmaBudget<NB>::kCtasPerSm >= 2) {
      static bool opted[64] = {false};
      if (!opted[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
          opted[dev] = true;
        } else {
          cudaGetLastError();
        }
      }
      if (opted[dev] && clusters_resident(big) > 0) return big;
    }
  }
  // the split that puts the most SMs to work with every cluster resident at once
  int best = 0;
  for (int split = 8; split >= 2; --split) {
    if (split > p.k_tiles || p.n_tiles * split > sms) continue;
    // (the query counts one CTA per SM; CTAs this small share an SM, and clusters beyond the
    // resident ones simply start as earlier ones finish: nothing waits across clusters)
    if (clusters_resident(split) * UmmaBudget<NB>::kCtasPerSm >= p.n_tiles) {
      best = split;
      break;
    }
  }
  return best;
}

template <int NB, int EPI>
cudaError_t launch_cluster_one(const FcParams& p, int m_base, int split, cudaStream_t s) {
  using L = ClusterLayout<NB>;
  size_t smem = (size_t)L::kSmemBytes;
  if (p.prologue) {
    if (!fc_prologue_supported(p.m, p.k) || NB != 16 || m_base != 0) return cudaErrorInvalidValue;
    smem += (size_t)((p.k_tiles + split - 1) / split + 1) * L::kQBytes;
  }
  if (p.push_ranks > 1 && (EPI != kEpiHybridF32 || m_base != 0 || !p.push_step_epoch)) return cudaErrorInvalidValue;
  return launch_chained_cluster(fc_cluster_kernel<NB, EPI>, dim3(p.n_tiles * split), dim3(kUmmaThreads), smem, split, s,
                                p, m_base, split);
}

// One pass of nb <= 64 activation rows: the cluster kernel when the shape suits it. Returns
// cudaErrorNotSupported when the caller should use the stream-K kernel instead.
template <int EPI>
cudaError_t try_cluster_pass(const FcParams& p, int m_base, int nb, cudaStream_t s) {
  int split = 0;
  switch (nb) {
    case 16:
      split = plan_cluster_split<16, EPI>(p);
      return split ? launch_cluster_one<16, EPI>(p, m_base, split, s) : cudaErrorNotSupported;
    case 32:
      split = plan_cluster_split<32, EPI>(p);
      return split ? launch_cluster_one<32, EPI>(p, m_base, split, s) : cudaErrorNotSupported;
    case 64:
      split = plan_cluster_split<64, EPI>(p);
      return split ? launch_cluster_one<64, EPI>(p, m_base, split, s) : cudaErrorNotSupported;
    default:
      return cudaErrorNotSupported;
  }
}

template <int EPI>
cudaError_t launch_all(const FcParams& p, cudaStream_t s) {
  int nb = umma_rows_per_pass(p.m);
  if (nb <= 64) {  // decode-sized: one pass, cluster split-K where the shape suits it
    const cudaError_t e = try_cluster_pass<EPI>(p, 0, nb, s);
    if (e != cudaErrorNotSupported) return e;
    if (p.push_ranks > 1) return cudaErrorInvalidValue;  // only the cluster kernel pushes its outputs to the peers
    return launch_umma_nb<EPI>(p, 0, nb, 1, s);
  }
  if (p.push_ranks > 1) return cudaErrorInvalidValue;
  const int sms = device_sm_count();
  if (p.m <= 128 && p.n_tiles * 2 < sms && p.m_alloc % 64 == 0) {
    // a little over one decode pass, few n tiles: 64 rows at a time through the cluster kernel
    for (int m_base = 0; m_base < p.m; m_base += 64) {
      const cudaError_t e = try_cluster_pass<EPI>(p, m_base, 64, s);
      if (e == cudaErrorNotSupported && m_base == 0) break;
      if (e != cudaSuccess) return e;
      if (m_base + 64 >= p.m) return cudaSuccess;
    }
  }
  // Prefill-sized: persistent CTAs over (n tile, pass of 256 activation rows) units. (Passes of 128 rows
  // through the decode kernel, which give twice the CTAs when there are few n tiles, measured no faster
  // for any shape once the epilogue stopped being the limit: 10.4 against 22.5 us at m = 1024, n = 2560,
  // k = 2048.) B200_FC_NB=128 keeps that launch for measurements.
  if (const char* e = tuning_env("B200_FC_NB")) {  // measurement knob
    const int v = atoi(e);
    if (v == 128 || v == 256) nb = v;
  }
  if (p.m_alloc % nb != 0) return cudaErrorInvalidValue;
  if (nb == 256) return launch_prefill<EPI>(p, s);
  const int passes = (p.m + nb - 1) / nb;
  FcParams q = p;
  // Whole n tiles per CTA. B200_FC_SPLIT_PASSES=1 (measurement knob) instead shares the SMs out among
  // the passes and splits each pass's reduction (stream-K): measured slower on B200 for the shapes
  // that leave SMs idle here (prompt chunk of 512 rows; qkv / o / down projections 26 / 17 / 77 us as
  // whole tiles, 57 us on average when split): the merge of 128-row partials through memory costs
  // more than the idle SMs.
  q.split_passes = 0;
  if (const char* e = tuning_env("B200_FC_SPLIT_PASSES")) q.split_passes = atoi(e) ? 1 : 0;
  q.force_whole_tiles = q.split_passes ? 0 : 1;
  return launch_umma_nb<EPI>(q, 0, nb, passes, s);
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

int fc_argmax_ctas(int n) {
  const int sms = device_sm_count();
  return std::min(tiles_n(n), sms * UmmaBudget<16>::kCtasPerSm);
}

bool fc_cluster_planned(int m, int n, int k) {
  if (m < 1 || m > 16) return false;
  FcParams p;
  memset(&p, 0, sizeof(p));
  p.m = m, p.n = n, p.k = k;
  p.n_tiles = tiles_n(n);
  p.k_tiles = tiles_k8(k);
  return plan_cluster_split<16, kEpiHybridF32>(p) != 0;
}

bool fc_prologue_supported(int m, int k) { return m >= 1 && m <= kPrologueMaxM && k >= 1 && k <= kPrologueMaxK; }

int umma_rows_per_pass(int m) {
  int nb = 16;
  while (nb < m && nb < 256) nb *= 2;
  return nb;
}

// The hybrid projection with the greedy pick in its epilogue: one pass of up to 16 rows, whole n tiles per
// CTA, one candidate slot per CTA and row.
static cudaError_t launch_pick(const FcParams& p, cudaStream_t s) {
  if (umma_rows_per_pass(p.m) != 16 || !p.argmax_val || !p.argmax_idx) return cudaErrorInvalidValue;
  FcParams q = p;
  q.force_whole_tiles = 1;
  if (fc_argmax_ctas(q.n) > q.argmax_parts) return cudaErrorInvalidValue;
  return launch_umma_one<16, kEpiHybridPick>(q, 0, 1, s);
}

cudaError_t launch_fc_i8_umma(const FcParams& p, FcEpilogue epi, cudaStream_t s) {
  if (epi == kEpiHybridPick) return launch_pick(p, s);
  if (epi == kEpiHybridF32) return launch_all<kEpiHybridF32>(p, s);
  if (epi == kEpiRequantI8) return launch_all<kEpiRequantI8>(p, s);
  return launch_all<kEpiRawI32>(p, s);
}

}  // namespace b200
