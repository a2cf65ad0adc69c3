// Blockwise 4-bit weights on the 5th-generation tensor cores:
// Y[m,n] = (sum_k (W4[n,k] * scale[n, k/32]) * Q[m,k] - zp[m] * kfsum[n]) * in_scale[m] + bias[n]
// (tflite/kernels/fully_connected.cc:1014-1086), with the accumulators in TMEM.
//
// The per-block scales rule out an integer accumulator that runs over the whole reduction, and
// reading one out of TMEM for every block of 32 would cost far more than the MMAs. So the scales
// are folded into the weights on their way to the tensor core: converter warps turn each 4-bit
// weight into the fp16 number RN(w * scale) (both factors are exact in fp16; the product is rounded
// once, relative error at most 2^-11), written straight into the 128-byte-swizzled K-major operand
// tile; the activations travel as the fp16 images of their int8 quantization (exact), and
// tcgen05.mma kind::f16 accumulates in fp32. The result differs from the reference's block-by-block
// float sums by rounding noise of a few 1e-4 of the output's magnitude.
//
// Roles inside a CTA (one CTA per SM, 512 threads):
//   warp 0, one lane   weight producer: linear bulk copies of 18 KiB packed tiles (256 reduction
//                      elements of 128 output channels: nibbles + block scales) into a ring;
//                      the weights are constants, so this runs ahead of the kernel's dependencies;
//   warp 2, one lane   activation producer: one fp16 tile (NB rows x 64 reduction elements) per step;
//   warps 8..15        converters: nibbles -> scaled fp16 operand tile (128 x 64), one per step;
//   warp 1, one lane   MMA issuer: four tcgen05.mma (M = 128 output channels, N = NB activation
//                      rows, K = 16) per step; tcgen05.commit frees the step's tiles;
//   warps 4..7         epilogue: TMEM -> registers -> zero-point term, row scale, bias -> global.
// Work units are (n tile, pass of NB activation rows, k range); CTAs take units round-robin. With
// few n tiles the reduction is cut into `ksplit` ranges whose fp32 partials meet in a scratch slot
// per unit; the CTA that completes a tile's count adds them in range order, so the result does not
// depend on timing. Every wait is bounded; TMEM is always freed.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

namespace {

constexpr int kW4Threads = 512;
constexpr int kW4ConvWarps = 8;
constexpr int kW4EpiThreads = 128;
constexpr int kW4ATileBytes = kTileN * 128;  // 128 channels x 64 fp16

template <int NB>
struct W4Layout {
  static constexpr int kBBytes = NB * 128;  // NB rows x 64 fp16
  static constexpr int kRawStages = NB <= 16 ? 8 : (NB <= 32 ? 6 : (NB <= 64 ? 4 : 2));
  static constexpr int kBStages = NB <= 128 ? 8 : 4;
  static constexpr int kAStages = NB <= 64 ? 3 : 2;
  static constexpr int kAOff = 0;
  static constexpr int kBOff = kAOff + kAStages * kW4ATileBytes;
  static constexpr int kRawOff = kBOff + kBStages * kBBytes;
  static constexpr int kBarOff = kRawOff + kRawStages * kTile4Bytes;
  static constexpr int kBarriers = 2 * (kRawStages + kBStages + kAStages) + 4;
  static constexpr int kSharedOff = kBarOff + kBarriers * 8;
  static constexpr int kTmemCols = 2 * NB < 32 ? 32 : 2 * NB;
};

struct W4Shared {
  uint32_t tmem_base;
  int abort_flag;
  int last;
  int pad;
  float in_scale[256];
  float in_zp[256];
};

template <int NB>
constexpr int w4_smem_bytes() {
  return W4Layout<NB>::kSharedOff + (int)sizeof(W4Shared) + 1024;  // + alignment slack
}

// Instruction descriptor, kind::f16: f16 x f16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int n) {
  return (1u << 4) /* D = f32 */ | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Makes this thread's ordinary shared-memory writes visible to the tensor core's (async proxy) reads.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

struct W4Unit {
  int nt, pass, kt_begin, kt_end;  // k range in 256-element tiles
};
__device__ __forceinline__ W4Unit w4_unit(const FcParams& p, int u, int ksplit) {
  W4Unit w;
  const int ks = u % ksplit, rest = u / ksplit;
  w.nt = rest % p.n_tiles;
  w.pass = rest / p.n_tiles;
  w.kt_begin = (int)((long long)p.k_tiles * ks / ksplit);
  w.kt_end = (int)((long long)p.k_tiles * (ks + 1) / ksplit);
  return w;
}

// Eight 4-bit weights of one row (one packed word) times their block scale -> eight fp16.
__device__ __forceinline__ uint4 w4_convert_word(uint32_t word, __half2 scale2) {
  const __half2 bias = __floats2half2_rn(1032.0f, 1032.0f);  // 1024 from the exponent trick + 8 offset binary
  uint32_t out[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t bits = ((word >> (4 * q)) & 0x000F000Fu) | 0x64006400u;  // the halves 1024 + u
    const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&bits), bias), scale2);
    out[q] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

template <int NB>
__global__ void __launch_bounds__(kW4Threads, 1) fc_w4_umma_kernel(const FcParams p, const int units, const int ksplit) {
  using L = W4Layout<NB>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* raw_empty = raw_full + L::kRawStages;
  uint64_t* b_full = raw_empty + L::kRawStages;
  uint64_t* b_empty = b_full + L::kBStages;
  uint64_t* a_full = b_empty + L::kBStages;
  uint64_t* a_empty = a_full + L::kAStages;
  uint64_t* acc_full = a_empty + L::kAStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  W4Shared* sh = reinterpret_cast<W4Shared*>(smem + L::kSharedOff);
  volatile int* abort_flag = &sh->abort_flag;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < L::kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], kW4ConvWarps);
    }
    for (int s = 0; s < L::kBStages; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 1);
    }
    for (int s = 0; s < L::kAStages; ++s) {
      mbar_init(&a_full[s], kW4ConvWarps);
      mbar_init(&a_empty[s], 1);
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
  const int m_groups_alloc = p.m_alloc / 8;

  if (warp == 0) {
    // ---------------- weight producer ----------------
    if (lane == 0) {
      pdl_launch_dependents();
      const uint64_t stream_policy = l2_policy_evict_first();
      uint32_t it = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const W4Unit w = w4_unit(p, u, ksplit);
        for (int kt = w.kt_begin; kt < w.kt_end; ++kt, ++it) {
          const int s = it % L::kRawStages;
          mbar_wait_bounded(&raw_empty[s], ((it / L::kRawStages) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
          mbar_arrive_expect_tx(&raw_full[s], (uint32_t)kTile4Bytes);
          bulk_g2s_hint(smem + L::kRawOff + (size_t)s * kTile4Bytes,
                        p.w_packed + ((size_t)w.nt * p.k_tiles + kt) * kTile4Bytes, kTile4Bytes, &raw_full[s], stream_policy);
        }
      }
      // never leave with copies in flight (only possible after an abort)
      for (uint32_t back = 0; back < (uint32_t)L::kRawStages && back < it; ++back) {
        const uint32_t j = it - 1 - back;
        mbar_wait_bounded(&raw_full[j % L::kRawStages], (j / L::kRawStages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
      }
    }
  } else if (warp == 2) {
    // ---------------- activation producer ----------------
    if (lane == 0) {
      pdl_wait();
      uint32_t it = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const W4Unit w = w4_unit(p, u, ksplit);
        const int mg_base = w.pass * (NB / 8);
        for (int k64 = w.kt_begin * 4; k64 < w.kt_end * 4; ++k64, ++it) {
          const int s = it % L::kBStages;
          mbar_wait_bounded(&b_empty[s], ((it / L::kBStages) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
          mbar_arrive_expect_tx(&b_full[s], (uint32_t)L::kBBytes);
          const size_t off = (((size_t)k64 * m_groups_alloc) + mg_base) * 1024;
          bulk_g2s(smem + L::kBOff + (size_t)s * L::kBBytes, reinterpret_cast<const uint8_t*>(p.q_tiled) + off, L::kBBytes,
                   &b_full[s]);
        }
      }
      for (uint32_t back = 0; back < (uint32_t)L::kBStages && back < it; ++back) {
        const uint32_t j = it - 1 - back;
        mbar_wait_bounded(&b_full[j % L::kBStages], (j / L::kBStages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(NB);
      uint32_t it = 0, done = 0;
      for (int u = blockIdx.x; u < units; u += gridDim.x, ++done) {
        const W4Unit w = w4_unit(p, u, ksplit);
        const uint32_t ab = done & 1u;
        mbar_wait_bounded(&acc_empty[ab], ((done >> 1) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * NB;
        const int steps = (w.kt_end - w.kt_begin) * 4;
        for (int st = 0; st < steps; ++st, ++it) {
          const int sa = it % L::kAStages, sb = it % L::kBStages;
          mbar_wait_bounded(&a_full[sa], (it / L::kAStages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
          mbar_wait_bounded(&b_full[sb], (it / L::kBStages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + L::kAOff + (size_t)sa * kW4ATileBytes);
          const uint32_t b_addr = smem_u32(smem + L::kBOff + (size_t)sb * L::kBBytes);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            // 16 fp16 of the reduction per MMA: 32 B further along the swizzled rows
            umma_f16(d_tmem, umma_smem_desc(a_addr + ks * 32), umma_smem_desc(b_addr + ks * 32), idesc,
                     (st == 0 && ks == 0) ? 0u : 1u);
          }
          umma_commit(&a_empty[sa]);
          umma_commit(&b_empty[sb]);
        }
        umma_commit(&acc_full[ab]);
      }
      for (uint32_t back = 0; back < 2 && back < done; ++back) {
        const uint32_t i = done - 1 - back;
        mbar_wait_bounded(&acc_full[i & 1u], (i >> 1) & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      }
    }
  } else if (warp >= 8) {
    // ---------------- converters ----------------
    const int ctid = tid - 256;
    const int row = ctid & 127;
    const int blk = ctid >> 7;  // which block of 32 of the 64-element step: words 4*blk .. 4*blk+3
    uint32_t it_raw = 0, it_a = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const W4Unit w = w4_unit(p, u, ksplit);
      for (int kt = w.kt_begin; kt < w.kt_end; ++kt, ++it_raw) {
        const int sr = it_raw % L::kRawStages;
        mbar_wait_bounded(&raw_full[sr], (it_raw / L::kRawStages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
        const uint8_t* raw = smem + L::kRawOff + (size_t)sr * kTile4Bytes;
#pragma unroll 1
        for (int sub = 0; sub < 4; ++sub, ++it_a) {
          const uint8_t* rs = raw + sub * kTile4SubBytes;
          const uint4 w4 = reinterpret_cast<const uint4*>(rs)[blk * 128 + row];
          const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
          const __half sc = reinterpret_cast<const __half*>(rs + kTile4SubWordBytes)[blk * 128 + row];
          const __half2 sc2 = __half2half2(sc);
          uint4 vals[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) vals[j] = w4_convert_word(words[j], sc2);
          const int sa = it_a % L::kAStages;
          mbar_wait_bounded(&a_empty[sa], ((it_a / L::kAStages) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTimeoutEmpty);
          uint8_t* a_row = smem + L::kAOff + (size_t)sa * kW4ATileBytes + (row >> 3) * 1024;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(a_row + swz_chunk_offset(row & 7, blk * 4 + j)) = vals[j];
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[sa]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[sr]);
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue (warps 4..7) ----------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int etid = tid - 128;
    float* y = static_cast<float*>(p.y);
    pdl_wait();
    uint32_t done = 0;
    int staged_pass = -1;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++done) {
      const W4Unit w = w4_unit(p, u, ksplit);
      const int m_base = w.pass * NB;
      const int m_valid = p.m - m_base < NB ? p.m - m_base : NB;
      const uint32_t ab = done & 1u;
      if (w.pass != staged_pass) {
        named_barrier(1, kW4EpiThreads);
        for (int i = etid; i < NB; i += kW4EpiThreads) {
          const int m = m_base + i;
          sh->in_scale[i] = m < p.m ? p.in_scales[m] : 0.0f;
          sh->in_zp[i] = m < p.m ? (float)p.in_zps[m] : 0.0f;
        }
        named_barrier(1, kW4EpiThreads);
        staged_pass = w.pass;
      }
      const int n = w.nt * kTileN + row_in_tile;
      const bool row_ok = n < p.n;
      const float kf = row_ok ? p.kfsum[n] : 0.0f;
      const float bias = (row_ok && p.bias_f32) ? p.bias_f32[n] : 0.0f;
      const bool has_bias = p.bias_f32 != nullptr;
      // tflite/kernels/fully_connected.cc:1077-1082: subtract zp * kfsum, scale by the row, add the bias
      auto finish = [&](float acc, int mi) {
        float out = __fsub_rn(acc, __fmul_rn(sh->in_zp[mi], kf));
        out = __fmul_rn(out, sh->in_scale[mi]);
        if (has_bias) out = __fadd_rn(out, bias);
        return out;
      };
      mbar_wait_bounded(&acc_full[ab], (done >> 1) & 1u, abort_flag, p.status, kStatusWaitTimeoutTmem);
      tc_fence_after();
      const uint32_t taddr = tmem_base + ab * NB + ((uint32_t)(quarter * 32) << 16);
      if (ksplit == 1) {
#pragma unroll 1
        for (int c = 0; c < NB / 16; ++c) {
          if (c * 16 >= m_valid) break;
          int r[16];
          tmem_ld16(taddr + c * 16, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int mi = c * 16 + j;
              if (mi < m_valid) y[(size_t)(m_base + mi) * p.n + n] = finish(__int_as_float(r[j]), mi);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      } else {
        // this unit's partial sums to its scratch slot; whoever completes the tile's count adds the
        // ranges' slots in range order and finishes the outputs
        float* mine = reinterpret_cast<float*>(p.ws_part) + (size_t)u * kZeroWsSlotInts;
#pragma unroll 1
        for (int c = 0; c < NB / 16; ++c) {
          if (c * 16 >= m_valid) break;
          int r[16];
          tmem_ld16(taddr + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int mi = c * 16 + j;
            if (mi < m_valid) __stcg(&mine[mi * kTileN + row_in_tile], __int_as_float(r[j]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
        named_barrier(1, kW4EpiThreads);
        const int tile_id = u / ksplit;
        if (etid == 0) {
          __threadfence();
          const int old = atomicAdd(&p.ws_count[tile_id], 1);
          sh->last = (old + 1 == ksplit) ? 1 : 0;
        }
        named_barrier(1, kW4EpiThreads);
        if (sh->last) {
          __threadfence();
          const float* first = reinterpret_cast<const float*>(p.ws_part) + (size_t)tile_id * ksplit * kZeroWsSlotInts + row_in_tile;
          for (int m0 = 0; m0 < m_valid; m0 += 8) {
            float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            for (int ks = 0; ks < ksplit; ++ks) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (m0 + j < m_valid) v[j] = __fadd_rn(v[j], __ldcg(first + (size_t)ks * kZeroWsSlotInts + (m0 + j) * kTileN));
            }
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (m0 + j < m_valid) y[(size_t)(m_base + m0 + j) * p.n + n] = finish(v[j], m0 + j);
            }
          }
          if (etid == 0) p.ws_count[tile_id] = 0;
        }
        named_barrier(1, kW4EpiThreads);  // sh->last is rewritten by the next unit
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::kTmemCols);
}

template <int NB>
cudaError_t launch_w4_nb(const FcParams& p, cudaStream_t s) {
  static_assert(w4_smem_bytes<NB>() <= 227 * 1024, "4-bit GEMM: shared memory over the per-CTA limit");
  static bool configured[64] = {false};
  auto kernel = fc_w4_umma_kernel<NB>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, w4_smem_bytes<NB>());
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int sms = device_sm_count();
  const int passes = (p.m + NB - 1) / NB;
  const int tiles = p.n_tiles * passes;
  // few tiles: cut the reduction so that every SM streams a share of the weights
  int ksplit = 1;
  if (tiles * 2 <= sms) {
    ksplit = sms / tiles;
    if (ksplit > p.k_tiles) ksplit = p.k_tiles;
    while (ksplit > 1 && tiles * ksplit > kZeroWsSlots) --ksplit;
    if (ksplit < 1) ksplit = 1;
  }
  const int units = tiles * ksplit;
  const int ctas = units < sms ? units : sms;
  return launch_chained(kernel, dim3(ctas), dim3(kW4Threads), (size_t)w4_smem_bytes<NB>(), s, p, units, ksplit);
}

}  // namespace

int w4_rows_per_pass(int m) {
  int nb = 16;
  while (nb < m && nb < 256) nb *= 2;
  return nb;
}

cudaError_t launch_fc_w4(const FcParams& p, cudaStream_t s) {
  switch (w4_rows_per_pass(p.m)) {
    case 16: return launch_w4_nb<16>(p, s);
    case 32: return launch_w4_nb<32>(p, s);
    case 64: return launch_w4_nb<64>(p, s);
    case 128: return launch_w4_nb<128>(p, s);
    default: return launch_w4_nb<256>(p, s);
  }
}

}  // namespace b200
