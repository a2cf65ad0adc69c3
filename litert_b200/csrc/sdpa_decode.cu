// Flash-decode for odml.scaled_dot_product_attention with one query token per
// sequence: ragged key/value lengths, grouped-query heads, fp16 / int8 / fp32
// key-value caches, optional additive mask and logit cap.
//
// Math (tflite/experimental/genai/sdpa.cc:361-662): for each query head n of
// batch entry b, out = softmax_s(scale * q.k_s + mask_s) . v_s over the first
// len[b] cached tokens of kv head n / (N / Nkv).
//
// HBM-bound: every K and V row is read exactly once, straight from global
// memory into MMA fragments (no shared-memory staging, no transposes):
//  * the up-to-8 query heads sharing a kv head form the 8-wide MMA dimension,
//    16 cached tokens the 16-row one: S^T[token, head] = K[token, :] . Q^T.
//    K rows are the row-major A operand as they lie in memory; a thread's
//    16-byte load is two k-steps of its token row (the order of the head
//    dimension inside the dot product is permuted identically for Q);
//  * O^T[d, head] += V^T[d, token] . P^T[token, head]: the thread loads 16
//    consecutive head-dim elements of four token rows and pairs them up with
//    byte permutes into the A operand; P^T comes from the S^T accumulators via
//    one 8x8 matrix transpose per 8 tokens;
//  * tokens are split over CTAs (grid.x) and warps; every warp keeps an online
//    softmax state; warps merge in shared memory, CTAs through a small
//    workspace that a second kernel reduces.
#include <math_constants.h>

#include "common.cuh"
#include "kernels.h"
#include "quant.cuh"

namespace b200 {

namespace {

constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

enum : int { kKvF16 = 0, kKvI8 = 1, kKvF32 = 2 };

// Loads 8 consecutive head-dim elements of one cached row as four f16x2 words.
// SRC: where the row lives. kSrcGlobal: read-only path; kSrcGlobalCoherent: ordinary loads (the
// kernel itself wrote one of the rows earlier); kSrcShared: a shared-memory copy (ld.shared, free to
// be scheduled early: the copy does not change while it is read).
enum : int { kSrcGlobal = 0, kSrcGlobalCoherent = 1, kSrcShared = 2 };

__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ uint2 lds64(const void* p) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(smem_u32(p)));
  return v;
}

template <int KV, int SRC = kSrcGlobal>
__device__ __forceinline__ void load8(const void* row, int d0, bool valid, uint32_t (&out)[4]) {
  if (!valid) {
    out[0] = out[1] = out[2] = out[3] = 0u;
    return;
  }
  if constexpr (KV == kKvF16) {
    const uint4* ptr = reinterpret_cast<const uint4*>(static_cast<const __half*>(row) + d0);
    const uint4 v = SRC == kSrcShared ? lds128(ptr) : (SRC == kSrcGlobalCoherent ? *ptr : __ldg(ptr));
    out[0] = v.x;
    out[1] = v.y;
    out[2] = v.z;
    out[3] = v.w;
  } else if constexpr (KV == kKvI8) {
    const uint2* ptr = reinterpret_cast<const uint2*>(static_cast<const int8_t*>(row) + d0);
    const uint2 v = SRC == kSrcShared ? lds64(ptr) : (SRC == kSrcGlobalCoherent ? *ptr : __ldg(ptr));
    // int8 -> f16, exact: bias to unsigned, splice into 1024 + u, subtract 1152
    const uint32_t w[2] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u};
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t lo = __byte_perm(w[i], 0x64646464u, 0x4140);  // bytes: b0,0x64,b1,0x64
      uint32_t hi = __byte_perm(w[i], 0x64646464u, 0x4342);
      __half2 l = __hsub2(*reinterpret_cast<__half2*>(&lo), bias);
      __half2 h = __hsub2(*reinterpret_cast<__half2*>(&hi), bias);
      out[2 * i] = *reinterpret_cast<uint32_t*>(&l);
      out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(row) + d0));
    const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(row) + d0 + 4));
    __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
    __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
    out[0] = *reinterpret_cast<uint32_t*>(&h0);
    out[1] = *reinterpret_cast<uint32_t*>(&h1);
    out[2] = *reinterpret_cast<uint32_t*>(&h2);
    out[3] = *reinterpret_cast<uint32_t*>(&h3);
  }
}

template <int KV>
__device__ __forceinline__ size_t kv_elem_bytes() {
  return KV == kKvF16 ? 2 : (KV == kKvI8 ? 1 : 4);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t transpose8x8(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Partial record per (batch, kv head, chunk, head-in-group): H floats of
// un-normalised output followed by the running max (log2 domain) and sum.
__host__ __device__ inline size_t partial_stride(int h) { return (size_t)h + 2; }

// Attention of the warp's share of the tokens [c0, c1) of one (batch entry, kv head): online
// softmax state for heads 2t and 2t+1 (log2 domain) and the un-normalised outputs, in registers.
// GPI = groups of 16 tokens a warp takes per pass (1, 2 or 4): small for short caches, where the
// kernel is latency-bound and wants as many warps as possible, 4 for long ones.

template <int KV, int H, int GPI>
struct WarpAttention {
  static constexpr int DB = H < 128 ? H : 128;  // head-dim block of the PV step
  static constexpr int NBLK = H / DB;
  static constexpr int TPB = DB / 16;           // m16 tiles per block
  static constexpr int DPT = DB / 8;            // head-dim elements per thread per block (8 or 16)
  static constexpr int KSTEPS = H / 32;         // 16-byte K pieces per thread per row
  static constexpr int kTokensPerWarpIter = 16 * GPI;

  float m_run[2], l_run[2];
  float o[NBLK * TPB][4];

  __device__ __forceinline__ void clear() {
    m_run[0] = m_run[1] = -CUDART_INF_F;
    l_run[0] = l_run[1] = 0.0f;
#pragma unroll
    for (int i = 0; i < NBLK * TPB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  }

  // Where the rows come from: `k` / `v` point at token 0's row (global cache or a shared-memory
  // copy biased by the copy's first token), rows `stride` bytes apart; per-token scales (int8).
  struct Rows {
    const uint8_t* k;
    const uint8_t* v;
    size_t stride;
    const float* k_scale;
    const float* v_scale;
    int scale_stride;
  };
  static __device__ __forceinline__ Rows cache_rows(const SdpaParams& p, int b, int kvh) {
    Rows r;
    r.stride = (size_t)p.nkv * H * kv_elem_bytes<KV>();
    const size_t seq = p.shared_kv ? (size_t)0 : (size_t)(p.rows_per_kv > 1 ? b / p.rows_per_kv : b);
    const size_t first = seq * p.s_max * p.nkv + kvh;
    r.k = static_cast<const uint8_t*>(p.k) + first * H * kv_elem_bytes<KV>();
    r.v = static_cast<const uint8_t*>(p.v) + first * H * kv_elem_bytes<KV>();
    r.k_scale = p.k_scale ? p.k_scale + first : nullptr;
    r.v_scale = p.v_scale ? p.v_scale + first : nullptr;
    r.scale_stride = p.nkv;
    return r;
  }

  // Tokens first, first + step, ... (blocks of kTokensPerWarpIter) below `c1`.
    // `fresh` false continues the running softmax state of an earlier call; `finish` false leaves the
  // denominators per thread for a later call to complete (calls over consecutive pieces of a chunk).
  // EXTRAS false: the caller knows that there is neither a logit cap nor a mask, and the tests for them
  // leave the loop (a warp alone on its scheduler pays each branch's latency in full). Rows beyond c1 are
  // not skipped by a branch either: they read the last valid row, and their logits are set to -inf.
  template <int SRC, bool EXTRAS = true>
  __device__ __forceinline__ void run(const SdpaParams& p, const uint32_t (&qf)[KSTEPS][4], const Rows& rows_src, int b,
                                      int first, int step, int c1, int lane, bool fresh = true, bool finish = true) {
    const int g = lane >> 2, t = lane & 3;
    if (fresh) clear();
  const size_t row_stride = rows_src.stride;
  const uint8_t* kbase = rows_src.k;
  const uint8_t* vbase = rows_src.v;
  const float* ksc = rows_src.k_scale;
  const float* vsc = rows_src.v_scale;
  const int sc_stride = rows_src.scale_stride;
  const float* maskp = (EXTRAS && p.mask) ? p.mask + (size_t)b * p.s_max : nullptr;
  const int last_tok = c1 - 1;

  const float scale_log2 = p.scale * kLog2e;

  for (int base = first; base < c1; base += step) {
    // ---- S^T = K Q^T for GPI groups of 16 tokens ----
    float s[GPI][4];
#pragma unroll
    for (int gi = 0; gi < GPI; ++gi) {
      const int ta = base + gi * 16 + g, tb = ta + 8;
      const bool va = ta < c1, vb = tb < c1;
      const void* ra = kbase + (size_t)min(ta, last_tok) * row_stride;
      const void* rb = kbase + (size_t)min(tb, last_tok) * row_stride;
      // four independent accumulation chains: a chain of 2 * KSTEPS dependent MMAs would leave the
      // tensor pipe idle for its whole latency between steps
      float part[4][4];
#pragma unroll
      for (int c = 0; c < 4; ++c) part[c][0] = part[c][1] = part[c][2] = part[c][3] = 0.0f;
#pragma unroll
      for (int i = 0; i < KSTEPS; ++i) {
        uint32_t ka[4], kb[4];
        const int d0 = 8 * (t + 4 * i);
        load8<KV, SRC>(ra, d0, true, ka);
        load8<KV, SRC>(rb, d0, true, kb);
        mma_f16(part[(2 * i) & 3], ka[0], kb[0], ka[1], kb[1], qf[i][0], qf[i][1]);
        mma_f16(part[(2 * i + 1) & 3], ka[2], kb[2], ka[3], kb[3], qf[i][2], qf[i][3]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) s[gi][e] = (part[0][e] + part[1][e]) + (part[2][e] + part[3][e]);
      // scale (and dequantise), cap, mask; work in the log2 domain
      float fa = scale_log2, fb = scale_log2;
      if constexpr (KV == kKvI8) {
        fa *= va ? ksc[(size_t)ta * sc_stride] : 0.0f;
        fb *= vb ? ksc[(size_t)tb * sc_stride] : 0.0f;
      }
      s[gi][0] *= fa;
      s[gi][1] *= fa;
      s[gi][2] *= fb;
      s[gi][3] *= fb;
      if (EXTRAS && p.logit_cap > 0.0f) {
        const float c = p.logit_cap * kLog2e, ic = 1.0f / c;
#pragma unroll
        for (int e = 0; e < 4; ++e) s[gi][e] = c * tanhf(s[gi][e] * ic);
      }
      if (EXTRAS && maskp) {
        const float ma = va ? maskp[ta] * kLog2e : 0.0f, mb = vb ? maskp[tb] * kLog2e : 0.0f;
        s[gi][0] += ma;
        s[gi][1] += ma;
        s[gi][2] += mb;
        s[gi][3] += mb;
      }
      s[gi][0] = va ? s[gi][0] : -CUDART_INF_F;
      s[gi][1] = va ? s[gi][1] : -CUDART_INF_F;
      s[gi][2] = vb ? s[gi][2] : -CUDART_INF_F;
      s[gi][3] = vb ? s[gi][3] : -CUDART_INF_F;
    }
    // ---- online softmax over these tokens ----
    float mx[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float v = fmaxf(s[0][e], s[0][e + 2]);
#pragma unroll
      for (int gi = 1; gi < GPI; ++gi) v = fmaxf(v, fmaxf(s[gi][e], s[gi][e + 2]));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
      mx[e] = v;
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float m_new = fmaxf(m_run[e], mx[e]);
      m_use[e] = m_new == -CUDART_INF_F ? 0.0f : m_new;  // everything masked so far
      alpha[e] = exp2f(m_run[e] - m_use[e]);             // exp2(-inf) = 0 on the first pass
      m_run[e] = m_new;
      l_run[e] *= alpha[e];
    }
#pragma unroll
    for (int i = 0; i < NBLK * TPB; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[1];
      o[i][2] *= alpha[0];
      o[i][3] *= alpha[1];
    }
    // ---- O^T += V^T P^T ----
#pragma unroll
    for (int gi = 0; gi < GPI; ++gi) {
      float pa0 = exp2f(s[gi][0] - m_use[0]), pa1 = exp2f(s[gi][1] - m_use[1]);
      float pb0 = exp2f(s[gi][2] - m_use[0]), pb1 = exp2f(s[gi][3] - m_use[1]);
      l_run[0] += pa0 + pb0;
      l_run[1] += pa1 + pb1;
      if constexpr (KV == kKvI8) {
        const int ta = base + gi * 16 + g, tb = ta + 8;
        const float sa = ta < c1 ? vsc[(size_t)ta * sc_stride] : 0.0f;
        const float sb = tb < c1 ? vsc[(size_t)tb * sc_stride] : 0.0f;
        pa0 *= sa;
        pa1 *= sa;
        pb0 *= sb;
        pb1 *= sb;
      }
      // rows = tokens g (g+8), columns = heads 2t, 2t+1 -> transposed fragments
      const uint32_t pt0 = transpose8x8(pack_half2(pa0, pa1));  // head g; tokens 2t, 2t+1
      const uint32_t pt1 = transpose8x8(pack_half2(pb0, pb1));  // head g; tokens 2t+8, 2t+9
      const int r0 = base + gi * 16 + 2 * t;
      const int rows[4] = {r0, r0 + 1, r0 + 8, r0 + 9};
#pragma unroll
      for (int blk = 0; blk < NBLK; ++blk) {
        uint32_t vr[4][DPT / 2];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const void* row = vbase + (size_t)min(rows[r], last_tok) * row_stride;  // (its weight is 0 beyond c1)
          const bool ok = true;
#pragma unroll
          for (int hlf = 0; hlf < DPT / 8; ++hlf) {
            uint32_t tmp[4];
            load8<KV, SRC>(row, blk * DB + DPT * g + 8 * hlf, ok, tmp);
            vr[r][4 * hlf + 0] = tmp[0];
            vr[r][4 * hlf + 1] = tmp[1];
            vr[r][4 * hlf + 2] = tmp[2];
            vr[r][4 * hlf + 3] = tmp[3];
          }
        }
#pragma unroll
        for (int i = 0; i < TPB; ++i) {
          // tile i: MMA row g <-> d = DPT g + 2 i, row g+8 <-> d + 1
          const uint32_t a0 = __byte_perm(vr[0][i], vr[1][i], 0x5410);
          const uint32_t a1 = __byte_perm(vr[0][i], vr[1][i], 0x7632);
          const uint32_t a2 = __byte_perm(vr[2][i], vr[3][i], 0x5410);
          const uint32_t a3 = __byte_perm(vr[2][i], vr[3][i], 0x7632);
          mma_f16(o[blk * TPB + i], a0, a1, a2, a3, pt0, pt1);
        }
      }
    }
  }

    // l is still per-thread; reduce over the token lanes
    if (finish) finish_sums();
  }

  __device__ __forceinline__ void finish_sums() {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float v = l_run[e];
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      l_run[e] = v;
    }
  }

  // Parks the warp's state in shared memory (sm_o rows are H + 4 floats).
  __device__ __forceinline__ void park(float (*sm_m)[8], float (*sm_l)[8], float (*sm_o)[8][H + 4], int warp, int lane) const {
    const int g = lane >> 2, t = lane & 3;
    if (g == 0) {
      sm_m[warp][2 * t] = m_run[0];
      sm_m[warp][2 * t + 1] = m_run[1];
      sm_l[warp][2 * t] = l_run[0];
      sm_l[warp][2 * t + 1] = l_run[1];
    }
#pragma unroll
    for (int blk = 0; blk < NBLK; ++blk)
#pragma unroll
      for (int i = 0; i < TPB; ++i) {
        const int d = blk * DB + DPT * g + 2 * i;
        sm_o[warp][2 * t][d] = o[blk * TPB + i][0];
        sm_o[warp][2 * t + 1][d] = o[blk * TPB + i][1];
        sm_o[warp][2 * t][d + 1] = o[blk * TPB + i][2];
        sm_o[warp][2 * t + 1][d + 1] = o[blk * TPB + i][3];
      }
  }
};

template <int KV, int H, bool QF32, int GPI>
__global__ void __launch_bounds__(kWarps * 32) sdpa_decode_kernel(const SdpaParams p, const int chunk_tokens,
                                                                  const int chunks_max) {
  using WA = WarpAttention<KV, H, GPI>;
  constexpr int KSTEPS = WA::KSTEPS;
  pdl_enter();
  const int b = blockIdx.z, kvh = blockIdx.y, chunk = blockIdx.x;
  const int len = p.lengths ? max(0, min(p.lengths[b], p.s_max)) : p.s_max;
  const int c0 = chunk * chunk_tokens;
  if (c0 >= len) return;
  const int c1 = min(len, c0 + chunk_tokens);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.n / p.nkv;  // query heads per kv head (<= 8)

  // ---- Q fragments: thread (g,t) keeps head g, 16-byte pieces t + 4 i ----
  uint32_t qf[KSTEPS][4];
  {
    const bool head_ok = g < group;
    const int head = kvh * group + (head_ok ? g : 0);
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) {
      const int d0 = 8 * (t + 4 * i);
      if (!head_ok) {
        qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
      } else if constexpr (QF32) {
        const float* q = static_cast<const float*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF32>(q, 0, true, qf[i]);
      } else {
        const __half* q = static_cast<const __half*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF16>(q, 0, true, qf[i]);
      }
    }
  }
  WA wa;
  wa.template run<kSrcGlobal>(p, qf, WA::cache_rows(p, b, kvh), b, c0 + warp * WA::kTokensPerWarpIter, kWarps * WA::kTokensPerWarpIter, c1, lane);

  // ---- merge the warps of this CTA ----
  __shared__ float sm_m[kWarps][8], sm_l[kWarps][8];
  __shared__ float sm_o[kWarps][8][H + 4];
  wa.park(sm_m, sm_l, sm_o, warp, lane);
  __syncthreads();
  float* part = p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max + chunk) * 8) * partial_stride(H);
  for (int idx = tid; idx < group * H; idx += kWarps * 32) {
    const int head = idx / H, d = idx % H;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, sm_m[w][head]);
    const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = exp2f(sm_m[w][head] - muse);
      acc += f * sm_o[w][head][d];
      l += f * sm_l[w][head];
    }
    float* rec = part + (size_t)head * partial_stride(H);
    rec[d] = acc;
    if (d == 0) {
      rec[H] = mm;
      rec[H + 1] = l;
    }
  }
}

// Staged variant of the kernel above for fp16 / int8 caches: the CTA's chunk goes through a ring of
// shared-memory stages of kRingTokens tokens, every cached row fetched by one bulk asynchronous copy
// (one row per thread and stage: keys by the lower half of the CTA, values by the upper), so a
// CTA keeps up to stages x 64 KB in flight without holding registers for it, and the warps read
// their MMA fragments from shared memory (the loads straight from global memory of the kernel
// above leave the SMs waiting on the long scoreboard with ~7 warps each). Same chunking, same
// partial records.
constexpr int kRingTokens = 64;
constexpr int kRingStagesMax = 3;

template <int KV, int H>
struct RingLayout {
  static constexpr int kRowBytes = H * (KV == kKvI8 ? 1 : 2);
  static constexpr int kPitch = kRowBytes + 16;  // rows 16 bytes apart in the banks
  static constexpr int kStageBytes = 2 * kRingTokens * kPitch;
  static constexpr int kParkBytes = (int)sizeof(float) * kWarps * 8 * (H + 4);
  static size_t smem_bytes(int stages) {
    const size_t ring = (size_t)stages * kStageBytes;
    return (ring > (size_t)kParkBytes ? ring : (size_t)kParkBytes) + 128;
  }
};

template <int KV, int H, bool QF32>
__global__ void __launch_bounds__(kWarps * 32) sdpa_decode_ring_kernel(const SdpaParams p, const int chunk_tokens,
                                                                       const int chunks_max, const int stages,
                                                                       const int stage_tokens) {
  using WA = WarpAttention<KV, H, 1>;
  using L = RingLayout<KV, H>;
  constexpr int KSTEPS = WA::KSTEPS;
  static_assert(kWarps * 32 == 2 * kRingTokens, "one row copy per thread and stage");
  static_assert(kWarps * 16 == kRingTokens, "one 16-token group per warp and stage");
  // `stage_tokens` (a multiple of 16, at most kRingTokens) tokens per stage: two stages must fit beside a
  // second CTA on the SM, so that the copy of the next stage runs under the arithmetic of this one
  const int stage_bytes = 2 * stage_tokens * L::kPitch;
  extern __shared__ __align__(128) uint8_t ring_smem[];
  __shared__ float sm_m[kWarps][8], sm_l[kWarps][8];
  __shared__ int s_abort;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring_smem);  // [kRingStagesMax], 128 bytes reserved
  uint8_t* ring = ring_smem + 128;
  float (*sm_o)[8][H + 4] = reinterpret_cast<float (*)[8][H + 4]>(ring);  // after the loop
  volatile int* abort_flag = &s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < kRingStagesMax; ++i) mbar_init(&full_bar[i], 1);
    s_abort = 0;
    mbar_fence_init();
  }
  pdl_enter();
  __syncthreads();
  const int b = blockIdx.z, kvh = blockIdx.y, chunk = blockIdx.x;
  const int len = p.lengths ? max(0, min(p.lengths[b], p.s_max)) : p.s_max;
  const int c0 = chunk * chunk_tokens;
  if (c0 >= len) return;  // uniform over the CTA, nothing in flight
  const int c1 = min(len, c0 + chunk_tokens);
  const int n_sub = (c1 - c0 + stage_tokens - 1) / stage_tokens;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.n / p.nkv;
  const typename WA::Rows cache = WA::cache_rows(p, b, kvh);
  // With one kv head the cached rows of consecutive tokens follow one another in memory: a stage is then
  // ONE bulk copy per operand (32 KB of fp16 rows) instead of one per row, unpadded in shared memory. (128
  // copies of 512 bytes per stage keep the copy engine busier issuing than moving; the 2- to 4-way bank
  // conflicts of the unpadded rows cost the fragment loads less than that.)
  const bool contiguous = cache.stride == (size_t)L::kRowBytes;
  const int pitch = contiguous ? L::kRowBytes : L::kPitch;

  // stage `s` <- tokens [c0 + j * 64, ...): thread r (< 64) fetches key row r, thread 64 + r value row r
  auto issue = [&](int j) {
    const int s = j % stages;
    const int t0 = c0 + j * stage_tokens;
    const int rows = min(stage_tokens, c1 - t0);
    uint8_t* stage = ring + (size_t)s * stage_bytes;
    if (tid == 0) mbar_arrive_expect_tx(&full_bar[s], (uint32_t)(2 * rows * L::kRowBytes));
    if (contiguous) {
      if (tid == 0) {
        bulk_g2s(stage, cache.k + (size_t)t0 * cache.stride, (uint32_t)(rows * L::kRowBytes), &full_bar[s]);
        bulk_g2s(stage + (size_t)stage_tokens * L::kPitch, cache.v + (size_t)t0 * cache.stride, (uint32_t)(rows * L::kRowBytes),
                 &full_bar[s]);
      }
      return;
    }
    const int r = tid & (kRingTokens - 1);
    if (r < rows) {
      const bool is_v = tid >= kRingTokens;
      const uint8_t* src = (is_v ? cache.v : cache.k) + (size_t)(t0 + r) * cache.stride;
      bulk_g2s(stage + (size_t)(is_v ? stage_tokens : 0) * L::kPitch + (size_t)r * L::kPitch, src, L::kRowBytes, &full_bar[s]);
    }
  };
  int issued = min(stages, n_sub);
  for (int j = 0; j < issued; ++j) issue(j);

  // ---- Q fragments (as above) while the first stages land ----
  uint32_t qf[KSTEPS][4];
  {
    const bool head_ok = g < group;
    const int head = kvh * group + (head_ok ? g : 0);
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) {
      const int d0 = 8 * (t + 4 * i);
      if (!head_ok) {
        qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
      } else if constexpr (QF32) {
        const float* q = static_cast<const float*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF32>(q, 0, true, qf[i]);
      } else {
        const __half* q = static_cast<const __half*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF16>(q, 0, true, qf[i]);
      }
    }
  }
  WA wa;
  wa.clear();
  for (int j = 0; j < n_sub; ++j) {
    const int s = j % stages;
    mbar_wait_bounded(&full_bar[s], (uint32_t)(j / stages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
    const int t0 = c0 + j * stage_tokens;
    const int t1 = min(c1, t0 + stage_tokens);
    const int first = t0 + warp * 16;
    if (first < t1 && !*abort_flag) {
      typename WA::Rows rows = cache;  // scales stay in global memory
      const uint8_t* stage = ring + (size_t)s * stage_bytes;
      rows.k = stage - (ptrdiff_t)t0 * pitch;  // indexed by absolute token
      rows.v = stage + (size_t)stage_tokens * L::kPitch - (ptrdiff_t)t0 * pitch;
      rows.stride = pitch;
      wa.template run<kSrcShared>(p, qf, rows, b, first, kRingTokens, t1, lane, /*fresh=*/false, /*finish=*/false);
    }
    __syncthreads();  // every warp is done with stage s
    if (issued < n_sub && !*abort_flag) {  // (abort_flag cannot change between the barrier above and here)
      issue(issued);
      ++issued;
    }
  }
  wa.finish_sums();
  // after an abort: the latest copies towards each stage may still be in flight
  if (*abort_flag)
    for (int j = max(0, issued - stages); j < issued; ++j)
      mbar_drain_bounded(&full_bar[j % stages], (uint32_t)(j / stages) & 1u);
  __syncthreads();

  // ---- merge the warps of this CTA (the parked outputs reuse the ring) ----
  wa.park(sm_m, sm_l, sm_o, warp, lane);
  __syncthreads();
  float* part = p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max + chunk) * 8) * partial_stride(H);
  for (int idx = tid; idx < group * H; idx += kWarps * 32) {
    const int head = idx / H, d = idx % H;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, sm_m[w][head]);
    const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = exp2f(sm_m[w][head] - muse);
      acc += f * sm_o[w][head][d];
      l += f * sm_l[w][head];
    }
    float* rec = part + (size_t)head * partial_stride(H);
    rec[d] = acc;
    if (d == 0) {
      rec[H] = mm;
      rec[H + 1] = l;
    }
  }
}

// Prompt-pass variant (SdpaParams::shared_kv): the rows of the batch are consecutive tokens of ONE
// sequence and all read the same cache, row b up to lengths[b]. Here a WARP owns a row: the warps of a
// CTA walk the same chunk of the cache for kWarps neighbouring rows at nearly the same pace, so the
// chunk comes through L2 once per CTA instead of once per row. Every warp writes the partial record
// of its own (row, chunk); the merge kernels are the same.
template <int KV, int H, bool QF32, int GPI>
__global__ void __launch_bounds__(kWarps * 32) sdpa_rows_kernel(const SdpaParams p, const int chunk_tokens,
                                                                const int chunks_max) {
  using WA = WarpAttention<KV, H, GPI>;
  constexpr int KSTEPS = WA::KSTEPS;
  __shared__ float sm_m[kWarps][8], sm_l[kWarps][8];
  __shared__ float sm_o[kWarps][8][H + 4];
  pdl_enter();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = (int)blockIdx.z * kWarps + warp, kvh = blockIdx.y, chunk = blockIdx.x;
  if (b >= p.b) return;  // (no block-wide barrier below)
  const int len = p.lengths ? max(0, min(p.lengths[b], p.s_max)) : p.s_max;
  const int c0 = chunk * chunk_tokens;
  if (c0 >= len) return;
  const int c1 = min(len, c0 + chunk_tokens);
  const int g = lane >> 2, t = lane & 3;
  const int group = p.n / p.nkv;
  uint32_t qf[KSTEPS][4];
  {
    const bool head_ok = g < group;
    const int head = kvh * group + (head_ok ? g : 0);
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) {
      const int d0 = 8 * (t + 4 * i);
      if (!head_ok) {
        qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
      } else if constexpr (QF32) {
        const float* q = static_cast<const float*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF32>(q, 0, true, qf[i]);
      } else {
        const __half* q = static_cast<const __half*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF16>(q, 0, true, qf[i]);
      }
    }
  }
  WA wa;
  wa.template run<kSrcGlobal>(p, qf, WA::cache_rows(p, b, kvh), b, c0, WA::kTokensPerWarpIter, c1, lane);
  wa.park(sm_m, sm_l, sm_o, warp, lane);
  __syncwarp();
  float* part = p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max + chunk) * 8) * partial_stride(H);
  for (int idx = lane; idx < group * H; idx += 32) {
    const int head = idx / H, d = idx % H;
    float* rec = part + (size_t)head * partial_stride(H);
    rec[d] = sm_o[warp][head][d];
    if (d == 0) {
      rec[H] = sm_m[warp][head];
      rec[H + 1] = sm_l[warp][head];
    }
  }
}

// Prompt pass with staging (fp16 / int8 caches): a CTA takes kWarps neighbouring rows and one chunk of
// the shared cache; the chunk goes through the 64-token ring stages of sdpa_decode_ring_kernel ONCE
// for all the CTA's rows, and every warp runs its own row (its own query, softmax state and partial
// record) over each stage, masked at the row's own length.
template <int KV, int H, bool QF32>
__global__ void __launch_bounds__(kWarps * 32) sdpa_rows_ring_kernel(const SdpaParams p, const int chunk_tokens,
                                                                     const int chunks_max, const int stages,
                                                                     const int stage_tokens) {
  using WA = WarpAttention<KV, H, 4>;  // one pass of 64 tokens per stage
  using L = RingLayout<KV, H>;
  constexpr int KSTEPS = WA::KSTEPS;
  static_assert(WA::kTokensPerWarpIter == kRingTokens, "a warp takes a whole stage per pass");
  const int stage_bytes = 2 * stage_tokens * L::kPitch;  // (stage_tokens <= kRingTokens: see the decode kernel's launcher)
  extern __shared__ __align__(128) uint8_t ring_smem[];
  __shared__ float sm_m[kWarps][8], sm_l[kWarps][8];
  __shared__ int s_abort;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring_smem);
  uint8_t* ring = ring_smem + 128;
  float (*sm_o)[8][H + 4] = reinterpret_cast<float (*)[8][H + 4]>(ring);  // after the loop
  volatile int* abort_flag = &s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < kRingStagesMax; ++i) mbar_init(&full_bar[i], 1);
    s_abort = 0;
    mbar_fence_init();
  }
  pdl_enter();
  __syncthreads();
  const int row0 = (int)blockIdx.z * kWarps, kvh = blockIdx.y, chunk = blockIdx.x;
  const int b = min(row0 + warp, p.b - 1);          // this warp's row (a surplus warp repeats the last one, unused)
  const bool row_ok = row0 + warp < p.b;
  const int b_last = min(row0 + kWarps, p.b) - 1;   // lengths grow with the row: the CTA's longest
  auto length_of = [&](int r) { return p.lengths ? max(0, min(p.lengths[r], p.s_max)) : p.s_max; };
  int len_cta = 0;
  for (int r = row0; r <= b_last; ++r) len_cta = max(len_cta, length_of(r));
  const int c0 = chunk * chunk_tokens;
  if (c0 >= len_cta) return;  // uniform over the CTA, nothing in flight
  const int c1 = min(len_cta, c0 + chunk_tokens);
  const int len_w = row_ok ? length_of(b) : 0;
  const int n_sub = (c1 - c0 + stage_tokens - 1) / stage_tokens;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.n / p.nkv;
  const typename WA::Rows cache = WA::cache_rows(p, 0, kvh);  // shared_kv: one cache for all rows

  auto issue = [&](int j) {
    const int s = j % stages;
    const int t0 = c0 + j * stage_tokens;
    const int rows = min(stage_tokens, c1 - t0);
    uint8_t* stage = ring + (size_t)s * stage_bytes;
    if (tid == 0) mbar_arrive_expect_tx(&full_bar[s], (uint32_t)(2 * rows * L::kRowBytes));
    const int r = tid & (kRingTokens - 1);
    if (r < rows) {
      const bool is_v = tid >= kRingTokens;
      const uint8_t* src = (is_v ? cache.v : cache.k) + (size_t)(t0 + r) * cache.stride;
      bulk_g2s(stage + (size_t)(is_v ? stage_tokens : 0) * L::kPitch + (size_t)r * L::kPitch, src, L::kRowBytes, &full_bar[s]);
    }
  };
  int issued = min(stages, n_sub);
  for (int j = 0; j < issued; ++j) issue(j);

  uint32_t qf[KSTEPS][4];
  {
    const bool head_ok = g < group;
    const int head = kvh * group + (head_ok ? g : 0);
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) {
      const int d0 = 8 * (t + 4 * i);
      if (!head_ok) {
        qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
      } else if constexpr (QF32) {
        const float* q = static_cast<const float*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF32>(q, 0, true, qf[i]);
      } else {
        const __half* q = static_cast<const __half*>(p.q) + ((size_t)b * p.n + head) * H + d0;
        load8<kKvF16>(q, 0, true, qf[i]);
      }
    }
  }
  WA wa;
  wa.clear();
  for (int j = 0; j < n_sub; ++j) {
    const int s = j % stages;
    mbar_wait_bounded(&full_bar[s], (uint32_t)(j / stages) & 1u, abort_flag, p.status, kStatusWaitTimeoutFull);
    const int t0 = c0 + j * stage_tokens;
    const int t1 = min(min(c1, t0 + stage_tokens), len_w);  // this row's own causal limit
    if (t0 < t1 && !*abort_flag) {
      typename WA::Rows rows = cache;
      const uint8_t* stage = ring + (size_t)s * stage_bytes;
      rows.k = stage - (ptrdiff_t)t0 * L::kPitch;
      rows.v = stage + (size_t)stage_tokens * L::kPitch - (ptrdiff_t)t0 * L::kPitch;
      rows.stride = L::kPitch;
      wa.template run<kSrcShared>(p, qf, rows, b, t0, kRingTokens, t1, lane, /*fresh=*/false, /*finish=*/false);
    }
    __syncthreads();  // every warp is done with stage s
    if (issued < n_sub && !*abort_flag) {
      issue(issued);
      ++issued;
    }
  }
  wa.finish_sums();
  if (*abort_flag)
    for (int j = max(0, issued - stages); j < issued; ++j) mbar_drain_bounded(&full_bar[j % stages], (uint32_t)(j / stages) & 1u);
  __syncthreads();
  wa.park(sm_m, sm_l, sm_o, warp, lane);
  __syncwarp();
  if (!row_ok || c0 >= len_w) return;  // (the merge reads only the chunks below the row's length)
  float* part = p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max + chunk) * 8) * partial_stride(H);
  for (int idx = lane; idx < group * H; idx += 32) {
    const int head = idx / H, d = idx % H;
    float* rec = part + (size_t)head * partial_stride(H);
    rec[d] = sm_o[warp][head][d];
    if (d == 0) {
      rec[H] = sm_m[warp][head];
      rec[H + 1] = sm_l[warp][head];
    }
  }
}

// ---- one decode step of a decoder layer's attention in ONE launch -------------------------------
// For a fused q/k/v projection output with a single KV head (multi-query attention) and at most
// eight query heads: rotary embedding of q and of the new key, append of the new key / value row to
// the cache, attention over the cached tokens, and the per-row asymmetric int8 quantization that
// the output projection (a hybrid FULLY_CONNECTED) applies to its input. One cluster of
// kAttnCluster CTAs per sequence: the CTAs split the tokens, merge their softmax states through
// distributed shared memory (CTA r finishes head r), exchange the finished heads' min / max the
// same way, and each writes its head's quantized bytes in the tiled activation layout.
constexpr int kAttnCluster = 8;
// Warps per CTA. Measured on B200 (batch 1, 1040 cached tokens): 4 warps x 3 passes of 16 tokens
// take 4.6 us in the token loop, 8 warps x 2 passes 5.4 us: the loop's cost is mostly fixed (cold
// instruction and data fetches after the weight stream has swept L2), not per token.
constexpr int kAttnWarps = 4;

template <int H>
struct AttnStepSmem {
  static constexpr int kRec = H + 4;  // outputs, maximum, sum, two floats of padding: whole 16-byte pieces
  float2 cs[H / 2];               // cos, sin per rotation pair
  float q[8][H];                  // rotated query heads
  float sm_m[kAttnWarps][8], sm_l[kAttnWarps][8], wf[kAttnWarps][8];
  __align__(16) float rec[8][kRec];             // this CTA's merged state per head
  __align__(16) float inbox[kAttnCluster][kRec];  // the states of the head this CTA finishes, from every CTA
  float own[H];                   // finished head
  __align__(8) float2 mmbox[kAttnCluster];  // min / max of every CTA's finished head
  float2 red[kAttnWarps];
  // the two exchanges of the cluster complete on these (transaction bytes carried by the remote stores
  // themselves): [0] the head states have arrived in `inbox`, [1] the min / max pairs in `mmbox`
  __align__(8) uint64_t xbar[2];
  int abort_flag;
  // followed by the staging area (`stage_rows` key rows then as many value rows, each padded by
  // 16 bytes against bank conflicts) and the warps' parked outputs
};
template <int KV, int H>
__host__ __device__ constexpr int attn_row_pitch() {
  return H * (KV == kKvI8 ? 1 : 2) + 16;
}
template <int H>
constexpr size_t attn_park_bytes() {
  return sizeof(float) * kAttnWarps * 8 * (H + 4);
}

// x * cos + rotate_half(x) * sin, every product and sum rounded on its own (separate MUL and ADD ops
// in the graph, tensor/examples/gemma3/gemma3_graph.cc:150-176); r = {cos, sin}.
__device__ __forceinline__ float rope_lo(float x1, float x2, float2 r) {
  return __fsub_rn(__fmul_rn(x1, r.x), __fmul_rn(x2, r.y));
}
__device__ __forceinline__ float rope_hi(float x1, float x2, float2 r) {
  return __fadd_rn(__fmul_rn(x2, r.x), __fmul_rn(x1, r.y));
}

template <int KV, int H, int GPI>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_step_cluster_kernel(const AttnStepParams p, const int stage_rows) {
  using WA = WarpAttention<KV, H, GPI>;
  constexpr int KSTEPS = WA::KSTEPS;
  constexpr int C = kAttnCluster, HALF = H / 2, REC = AttnStepSmem<H>::kRec;
  constexpr int PITCH = attn_row_pitch<KV, H>();
  constexpr int ROW_BYTES = H * (KV == kKvI8 ? 1 : 2);
  extern __shared__ __align__(128) uint8_t attn_smem_raw[];
  AttnStepSmem<H>& sm = *reinterpret_cast<AttnStepSmem<H>*>(attn_smem_raw);
  uint8_t* stage_k = attn_smem_raw + ((sizeof(AttnStepSmem<H>) + 127) / 128) * 128;
  uint8_t* stage_v = stage_k + (size_t)stage_rows * PITCH;
  // the warps' parked outputs reuse the staging area once every warp has left the token loop
  float (*sm_o)[8][H + 4] = reinterpret_cast<float (*)[8][H + 4]>(stage_k);

  const bool tracer = p.trace && blockIdx.x == 0 && threadIdx.x == 0;
  if (tracer) p.trace[0] = global_timer_ns();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    mbar_init(&sm.xbar[0], 1);
    mbar_init(&sm.xbar[1], 1);
    sm.abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  cluster_arrive();  // phase 0: this CTA runs and its barriers exist (waited for before the first remote store)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rank = (int)cluster_ctarank();
  const int b = blockIdx.x / C;
  // The positions and every cached row below the new token date from earlier steps: they can be
  // read before the kernel that produces this step's q / k / v has finished.
  const int pos = p.positions[b];
  if (tracer) p.trace[9] = global_timer_ns() + (pos == -12345);
  const bool append = pos < p.s_max;  // a full cache ignores the step's key / value
  const int len = append ? pos + 1 : p.s_max;
  // tokens of this CTA: equal shares, a multiple of 16
  const int per = (((len + C - 1) / C) + 15) / 16 * 16;
  const int c0 = rank * per;
  const int c1 = min(len, c0 + per);
  // The first `stage_rows` rows of the share are staged in shared memory; a share a little longer than
  // the staging area reads its last rows straight from the cache (a context that outgrows the staging
  // area by a few tokens must not fall off a cliff), a much longer one reads all of them from there.
  const bool staged = c1 - c0 <= stage_rows + 64;
  const int s_end = min(c1, c0 + stage_rows);      // staged rows: [c0, s_end)
  const int old_end = append ? min(c1, pos) : c1;  // rows [c0, old_end) are already in the cache
  const uint8_t* kglob = static_cast<const uint8_t*>(p.k_cache) + (size_t)b * p.s_max * ROW_BYTES;
  const uint8_t* vglob = static_cast<const uint8_t*>(p.v_cache) + (size_t)b * p.s_max * ROW_BYTES;
  if (staged) {
    // 16-byte asynchronous copies, all in flight at once (no registers held): the rows land padded
    constexpr int PIECES = ROW_BYTES / 16;
    const int n_pieces = (min(old_end, s_end) - c0) * PIECES;
    for (int i = tid; i < n_pieces; i += kAttnWarps * 32) {
      const int r = i / PIECES, c = i % PIECES;
      cp_async16(stage_k + (size_t)r * PITCH + c * 16, kglob + (size_t)(c0 + r) * ROW_BYTES + c * 16);
      cp_async16(stage_v + (size_t)r * PITCH + c * 16, vglob + (size_t)(c0 + r) * ROW_BYTES + c * 16);
    }
    cp_async_commit();
  }
  if (tracer) p.trace[10] = global_timer_ns();
  // cos / sin of this position's rotation angles, from the table the host side prepared
  for (int i = tid; i < HALF; i += kAttnWarps * 32) sm.cs[i] = p.rope_cs[(size_t)min(pos, p.s_max) * HALF + i];
  if (tracer) p.trace[11] = global_timer_ns();
  // (Running the code below once ahead of the dependency wait, on stale q / k / v, to warm the caches was
  // measured on B200 and does not pay here: the early run outlasts the projection kernel by 8 us and the
  // real one is no faster. The row kernels of the decoder keep theirs.)
  {
    constexpr bool live = true;
    if (live) {
      pdl_wait();  // this step's q / k / v
      if (tracer) p.trace[1] = global_timer_ns();
    }
    __syncthreads();
    const float* src = p.qkv + (size_t)b * (p.n + 2) * H;
    for (int idx = tid; idx < p.n * HALF; idx += kAttnWarps * 32) {
      const int head = idx / HALF, i = idx % HALF;
      const float x1 = __ldcg(src + head * H + i), x2 = __ldcg(src + head * H + i + HALF);  // past L1: the dry run read them too
      const float2 r = sm.cs[i];
      sm.q[head][i] = rope_lo(x1, x2, r);
      sm.q[head][i + HALF] = rope_hi(x1, x2, r);
    }
    if (append && pos >= c0 && pos < c1) {
      // The CTA whose share holds the new token writes its row: to the cache, and to the staged
      // copy it is about to read (the same rounded values later steps will find in the cache).
      const float* ksrc = src + (size_t)p.n * H;
      const float* vsrc = ksrc + H;
      const size_t tok = (size_t)b * p.s_max + pos;
      if constexpr (KV == kKvI8) {
        // symmetric per token: scale = max|row| / 127 (key after the rotation)
        float ka = 0.0f, va = 0.0f;
        for (int i = tid; i < HALF; i += kAttnWarps * 32) {
          const float2 r = sm.cs[i];
          const float x1 = __ldcg(ksrc + i), x2 = __ldcg(ksrc + i + HALF);
          ka = fmaxf(ka, fmaxf(fabsf(rope_lo(x1, x2, r)), fabsf(rope_hi(x1, x2, r))));
          va = fmaxf(va, fmaxf(fabsf(__ldcg(vsrc + i)), fabsf(__ldcg(vsrc + i + HALF))));
        }
  #pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
          va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o));
        }
        if (lane == 0) sm.red[warp] = make_float2(ka, va);
        __syncthreads();
        ka = sm.red[0].x, va = sm.red[0].y;
  #pragma unroll
        for (int w = 1; w < kAttnWarps; ++w) {
          ka = fmaxf(ka, sm.red[w].x);
          va = fmaxf(va, sm.red[w].y);
        }
        const float ks = ka > 0.0f ? __fdiv_rn(ka, 127.0f) : 1.0f, vs = va > 0.0f ? __fdiv_rn(va, 127.0f) : 1.0f;
        int8_t* kd = static_cast<int8_t*>(p.k_cache) + tok * H;
        int8_t* vd = static_cast<int8_t*>(p.v_cache) + tok * H;
        int8_t* ks_row = reinterpret_cast<int8_t*>(stage_k + (size_t)(pos - c0) * PITCH);
        int8_t* vs_row = reinterpret_cast<int8_t*>(stage_v + (size_t)(pos - c0) * PITCH);
        for (int i = tid; i < HALF; i += kAttnWarps * 32) {
          const float2 r = sm.cs[i];
          const float x1 = __ldcg(ksrc + i), x2 = __ldcg(ksrc + i + HALF);
          const int8_t k1 = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(rope_lo(x1, x2, r), ks))));
          const int8_t k2 = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(rope_hi(x1, x2, r), ks))));
          const int8_t v1 = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(__ldcg(vsrc + i), vs))));
          const int8_t v2 = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(__ldcg(vsrc + i + HALF), vs))));
          if (live) kd[i] = k1, kd[i + HALF] = k2, vd[i] = v1, vd[i + HALF] = v2;
          if (staged && pos < s_end) ks_row[i] = k1, ks_row[i + HALF] = k2, vs_row[i] = v1, vs_row[i + HALF] = v2;
        }
        if (tid == 0 && live) {
          p.k_scale[tok] = ks;
          p.v_scale[tok] = vs;
        }
      } else {
        __half* kd = static_cast<__half*>(p.k_cache) + tok * H;
        __half* vd = static_cast<__half*>(p.v_cache) + tok * H;
        __half* ks_row = reinterpret_cast<__half*>(stage_k + (size_t)(pos - c0) * PITCH);
        __half* vs_row = reinterpret_cast<__half*>(stage_v + (size_t)(pos - c0) * PITCH);
        for (int i = tid; i < HALF; i += kAttnWarps * 32) {
          const float2 r = sm.cs[i];
          const float x1 = __ldcg(ksrc + i), x2 = __ldcg(ksrc + i + HALF);
          const __half k1 = __float2half_rn(rope_lo(x1, x2, r)), k2 = __float2half_rn(rope_hi(x1, x2, r));
          const __half v1 = __float2half_rn(__ldcg(vsrc + i)), v2 = __float2half_rn(__ldcg(vsrc + i + HALF));
          if (live) kd[i] = k1, kd[i + HALF] = k2, vd[i] = v1, vd[i + HALF] = v2;
          if (staged && pos < s_end) ks_row[i] = k1, ks_row[i + HALF] = k2, vs_row[i] = v1, vs_row[i + HALF] = v2;
        }
      }
    }
    cp_async_wait_all();
    __syncthreads();  // rotated queries, staged rows and the new row (staged copy, or the cache through this CTA's own stores) in place

    if (tracer && live) p.trace[2] = global_timer_ns();
    uint32_t qf[KSTEPS][4];
  #pragma unroll
    for (int i = 0; i < KSTEPS; ++i) {
      const int d0 = 8 * (t + 4 * i);
      if (g < p.n) {
        const float* q = &sm.q[g][d0];
        qf[i][0] = pack_half2(q[0], q[1]);
        qf[i][1] = pack_half2(q[2], q[3]);
        qf[i][2] = pack_half2(q[4], q[5]);
        qf[i][3] = pack_half2(q[6], q[7]);
      } else {
        qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
      }
    }
    SdpaParams sp;
    sp.mask = nullptr;
    sp.nkv = 1;
    sp.s_max = p.s_max;
    sp.scale = p.scale;
    sp.logit_cap = 0.0f;
    typename WA::Rows rows;
    rows.k_scale = p.k_scale ? p.k_scale + (size_t)b * p.s_max : nullptr;
    rows.v_scale = p.v_scale ? p.v_scale + (size_t)b * p.s_max : nullptr;
    rows.scale_stride = 1;
    if (staged) {
      rows.k = stage_k - (ptrdiff_t)c0 * PITCH;  // indexed by absolute token
      rows.v = stage_v - (ptrdiff_t)c0 * PITCH;
      rows.stride = PITCH;
    } else {
      rows.k = kglob;
      rows.v = vglob;
      rows.stride = ROW_BYTES;
    }
    if (tracer && live) p.trace[3] = global_timer_ns();
    // the warps take equal contiguous shares of the CTA's tokens (multiples of 16)
    // Staged rows are read from shared memory, where passes are cheap: the smallest loop body (16
    // tokens per pass) whatever the cache's capacity. Rows read from the cache itself (a share
    // longer than the staging area) want the long passes the kernel was instantiated with.
    if (staged) {
      using WA1 = WarpAttention<KV, H, 1>;
      WA1 wa;
      typename WA1::Rows rows1;
      rows1.k = rows.k;
      rows1.v = rows.v;
      rows1.stride = rows.stride;
      rows1.k_scale = rows.k_scale;
      rows1.v_scale = rows.v_scale;
      rows1.scale_stride = rows.scale_stride;
      wa.clear();
      {
        const int wper = ((((s_end - c0) + kAttnWarps - 1) / kAttnWarps) + 15) / 16 * 16;
        const int first = c0 + warp * wper;
        const int last = min(s_end, first + wper);
        if (first < last) wa.template run<kSrcShared, false>(sp, qf, rows1, b, first, 16, last, lane, /*fresh=*/false, /*finish=*/false);
      }
      if (s_end < c1) {  // the share's rows beyond the staging area, from the cache (this CTA's own append included)
        rows1.k = kglob;
        rows1.v = vglob;
        rows1.stride = ROW_BYTES;
        const int wper = ((((c1 - s_end) + kAttnWarps - 1) / kAttnWarps) + 15) / 16 * 16;
        const int first = s_end + warp * wper;
        const int last = min(c1, first + wper);
        if (first < last)
          wa.template run<kSrcGlobalCoherent, false>(sp, qf, rows1, b, first, 16, last, lane, /*fresh=*/false, /*finish=*/false);
      }
      wa.finish_sums();
      if (tracer && live) p.trace[4] = global_timer_ns();
      __syncthreads();  // the staged rows are dead: the parked outputs take their place
      wa.park(sm.sm_m, sm.sm_l, sm_o, warp, lane);
    } else {
      const int wper = ((((c1 - c0) + kAttnWarps - 1) / kAttnWarps) + 15) / 16 * 16;
      const int first = c0 + warp * wper;
      const int last = min(c1, first + wper);
      WA wa;
      if (first >= last) {
        wa.clear();
      } else {
        wa.template run<kSrcGlobalCoherent, false>(sp, qf, rows, b, first, WA::kTokensPerWarpIter, last, lane);
      }
      if (tracer && live) p.trace[4] = global_timer_ns();
      wa.park(sm.sm_m, sm.sm_l, sm_o, warp, lane);
    }
    __syncthreads();
    // this CTA's state per head: the warps merged (weights per warp and head computed once)
    if (tid < 8) {
      const int head = tid;
      float mm = -CUDART_INF_F;
  #pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, sm.sm_m[w][head]);
      const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
      float l = 0.0f;
  #pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        const float f = exp2f(sm.sm_m[w][head] - muse);
        sm.wf[w][head] = f;
        l += f * sm.sm_l[w][head];
      }
      sm.rec[head][H] = mm;
      sm.rec[head][H + 1] = l;
    }
    __syncthreads();
    for (int idx = tid; idx < p.n * H; idx += kAttnWarps * 32) {
      const int head = idx / H, d = idx % H;
      float acc = 0.0f;
  #pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) acc += sm.wf[w][head] * sm_o[w][head][d];
      sm.rec[head][d] = acc;
    }
    __syncthreads();
    if (tracer && live) p.trace[5] = global_timer_ns();
    cluster_wait();  // phase 0
    // Head h goes to CTA h (n <= 8 = cluster size). Every float sent also counts as four transaction bytes on
    // the receiving CTA's barrier (st.async): a CTA knows that its head's states are in without a cluster-wide
    // barrier, which costs 0.4 us more (measured on B200 on the same exchange).
    const bool owner = rank < p.n;
    volatile int* abort_flag = &sm.abort_flag;
    if (tid == 0) {
      mbar_arrive_expect_tx(&sm.xbar[0], owner ? (uint32_t)(C * REC * 4) : 0u);
      mbar_arrive_expect_tx(&sm.xbar[1], (uint32_t)(C * 8));
    }
    for (int head = 0; head < p.n; ++head) {
      const uint32_t dst = map_to_rank(smem_u32(&sm.inbox[rank][0]), (uint32_t)head);
      const uint32_t bar = map_to_rank(smem_u32(&sm.xbar[0]), (uint32_t)head);
      for (int i = tid; i < REC / 4; i += kAttnWarps * 32)  // 16 bytes per message
        st_async_cluster_f32x4(dst + 16u * (uint32_t)i, *reinterpret_cast<const float4*>(&sm.rec[head][4 * i]), bar);
    }
    mbar_wait_bounded(&sm.xbar[0], 0, abort_flag, p.status, kStatusWaitTimeoutFull);
    if (tracer && live) p.trace[6] = global_timer_ns();
    float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
    if (owner) {
      float mm = -CUDART_INF_F;
  #pragma unroll
      for (int c = 0; c < C; ++c) mm = fmaxf(mm, sm.inbox[c][H]);
      const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
      float f[C], l = 0.0f;
  #pragma unroll
      for (int c = 0; c < C; ++c) {
        f[c] = exp2f(sm.inbox[c][H] - muse);
        l += f[c] * sm.inbox[c][H + 1];
      }
      for (int d = tid; d < H; d += kAttnWarps * 32) {
        float acc = 0.0f;
  #pragma unroll
        for (int c = 0; c < C; ++c) acc += f[c] * sm.inbox[c][d];
        const float v = acc / l;
        sm.own[d] = v;
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
    }
  #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) sm.red[warp] = make_float2(mn, mx);
    __syncthreads();
    if (tid < C) {
      float lo = sm.red[0].x, hi = sm.red[0].y;
  #pragma unroll
      for (int w = 1; w < kAttnWarps; ++w) {
        lo = fminf(lo, sm.red[w].x);
        hi = fmaxf(hi, sm.red[w].y);
      }
      st_async_cluster_f32x2(map_to_rank(smem_u32(&sm.mmbox[rank]), (uint32_t)tid), lo, hi,
                             map_to_rank(smem_u32(&sm.xbar[1]), (uint32_t)tid));
    }
    mbar_wait_bounded(&sm.xbar[1], 0, abort_flag, p.status, kStatusWaitTimeoutFull);
    if (tracer && live) p.trace[7] = global_timer_ns();
    float lo = sm.mmbox[0].x, hi = sm.mmbox[0].y;
  #pragma unroll
    for (int c = 1; c < C; ++c) {
      lo = fminf(lo, sm.mmbox[c].x);
      hi = fmaxf(hi, sm.mmbox[c].y);
    }
    float sf, inv;
    int zp, zero_row;
    row_quant_params(lo, hi, true, &sf, &inv, &zp, &zero_row);
    const float zpf = (float)zp;
    if (owner) {
      for (int d4 = tid * 4; d4 < H; d4 += kAttnWarps * 32 * 4) {
        uint32_t word = 0;
  #pragma unroll
        for (int e = 0; e < 4; ++e)
          if (!zero_row) word |= quantize_value(sm.own[d4 + e], inv, zpf, true) << (8 * e);
        if (live) *reinterpret_cast<uint32_t*>(p.q_tiled_out + q_tiled_offset(b, rank * H + d4, p.m_alloc)) = word;
      }
    }
    if (rank == 0 && live) {
      const int width = p.n * H, k_pad = (width + 127) / 128 * 128;
      for (int k4 = width + tid * 4; k4 < k_pad; k4 += kAttnWarps * 32 * 4)
        *reinterpret_cast<uint32_t*>(p.q_tiled_out + q_tiled_offset(b, k4, p.m_alloc)) = 0u;
      if (tid == 0) {
        p.out_scales[b] = sf;
        p.out_zps[b] = zp;
      }
    }
    if (tracer && live) p.trace[8] = global_timer_ns();
  }
}

// Reduces the per-chunk partials of one (batch, query head): grid (n, b), H threads. The kernel is a chain
// of L2 round trips, so they are made to overlap: every thread requests its element of the first chunks
// at once, the first warp meanwhile gathers the chunks' maxima and sums (one chunk per lane and step) and
// leaves the chunks' weights in shared memory, and the remaining chunks are summed eight loads at a time.
template <int H, bool QF32>
__global__ void sdpa_merge_kernel(const SdpaParams p, const int chunk_tokens, const int chunks_max) {
  extern __shared__ float merge_w[];  // [chunks_max] weights exp2(m_chunk - m)
  __shared__ float s_l;
  pdl_enter();
  const int b = blockIdx.y, head = blockIdx.x, d = threadIdx.x;
  const int group = p.n / p.nkv;
  const int kvh = head / group, hg = head % group;
  const int len = p.lengths ? max(0, min(p.lengths[b], p.s_max)) : p.s_max;
  const int chunks = (len + chunk_tokens - 1) / chunk_tokens;
  const float* base = p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max) * 8 + hg) * partial_stride(H);
  const size_t cstride = 8 * partial_stride(H);
  constexpr int kPre = 16;
  float pre[kPre];
#pragma unroll
  for (int j = 0; j < kPre; ++j) pre[j] = j < chunks ? base[j * cstride + d] : 0.0f;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mm = -CUDART_INF_F;
    for (int c = lane; c < chunks; c += 32) mm = fmaxf(mm, base[c * cstride + H]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
    float l = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      const float f = exp2f(base[c * cstride + H] - muse);
      merge_w[c] = f;
      l += f * base[c * cstride + H + 1];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) s_l = l;
  }
  __syncthreads();
  float acc = 0.0f;
  const int npre = chunks < kPre ? chunks : kPre;
#pragma unroll
  for (int j = 0; j < kPre; ++j)
    if (j < npre) acc += merge_w[j] * pre[j];
  for (int c = kPre; c < chunks; c += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = c + j < chunks ? base[(size_t)(c + j) * cstride + d] : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c + j < chunks) acc += merge_w[c + j] * v[j];
  }
  const float l = s_l;
  const float out = l > 0.0f ? acc / l : 0.0f;  // no cached token (or every key masked out): zeros, not 0 / 0
  const size_t oi = ((size_t)b * p.n + head) * H + d;
  if constexpr (QF32) {
    static_cast<float*>(p.out)[oi] = out;
  } else {
    static_cast<__half*>(p.out)[oi] = __float2half_rn(out);
  }
}

// Merge of the per-chunk partials fused with the per-row asymmetric int8 quantization the next
// hybrid FULLY_CONNECTED applies to the attention output: grid (b), one CTA per sequence over all
// n*h outputs. Writes the tiled int8 row (+ scale, zero point) and, when p.out is set, the floats.
template <int H>
__global__ void __launch_bounds__(1024) sdpa_merge_quant_kernel(const SdpaParams p, const int chunk_tokens,
                                                              const int chunks_max) {
  extern __shared__ float xs[];        // n * H merged outputs, then n * chunks_max weights
  __shared__ float red[32];
  __shared__ float s_linv[64];         // 1 / softmax denominator per head
  pdl_enter();
  const int b = blockIdx.x;
  const int group = p.n / p.nkv;
  const int len = p.lengths ? max(0, min(p.lengths[b], p.s_max)) : p.s_max;
  const int chunks = (len + chunk_tokens - 1) / chunk_tokens;
  const size_t cstride = 8 * partial_stride(H);
  const int width = p.n * H;
  float* wts = xs + width;              // [head][chunk]: exp2(m_chunk - m_head)
  auto head_base = [&](int head) {
    const int kvh = head / group, hg = head % group;
    return p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max) * 8 + hg) * partial_stride(H);
  };
  // The partial outputs of this thread's first two elements (first kPre chunks) are requested
  // before anything else, so that their L2 round trips overlap the per-head statistics below.
  constexpr int kPre = 16;
  float pre[2][kPre];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int idx = threadIdx.x + e * blockDim.x;
    const float* base = idx < width ? head_base(idx / H) + idx % H : nullptr;
#pragma unroll
    for (int j = 0; j < kPre; ++j) pre[e][j] = (base && j < chunks) ? base[j * cstride] : 0.0f;
  }
  // one warp per head: maximum over the chunks, the chunks' weights and the denominator
  for (int head = threadIdx.x >> 5; head < p.n; head += blockDim.x >> 5) {
    const int lane = threadIdx.x & 31;
    const float* base = head_base(head);
    float mm = -CUDART_INF_F;
    for (int c = lane; c < chunks; c += 32) mm = fmaxf(mm, base[c * cstride + H]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
    float l = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      const float f = exp2f(base[c * cstride + H] - muse);
      wts[head * chunks_max + c] = f;
      l += f * base[c * cstride + H + 1];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) s_linv[head & 63] = l;
  }
  __syncthreads();
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  int e = 0;
  for (int idx = threadIdx.x; idx < width; idx += blockDim.x, ++e) {
    const int head = idx / H, d = idx % H;
    const float* base = head_base(head) + d;
    const float* w = wts + head * chunks_max;
    float acc = 0.0f;
    int c = 0;
    if (e < 2) {
      const int npre = chunks < kPre ? chunks : kPre;
#pragma unroll
      for (int j = 0; j < kPre; ++j)
        if (j < npre) acc += w[j] * (e == 0 ? pre[0][j] : pre[1][j]);
      c = npre;
    }
    for (; c + 8 <= chunks; c += 8) {   // eight independent loads in flight per thread
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = base[(c + j) * cstride];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += w[c + j] * a[j];
    }
    for (; c < chunks; ++c) acc += w[c] * base[c * cstride];
    const float l = s_linv[head & 63];
    const float v = l > 0.0f ? acc / l : 0.0f;  // an empty sequence gives a zero row
    xs[idx] = v;
    if (p.out) static_cast<float*>(p.out)[(size_t)b * width + idx] = v;
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  const int k_pad = (width + 127) / 128 * 128;
  quantize_smem_row(xs, width, k_pad, b, p.m_alloc, mn, mx, p.q_tiled_out, p.out_scales, p.out_zps, red);
}

// Generic fallback (any head size / group size): one warp per (batch, head),
// plain fp32 loops. Correct for every shape the composite admits with one
// query token; used when the fast path's shape constraints do not hold.
template <int KV, bool QF32>
__global__ void sdpa_decode_generic_kernel(const SdpaParams p) {
  const int b = blockIdx.y, head = blockIdx.x, lane = threadIdx.x;
  const int group = p.n / p.nkv, kvh = head / group;
  const int len = p.lengths ? max(0, min(p.lengths[b], p.s_max)) : p.s_max;
  const int h = p.h;
  extern __shared__ float sh[];  // h floats of q, then s_max logits
  float* q = sh;
  float* logits = sh + h;
  for (int d = lane; d < h; d += 32) {
    const size_t qi = ((size_t)b * p.n + head) * h + d;
    q[d] = (QF32 ? static_cast<const float*>(p.q)[qi] : __half2float(static_cast<const __half*>(p.q)[qi])) * p.scale;
  }
  __syncwarp();
  auto kv_at = [&](const void* basep, const float* sc, int s, int d) -> float {
    const size_t tok = ((size_t)(p.shared_kv ? 0 : (p.rows_per_kv > 1 ? b / p.rows_per_kv : b)) * p.s_max + s) * p.nkv + kvh;
    const size_t idx = tok * h + d;
    if (KV == kKvF16) return __half2float(static_cast<const __half*>(basep)[idx]);
    if (KV == kKvF32) return static_cast<const float*>(basep)[idx];
    return (float)static_cast<const int8_t*>(basep)[idx] * sc[tok];
  };
  float mx = -CUDART_INF_F;
  for (int s = lane; s < len; s += 32) {
    float acc = 0.0f;
    for (int d = 0; d < h; ++d) acc += q[d] * kv_at(p.k, p.k_scale, s, d);
    if (p.logit_cap > 0.0f) acc = p.logit_cap * tanhf(acc / p.logit_cap);
    if (p.mask) acc += p.mask[(size_t)b * p.s_max + s];
    logits[s] = acc;
    mx = fmaxf(mx, acc);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.0f;
  for (int s = lane; s < len; s += 32) {
    const float e = expf(logits[s] - mx);
    logits[s] = e;
    sum += e;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int d = lane; d < h; d += 32) {
    float acc = 0.0f;
    for (int s = 0; s < len; ++s) acc += logits[s] * kv_at(p.v, p.v_scale, s, d);
    const float out = sum > 0.0f ? acc / sum : 0.0f;
    const size_t oi = ((size_t)b * p.n + head) * h + d;
    if (QF32) {
      static_cast<float*>(p.out)[oi] = out;
    } else {
      static_cast<__half*>(p.out)[oi] = __float2half_rn(out);
    }
  }
}

// Tokens per CTA. The kernel is latency-bound on short caches (one decode step of a small batch
// reads ~1 MB) and bandwidth-bound on long ragged batches: small chunks give many warps one short
// pass each, large chunks amortise the partial records. Depends only on (batch, s_max) so that the
// workspace size can be computed without the lengths.
int pick_chunk_tokens(int b, int s_max, int shared_kv) {
  // prompt pass (a warp per row and chunk): measured on B200 (1024 rows of one sequence, 8 query
  // heads x 256): 64-token chunks 128 us, 128 tokens 101 us, 256 tokens 95 us per layer
  if (shared_kv) {
    static const int chunk = [] {  // B200_ROWS_CHUNK: measurement knob
      const char* e = tuning_env("B200_ROWS_CHUNK");
      const int v = e ? atoi(e) : 0;
      return (v == 64 || v == 128 || v == 256 || v == 512) ? v : 256;
    }();
    return chunk;
  }
  static const int forced = [] {  // B200_SDPA_CHUNK: measurement knob
    const char* e = tuning_env("B200_SDPA_CHUNK");
    const int v = e ? atoi(e) : 0;
    return (v == 64 || v == 128 || v == 256 || v == 512) ? v : 0;
  }();
  if (forced) return forced;
  const long long tokens = (long long)b * s_max;
  if (tokens <= 16384) return 64;
  if (tokens <= 65536) return 128;
  if (tokens <= 262144) return 256;
  return 512;
}

template <int KV, int H, bool QF32>
cudaError_t launch_fast(const SdpaParams& p, cudaStream_t s) {
  const int chunk_tokens = pick_chunk_tokens(p.b, p.s_max, p.shared_kv);
  const int chunks_max = (p.s_max + chunk_tokens - 1) / chunk_tokens;
  dim3 grid(chunks_max, p.nkv, p.b);
  cudaError_t e;
  bool staged = false;
  static const bool ring_env = [] {  // B200_SDPA_RING=0: measurement knob, keeps the register-fed kernel
    const char* e = tuning_env("B200_SDPA_RING");
    return !(e && e[0] == '0');
  }();
  if constexpr (KV != kKvF32) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) == 0;
    if (ring_env && !p.shared_kv && aligned && chunk_tokens % kRingTokens == 0) {
      using L = RingLayout<KV, H>;
      // As many stages as keep two or three CTAs on an SM: the token loop is latency-bound and wants
      // warps more than it wants depth. Measured on B200, 16 ragged sequences up to 8192 tokens, head
      // size 256: fp16 rows (68 KB per stage) 23.4 us with one stage, 31.4 with three (one CTA per
      // SM); int8 rows (35 KB) 18.4 us with three, 21.9 with one. The register-fed kernel: 24.8 / 68 us.
      // Two CTAs per SM (about 104 KB each), at least two stages per CTA so that the next stage's copy runs
      // under this stage's arithmetic: with ONE 64-token stage per CTA (three CTAs per SM) every CTA of the
      // grid loads, computes, loads ... in step with the others, HBM idle half of the time (device-timer
      // stamps of one CTA, 16 ragged sequences, fp16 rows: 2.0 us copy + 1.8 us arithmetic per stage, strictly
      // in turn). Rows that do not fit two 64-token stages get shorter stages (fp16 at head size 256: 48).
      int stage_tokens = kRingTokens;
      while (stage_tokens > 16 && 2 * (2 * stage_tokens * L::kPitch) > 104 * 1024) stage_tokens -= 16;
      const int stage_bytes = 2 * stage_tokens * L::kPitch;
      int stages = std::min(kRingStagesMax, (chunk_tokens + stage_tokens - 1) / stage_tokens);
      stages = std::min(stages, std::max(1, (104 * 1024) / stage_bytes));
      static const int stages_env = [] {  // B200_SDPA_STAGES: measurement knob
        const char* e = tuning_env("B200_SDPA_STAGES");
        return e ? atoi(e) : 0;
      }();
      if (stages_env >= 1 && stages_env <= kRingStagesMax) stages = std::min(stages, stages_env);
      static const int tokens_env = [] {  // B200_SDPA_STAGE_TOKENS: measurement knob
        const char* e = tuning_env("B200_SDPA_STAGE_TOKENS");
        return e ? atoi(e) : 0;
      }();
      if (tokens_env == 16 || tokens_env == 32 || tokens_env == 48 || tokens_env == 64) stage_tokens = tokens_env;
      const size_t ring_bytes = (size_t)stages * (2 * stage_tokens * L::kPitch);
      const size_t smem = (ring_bytes > (size_t)L::kParkBytes ? ring_bytes : (size_t)L::kParkBytes) + 128;
      auto kernel = sdpa_decode_ring_kernel<KV, H, QF32>;
      static size_t configured[64] = {0};
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev < 0 || dev >= 64) dev = 0;
      if (configured[dev] < smem) {
        cudaError_t ea = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::smem_bytes(kRingStagesMax));
        if (ea != cudaSuccess) return ea;
        configured[dev] = L::smem_bytes(kRingStagesMax);
      }
      e = launch_chained(kernel, grid, dim3(kWarps * 32), smem, s, p, chunk_tokens, chunks_max, stages, stage_tokens);
      staged = true;
    }
  }
  if constexpr (KV != kKvF32) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) == 0;
    if (ring_env && p.shared_kv && aligned && chunk_tokens % kRingTokens == 0) {
      using L = RingLayout<KV, H>;
      // Whole 64-token stages here, even when only one fits: a warp's pass covers 64 tokens, and this kernel
      // is bound by its arithmetic, not by the copies (1024-token prompt, fp16 rows, measured per layer:
      // 65.7 us with one 64-token stage, 75.8 with two of 48, 90.2 with three of 32).
      int stage_tokens = kRingTokens;
      static const int rtokens_env = [] {  // B200_ROWS_STAGE_TOKENS: measurement knob
        const char* e = tuning_env("B200_ROWS_STAGE_TOKENS");
        return e ? atoi(e) : 0;
      }();
      if (rtokens_env == 16 || rtokens_env == 32 || rtokens_env == 48 || rtokens_env == 64) stage_tokens = rtokens_env;
      const int stage_bytes = 2 * stage_tokens * L::kPitch;
      int stages = std::min(kRingStagesMax, (chunk_tokens + stage_tokens - 1) / stage_tokens);
      stages = std::min(stages, std::max(1, (104 * 1024) / stage_bytes));
      const size_t ring_bytes = (size_t)stages * stage_bytes;
      const size_t smem = (ring_bytes > (size_t)L::kParkBytes ? ring_bytes : (size_t)L::kParkBytes) + 128;
      auto kernel = sdpa_rows_ring_kernel<KV, H, QF32>;
      static bool configured[64] = {false};
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev < 0 || dev >= 64) dev = 0;
      if (!configured[dev]) {
        cudaError_t ea = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::smem_bytes(kRingStagesMax));
        if (ea != cudaSuccess) return ea;
        configured[dev] = true;
      }
      const dim3 rgrid(chunks_max, p.nkv, (p.b + kWarps - 1) / kWarps);
      e = launch_chained(kernel, rgrid, dim3(kWarps * 32), smem, s, p, chunk_tokens, chunks_max, stages, stage_tokens);
      staged = true;
    }
  }
  if (staged) {
    // (the merge below is common to all variants)
  } else if (p.shared_kv) {
    // prompt pass: a warp per row, the CTA's rows share the chunk's traffic; long passes
    const dim3 rgrid(chunks_max, p.nkv, (p.b + kWarps - 1) / kWarps);
    static const int gpi = [] {  // B200_ROWS_GPI: measurement knob
      const char* e = tuning_env("B200_ROWS_GPI");
      return e ? atoi(e) : 4;
    }();
    if (gpi == 1) {
      e = launch_chained(sdpa_rows_kernel<KV, H, QF32, 1>, rgrid, dim3(kWarps * 32), 0, s, p, chunk_tokens, chunks_max);
    } else if (gpi == 4) {
      e = launch_chained(sdpa_rows_kernel<KV, H, QF32, 4>, rgrid, dim3(kWarps * 32), 0, s, p, chunk_tokens, chunks_max);
    } else {
      e = launch_chained(sdpa_rows_kernel<KV, H, QF32, 2>, rgrid, dim3(kWarps * 32), 0, s, p, chunk_tokens, chunks_max);
    }
  } else if (chunk_tokens == 64) {
    e = launch_chained(sdpa_decode_kernel<KV, H, QF32, 1>, grid, dim3(kWarps * 32), 0, s, p, chunk_tokens, chunks_max);
  } else if (chunk_tokens == 128) {
    e = launch_chained(sdpa_decode_kernel<KV, H, QF32, 2>, grid, dim3(kWarps * 32), 0, s, p, chunk_tokens, chunks_max);
  } else {
    e = launch_chained(sdpa_decode_kernel<KV, H, QF32, 4>, grid, dim3(kWarps * 32), 0, s, p, chunk_tokens, chunks_max);
  }
  if (e != cudaSuccess) return e;
  if (p.q_tiled_out) {
    if (p.n > 64) return cudaErrorInvalidValue;
    const size_t smem = sizeof(float) * ((size_t)p.n * H + (size_t)p.n * chunks_max);
    if (smem > 48 * 1024) {
      cudaError_t ea = cudaFuncSetAttribute(sdpa_merge_quant_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ea != cudaSuccess) return ea;
    }
    // a few rows (a decode step): the widest block per row; many rows (a prompt chunk): several rows per SM
    return launch_chained(sdpa_merge_quant_kernel<H>, dim3(p.b), dim3(p.b > 32 ? 256 : 1024), smem, s, p, chunk_tokens, chunks_max);
  }
  return launch_chained(sdpa_merge_kernel<H, QF32>, dim3(p.n, p.b), dim3(H), sizeof(float) * (size_t)chunks_max, s, p,
                        chunk_tokens, chunks_max);
}

template <int KV, bool QF32>
cudaError_t launch_kv(const SdpaParams& p, cudaStream_t s) {
  const int group = p.nkv > 0 ? p.n / p.nkv : 0;
  const bool fast = group >= 1 && group <= 8 && p.n % p.nkv == 0 && p.ws != nullptr &&
                    p.ws_bytes >= sdpa_workspace_bytes(p.b, p.n, p.nkv, p.h, p.s_max, p.shared_kv);
  if (p.q_tiled_out && (!fast || !QF32 || (p.h != 256 && p.h != 128 && p.h != 64)))
    return cudaErrorInvalidValue;  // fused output quantization exists on the fast f32-query path only
  if (fast && p.h == 256) return launch_fast<KV, 256, QF32>(p, s);
  if (fast && p.h == 128) return launch_fast<KV, 128, QF32>(p, s);
  if (fast && p.h == 64) return launch_fast<KV, 64, QF32>(p, s);
  const size_t smem = sizeof(float) * ((size_t)p.h + p.s_max);
  auto kernel = sdpa_decode_generic_kernel<KV, QF32>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  kernel<<<dim3(p.n, p.b), 32, smem, s>>>(p);
  return cudaGetLastError();
}

template <int KV, int H>
cudaError_t launch_attn_step_h(const AttnStepParams& p, cudaStream_t s) {
  constexpr size_t kBudget = 224 * 1024;
  const size_t fixed = ((sizeof(AttnStepSmem<H>) + 127) / 128) * 128;
  const int pitch = attn_row_pitch<KV, H>();
  // as many staged rows as a CTA's share of the longest cache needs, within the budget (the warps'
  // parked outputs take the staging area's place after the token loop)
  const int per_max = ((p.s_max + kAttnCluster - 1) / kAttnCluster + 15) / 16 * 16;
  int rows = (int)((kBudget - fixed) / (2 * (size_t)pitch));
  rows = rows / 8 * 8;
  if (rows > per_max) rows = per_max;
  const size_t staging = 2 * (size_t)rows * pitch;
  const size_t smem = fixed + (staging > attn_park_bytes<H>() ? staging : attn_park_bytes<H>());
  auto go = [&](auto kernel) -> cudaError_t {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    return launch_chained_cluster(kernel, dim3(p.b * kAttnCluster), dim3(kAttnWarps * 32), smem, kAttnCluster, s, p, rows);
  };
  // Staged rows are read from shared memory: passes are cheap, and the smallest loop body (16
  // tokens per warp and pass) costs the fewest instruction-cache misses, which dominate a kernel
  // that runs once per layer between large GEMVs. Rows read from the cache want long passes.
  if (per_max <= rows + 16 || per_max <= 64) return go(attn_step_cluster_kernel<KV, H, 1>);
  if (per_max <= 128) return go(attn_step_cluster_kernel<KV, H, 2>);
  return go(attn_step_cluster_kernel<KV, H, 4>);
}

}  // namespace

size_t sdpa_workspace_bytes(int b, int n, int nkv, int h, int s_max, int shared_kv) {
  (void)n;
  const int chunk_tokens = pick_chunk_tokens(b, s_max, shared_kv);
  const int chunks_max = (s_max + chunk_tokens - 1) / chunk_tokens;
  // [b][nkv][chunks][8 (query heads of the group, padded)][h + 2] floats
  return (size_t)b * nkv * chunks_max * 8 * partial_stride(h) * sizeof(float);
}

cudaError_t launch_sdpa_decode(const SdpaParams& p, cudaStream_t s) {
  const bool qf32 = p.q_dtype == 1;
  switch (p.kv_dtype) {
    case kKvF16: return qf32 ? launch_kv<kKvF16, true>(p, s) : launch_kv<kKvF16, false>(p, s);
    case kKvI8: return qf32 ? launch_kv<kKvI8, true>(p, s) : launch_kv<kKvI8, false>(p, s);
    case kKvF32: return qf32 ? launch_kv<kKvF32, true>(p, s) : launch_kv<kKvF32, false>(p, s);
    default: return cudaErrorInvalidValue;
  }
}

bool attn_step_supported(int n, int nkv, int h, int kv_dtype) {
  return nkv == 1 && n >= 1 && n <= 8 && (h == 64 || h == 128 || h == 256) && (kv_dtype == kKvF16 || kv_dtype == kKvI8);
}

cudaError_t launch_attn_step(const AttnStepParams& p, cudaStream_t s) {
  if (!attn_step_supported(p.n, 1, p.h, p.kv_dtype) || p.b < 1) return cudaErrorInvalidValue;
  if (p.kv_dtype == kKvI8) {
    if (p.h == 256) return launch_attn_step_h<kKvI8, 256>(p, s);
    if (p.h == 128) return launch_attn_step_h<kKvI8, 128>(p, s);
    return launch_attn_step_h<kKvI8, 64>(p, s);
  }
  if (p.h == 256) return launch_attn_step_h<kKvF16, 256>(p, s);
  if (p.h == 128) return launch_attn_step_h<kKvF16, 128>(p, s);
  return launch_attn_step_h<kKvF16, 64>(p, s);
}

}  // namespace b200
