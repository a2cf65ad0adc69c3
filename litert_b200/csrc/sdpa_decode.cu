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
template <int KV>
__device__ __forceinline__ void load8(const void* row, int d0, bool valid, uint32_t (&out)[4]) {
  if (!valid) {
    out[0] = out[1] = out[2] = out[3] = 0u;
    return;
  }
  if constexpr (KV == kKvF16) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(row) + d0));
    out[0] = v.x;
    out[1] = v.y;
    out[2] = v.z;
    out[3] = v.w;
  } else if constexpr (KV == kKvI8) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(static_cast<const int8_t*>(row) + d0));
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

// GPI = groups of 16 tokens a warp takes per pass (1, 2 or 4): small for short caches, where the
// kernel is latency-bound and wants as many warps as possible, 4 for long ones.
template <int KV, int H, bool QF32, int GPI>
__global__ void __launch_bounds__(kWarps * 32) sdpa_decode_kernel(const SdpaParams p, const int chunk_tokens,
                                                                  const int chunks_max) {
  constexpr int DB = H < 128 ? H : 128;  // head-dim block of the PV step
  constexpr int NBLK = H / DB;
  constexpr int TPB = DB / 16;           // m16 tiles per block
  constexpr int DPT = DB / 8;            // head-dim elements per thread per block (8 or 16)
  constexpr int KSTEPS = H / 32;         // 16-byte K pieces per thread per row
  constexpr int kTokensPerWarpIter = 16 * GPI;

  pdl_enter();
  const int b = blockIdx.z, kvh = blockIdx.y, chunk = blockIdx.x;
  const int len = p.lengths ? min(p.lengths[b], p.s_max) : p.s_max;
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

  const size_t row_stride = (size_t)p.nkv * H * kv_elem_bytes<KV>();
  const uint8_t* kbase = static_cast<const uint8_t*>(p.k) + ((size_t)b * p.s_max * p.nkv + kvh) * H * kv_elem_bytes<KV>();
  const uint8_t* vbase = static_cast<const uint8_t*>(p.v) + ((size_t)b * p.s_max * p.nkv + kvh) * H * kv_elem_bytes<KV>();
  const float* ksc = p.k_scale ? p.k_scale + (size_t)b * p.s_max * p.nkv + kvh : nullptr;
  const float* vsc = p.v_scale ? p.v_scale + (size_t)b * p.s_max * p.nkv + kvh : nullptr;
  const float* maskp = p.mask ? p.mask + (size_t)b * p.s_max : nullptr;

  // online softmax state for heads 2t and 2t+1 (log2 domain)
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l_run[2] = {0.0f, 0.0f};
  float o[NBLK * TPB][4];
#pragma unroll
  for (int i = 0; i < NBLK * TPB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  const float scale_log2 = p.scale * kLog2e;

  for (int base = c0 + warp * kTokensPerWarpIter; base < c1; base += kWarps * kTokensPerWarpIter) {
    // ---- S^T = K Q^T for GPI groups of 16 tokens ----
    float s[GPI][4];
#pragma unroll
    for (int gi = 0; gi < GPI; ++gi) {
      s[gi][0] = s[gi][1] = s[gi][2] = s[gi][3] = 0.0f;
      const int ta = base + gi * 16 + g, tb = ta + 8;
      const bool va = ta < c1, vb = tb < c1;
      const void* ra = kbase + (size_t)ta * row_stride;
      const void* rb = kbase + (size_t)tb * row_stride;
#pragma unroll
      for (int i = 0; i < KSTEPS; ++i) {
        uint32_t ka[4], kb[4];
        const int d0 = 8 * (t + 4 * i);
        load8<KV>(ra, d0, va, ka);
        load8<KV>(rb, d0, vb, kb);
        mma_f16(s[gi], ka[0], kb[0], ka[1], kb[1], qf[i][0], qf[i][1]);
        mma_f16(s[gi], ka[2], kb[2], ka[3], kb[3], qf[i][2], qf[i][3]);
      }
      // scale (and dequantise), cap, mask; work in the log2 domain
      float fa = scale_log2, fb = scale_log2;
      if constexpr (KV == kKvI8) {
        fa *= va ? ksc[(size_t)ta * p.nkv] : 0.0f;
        fb *= vb ? ksc[(size_t)tb * p.nkv] : 0.0f;
      }
      s[gi][0] *= fa;
      s[gi][1] *= fa;
      s[gi][2] *= fb;
      s[gi][3] *= fb;
      if (p.logit_cap > 0.0f) {
        const float c = p.logit_cap * kLog2e, ic = 1.0f / c;
#pragma unroll
        for (int e = 0; e < 4; ++e) s[gi][e] = c * tanhf(s[gi][e] * ic);
      }
      if (maskp) {
        const float ma = va ? maskp[ta] * kLog2e : 0.0f, mb = vb ? maskp[tb] * kLog2e : 0.0f;
        s[gi][0] += ma;
        s[gi][1] += ma;
        s[gi][2] += mb;
        s[gi][3] += mb;
      }
      if (!va) s[gi][0] = s[gi][1] = -CUDART_INF_F;
      if (!vb) s[gi][2] = s[gi][3] = -CUDART_INF_F;
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
        const float sa = ta < c1 ? vsc[(size_t)ta * p.nkv] : 0.0f;
        const float sb = tb < c1 ? vsc[(size_t)tb * p.nkv] : 0.0f;
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
          const void* row = vbase + (size_t)rows[r] * row_stride;
          const bool ok = rows[r] < c1;
#pragma unroll
          for (int hlf = 0; hlf < DPT / 8; ++hlf) {
            uint32_t tmp[4];
            load8<KV>(row, blk * DB + DPT * g + 8 * hlf, ok, tmp);
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

  // ---- merge the warps of this CTA ----
  // l is still per-thread; reduce over the token lanes
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float v = l_run[e];
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    l_run[e] = v;
  }
  __shared__ float sm_m[kWarps][8], sm_l[kWarps][8];
  __shared__ float sm_o[kWarps][8][H + 4];
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

// Reduces the per-chunk partials of one (batch, query head): grid (n, b),
// H threads.
template <int H, bool QF32>
__global__ void sdpa_merge_kernel(const SdpaParams p, const int chunk_tokens, const int chunks_max) {
  pdl_enter();
  const int b = blockIdx.y, head = blockIdx.x, d = threadIdx.x;
  const int group = p.n / p.nkv;
  const int kvh = head / group, hg = head % group;
  const int len = p.lengths ? min(p.lengths[b], p.s_max) : p.s_max;
  const int chunks = (len + chunk_tokens - 1) / chunk_tokens;
  const float* base = p.ws + ((((size_t)b * p.nkv + kvh) * chunks_max) * 8 + hg) * partial_stride(H);
  const size_t cstride = 8 * partial_stride(H);
  float mm = -CUDART_INF_F;
  for (int c = 0; c < chunks; ++c) mm = fmaxf(mm, base[c * cstride + H]);
  const float muse = mm == -CUDART_INF_F ? 0.0f : mm;
  float acc = 0.0f, l = 0.0f;
  for (int c = 0; c < chunks; ++c) {
    const float f = exp2f(base[c * cstride + H] - muse);
    acc += f * base[c * cstride + d];
    l += f * base[c * cstride + H + 1];
  }
  const float out = acc / l;
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
  const int len = p.lengths ? min(p.lengths[b], p.s_max) : p.s_max;
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
    const float v = acc / s_linv[head & 63];
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
  const int len = p.lengths ? min(p.lengths[b], p.s_max) : p.s_max;
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
    const size_t idx = (((size_t)b * p.s_max + s) * p.nkv + kvh) * h + d;
    if (KV == kKvF16) return __half2float(static_cast<const __half*>(basep)[idx]);
    if (KV == kKvF32) return static_cast<const float*>(basep)[idx];
    return (float)static_cast<const int8_t*>(basep)[idx] * sc[((size_t)b * p.s_max + s) * p.nkv + kvh];
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
    const float out = acc / sum;
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
int pick_chunk_tokens(int b, int s_max) {
  const long long tokens = (long long)b * s_max;
  if (tokens <= 16384) return 64;
  if (tokens <= 65536) return 128;
  if (tokens <= 262144) return 256;
  return 512;
}

template <int KV, int H, bool QF32>
cudaError_t launch_fast(const SdpaParams& p, cudaStream_t s) {
  const int chunk_tokens = pick_chunk_tokens(p.b, p.s_max);
  const int chunks_max = (p.s_max + chunk_tokens - 1) / chunk_tokens;
  dim3 grid(chunks_max, p.nkv, p.b);
  cudaError_t e;
  if (chunk_tokens == 64) {
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
    return launch_chained(sdpa_merge_quant_kernel<H>, dim3(p.b), dim3(1024), smem, s, p, chunk_tokens, chunks_max);
  }
  return launch_chained(sdpa_merge_kernel<H, QF32>, dim3(p.n, p.b), dim3(H), 0, s, p, chunk_tokens, chunks_max);
}

template <int KV, bool QF32>
cudaError_t launch_kv(const SdpaParams& p, cudaStream_t s) {
  const int group = p.nkv > 0 ? p.n / p.nkv : 0;
  const bool fast = group >= 1 && group <= 8 && p.n % p.nkv == 0 && p.ws != nullptr &&
                    p.ws_bytes >= sdpa_workspace_bytes(p.b, p.n, p.nkv, p.h, p.s_max);
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

}  // namespace

size_t sdpa_workspace_bytes(int b, int n, int nkv, int h, int s_max) {
  (void)n;
  const int chunk_tokens = pick_chunk_tokens(b, s_max);
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

}  // namespace b200
