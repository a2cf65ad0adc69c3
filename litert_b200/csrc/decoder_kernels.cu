// Glue kernels of the decode step of a Gemma-shaped decoder: everything between
// the quantized projections and the attention kernel. Each one fuses an
// elementwise stage with the per-row int8 quantization the next hybrid
// FULLY_CONNECTED needs, and writes the quantized row directly in the tiled
// layout the GEMM streams, so the only float activations that touch HBM are
// the residual stream and the projection outputs.
// The ops are the ones tensor/examples/gemma3/gemma3_graph.cc authors out of
// TFLite builtins: RMS norm, rotary embedding (x*cos + rotate_half(x)*sin,
// :150-176), GELU(tanh) * up (:118-146), residual add, hybrid embedding lookup
// (tflite/kernels/embedding_lookup.cc), first-index argmax.
#include <cooperative_groups.h>
#include <math_constants.h>

#include "argmax.cuh"
#include "common.cuh"
#include "decoder_kernels.h"
#include "quant.cuh"

namespace b200 {

namespace {

constexpr int kRowThreads = 256;
constexpr int kNormThreads = 1024;

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ float ld_peer(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Handshake of one exchange (see TpExchange). Called by every thread of the CTA after the
// predecessor kernel has completed; CTA 0 signals, every CTA waits. A wait that runs out
// (one second) records kStatusTimeoutPeer and lets the kernel finish with whatever is there.
__device__ __forceinline__ void tp_handshake(const TpExchange& x, bool signaller) {
  const unsigned long long epoch = *x.step_epoch * (unsigned long long)x.per_step + (unsigned long long)x.seq + 1ull;
  const int j = threadIdx.x;
  if (j < x.tp_size && j != x.tp_rank) {
    if (signaller) {
      __threadfence_system();
      st_release_sys(x.flag_out[j], epoch);
    }
    // after one wait has run out the status stays set and later waits give up at once
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long budget = wait_budget_ns(x.status);
    while (ld_acquire_sys(x.flags_in + j) < epoch) {
      if (*reinterpret_cast<volatile int*>(x.status) != 0) break;
      if (global_timer_ns() - t0 > budget) {
        atomicCAS(x.status, 0, kStatusTimeoutPeer);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
}

// h[b,:] = int8 embedding row * its scale * embed_scale; also attn_len = positions + 1.
__global__ void __launch_bounds__(kRowThreads) embed_kernel(const int32_t* __restrict__ tokens,
                                                            const int8_t* __restrict__ table,
                                                            const float* __restrict__ row_scales, int vocab, int d,
                                                            float embed_scale, float* __restrict__ h,
                                                            const int32_t* __restrict__ positions,
                                                            int32_t* __restrict__ attn_len,
                                                            unsigned long long* __restrict__ step_epoch) {
  pdl_enter();
  if (step_epoch && blockIdx.x == 0 && threadIdx.x == 0) *step_epoch += 1ull;
  const int b = blockIdx.x;
  // an id outside the table reads row 0 (the reference's op fails the invocation instead,
  // tflite/kernels/embedding_lookup.cc: a kernel cannot, and must not read out of bounds)
  int tok = tokens[b];
  if (tok < 0 || tok >= vocab) tok = 0;
  const float s = row_scales[tok];
  const int8_t* row = table + (size_t)tok * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    h[(size_t)b * d + i] = __fmul_rn(__fmul_rn((float)row[i], s), embed_scale);
  if (attn_len && threadIdx.x == 0) attn_len[b] = positions[b] + 1;
}

// Up to this many rows a glue kernel is one link of a latency chain (widest blocks, dry run, a cluster
// per row); above it, a throughput kernel (several rows per SM, one pass).
constexpr int kLatencyRows = 32;

// h += delta (optional); x = h * rsqrt(mean(h^2) + eps) * gain; quantize x.
__global__ void __launch_bounds__(kNormThreads) add_norm_quant_kernel(float* __restrict__ h,
                                                                     const float* __restrict__ delta,
                                                                     const float* __restrict__ gain, int d, int d_pad,
                                                                     float eps, int m_alloc,
                                                                     int8_t* __restrict__ q_tiled,
                                                                     float* __restrict__ scales,
                                                                     int32_t* __restrict__ zps, TpExchange xch,
                                                                     int first_pass, int batched) {
  extern __shared__ float xs[];
  __shared__ float red[32];
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const bool exchange = xch.tp_size > 1;
  float* hr = h + (size_t)b * d;
  // Two passes over the same code. The first runs while the producing kernel is still busy, on
  // whatever the inputs hold, and stores nothing: it only pulls the instructions (and the gain
  // vector) into the caches, which is most of what this short kernel otherwise waits for. The
  // second, after the dependency wait, is the real one. (first_pass 1: no dry run -- with hundreds of
  // rows the kernel is no longer a latency chain and the dry run would only double its work.)
#pragma unroll 1
  for (int pass = first_pass; pass < 2; ++pass) {
    const bool live = pass == 1;
    if (live) {
      pdl_wait();
      if (exchange) tp_handshake(xch, blockIdx.x == 0);
    }
    // inputs written by earlier kernels are read past L1 (__ldcg): the dry run must leave no stale
    // line behind for the real pass
    float ss = 0.0f;
    if (!exchange && batched) {
      // The row is updated in place, so the load of one element may not pass the store of the one before:
      // a thread's elements are all requested first (one L2 round trip for the lot), then added and stored.
      constexpr int kBatch = 2;
      const float* dr = delta ? delta + (size_t)b * d : nullptr;
      for (int i0 = threadIdx.x; i0 < d; i0 += kBatch * blockDim.x) {
        float vh[kBatch], vd[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int i = i0 + j * blockDim.x;
          vh[j] = i < d ? __ldcg(hr + i) : 0.0f;
        }
        if (dr) {
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            const int i = i0 + j * blockDim.x;
            vd[j] = i < d ? __ldcg(dr + i) : 0.0f;
          }
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int i = i0 + j * blockDim.x;
          if (i < d) {
            float v = vh[j];
            if (dr) {
              v = __fadd_rn(v, vd[j]);
              if (live) hr[i] = v;
            }
            xs[i] = v;
            ss += v * v;
          }
        }
      }
    } else
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float v = __ldcg(hr + i);
      if (exchange) {
        // sum of the ranks' partial outputs, in rank order on every rank
        float sum = 0.0f;
        for (int j = 0; j < xch.tp_size; ++j) {
          const float* pj = xch.partial[j] + (size_t)b * d + i;
          const float t = j == xch.tp_rank ? __ldcg(pj) : ld_peer(pj);
          sum = j == 0 ? t : __fadd_rn(sum, t);
        }
        v = __fadd_rn(v, sum);
        if (live) hr[i] = v;
      } else if (delta) {
        v = __fadd_rn(v, __ldcg(delta + (size_t)b * d + i));
        if (live) hr[i] = v;
      }
      xs[i] = v;
      ss += v * v;
    }
    ss = block_reduce(ss, [](float a, float c) { return a + c; }, 0.0f, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float v = __fmul_rn(__fmul_rn(xs[i], inv), gain[i]);
      xs[i] = v;
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
    quantize_smem_row(xs, d, d_pad, b, m_alloc, mn, mx, q_tiled, scales, zps, red, live);
    __syncthreads();
  }
}

// The same stage for a decode step's rows of at most 2 * kNormThreads elements (even length): a thread keeps its two neighbouring elements in registers from the load to the quantized bytes: no
// staging of the row in shared memory, the gains fetched before the dependency wait, one 16-bit store per thread.
// Measured on B200 (one row of 2048, stamps of the device timer after the wait): the staged form spent 0.7 us in its
// normalising loop (shared memory and gains per element) and 0.5 us in its quantizing loop, of 3.7 us.
__global__ void __launch_bounds__(kNormThreads) add_norm_quant_pair_kernel(float* __restrict__ h,
                                                                          const float* __restrict__ delta,
                                                                          const float* __restrict__ gain, int d, int d_pad,
                                                                          float eps, int m_alloc,
                                                                          int8_t* __restrict__ q_tiled,
                                                                          float* __restrict__ scales,
                                                                          int32_t* __restrict__ zps, TpExchange xch) {
  __shared__ float red[32];
  __shared__ float2 s_mm[32];
  __shared__ float s_inv;
  __shared__ int s_zp, s_zero;
  pdl_launch_dependents();
  const bool exchange = xch.tp_size > 1;  // the addend is the sum of the ranks' partial outputs, fetched from the peers
  const int b = blockIdx.x;
  const int i = 2 * (int)threadIdx.x;
  const bool have = i < d;  // d is even: both elements or none
  float* hr = h + (size_t)b * d;
  const float* dr = delta ? delta + (size_t)b * d : nullptr;
  const float2 g = have ? *reinterpret_cast<const float2*>(gain + i) : make_float2(0.0f, 0.0f);  // constants
  // two passes over the same code, as in add_norm_quant_kernel: a dry run before the dependency wait, then the real one
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const bool live = pass == 1;
    const bool pushed = exchange && xch.push_in != nullptr;
    if (live) {
      pdl_wait();
      if (exchange && !pushed) tp_handshake(xch, blockIdx.x == 0);
    }
    float2 v = make_float2(0.0f, 0.0f), e = make_float2(0.0f, 0.0f);
    if (have) v = __ldcg(reinterpret_cast<const float2*>(hr + i));
    if (have && pushed) {
      // The peers' GEMVs pushed their partials here as {value, epoch} messages: poll this rank's own memory until
      // both of this thread's messages from every peer carry the exchange's epoch (bounded), then sum in rank order.
      const uint32_t epoch32 =
          (uint32_t)(*xch.step_epoch * (unsigned long long)xch.per_step + (unsigned long long)xch.seq + 1ull);
      float2 part[kMaxTpRanks];
#pragma unroll
      for (int j = 0; j < kMaxTpRanks; ++j) {
        part[j] = make_float2(0.0f, 0.0f);
        if (j >= xch.tp_size) continue;
        if (j == xch.tp_rank) {
          part[j] = __ldcg(reinterpret_cast<const float2*>(xch.partial[j] + (size_t)b * d + i));
          continue;
        }
        if (!live) continue;  // (the dry run has nothing to wait for)
        const uint2* msg = xch.push_in + (size_t)j * xch.push_stride + (size_t)b * d + i;
        uint32_t v0, e0, v1, e1;
        const unsigned long long t0 = global_timer_ns();
        const unsigned long long budget = wait_budget_ns(xch.status);
        for (uint32_t spin = 0;; ++spin) {
          asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v0), "=r"(e0) : "l"(msg) : "memory");
          asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v1), "=r"(e1) : "l"(msg + 1) : "memory");
          if (e0 == epoch32 && e1 == epoch32) break;
          if ((spin & 15u) == 15u) {
            if (*reinterpret_cast<volatile int*>(xch.status) != 0) break;  // after one wait has run out, give up at once
            if (global_timer_ns() - t0 > budget) {
              atomicCAS(xch.status, 0, kStatusTimeoutPeer);
              break;
            }
          }
        }
        part[j] = make_float2(__uint_as_float(v0), __uint_as_float(v1));
      }
      e = part[0];
#pragma unroll
      for (int j = 1; j < kMaxTpRanks; ++j)
        if (j < xch.tp_size) e = make_float2(__fadd_rn(e.x, part[j].x), __fadd_rn(e.y, part[j].y));
    } else if (have && exchange) {
      // every rank's partial is requested before the first is used; summed in rank order on every rank
      float2 part[kMaxTpRanks];
#pragma unroll
      for (int j = 0; j < kMaxTpRanks; ++j) {
        part[j] = make_float2(0.0f, 0.0f);
        if (j < xch.tp_size) {
          const float* pj = xch.partial[j] + (size_t)b * d + i;
          part[j] = j == xch.tp_rank ? __ldcg(reinterpret_cast<const float2*>(pj)) : make_float2(ld_peer(pj), ld_peer(pj + 1));
        }
      }
      e = part[0];
#pragma unroll
      for (int j = 1; j < kMaxTpRanks; ++j)
        if (j < xch.tp_size) e = make_float2(__fadd_rn(e.x, part[j].x), __fadd_rn(e.y, part[j].y));
    } else if (have && dr) {
      e = __ldcg(reinterpret_cast<const float2*>(dr + i));
    }
    if (dr || exchange) {
      v.x = __fadd_rn(v.x, e.x);
      v.y = __fadd_rn(v.y, e.y);
      if (live && have) *reinterpret_cast<float2*>(hr + i) = v;
    }
    float ss = v.x * v.x + v.y * v.y;
    ss = block_reduce(ss, [](float a, float c) { return a + c; }, 0.0f, red);
    const float inv_rms = 1.0f / sqrtf(ss / (float)d + eps);
    const float x0 = __fmul_rn(__fmul_rn(v.x, inv_rms), g.x), x1 = __fmul_rn(__fmul_rn(v.y, inv_rms), g.y);
    float mn = have ? fminf(x0, x1) : 3.402823466e+38f, mx = have ? fmaxf(x0, x1) : -3.402823466e+38f;
    block_minmax(mn, mx, s_mm);
    if (threadIdx.x == 0) {  // one thread: the parameters take three double-precision divisions
      float sf, inv;
      int zp, zero_row;
      row_quant_params(mn, mx, true, &sf, &inv, &zp, &zero_row);
      s_zero = zero_row;
      s_inv = inv;
      s_zp = zp;
      if (live) {
        scales[b] = sf;
        zps[b] = zp;
      }
    }
    __syncthreads();
    if (i < d_pad) {  // the tiled row ends at the padded length: zeros beyond d
      uint32_t pair = 0;
      if (have && !s_zero) {
        const float inv = s_inv, zpf = (float)s_zp;
        pair = quantize_value(x0, inv, zpf, true) | (quantize_value(x1, inv, zpf, true) << 8);
      }
      if (live) *reinterpret_cast<uint16_t*>(q_tiled + q_tiled_offset(b, i, m_alloc)) = (uint16_t)pair;
    }
    __syncthreads();  // the shared scratch is rewritten by the next pass
  }
}

// tanh(u) = 1 - 2 / (1 + e^(2u)) on the fast exponential and reciprocal units: absolute error about 1e-7
// (the result is used as 1 + tanh, so absolute error is what counts), saturating to +-1 through e^(2u) = inf / 0.
// tanhf's range-split polynomial costs five times the instructions, and a prompt pass evaluates 16 M of these
// per layer: the GeGLU kernel was bound by it (50 us per layer for 1024 rows, 134 MB read).
__device__ __forceinline__ float tanh_fast(float u) {
  const float e = exp2f(__fmul_rn(u, 2.885390081777927f));  // e^(2u) = 2^(2u log2 e)
  return __fsub_rn(1.0f, __fdividef(2.0f, __fadd_rn(1.0f, e)));
}

__device__ __forceinline__ float gelu_tanh(float v) {
  // every product and sum rounded on its own, in the order a C compiler without contraction gives
  // (left to right): the row is quantized to int8 next, where one ulp can flip a value
  const float k0 = 0.7978845608028654f;
  const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
  const float th = tanh_fast(__fmul_rn(k0, __fadd_rn(v, cube)));
  return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, th));
}

// f = gelu_tanh(gate) * up from the fused projection output [b, 2 f]; quantize f per row.
// A row (16384 elements at the benchmark's size) is spread over a cluster of kGegluCluster CTAs:
// each computes its slice into shared memory with its local min / max, the CTAs exchange those
// through distributed shared memory, and each then quantizes its slice with the row's parameters.
// With many rows (a prompt chunk) one CTA takes a whole row (CL = 1) and there is no dry run.
constexpr int kGegluCluster = 8;
constexpr int kGegluThreads = 512;

template <int CL>
__global__ void __launch_bounds__(kGegluThreads) geglu_quant_kernel(const float* __restrict__ gate_up, int f, int f_pad,
                                                                    int per_cta, int m_alloc,
                                                                    int8_t* __restrict__ q_tiled,
                                                                    float* __restrict__ scales,
                                                                    int32_t* __restrict__ zps) {
  namespace cg = cooperative_groups;
  extern __shared__ float xs[];
  __shared__ float2 s_mm[32];
  __shared__ __align__(8) float2 s_all[CL];  // every CTA's min / max, pushed here by the CTAs themselves
  __shared__ __align__(8) uint64_t s_bar[2];  // one per pass: completes when all CL messages are in
  cg::cluster_group cluster = cg::this_cluster();
  if (CL > 1 && threadIdx.x == 0) {
    mbar_init(&s_bar[0], 1);
    mbar_init(&s_bar[1], 1);
    mbar_fence_init();
  }
  const int rank = CL > 1 ? (int)cluster.block_rank() : 0;
  const int b = blockIdx.x / CL;
  pdl_launch_dependents();
  const float* g = gate_up + (size_t)b * 2 * f;
  const float* u = g + f;
  const int lo = rank * per_cta, hi = min(f, lo + per_cta);
  const bool vec = (f & 3) == 0;  // rows and slices then start on 16-byte boundaries
  if (CL > 1) cluster.sync();  // every CTA of the cluster runs: remote stores are legal from here on
  // two passes over the same code: a dry run that warms the instruction caches while the producing
  // kernel is still busy (nothing stored), then the real one after the dependency wait
#pragma unroll 1
  for (int pass = CL > 1 ? 0 : 1; pass < 2; ++pass) {
    const bool live = pass == 1;
    if (live) pdl_wait();
    float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
    if (vec) {
      for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
        const float4 gv = __ldcg(reinterpret_cast<const float4*>(g + i));  // past L1: see add_norm_quant_kernel
        const float4 uv = __ldcg(reinterpret_cast<const float4*>(u + i));
        float4 v;
        v.x = __fmul_rn(gelu_tanh(gv.x), uv.x);
        v.y = __fmul_rn(gelu_tanh(gv.y), uv.y);
        v.z = __fmul_rn(gelu_tanh(gv.z), uv.z);
        v.w = __fmul_rn(gelu_tanh(gv.w), uv.w);
        *reinterpret_cast<float4*>(xs + (i - lo)) = v;
        mn = fminf(fminf(mn, fminf(v.x, v.y)), fminf(v.z, v.w));
        mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
      }
    } else {
      for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = __fmul_rn(gelu_tanh(__ldcg(g + i)), __ldcg(u + i));
        xs[i - lo] = v;
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
    }
    block_minmax(mn, mx, s_mm);
    if (CL > 1) {
      // The slices' extremes go to every CTA of the cluster by remote stores that also count as transaction
      // bytes on the receiver's barrier (st.async): nobody waits for a remote read or for a cluster-wide
      // barrier (0.4 us dearer per launch, measured on B200), and every thread derives the row's parameters
      // itself.
      if (threadIdx.x == 0) mbar_arrive_expect_tx(&s_bar[pass], CL * 8u);
      if (threadIdx.x < CL)
        st_async_cluster_f32x2(map_to_rank(smem_u32(&s_all[rank]), threadIdx.x), mn, mx,
                               map_to_rank(smem_u32(&s_bar[pass]), threadIdx.x));
      mbar_drain_bounded(&s_bar[pass], 0);  // (bounded: a lost message ends in wrong numbers, never in a hang)
#pragma unroll
      for (int r = 0; r < CL; ++r) {
        mn = fminf(mn, s_all[r].x);
        mx = fmaxf(mx, s_all[r].y);
      }
    }
    float sf, inv;
    int zp, zero_row;
    row_quant_params(mn, mx, true, &sf, &inv, &zp, &zero_row);
    if (threadIdx.x == 0 && rank == 0 && live) {
      scales[b] = sf;
      zps[b] = zp;
    }
    const bool zero = zero_row != 0;
    const float zpf = (float)zp;
    const int k_end = min(lo + per_cta, f_pad);  // the tiled row ends at the padded length
    for (int k4 = lo + threadIdx.x * 4; k4 < k_end; k4 += blockDim.x * 4) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (k4 + e < f && !zero) word |= quantize_value(xs[k4 + e - lo], inv, zpf, true) << (8 * e);
      if (live) *reinterpret_cast<uint32_t*>(q_tiled + q_tiled_offset(b, k4, m_alloc)) = word;
    }
    // (no barrier at the end: a CTA cannot leave before all the messages addressed to it have arrived, and
    // each pass has a barrier of its own, so a fast CTA's second message cannot complete a slow one's first)
    __syncthreads();  // xs and s_mm are rewritten by the next pass
  }
}

// Rotary embedding of q and k from the fused qkv projection output, and the
// cache append. grid (b, heads + kv_heads + kv_heads), head_dim / 2 threads. Row b appends to the
// cache of sequence b, or, with one_sequence (a prompt pass), every row to the cache passed in.
// The rotation is the graph's x * cos + rotate_half(x) * sin over the cos / sin tensors the host side
// prepares (tensor/examples/gemma3/gemma3_graph.cc:150-176): rope_cs[pos][i] = {cos, sin} of pair i,
// max_seq + 1 positions; every product and sum rounded on its own, as separate MUL and ADD ops give.
template <bool KV_I8>
__global__ void rope_cache_kernel(const float* __restrict__ qkv, int heads, int kv_heads, int head_dim,
                                  const float2* __restrict__ rope_cs, const int32_t* __restrict__ positions, int max_seq,
                                  float* __restrict__ q_out, void* __restrict__ k_cache, void* __restrict__ v_cache,
                                  float* __restrict__ k_scale, float* __restrict__ v_scale, int one_sequence) {
  __shared__ float red[32];
  pdl_enter();
  const int b = blockIdx.x, slot = blockIdx.y, i = threadIdx.x, half = head_dim / 2;
  const int pos = positions[b];
  const float* src = qkv + ((size_t)b * (heads + 2 * kv_heads) + slot) * head_dim;
  float x1 = src[i], x2 = src[i + half];
  const bool is_v = slot >= heads + kv_heads;
  if (!is_v) {
    const float2 r = rope_cs[(size_t)min(pos, max_seq) * half + i];
    const float r1 = __fsub_rn(__fmul_rn(x1, r.x), __fmul_rn(x2, r.y));
    const float r2 = __fadd_rn(__fmul_rn(x2, r.x), __fmul_rn(x1, r.y));
    x1 = r1;
    x2 = r2;
  }
  if (slot < heads) {
    float* dst = q_out + ((size_t)b * heads + slot) * head_dim;
    dst[i] = x1;
    dst[i + half] = x2;
    return;
  }
  const int kvh = is_v ? slot - heads - kv_heads : slot - heads;
  if (pos >= max_seq) return;  // cache full: the step is ignored for this sequence
  const size_t tok = ((size_t)(one_sequence ? 0 : b) * max_seq + pos) * kv_heads + kvh;
  if constexpr (KV_I8) {
    // symmetric per token and kv head: scale = max|row| / 127
    float amax = fmaxf(fabsf(x1), fabsf(x2));
    amax = block_reduce(amax, [](float a, float c) { return fmaxf(a, c); }, 0.0f, red);
    const float sc = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    int8_t* dst = static_cast<int8_t*>(is_v ? v_cache : k_cache) + tok * head_dim;
    dst[i] = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(x1, sc))));
    dst[i + half] = (int8_t)max(-127, min(127, __float2int_rn(__fdiv_rn(x2, sc))));
    if (i == 0) (is_v ? v_scale : k_scale)[tok] = sc;
  } else {
    __half* dst = static_cast<__half*>(is_v ? v_cache : k_cache) + tok * head_dim;
    dst[i] = __float2half_rn(x1);
    dst[i + half] = __float2half_rn(x2);
  }
}

// grid (parts, b): each CTA scans a slice of the row.
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits, int n, int parts,
                                                             float soft_cap, float* __restrict__ part_val,
                                                             int32_t* __restrict__ part_idx) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_enter();
  const int b = blockIdx.y, part = blockIdx.x;
  const int per = (n + parts - 1) / parts;
  const int lo = part * per, hi = min(n, lo + per);
  const float* row = logits + (size_t)b * n;
  BestPick best{lo < n ? soft_capped(row[lo], soft_cap) : -CUDART_INF_F, lo < n ? lo : 0x7fffffff};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) best = better_pick(best, BestPick{soft_capped(row[i], soft_cap), i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPick other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better_pick(best, other);
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best.v;
    si[threadIdx.x >> 5] = best.i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) best = better_pick(best, BestPick{sv[w], si[w]});
    part_val[(size_t)b * parts + part] = best.v;
    part_idx[(size_t)b * parts + part] = best.i;
  }
}

// grid b, 32 threads: final reduction; also advances the sequence position.
__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int32_t* __restrict__ part_idx,
                                    int parts, int idx_offset, int32_t* __restrict__ next_tokens,
                                    int32_t* __restrict__ positions, int max_seq, float2* __restrict__ pair_out) {
  pdl_enter();
  const int b = blockIdx.x;
  BestPick best{part_val[(size_t)b * parts], part_idx[(size_t)b * parts]};
  for (int i = threadIdx.x; i < parts; i += 32)
    best = better_pick(best, BestPick{part_val[(size_t)b * parts + i], part_idx[(size_t)b * parts + i]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    BestPick other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better_pick(best, other);
  }
  if (threadIdx.x == 0) {
    if (pair_out) {
      pair_out[b] = make_float2(best.v, (float)(best.i + idx_offset));  // exact below 2^24
    } else {
      next_tokens[b] = best.i + idx_offset;
      if (positions && positions[b] < max_seq) positions[b] += 1;
    }
  }
}

struct PairTable {
  const float2* p[kMaxTpRanks];
};

// grid b, 32 threads: winner over the ranks' candidates (larger value, then lower index).
__global__ void argmax_pick_kernel(PairTable pairs, int tp_size, int32_t* __restrict__ next_tokens,
                                   int32_t* __restrict__ positions, int max_seq, TpExchange xch) {
  pdl_enter();
  if (xch.tp_size > 1) tp_handshake(xch, blockIdx.x == 0);
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    BestPick best{-CUDART_INF_F, 0x7fffffff};
    for (int j = 0; j < tp_size; ++j) {
      const float* pj = reinterpret_cast<const float*>(pairs.p[j] + b);
      const float v = ld_peer(pj), fi = ld_peer(pj + 1);
      const BestPick cand{v, (int)fi};
      best = j == 0 ? cand : better_pick(best, cand);
    }
    next_tokens[b] = best.i;
    if (positions[b] < max_seq) positions[b] += 1;
  }
}

}  // namespace

void fill_rope_table(float* cs, int positions, int head_dim, float base) {
  const int half = head_dim / 2;
  for (int pos = 0; pos < positions; ++pos)
    for (int i = 0; i < half; ++i) {
      const float freq = powf(base, -2.0f * (float)i / (float)head_dim);
      const float ang = (float)pos * freq;
      cs[((size_t)pos * half + i) * 2] = cosf(ang);
      cs[((size_t)pos * half + i) * 2 + 1] = sinf(ang);
    }
}

cudaError_t launch_embed(const int32_t* tokens, const int8_t* table, const float* row_scales, int batch, int vocab, int d,
                         float embed_scale, float* h, const int32_t* positions, int32_t* attn_len,
                         unsigned long long* step_epoch, cudaStream_t s) {
  return launch_chained(embed_kernel, dim3(batch), dim3(kRowThreads), 0, s, tokens, table, row_scales, vocab, d, embed_scale, h, positions,
                        attn_len, step_epoch);
}

cudaError_t launch_add_norm_quant(float* h, const float* delta, const float* gain, int batch, int d, float eps,
                                  int m_alloc, int8_t* q_tiled, float* scales, int32_t* zps, const TpExchange* xch,
                                  cudaStream_t s) {
  const int d_pad = (d + 127) / 128 * 128;
  const TpExchange x = xch ? *xch : TpExchange();
  // a decode step's few rows: the widest block and a dry run; a prompt chunk's many rows: several rows per SM
  const bool many = batch > kLatencyRows;
  const bool pair_ok = !many && d % 2 == 0 && d_pad <= 2 * kNormThreads && (reinterpret_cast<uintptr_t>(h) & 7) == 0 &&
                       (reinterpret_cast<uintptr_t>(delta) & 7) == 0 && (reinterpret_cast<uintptr_t>(gain) & 7) == 0;
  if (x.push_in && !pair_ok) return cudaErrorInvalidValue;  // pushed partials are only read by the register-resident kernel
  if (!many && d % 2 == 0 && d_pad <= 2 * kNormThreads && (reinterpret_cast<uintptr_t>(h) & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(delta) & 7) == 0 && (reinterpret_cast<uintptr_t>(gain) & 7) == 0 && !tuning_env("B200_NORM_STAGED"))
    return launch_chained(add_norm_quant_pair_kernel, dim3(batch), dim3(kNormThreads), 0, s, h, delta, gain, d, d_pad, eps, m_alloc,
                          q_tiled, scales, zps, x);
  int batched = 1;
  if (const char* e = tuning_env("B200_NORM_BATCHED")) batched = atoi(e);  // measurement knob
  return launch_chained(add_norm_quant_kernel, dim3(batch), dim3(many ? 256 : kNormThreads), sizeof(float) * d, s, h, delta, gain,
                        d, d_pad, eps, m_alloc, q_tiled, scales, zps, x, many ? 1 : 0, batched);
}

cudaError_t launch_geglu_quant(const float* gate_up, int batch, int f, int m_alloc, int8_t* q_tiled, float* scales,
                               int32_t* zps, cudaStream_t s) {
  const int f_pad = (f + 127) / 128 * 128;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (batch > kLatencyRows && sizeof(float) * f_pad <= 160 * 1024) {
    // many rows: a CTA per row
    const size_t smem = sizeof(float) * f_pad;
    static bool configured1[64] = {false};
    if (!configured1[dev] && smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(geglu_quant_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e != cudaSuccess) return e;
      configured1[dev] = true;
    }
    return launch_chained(geglu_quant_kernel<1>, dim3(batch), dim3(kGegluThreads), smem, s, gate_up, f, f_pad, f_pad, m_alloc,
                          q_tiled, scales, zps);
  }
  // slice per CTA: a multiple of 128 elements so that slices tile the padded row exactly
  const int per_cta = ((f_pad / 128 + kGegluCluster - 1) / kGegluCluster) * 128;
  const size_t smem = sizeof(float) * per_cta;
  if (smem > 160 * 1024) return cudaErrorInvalidValue;
  static bool configured[64] = {false};
  if (!configured[dev] && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(geglu_quant_kernel<kGegluCluster>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_chained_cluster(geglu_quant_kernel<kGegluCluster>, dim3(batch * kGegluCluster), dim3(kGegluThreads), smem,
                                kGegluCluster, s, gate_up, f, f_pad, per_cta, m_alloc, q_tiled, scales, zps);
}

cudaError_t launch_rope_cache(const float* qkv, int batch, int heads, int kv_heads, int head_dim, const float2* rope_cs,
                              const int32_t* positions, int max_seq, float* q_out, void* k_cache, void* v_cache,
                              float* k_scale, float* v_scale, int kv_int8, int one_sequence, cudaStream_t s) {
  dim3 grid(batch, heads + 2 * kv_heads);
  if (kv_int8) {
    return launch_chained(rope_cache_kernel<true>, grid, dim3(head_dim / 2), 0, s, qkv, heads, kv_heads, head_dim, rope_cs,
                          positions, max_seq, q_out, k_cache, v_cache, k_scale, v_scale, one_sequence);
  }
  return launch_chained(rope_cache_kernel<false>, grid, dim3(head_dim / 2), 0, s, qkv, heads, kv_heads, head_dim, rope_cs,
                        positions, max_seq, q_out, k_cache, v_cache, k_scale, v_scale, one_sequence);
}

cudaError_t launch_argmax(const float* logits, int batch, int n, int idx_offset, float soft_cap, float* part_val,
                          int32_t* part_idx, int32_t* next_tokens, int32_t* positions, int max_seq, float2* pair_out,
                          cudaStream_t s) {
  cudaError_t e = launch_chained(argmax_partial_kernel, dim3(kArgmaxParts, batch), dim3(256), 0, s, logits, n, (int)kArgmaxParts,
                                 soft_cap, part_val, part_idx);
  if (e != cudaSuccess) return e;
  return launch_chained(argmax_final_kernel, dim3(batch), dim3(32), 0, s, (const float*)part_val, (const int32_t*)part_idx,
                        (int)kArgmaxParts, idx_offset, next_tokens, positions, max_seq, pair_out);
}

cudaError_t launch_argmax_final(const float* part_val, const int32_t* part_idx, int batch, int parts, int idx_offset,
                                int32_t* next_tokens, int32_t* positions, int max_seq, float2* pair_out, cudaStream_t s) {
  return launch_chained(argmax_final_kernel, dim3(batch), dim3(32), 0, s, part_val, part_idx, parts, idx_offset, next_tokens,
                        positions, max_seq, pair_out);
}

cudaError_t launch_argmax_pick(const float2* const* pairs, int tp_size, int batch, int32_t* next_tokens,
                               int32_t* positions, int max_seq, const TpExchange* xch, cudaStream_t s) {
  if (tp_size < 1 || tp_size > kMaxTpRanks) return cudaErrorInvalidValue;
  PairTable t;
  for (int j = 0; j < kMaxTpRanks; ++j) t.p[j] = j < tp_size ? pairs[j] : nullptr;
  const TpExchange x = xch ? *xch : TpExchange();
  return launch_chained(argmax_pick_kernel, dim3(batch), dim3(32), 0, s, t, tp_size, next_tokens, positions, max_seq, x);
}

}  // namespace b200
