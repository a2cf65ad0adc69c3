// Resident Gemma-shaped decoder: weights packed once on the device, KV cache on
// the device, one decode step = one CUDA graph over the GEMV, attention and glue
// kernels. C ABI in include/litert_b200.h (b200_decoder_*).
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>

#include "../../include/litert_b200.h"
#include "common.cuh"
#include "decoder_kernels.h"
#include "kernels.h"

namespace {

using namespace b200;

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  ~DevBuf() { release(); }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
    bytes = 0;
  }
  cudaError_t alloc(size_t n) {
    release();
    if (n == 0) return cudaSuccess;
    cudaError_t e = cudaMalloc(&p, n);
    if (e == cudaSuccess) bytes = n;
    return e;
  }
  template <typename T>
  T* as() const { return static_cast<T*>(p); }
};

// One packed projection: y[n] = hybrid_fc(x[k]).
struct Projection {
  int n = 0, k = 0;
  DevBuf packed, row_sums, scales;
};

struct Layer {
  Projection qkv, o, gate_up, down;
  DevBuf norm1, norm2;
  DevBuf k_cache, v_cache, k_scale, v_scale;
};

// Scratch of a prompt pass: the decode step's buffers hold max_batch rows, a prompt chunk up to `rows`.
struct PrefillBufs {
  int rows = 0;
  DevBuf tokens, positions, attn_len, h, qkv, q, gate_up, proj, down_out;
  DevBuf q_d, q_a, q_f, sc_d, sc_a, sc_f, zp_d, zp_a, zp_f, sdpa_ws;
  int32_t* h_stage = nullptr;  // pinned: tokens then positions of one chunk
  ~PrefillBufs() {
    if (h_stage) cudaFreeHost(h_stage);
  }
};

}  // namespace

struct b200_decoder {
  b200_decoder_config cfg;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  std::vector<std::unique_ptr<Layer>> layers;
  Projection lm_head;
  DevBuf embed_table, embed_scales, final_norm;
  DevBuf rope_cs;  // {cos, sin} of the rotation angles, [max_seq + 1][head_dim / 2], computed on the host
  // activations and scratch
  DevBuf tokens, next_tokens, positions, attn_len;
  DevBuf h, h2, qkv, q, attn, gate_up, logits;  // h / h2: residual stream, ping-pong when the norm is fused into a GEMV
  float *proj = nullptr, *down_out = nullptr;  // inside comm
  DevBuf q_d, q_a, q_f;         // tiled int8 activations for K = d_model, heads*head_dim, d_ff
  DevBuf sc_d, sc_a, sc_f, zp_d, zp_a, zp_f;
  DevBuf zero_ws, sdpa_ws, arg_val, arg_idx;
  DevBuf trace;        // B200_DEC_TRACE=<file>: 4 timer stamps per GEMV launch of a step
  int trace_next = 0;  // slot of the next GEMV launch while a step is being enqueued
  int32_t *h_tokens_pinned = nullptr, *h_next_pinned = nullptr;
  // tensor parallelism: this rank's share of the heads, KV heads, feed-forward units and vocabulary rows
  int hl = 0, kvl = 0, fl = 0, vl = 0;
  // Exchange buffer (one cudaMalloc, exported to the peers): flags | step counter | o-projection
  // partial | down-projection partial | argmax candidate pairs. proj / down_out point into it.
  DevBuf comm, gather;
  size_t off_epoch = 0, off_part_a = 0, off_part_b = 0, off_pairs = 0;
  // message areas of the pushed exchanges (decode-sized batches): [tp_size][kTpPushRows * d_model] 8-byte messages each
  size_t off_push_a = 0, off_push_b = 0, push_stride = 0;
  uint8_t* peer_comm[b200::kMaxTpRanks] = {nullptr};  // peers' exchange buffers mapped here (own entry: comm.p)
  bool peers_connected = false;
  bool peers_are_ipc = true;  // peer_comm entries came from cudaIpcOpenMemHandle (closed at destroy)
  b200_allreduce_fn allreduce = nullptr;
  void* allreduce_user = nullptr;
  void* nccl_comm = nullptr;
  cudaGraphExec_t graph[257] = {nullptr};  // indexed by batch
  std::unique_ptr<PrefillBufs> pf;         // allocated by the first prompt pass
  int launches = 0;
  float soft_cap = 0.0f;  // logits soft-cap of the greedy pick (0 = none)
  // per-kernel-class timing of one eager step (b200_decoder_profile_step)
  bool profiling = false;
  std::vector<cudaEvent_t> prof_events;  // start/stop pairs
  std::vector<int> prof_class;           // 0 = GEMV, 1 = attention, 2 = glue
};

namespace {

thread_local char g_dec_error[512] = "";
int dec_fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) {
    snprintf(g_dec_error, sizeof(g_dec_error), "%s: %s", what, cudaGetErrorString(e));
  } else {
    snprintf(g_dec_error, sizeof(g_dec_error), "%s", what);
  }
  return code;
}
#define DEC_CUDA(expr)                                              \
  do {                                                              \
    cudaError_t _e = (expr);                                        \
    if (_e != cudaSuccess) return dec_fail(B200_ERR_CUDA, #expr, _e); \
  } while (0)

// ---- NCCL, loaded at run time (no link-time dependency) ---------------------------------------
// Only the four calls the decoder needs, through the library's stable C ABI: the unique id is a
// 128-byte struct passed by value, data type 7 is float32, reduction 0 is sum.
struct NcclId {
  char bytes[128];
};
struct NcclApi {
  void* lib = nullptr;
  int (*get_unique_id)(NcclId*) = nullptr;
  int (*comm_init_rank)(void**, int, NcclId, int) = nullptr;
  int (*all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*comm_destroy)(void*) = nullptr;
  const char* (*get_error_string)(int) = nullptr;
};
NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    // a process that already holds an NCCL (PyTorch's, say) gets that one back
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (lib) {
      api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(lib, "ncclGetUniqueId"));
      api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(lib, "ncclCommInitRank"));
      api.all_reduce = reinterpret_cast<decltype(api.all_reduce)>(dlsym(lib, "ncclAllReduce"));
      api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(lib, "ncclCommDestroy"));
      api.get_error_string = reinterpret_cast<decltype(api.get_error_string)>(dlsym(lib, "ncclGetErrorString"));
      if (api.get_unique_id && api.comm_init_rank && api.all_reduce && api.comm_destroy) api.lib = lib;
    }
  }
  return api.lib ? &api : nullptr;
}
int nccl_allreduce_cb(void* user, float* buf, size_t count, void* stream) {
  NcclApi* api = nccl_api();
  if (!api || !user) return 1;
  return api->all_reduce(buf, buf, count, /*ncclFloat32=*/7, /*ncclSum=*/0, user, static_cast<cudaStream_t>(stream));
}
void nccl_release(b200_decoder* d) {
  NcclApi* api = nccl_api();
  if (api && d->nccl_comm) api->comm_destroy(d->nccl_comm);
  d->nccl_comm = nullptr;
}

struct ProfScope {
  b200_decoder* d;
  ProfScope(b200_decoder* dec, int cls) : d(dec) {
    if (!d->profiling) return;
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    d->prof_events.push_back(a);
    d->prof_events.push_back(b);
    d->prof_class.push_back(cls);
    cudaEventRecord(a, d->stream);
  }
  ~ProfScope() {
    if (d->profiling) cudaEventRecord(d->prof_events.back(), d->stream);
  }
};

#define GLUE_CUDA(expr)      \
  do {                       \
    ProfScope _scope(d, 2);  \
    DEC_CUDA(expr);          \
  } while (0)

size_t q_tiled_bytes(int m_alloc, int k) { return (size_t)tiles_k8(k) * m_alloc * 128; }

// Concatenates row-major [n_i, k] int8 matrices (and their scales) and packs them as one projection.
int build_projection(b200_decoder* d, Projection* pr, int k, std::initializer_list<const int8_t*> ws,
                     std::initializer_list<const float*> ss, std::initializer_list<int> ns) {
  int n = 0;
  for (int v : ns) n += v;
  pr->n = n;
  pr->k = k;
  DevBuf staging;
  DEC_CUDA(staging.alloc((size_t)n * k));
  DEC_CUDA(pr->scales.alloc(sizeof(float) * n));
  DEC_CUDA(pr->row_sums.alloc(sizeof(int32_t) * n));
  DEC_CUDA(pr->packed.alloc((size_t)tiles_n(n) * tiles_k8(k) * kTileBytes));
  size_t row = 0;
  auto wi = ws.begin();
  auto si = ss.begin();
  for (int v : ns) {
    DEC_CUDA(cudaMemcpyAsync(staging.as<int8_t>() + row * k, *wi, (size_t)v * k, cudaMemcpyDeviceToDevice, d->stream));
    DEC_CUDA(cudaMemcpyAsync(pr->scales.as<float>() + row, *si, sizeof(float) * v, cudaMemcpyDeviceToDevice, d->stream));
    row += v;
    ++wi;
    ++si;
  }
  DEC_CUDA(launch_pack_w8(staging.as<int8_t>(), n, k, pr->packed.as<uint8_t>(), pr->row_sums.as<int32_t>(), d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));  // staging dies here
  return B200_OK;
}

constexpr int kTraceSlots = 256;

// Residual add + RMS norm + quantization done inside the GEMV (FcParams::prologue).
struct FusedInput {
  const float* h_in;
  const float* delta;
  const float* gain;
  float* h_out;
};

// pick: the greedy pick fused into the projection's epilogue (the LM head at up to 16 rows): the CTAs'
// candidates go to arg_val / arg_idx, y may be null.
cudaError_t run_fc(b200_decoder* d, const Projection& pr, int batch, const int8_t* q_tiled, const float* scales,
                   const int32_t* zps, float* y, const FusedInput* fused = nullptr, bool pick = false,
                   int push_seq = -1) {
  FcParams p;
  memset(&p, 0, sizeof(p));
  if (push_seq >= 0) {  // tensor-parallel, decode-sized: the outputs also go to every peer as messages
    const b200_decoder_config& c = d->cfg;
    const size_t off = (push_seq & 1) ? d->off_push_b : d->off_push_a;  // even: attention output, odd: down
    for (int j = 0; j < c.tp_size; ++j)
      p.push_out[j] = reinterpret_cast<uint2*>(d->peer_comm[j] + off) + (size_t)c.tp_rank * d->push_stride;
    p.push_ranks = c.tp_size;
    p.push_rank = c.tp_rank;
    p.push_seq = push_seq;
    p.push_per_step = 2 * c.n_layers + 1;
    p.push_step_epoch = reinterpret_cast<const unsigned long long*>(d->comm.as<uint8_t>() + d->off_epoch);
  }
  if (fused) {
    p.prologue = 1;
    p.pro_h_in = fused->h_in;
    p.pro_delta = fused->delta;
    p.pro_gain = fused->gain;
    p.pro_h_out = fused->h_out;
    p.pro_eps = d->cfg.rms_eps;
  }
  p.w_packed = pr.packed.as<uint8_t>();
  p.q_tiled = q_tiled;
  p.m = batch;
  p.n = pr.n;
  p.k = pr.k;
  p.n_tiles = tiles_n(pr.n);
  p.k_tiles = tiles_k8(pr.k);
  p.m_alloc = m_alloc_for(batch);
  p.in_scales = scales;
  p.in_zps = zps;
  p.w_scales = pr.scales.as<float>();
  p.per_channel = 1;
  p.row_sums = pr.row_sums.as<int32_t>();
  p.activation = 0;
  p.y = y;
  if (pick) {
    p.argmax_val = d->arg_val.as<float>();
    p.argmax_idx = d->arg_idx.as<int32_t>();
    p.argmax_parts = fc_argmax_ctas(pr.n);
    p.soft_cap = d->soft_cap;
  }
  // Between two projections of a decode step run short row kernels that leave HBM idle, with this
  // projection's CTAs already resident and waiting: they pull a few of their weight tiles beyond the ring
  // towards L2 meanwhile. Measured on B200 (batch 1, step time, same run): none 0.859 ms, 2 tiles per CTA
  // 0.847, 4: 0.843, 6: 0.841, 8: 0.845, 12 and more (all of a layer's projection) 0.848: the requests
  // compete with the projection that is still streaming.
  {
    static const int pf_env = [] {
      const char* e = tuning_env("B200_L2_PREFETCH");  // measurement knob: tiles per CTA, 0 = off
      return e ? atoi(e) : -1;
    }();
    p.l2_prefetch_tiles = batch <= 16 ? 6 : 0;
    if (pf_env >= 0) p.l2_prefetch_tiles = pf_env;
  }
  uint8_t* z = d->zero_ws.as<uint8_t>();
  p.status = reinterpret_cast<int*>(z);
  p.ws_count = reinterpret_cast<int32_t*>(z + zero_ws_counter_off());
  p.ws_part = reinterpret_cast<int32_t*>(z + b200::zero_ws_part_off());
  ++d->launches;
  if (d->trace.p && d->trace_next < kTraceSlots) p.trace = d->trace.as<unsigned long long>() + 4 * d->trace_next++;
  ProfScope scope(d, 0);
  return launch_fc_i8_umma(p, pick ? kEpiHybridPick : kEpiHybridF32, d->stream);
}

// The exchange whose sum the next consuming kernel needs: partials at byte offset `off` of every
// rank's exchange buffer, `seq` = its number within the step.
TpExchange make_exchange(const b200_decoder* d, int seq, size_t off, bool pushed = false) {
  TpExchange x;
  if (pushed) {
    x.push_in = reinterpret_cast<const uint2*>(d->comm.as<uint8_t>() + (off == d->off_part_a ? d->off_push_a : d->off_push_b));
    x.push_stride = (int)d->push_stride;
  }
  const b200_decoder_config& c = d->cfg;
  x.tp_size = c.tp_size;
  x.tp_rank = c.tp_rank;
  x.seq = seq;
  x.per_step = 2 * c.n_layers + 1;
  for (int j = 0; j < c.tp_size; ++j) {
    x.partial[j] = reinterpret_cast<const float*>(d->peer_comm[j] + off);
    x.flag_out[j] = reinterpret_cast<unsigned long long*>(d->peer_comm[j]) + c.tp_rank;
  }
  x.flags_in = reinterpret_cast<const unsigned long long*>(d->comm.p);
  x.step_epoch = reinterpret_cast<const unsigned long long*>(d->comm.as<uint8_t>() + d->off_epoch);
  x.status = d->zero_ws.as<int>();
  return x;
}

// Enqueues one full decode step for `batch` sequences on the decoder's stream.
int enqueue_step(b200_decoder* d, int batch, float* d_logits_out) {
  const b200_decoder_config& c = d->cfg;
  cudaStream_t s = d->stream;
  const int m_alloc = m_alloc_for(batch);
  const bool tp = c.tp_size > 1;
  const bool fused = tp && d->peers_connected;  // sums fetched from peer memory inside the consuming kernels
  if (tp && !fused && !d->allreduce)
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "tensor-parallel decoder: connect the peers or set an all-reduce first");
  d->launches = 0;
  d->trace_next = 0;
  auto count = [&](int n = 1) { d->launches += n; };
  // sum over ranks of a partial projection output through the caller's collective (not a kernel of ours)
  auto reduce = [&](float* buf, size_t n) -> int {
    if (!tp || fused) return B200_OK;
    ProfScope scope(d, 2);
    if (d->allreduce(d->allreduce_user, buf, n, s) != 0) return dec_fail(B200_ERR_CUDA, "all-reduce callback failed");
    return B200_OK;
  };
  unsigned long long* epoch = fused ? reinterpret_cast<unsigned long long*>(d->comm.as<uint8_t>() + d->off_epoch) : nullptr;
  GLUE_CUDA(launch_embed(d->tokens.as<int32_t>(), d->embed_table.as<int8_t>(), d->embed_scales.as<float>(), batch,
                        c.vocab, c.d_model, c.embed_scale, d->h.as<float>(), d->positions.as<int32_t>(),
                        d->attn_len.as<int32_t>(), epoch, s));
  count();
  // Opt-in (B200_FUSED_PROLOGUE=1): with one GPU and a decode-sized batch the residual add, RMS norm
  // and quantization in front of the qkv, gate/up and LM-head projections run inside those GEMVs
  // (no kernel of their own); the residual stream then alternates between two buffers, because every
  // CTA reads the old one. Measured on B200 at batch 1 this is 7 % SLOWER than the separate kernel
  // (1.40 vs 1.30 ms per step): a GEMV's CTAs cannot become resident while the previous GEMV holds
  // the shared memory, so the prologue's latency is exposed, whereas the small separate kernel runs
  // beside the previous GEMV and the next one fills its ring meanwhile. Kept for wider rows per SM.
  static const bool fuse_env = [] {
    const char* e = tuning_env("B200_FUSED_PROLOGUE");
    return e && e[0] == '1';
  }();
  const bool fuse_norm = fuse_env && !tp && fc_prologue_supported(batch, c.d_model);
  // Measurement knob: leave kernels out of the step to read their marginal cost off the step time
  // (the results are then meaningless). Bits: 1 norm, 2 rope, 4 attention, 8 GeGLU, 16 qkv, 32 o,
  // 64 gate/up, 128 down, 256 LM head.
  static const int skip = [] {
    const char* e = tuning_env("B200_DEC_SKIP");
    return e ? atoi(e) : 0;
  }();
  // Rotary embedding, cache append, attention and output quantization as one cluster kernel where
  // the shape allows (one KV head on this rank, at most eight query heads); B200_ATTN_STEP=0 keeps
  // the three separate kernels.
  static const bool attn_env = [] {
    const char* e = tuning_env("B200_ATTN_STEP");
    return !(e && e[0] == '0');
  }();
  // (one cluster of 8 CTAs per sequence, each with most of an SM's shared memory: beyond about a
  // sixth of the SMs in sequences the chunked kernels do better: 1.69 vs 1.86 ms per step at batch 32)
  const bool attn_one_launch = attn_env && batch * 8 <= device_sm_count() / 2 &&
                               attn_step_supported(d->hl, d->kvl, c.head_dim, c.kv_dtype == B200_DTYPE_I8 ? 1 : 0);
  // Tensor-parallel exchange of decode-sized batches: the attention-output and down GEMVs push their partials to
  // the peers as self-validating messages, and the norm stage that consumes the sum polls its own memory (no flag
  // handshake, no fence, no remote read).
  static const bool push_env = [] {
    const char* e = tuning_env("B200_TP_PUSH");  // measurement knob: 0 keeps the flag handshake
    return !(e && e[0] == '0');
  }();
  const bool push = push_env && fused && batch <= kTpPushRows && c.d_model % 2 == 0 && c.d_model <= 2048 &&
                    fc_cluster_planned(batch, c.d_model, d->hl * c.head_dim) && fc_cluster_planned(batch, c.d_model, d->fl);
  float* hbuf[2] = {d->h.as<float>(), d->h2.as<float>()};
  int cur = 0;
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = *d->layers[l];
    if (fuse_norm) {
      const FusedInput fi{hbuf[cur], l == 0 ? nullptr : d->down_out, L.norm1.as<float>(), hbuf[cur ^ 1]};
      if (!(skip & 16)) DEC_CUDA(run_fc(d, L.qkv, batch, nullptr, nullptr, nullptr, d->qkv.as<float>(), &fi));
      cur ^= 1;
    } else {
      const TpExchange x = fused && l > 0 ? make_exchange(d, 2 * l - 1, d->off_part_b, push) : TpExchange();
      if (!(skip & 1)) GLUE_CUDA(launch_add_norm_quant(d->h.as<float>(), l == 0 ? nullptr : d->down_out, L.norm1.as<float>(), batch,
                                     c.d_model, c.rms_eps, m_alloc, d->q_d.as<int8_t>(), d->sc_d.as<float>(),
                                     d->zp_d.as<int32_t>(), fused && l > 0 ? &x : nullptr, s));
      count();
      if (!(skip & 16)) DEC_CUDA(run_fc(d, L.qkv, batch, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(), d->qkv.as<float>()));
    }
    if (attn_one_launch) {
      AttnStepParams ap;
      memset(&ap, 0, sizeof(ap));
      ap.qkv = d->qkv.as<float>();
      ap.positions = d->positions.as<int32_t>();
      ap.k_cache = L.k_cache.p;
      ap.v_cache = L.v_cache.p;
      ap.k_scale = L.k_scale.as<float>();
      ap.v_scale = L.v_scale.as<float>();
      ap.b = batch;
      ap.n = d->hl;
      ap.h = c.head_dim;
      ap.s_max = c.max_seq;
      ap.kv_dtype = c.kv_dtype == B200_DTYPE_I8 ? 1 : 0;
      ap.rope_cs = d->rope_cs.as<float2>();
      ap.scale = 1.0f / sqrtf((float)c.head_dim);
      ap.q_tiled_out = d->q_a.as<int8_t>();
      ap.out_scales = d->sc_a.as<float>();
      ap.out_zps = d->zp_a.as<int32_t>();
      ap.m_alloc = m_alloc;
      ap.status = d->zero_ws.as<int>();
      if (d->trace.p) ap.trace = d->trace.as<unsigned long long>() + 4 * kTraceSlots + 16 * l;
      {
        ProfScope scope(d, 1);
        if (!(skip & 4)) DEC_CUDA(launch_attn_step(ap, s));
      }
      count();
    } else {
      if (!(skip & 2)) GLUE_CUDA(launch_rope_cache(d->qkv.as<float>(), batch, d->hl, d->kvl, c.head_dim, d->rope_cs.as<float2>(),
                                 d->positions.as<int32_t>(), c.max_seq, d->q.as<float>(), L.k_cache.p, L.v_cache.p,
                                 L.k_scale.as<float>(), L.v_scale.as<float>(), c.kv_dtype == B200_DTYPE_I8, 0, s));
      count();
      SdpaParams sp;
      memset(&sp, 0, sizeof(sp));
      sp.q = d->q.p;
      sp.k = L.k_cache.p;
      sp.v = L.v_cache.p;
      sp.k_scale = L.k_scale.as<float>();
      sp.v_scale = L.v_scale.as<float>();
      sp.lengths = d->attn_len.as<int32_t>();
      sp.out = nullptr;  // only the quantized rows are needed downstream
      sp.q_tiled_out = d->q_a.as<int8_t>();
      sp.out_scales = d->sc_a.as<float>();
      sp.out_zps = d->zp_a.as<int32_t>();
      sp.m_alloc = m_alloc;
      sp.b = batch;
      sp.n = d->hl;
      sp.nkv = d->kvl;
      sp.h = c.head_dim;
      sp.s_max = c.max_seq;
      sp.q_dtype = 1;
      sp.kv_dtype = c.kv_dtype == B200_DTYPE_I8 ? 1 : 0;
      sp.scale = 1.0f / sqrtf((float)c.head_dim);
      sp.ws = d->sdpa_ws.as<float>();
      sp.ws_bytes = d->sdpa_ws.bytes;
      sp.status = d->zero_ws.as<int>();
      {
        ProfScope scope(d, 1);
        if (!(skip & 4)) DEC_CUDA(launch_sdpa_decode(sp, s));
      }
      count(2);
    }
    if (!(skip & 32)) DEC_CUDA(run_fc(d, L.o, batch, d->q_a.as<int8_t>(), d->sc_a.as<float>(), d->zp_a.as<int32_t>(), d->proj, nullptr,
                                      false, push ? 2 * l : -1));
    if (int rc = reduce(d->proj, (size_t)batch * c.d_model)) return rc;
    if (fuse_norm) {
      const FusedInput fi{hbuf[cur], d->proj, L.norm2.as<float>(), hbuf[cur ^ 1]};
      if (!(skip & 64)) DEC_CUDA(run_fc(d, L.gate_up, batch, nullptr, nullptr, nullptr, d->gate_up.as<float>(), &fi));
      cur ^= 1;
    } else {
      const TpExchange x = fused ? make_exchange(d, 2 * l, d->off_part_a, push) : TpExchange();
      if (!(skip & 1)) GLUE_CUDA(launch_add_norm_quant(d->h.as<float>(), d->proj, L.norm2.as<float>(), batch, c.d_model, c.rms_eps,
                                     m_alloc, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(),
                                     fused ? &x : nullptr, s));
      count();
      if (!(skip & 64)) DEC_CUDA(run_fc(d, L.gate_up, batch, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(),
                      d->gate_up.as<float>()));
    }
    if (!(skip & 8)) GLUE_CUDA(launch_geglu_quant(d->gate_up.as<float>(), batch, d->fl, m_alloc, d->q_f.as<int8_t>(), d->sc_f.as<float>(),
                                d->zp_f.as<int32_t>(), s));
    count();
    if (!(skip & 128)) DEC_CUDA(run_fc(d, L.down, batch, d->q_f.as<int8_t>(), d->sc_f.as<float>(), d->zp_f.as<int32_t>(), d->down_out,
                                       nullptr, false, push ? 2 * l + 1 : -1));
    if (int rc = reduce(d->down_out, (size_t)batch * c.d_model)) return rc;
  }
  // One sequence batch on one GPU, at most 16 rows: the LM-head GEMV picks the greedy token in its own
  // epilogue (soft-cap, first index of the maximum, NaN rule), so that no logits are written unless the
  // caller asked for them, and one small kernel compares the CTAs' candidates.
  static const bool pick_env = [] {
    const char* e = tuning_env("B200_FUSED_PICK");  // measurement knob: 0 keeps the separate arg-max kernels
    return !(e && e[0] == '0');
  }();
  const bool fused_pick = pick_env && !tp && batch <= 16 && fc_argmax_ctas(d->lm_head.n) <= kArgmaxSlots;
  float* logits = d_logits_out ? d_logits_out : (fused_pick ? nullptr : d->logits.as<float>());
  if (fuse_norm) {
    const FusedInput fi{hbuf[cur], d->down_out, d->final_norm.as<float>(), hbuf[cur ^ 1]};
    if (!(skip & 256)) DEC_CUDA(run_fc(d, d->lm_head, batch, nullptr, nullptr, nullptr, logits, &fi, fused_pick));
  } else {
    const TpExchange x = fused ? make_exchange(d, 2 * c.n_layers - 1, d->off_part_b, push) : TpExchange();
    if (!(skip & 1)) GLUE_CUDA(launch_add_norm_quant(d->h.as<float>(), d->down_out, d->final_norm.as<float>(), batch, c.d_model, c.rms_eps,
                                   m_alloc, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(),
                                   fused ? &x : nullptr, s));
    count();
    if (!(skip & 256)) DEC_CUDA(run_fc(d, d->lm_head, batch, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(), logits, nullptr, fused_pick));
  }
  if (fused_pick) {
    GLUE_CUDA(launch_argmax_final(d->arg_val.as<float>(), d->arg_idx.as<int32_t>(), batch, fc_argmax_ctas(d->lm_head.n), 0,
                                 d->next_tokens.as<int32_t>(), d->positions.as<int32_t>(), c.max_seq, nullptr, s));
    count();
    return B200_OK;
  }
  if (!tp) {
    GLUE_CUDA(launch_argmax(logits, batch, c.vocab, 0, d->soft_cap, d->arg_val.as<float>(), d->arg_idx.as<int32_t>(),
                           d->next_tokens.as<int32_t>(), d->positions.as<int32_t>(), c.max_seq, nullptr, s));
    count(2);
    return B200_OK;
  }
  // every rank proposes the best of its vocabulary rows; the winner over ranks is the next token
  const float2* pairs[kMaxTpRanks] = {nullptr};
  if (fused) {
    float2* own = reinterpret_cast<float2*>(d->comm.as<uint8_t>() + d->off_pairs);
    GLUE_CUDA(launch_argmax(logits, batch, d->vl, c.tp_rank * d->vl, 0.0f, d->arg_val.as<float>(), d->arg_idx.as<int32_t>(),
                           nullptr, nullptr, c.max_seq, own, s));
    for (int j = 0; j < c.tp_size; ++j) pairs[j] = reinterpret_cast<const float2*>(d->peer_comm[j] + d->off_pairs);
    const TpExchange x = make_exchange(d, 2 * c.n_layers, d->off_pairs);
    GLUE_CUDA(launch_argmax_pick(pairs, c.tp_size, batch, d->next_tokens.as<int32_t>(), d->positions.as<int32_t>(),
                                c.max_seq, &x, s));
  } else {
    // gather through the sum collective: every rank fills its own slot of a zeroed table
    float2* table = d->gather.as<float2>();
    DEC_CUDA(cudaMemsetAsync(table, 0, sizeof(float2) * c.tp_size * c.max_batch, s));
    GLUE_CUDA(launch_argmax(logits, batch, d->vl, c.tp_rank * d->vl, 0.0f, d->arg_val.as<float>(), d->arg_idx.as<int32_t>(),
                           nullptr, nullptr, c.max_seq, table + (size_t)c.tp_rank * c.max_batch, s));
    if (int rc = reduce(reinterpret_cast<float*>(table), (size_t)2 * c.tp_size * c.max_batch)) return rc;
    for (int j = 0; j < c.tp_size; ++j) pairs[j] = table + (size_t)j * c.max_batch;
    GLUE_CUDA(launch_argmax_pick(pairs, c.tp_size, batch, d->next_tokens.as<int32_t>(), d->positions.as<int32_t>(),
                                c.max_seq, nullptr, s));
  }
  count(3);
  return B200_OK;
}

// Rows of one prompt chunk. The projections with few n tiles (attention output and down: 16 tiles
// of 128 channels) only fill the SMs when there are many passes of activation rows, so the chunk is
// large; the scratch is 140 KB per row at the benchmark's sizes. B200_PREFILL_ROWS overrides it
// (measurement knob, read when the first prompt pass allocates the scratch).
constexpr int kPrefillRows = 1024;

int ensure_prefill_bufs(b200_decoder* d) {
  if (d->pf) return B200_OK;
  const b200_decoder_config& c = d->cfg;
  auto pf = std::make_unique<PrefillBufs>();
  int R = kPrefillRows;
  if (const char* e = tuning_env("B200_PREFILL_ROWS")) {
    const int v = atoi(e);
    if (v >= 1 && v <= 8192) R = v;
  }
  const int m_alloc = m_alloc_for(R), qdim = d->hl * c.head_dim, kvdim = d->kvl * c.head_dim;
  pf->rows = R;
  DEC_CUDA(pf->tokens.alloc(sizeof(int32_t) * R));
  DEC_CUDA(pf->positions.alloc(sizeof(int32_t) * R));
  DEC_CUDA(pf->attn_len.alloc(sizeof(int32_t) * R));
  DEC_CUDA(pf->h.alloc(sizeof(float) * R * c.d_model));
  DEC_CUDA(pf->qkv.alloc(sizeof(float) * R * (qdim + 2 * kvdim)));
  DEC_CUDA(pf->q.alloc(sizeof(float) * R * qdim));
  DEC_CUDA(pf->gate_up.alloc(sizeof(float) * (size_t)R * 2 * d->fl));
  DEC_CUDA(pf->proj.alloc(sizeof(float) * R * c.d_model));
  DEC_CUDA(pf->down_out.alloc(sizeof(float) * R * c.d_model));
  DEC_CUDA(pf->q_d.alloc(q_tiled_bytes(m_alloc, c.d_model)));
  DEC_CUDA(pf->q_a.alloc(q_tiled_bytes(m_alloc, qdim)));
  DEC_CUDA(pf->q_f.alloc(q_tiled_bytes(m_alloc, d->fl)));
  for (DevBuf* b : {&pf->sc_d, &pf->sc_a, &pf->sc_f, &pf->zp_d, &pf->zp_a, &pf->zp_f}) DEC_CUDA(b->alloc(sizeof(float) * m_alloc));
  DEC_CUDA(pf->sdpa_ws.alloc(sdpa_workspace_bytes(R, d->hl, d->kvl, c.head_dim, c.max_seq, 1)));
  DEC_CUDA(cudaMallocHost(&pf->h_stage, sizeof(int32_t) * 2 * R));
  d->pf = std::move(pf);
  return B200_OK;
}

// Enqueues the layers over `rows` consecutive prompt tokens of sequence `seq` (tokens and positions
// already in the prompt scratch). Every projection is one GEMM over all the rows; the rows' keys and
// values are appended first, then row t attends over the cache up to its own position, which is the
// causal mask. With `pick`, the last row goes through the final norm, the LM head and the arg-max,
// whose token lands in next_tokens[seq].
int enqueue_prefill_chunk(b200_decoder* d, int seq, int rows, bool pick) {
  const b200_decoder_config& c = d->cfg;
  PrefillBufs& f = *d->pf;
  cudaStream_t s = d->stream;
  const int m_alloc = m_alloc_for(rows);
  const bool tp = c.tp_size > 1;
  const bool i8 = c.kv_dtype == B200_DTYPE_I8;
  auto reduce = [&](float* buf, size_t n) -> int {
    if (!tp) return B200_OK;
    if (d->allreduce(d->allreduce_user, buf, n, s) != 0) return dec_fail(B200_ERR_CUDA, "all-reduce callback failed");
    return B200_OK;
  };
  const size_t kv_first = (size_t)seq * c.max_seq * d->kvl;  // first token row of this sequence's cache
  const size_t kv_row = (size_t)c.head_dim * (i8 ? 1 : 2);
  DEC_CUDA(launch_embed(f.tokens.as<int32_t>(), d->embed_table.as<int8_t>(), d->embed_scales.as<float>(), rows, c.vocab, c.d_model,
                        c.embed_scale, f.h.as<float>(), f.positions.as<int32_t>(), f.attn_len.as<int32_t>(), nullptr, s));
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = *d->layers[l];
    void* kc = L.k_cache.as<uint8_t>() + kv_first * kv_row;
    void* vc = L.v_cache.as<uint8_t>() + kv_first * kv_row;
    float* ks = i8 ? L.k_scale.as<float>() + kv_first : nullptr;
    float* vs = i8 ? L.v_scale.as<float>() + kv_first : nullptr;
    DEC_CUDA(launch_add_norm_quant(f.h.as<float>(), l == 0 ? nullptr : f.down_out.as<float>(), L.norm1.as<float>(), rows, c.d_model,
                                   c.rms_eps, m_alloc, f.q_d.as<int8_t>(), f.sc_d.as<float>(), f.zp_d.as<int32_t>(), nullptr, s));
    DEC_CUDA(run_fc(d, L.qkv, rows, f.q_d.as<int8_t>(), f.sc_d.as<float>(), f.zp_d.as<int32_t>(), f.qkv.as<float>()));
    DEC_CUDA(launch_rope_cache(f.qkv.as<float>(), rows, d->hl, d->kvl, c.head_dim, d->rope_cs.as<float2>(), f.positions.as<int32_t>(),
                               c.max_seq, f.q.as<float>(), kc, vc, ks, vs, i8, 1, s));
    SdpaParams sp;
    memset(&sp, 0, sizeof(sp));
    sp.q = f.q.p;
    sp.k = kc;
    sp.v = vc;
    sp.k_scale = ks;
    sp.v_scale = vs;
    sp.shared_kv = 1;
    sp.lengths = f.attn_len.as<int32_t>();
    sp.q_tiled_out = f.q_a.as<int8_t>();
    sp.out_scales = f.sc_a.as<float>();
    sp.out_zps = f.zp_a.as<int32_t>();
    sp.m_alloc = m_alloc;
    sp.b = rows;
    sp.n = d->hl;
    sp.nkv = d->kvl;
    sp.h = c.head_dim;
    sp.s_max = c.max_seq;
    sp.q_dtype = 1;
    sp.kv_dtype = i8 ? 1 : 0;
    sp.scale = 1.0f / sqrtf((float)c.head_dim);
    sp.ws = f.sdpa_ws.as<float>();
    sp.ws_bytes = f.sdpa_ws.bytes;
    sp.status = d->zero_ws.as<int>();
    DEC_CUDA(launch_sdpa_decode(sp, s));
    DEC_CUDA(run_fc(d, L.o, rows, f.q_a.as<int8_t>(), f.sc_a.as<float>(), f.zp_a.as<int32_t>(), f.proj.as<float>()));
    if (int rc = reduce(f.proj.as<float>(), (size_t)rows * c.d_model)) return rc;
    DEC_CUDA(launch_add_norm_quant(f.h.as<float>(), f.proj.as<float>(), L.norm2.as<float>(), rows, c.d_model, c.rms_eps, m_alloc,
                                   f.q_d.as<int8_t>(), f.sc_d.as<float>(), f.zp_d.as<int32_t>(), nullptr, s));
    DEC_CUDA(run_fc(d, L.gate_up, rows, f.q_d.as<int8_t>(), f.sc_d.as<float>(), f.zp_d.as<int32_t>(), f.gate_up.as<float>()));
    DEC_CUDA(launch_geglu_quant(f.gate_up.as<float>(), rows, d->fl, m_alloc, f.q_f.as<int8_t>(), f.sc_f.as<float>(),
                                f.zp_f.as<int32_t>(), s));
    DEC_CUDA(run_fc(d, L.down, rows, f.q_f.as<int8_t>(), f.sc_f.as<float>(), f.zp_f.as<int32_t>(), f.down_out.as<float>()));
    if (int rc = reduce(f.down_out.as<float>(), (size_t)rows * c.d_model)) return rc;
  }
  if (!pick) return B200_OK;
  // the last prompt token predicts the first generated one: one row through the head
  const size_t last = (size_t)(rows - 1) * c.d_model;
  DEC_CUDA(launch_add_norm_quant(f.h.as<float>() + last, f.down_out.as<float>() + last, d->final_norm.as<float>(), 1, c.d_model,
                                 c.rms_eps, m_alloc_for(1), f.q_d.as<int8_t>(), f.sc_d.as<float>(), f.zp_d.as<int32_t>(), nullptr, s));
  float* logits = d->logits.as<float>();
  DEC_CUDA(run_fc(d, d->lm_head, 1, f.q_d.as<int8_t>(), f.sc_d.as<float>(), f.zp_d.as<int32_t>(), logits));
  int32_t* scratch_pos = f.attn_len.as<int32_t>();  // the arg-max advances a position: not the sequence's, set by the caller
  if (!tp) {
    DEC_CUDA(launch_argmax(logits, 1, c.vocab, 0, d->soft_cap, d->arg_val.as<float>(), d->arg_idx.as<int32_t>(),
                           d->next_tokens.as<int32_t>() + seq, scratch_pos, c.max_seq, nullptr, s));
    return B200_OK;
  }
  // every rank proposes the best of its vocabulary rows through the sum collective (zeroed table, own slot)
  float2* table = d->gather.as<float2>();
  DEC_CUDA(cudaMemsetAsync(table, 0, sizeof(float2) * c.tp_size * c.max_batch, s));
  DEC_CUDA(launch_argmax(logits, 1, d->vl, c.tp_rank * d->vl, 0.0f, d->arg_val.as<float>(), d->arg_idx.as<int32_t>(), nullptr, nullptr,
                         c.max_seq, table + (size_t)c.tp_rank * c.max_batch, s));
  if (int rc = reduce(reinterpret_cast<float*>(table), (size_t)2 * c.tp_size * c.max_batch)) return rc;
  const float2* pairs[kMaxTpRanks] = {nullptr};
  for (int j = 0; j < c.tp_size; ++j) pairs[j] = table + (size_t)j * c.max_batch;
  DEC_CUDA(launch_argmax_pick(pairs, c.tp_size, 1, d->next_tokens.as<int32_t>() + seq, scratch_pos, c.max_seq, nullptr, s));
  return B200_OK;
}

// After a wait has run out: the status word is sticky and an aborted launch may have left split-K
// counters or accumulator slots non-zero. Clears them (keeping the wait budget) so that the next call
// starts from a clean workspace.
int clear_fault(b200_decoder* d) {
  uint8_t* z = d->zero_ws.as<uint8_t>();
  DEC_CUDA(cudaMemsetAsync(z, 0, 8, d->stream));
  DEC_CUDA(cudaMemsetAsync(z + 16, 0, zero_ws_part_off() - 16, d->stream));
  return B200_OK;
}

// Graph of one step (default logits buffer), captured on first use per batch size.
int ensure_graph(b200_decoder* d, int batch) {
  if (d->graph[batch]) return B200_OK;
  // Run once uncaptured so that every kernel's one-time attribute setup happens outside capture.
  // The warm-up advances the positions (restored below) and writes one cache row and the scratch
  // buffers, all of which the next real step overwrites.
  std::vector<int32_t> saved(d->cfg.max_batch);
  DEC_CUDA(cudaMemcpyAsync(saved.data(), d->positions.p, sizeof(int32_t) * saved.size(), cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  int rc = enqueue_step(d, batch, nullptr);
  if (rc) return rc;
  DEC_CUDA(cudaMemcpyAsync(d->positions.p, saved.data(), sizeof(int32_t) * saved.size(), cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  cudaGraph_t g = nullptr;
  DEC_CUDA(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
  rc = enqueue_step(d, batch, nullptr);
  cudaError_t e = cudaStreamEndCapture(d->stream, &g);
  if (rc) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  if (e != cudaSuccess) return dec_fail(B200_ERR_CUDA, "cudaStreamEndCapture", e);
  e = cudaGraphInstantiate(&d->graph[batch], g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return dec_fail(B200_ERR_CUDA, "cudaGraphInstantiate", e);
  return B200_OK;
}

}  // namespace

extern "C" {

int b200_decoder_create(const b200_decoder_config* config, void* stream, b200_decoder** out) {
  if (!config || !out) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_create: null argument");
  const b200_decoder_config& c = *config;
  if (c.n_layers <= 0 || c.d_model <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.head_dim <= 0 || c.d_ff <= 0 ||
      c.vocab <= 0 || c.max_seq <= 0 || c.max_batch <= 0 || c.max_batch > 256 || c.n_heads % c.n_kv_heads != 0 ||
      c.head_dim % 2 != 0)
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_create: bad configuration");
  if (c.kv_dtype != B200_DTYPE_F16 && c.kv_dtype != B200_DTYPE_I8)
    return dec_fail(B200_ERR_UNSUPPORTED, "b200_decoder_create: kv_dtype must be f16 or int8");
  const int T = c.tp_size < 1 ? 1 : c.tp_size;
  if (T > kMaxTpRanks || c.tp_rank < 0 || c.tp_rank >= T)
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_create: tp_size must be 1..8 and tp_rank below it");
  if (c.n_heads % T != 0 || c.d_ff % T != 0 || c.vocab % T != 0 || (c.n_kv_heads % T != 0 && T % c.n_kv_heads != 0) ||
      (T > 1 && c.vocab >= (1 << 24)))
    return dec_fail(B200_ERR_UNSUPPORTED,
                    "b200_decoder_create: heads, d_ff and vocab must divide by tp_size (KV heads divide or are replicated)");
  auto d = std::make_unique<b200_decoder>();
  d->cfg = c;
  d->cfg.tp_size = T;
  if (T == 1) d->cfg.tp_rank = 0;
  d->hl = c.n_heads / T;
  d->kvl = c.n_kv_heads % T == 0 ? c.n_kv_heads / T : 1;
  d->fl = c.d_ff / T;
  d->vl = c.vocab / T;
  if (stream) {
    d->stream = static_cast<cudaStream_t>(stream);
  } else {
    DEC_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
    d->own_stream = true;
  }
  const int B = c.max_batch, m_alloc = m_alloc_for(B), qdim = d->hl * c.head_dim;
  const int kvdim = d->kvl * c.head_dim;
  DEC_CUDA(d->tokens.alloc(sizeof(int32_t) * B));
  DEC_CUDA(d->next_tokens.alloc(sizeof(int32_t) * B));
  DEC_CUDA(d->positions.alloc(sizeof(int32_t) * B));
  DEC_CUDA(d->attn_len.alloc(sizeof(int32_t) * B));
  DEC_CUDA(d->h.alloc(sizeof(float) * B * c.d_model));
  DEC_CUDA(d->h2.alloc(sizeof(float) * B * c.d_model));
  DEC_CUDA(d->qkv.alloc(sizeof(float) * B * (qdim + 2 * kvdim)));
  DEC_CUDA(d->q.alloc(sizeof(float) * B * qdim));
  DEC_CUDA(d->attn.alloc(sizeof(float) * B * qdim));
  DEC_CUDA(d->gate_up.alloc(sizeof(float) * (size_t)B * 2 * d->fl));
  DEC_CUDA(d->logits.alloc(sizeof(float) * (size_t)B * d->vl));
  {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t part = up(sizeof(float) * (size_t)B * c.d_model);
    d->off_epoch = 256;
    d->off_part_a = 512;
    d->off_part_b = d->off_part_a + part;
    d->off_pairs = d->off_part_b + part;
    d->push_stride = (size_t)kTpPushRows * c.d_model;
    d->off_push_a = d->off_pairs + up(sizeof(float2) * B);
    d->off_push_b = d->off_push_a + up(sizeof(uint2) * d->push_stride * T);
    const size_t total = d->off_push_b + up(sizeof(uint2) * d->push_stride * T);
    // whole 2 MiB pages, so that the exported allocation holds nothing else
    DEC_CUDA(d->comm.alloc((total + (2u << 20) - 1) / (2u << 20) * (2u << 20)));
    DEC_CUDA(cudaMemsetAsync(d->comm.p, 0, d->comm.bytes, d->stream));
    d->proj = reinterpret_cast<float*>(d->comm.as<uint8_t>() + d->off_part_a);
    d->down_out = reinterpret_cast<float*>(d->comm.as<uint8_t>() + d->off_part_b);
    d->peer_comm[d->cfg.tp_rank] = d->comm.as<uint8_t>();
    if (T > 1) DEC_CUDA(d->gather.alloc(sizeof(float2) * T * B));
  }
  DEC_CUDA(d->q_d.alloc(q_tiled_bytes(m_alloc, c.d_model)));
  DEC_CUDA(d->q_a.alloc(q_tiled_bytes(m_alloc, qdim)));
  DEC_CUDA(d->q_f.alloc(q_tiled_bytes(m_alloc, d->fl)));
  for (DevBuf* b : {&d->sc_d, &d->sc_a, &d->sc_f, &d->zp_d, &d->zp_a, &d->zp_f}) DEC_CUDA(b->alloc(sizeof(float) * m_alloc));
  DEC_CUDA(d->zero_ws.alloc(zero_ws_total_bytes()));
  if (tuning_env("B200_DEC_TRACE")) {
    DEC_CUDA(d->trace.alloc(sizeof(unsigned long long) * (4 * kTraceSlots + 16 * 64)));
    DEC_CUDA(cudaMemsetAsync(d->trace.p, 0, d->trace.bytes, d->stream));
  }
  DEC_CUDA(cudaMemsetAsync(d->zero_ws.p, 0, d->zero_ws.bytes, d->stream));
  size_t sdpa_bytes = 0;  // the chunking depends on the batch: size for the worst batch <= max_batch
  for (int b = 1; b <= B; ++b) sdpa_bytes = std::max(sdpa_bytes, sdpa_workspace_bytes(b, d->hl, d->kvl, c.head_dim, c.max_seq));
  DEC_CUDA(d->sdpa_ws.alloc(sdpa_bytes));
  DEC_CUDA(d->arg_val.alloc(sizeof(float) * B * kArgmaxSlots));
  DEC_CUDA(d->arg_idx.alloc(sizeof(int32_t) * B * kArgmaxSlots));
  DEC_CUDA(cudaMemsetAsync(d->positions.p, 0, sizeof(int32_t) * B, d->stream));
  DEC_CUDA(cudaMallocHost(&d->h_tokens_pinned, sizeof(int32_t) * B));
  DEC_CUDA(cudaMallocHost(&d->h_next_pinned, sizeof(int32_t) * (B + 1)));  // + the status word read back with the tokens
  const size_t kv_elems = (size_t)B * c.max_seq * kvdim;
  const size_t kv_bytes = kv_elems * (c.kv_dtype == B200_DTYPE_I8 ? 1 : 2);
  for (int l = 0; l < c.n_layers; ++l) {
    d->layers.emplace_back(new Layer());
    Layer& L = *d->layers.back();
    DEC_CUDA(L.k_cache.alloc(kv_bytes));
    DEC_CUDA(L.v_cache.alloc(kv_bytes));
    DEC_CUDA(cudaMemsetAsync(L.k_cache.p, 0, kv_bytes, d->stream));
    DEC_CUDA(cudaMemsetAsync(L.v_cache.p, 0, kv_bytes, d->stream));
    if (c.kv_dtype == B200_DTYPE_I8) {
      DEC_CUDA(L.k_scale.alloc(sizeof(float) * (size_t)B * c.max_seq * d->kvl));
      DEC_CUDA(L.v_scale.alloc(sizeof(float) * (size_t)B * c.max_seq * d->kvl));
    }
    DEC_CUDA(L.norm1.alloc(sizeof(float) * c.d_model));
    DEC_CUDA(L.norm2.alloc(sizeof(float) * c.d_model));
  }
  DEC_CUDA(d->final_norm.alloc(sizeof(float) * c.d_model));
  {
    // the graph's cos / sin inputs: prepared once on the host, as the reference's host side does
    std::vector<float> cs((size_t)(c.max_seq + 1) * (c.head_dim / 2) * 2);
    fill_rope_table(cs.data(), c.max_seq + 1, c.head_dim, c.rope_base);
    DEC_CUDA(d->rope_cs.alloc(sizeof(float) * cs.size()));
    DEC_CUDA(cudaMemcpy(d->rope_cs.p, cs.data(), sizeof(float) * cs.size(), cudaMemcpyHostToDevice));
  }
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  *out = d.release();
  return B200_OK;
}

void b200_decoder_destroy(b200_decoder* d) {
  if (!d) return;
  cudaStreamSynchronize(d->stream);
  if (d->trace.p) {  // measurement: the last step's stamps, one line per GEMV launch
    std::vector<unsigned long long> t(4 * kTraceSlots + 16 * 64);
    if (cudaMemcpy(t.data(), d->trace.p, d->trace.bytes, cudaMemcpyDeviceToHost) == cudaSuccess) {
      if (FILE* f = fopen(tuning_env("B200_DEC_TRACE"), "w")) {
        for (int i = 0; i < kTraceSlots && t[4 * i]; ++i)
          fprintf(f, "%d %llu %llu %llu %llu\n", i, t[4 * i], t[4 * i + 1], t[4 * i + 2], t[4 * i + 3]);
        for (int l = 0; l < 64 && l < d->cfg.n_layers; ++l) {  // attention step kernel, nine stamps per layer
          const unsigned long long* a = t.data() + 4 * kTraceSlots + 16 * l;
          if (!a[0]) break;
          fprintf(f, "attn %d", l);
          for (int j = 0; j < 12; ++j) fprintf(f, " %llu", a[j]);
          fprintf(f, "\n");
        }
        fclose(f);
      }
    }
  }
  for (auto& g : d->graph)
    if (g) cudaGraphExecDestroy(g);
  if (d->peers_connected && d->peers_are_ipc)
    for (int j = 0; j < d->cfg.tp_size; ++j)
      if (j != d->cfg.tp_rank && d->peer_comm[j]) cudaIpcCloseMemHandle(d->peer_comm[j]);
  nccl_release(d);
  if (d->h_tokens_pinned) cudaFreeHost(d->h_tokens_pinned);
  if (d->h_next_pinned) cudaFreeHost(d->h_next_pinned);
  if (d->own_stream) cudaStreamDestroy(d->stream);
  delete d;
}

int b200_decoder_set_layer(b200_decoder* d, int layer, const b200_decoder_layer_weights* w) {
  if (!d || !w || layer < 0 || layer >= d->cfg.n_layers) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_set_layer: bad argument");
  const b200_decoder_config& c = d->cfg;
  const int qdim = d->hl * c.head_dim, kvdim = d->kvl * c.head_dim;  // this rank's shard
  Layer& L = *d->layers[layer];
  int rc = build_projection(d, &L.qkv, c.d_model, {w->wq, w->wk, w->wv}, {w->sq, w->sk, w->sv}, {qdim, kvdim, kvdim});
  if (rc) return rc;
  rc = build_projection(d, &L.o, qdim, {w->wo}, {w->so}, {c.d_model});
  if (rc) return rc;
  rc = build_projection(d, &L.gate_up, c.d_model, {w->wgate, w->wup}, {w->sgate, w->sup}, {d->fl, d->fl});
  if (rc) return rc;
  rc = build_projection(d, &L.down, d->fl, {w->wdown}, {w->sdown}, {c.d_model});
  if (rc) return rc;
  DEC_CUDA(cudaMemcpyAsync(L.norm1.p, w->norm1, sizeof(float) * c.d_model, cudaMemcpyDeviceToDevice, d->stream));
  DEC_CUDA(cudaMemcpyAsync(L.norm2.p, w->norm2, sizeof(float) * c.d_model, cudaMemcpyDeviceToDevice, d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  return B200_OK;
}

int b200_decoder_set_embedding(b200_decoder* d, const int8_t* table, const float* row_scales, const float* final_norm) {
  if (!d || !table || !row_scales || !final_norm) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_set_embedding: null");
  const b200_decoder_config& c = d->cfg;
  DEC_CUDA(d->embed_table.alloc((size_t)c.vocab * c.d_model));
  DEC_CUDA(d->embed_scales.alloc(sizeof(float) * c.vocab));
  DEC_CUDA(cudaMemcpyAsync(d->embed_table.p, table, (size_t)c.vocab * c.d_model, cudaMemcpyDeviceToDevice, d->stream));
  DEC_CUDA(cudaMemcpyAsync(d->embed_scales.p, row_scales, sizeof(float) * c.vocab, cudaMemcpyDeviceToDevice, d->stream));
  DEC_CUDA(cudaMemcpyAsync(d->final_norm.p, final_norm, sizeof(float) * c.d_model, cudaMemcpyDeviceToDevice, d->stream));
  const size_t first = (size_t)c.tp_rank * d->vl;  // this rank's rows of the tied LM head
  return build_projection(d, &d->lm_head, c.d_model, {table + first * c.d_model}, {row_scales + first}, {d->vl});
}

int b200_decoder_set_allreduce(b200_decoder* d, b200_allreduce_fn fn, void* user) {
  if (!d) return dec_fail(B200_ERR_INVALID_ARGUMENT, "null decoder");
  d->allreduce = fn;
  d->allreduce_user = user;
  return B200_OK;
}

int b200_nccl_unique_id(void* out, size_t bytes) {
  NcclApi* api = nccl_api();
  if (!api) return dec_fail(B200_ERR_UNSUPPORTED, "b200_nccl_unique_id: libnccl.so.2 could not be loaded");
  if (!out || bytes < sizeof(NcclId)) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_nccl_unique_id: need 128 bytes");
  if (api->get_unique_id(static_cast<NcclId*>(out)) != 0) return dec_fail(B200_ERR_CUDA, "ncclGetUniqueId failed");
  return B200_OK;
}

int b200_decoder_init_nccl(b200_decoder* d, const void* unique_id) {
  if (!d || !unique_id) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_init_nccl: null argument");
  NcclApi* api = nccl_api();
  if (!api) return dec_fail(B200_ERR_UNSUPPORTED, "b200_decoder_init_nccl: libnccl.so.2 could not be loaded");
  NcclId id;
  memcpy(&id, unique_id, sizeof(id));
  nccl_release(d);
  const int rc = api->comm_init_rank(&d->nccl_comm, d->cfg.tp_size, id, d->cfg.tp_rank);
  if (rc != 0) {
    snprintf(g_dec_error, sizeof(g_dec_error), "ncclCommInitRank: %s", api->get_error_string ? api->get_error_string(rc) : "failed");
    return B200_ERR_CUDA;
  }
  d->allreduce = nccl_allreduce_cb;
  d->allreduce_user = d->nccl_comm;
  return B200_OK;
}

int b200_decoder_exchange_handle(b200_decoder* d, void* handle_out, size_t bytes) {
  if (!d || !handle_out || bytes < sizeof(cudaIpcMemHandle_t))
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_exchange_handle: need 64 bytes");
  cudaIpcMemHandle_t h;
  DEC_CUDA(cudaIpcGetMemHandle(&h, d->comm.p));
  memcpy(handle_out, &h, sizeof(h));
  return B200_OK;
}

int b200_decoder_connect_peers(b200_decoder* d, const void* handles, size_t bytes_per_handle) {
  if (!d || !handles || bytes_per_handle < sizeof(cudaIpcMemHandle_t))
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_connect_peers: bad argument");
  if (d->peers_connected) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_connect_peers: already connected");
  const int T = d->cfg.tp_size;
  for (int j = 0; j < T; ++j) {
    if (j == d->cfg.tp_rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)j * bytes_per_handle, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      for (int i = 0; i < j; ++i)
        if (i != d->cfg.tp_rank && d->peer_comm[i]) {
          cudaIpcCloseMemHandle(d->peer_comm[i]);
          d->peer_comm[i] = nullptr;
        }
      return dec_fail(B200_ERR_CUDA, "cudaIpcOpenMemHandle (peer exchange buffer)", e);
    }
    d->peer_comm[j] = static_cast<uint8_t*>(p);
  }
  d->peers_connected = T > 1;
  return B200_OK;
}

int b200_decoder_reset(b200_decoder* d) {
  if (!d) return dec_fail(B200_ERR_INVALID_ARGUMENT, "null decoder");
  DEC_CUDA(cudaMemsetAsync(d->positions.p, 0, sizeof(int32_t) * d->cfg.max_batch, d->stream));
  return clear_fault(d);
}

int b200_decoder_clear_fault(b200_decoder* d) {
  if (!d) return dec_fail(B200_ERR_INVALID_ARGUMENT, "null decoder");
  int rc = clear_fault(d);
  if (rc) return rc;
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  return B200_OK;
}

int b200_decoder_set_wait_budget(b200_decoder* d, unsigned long long nanoseconds) {
  if (!d) return dec_fail(B200_ERR_INVALID_ARGUMENT, "null decoder");
  DEC_CUDA(cudaMemcpyAsync(d->zero_ws.as<uint8_t>() + 4 * kStatusBudgetWordOffsetInts, &nanoseconds, sizeof(nanoseconds),
                           cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  return B200_OK;
}

size_t b200_decoder_exchange_bytes(const b200_decoder* d) { return d ? d->comm.bytes : 0; }

int b200_decoder_connect_peer_pointers(b200_decoder* d, void* const* d_exchange_buffers) {
  if (!d || !d_exchange_buffers) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_connect_peer_pointers: null argument");
  if (d->peers_connected) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_connect_peer_pointers: already connected");
  const int T = d->cfg.tp_size;
  for (int j = 0; j < T; ++j) {
    if (j == d->cfg.tp_rank) continue;
    if (!d_exchange_buffers[j]) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_connect_peer_pointers: null peer buffer");
    d->peer_comm[j] = static_cast<uint8_t*>(d_exchange_buffers[j]);
  }
  d->peers_connected = T > 1;
  d->peers_are_ipc = false;
  return B200_OK;
}

void* b200_decoder_exchange_buffer(b200_decoder* d) { return d ? d->comm.p : nullptr; }

int b200_decoder_set_logit_soft_cap(b200_decoder* d, float cap) {
  if (!d || !(cap >= 0.0f)) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_set_logit_soft_cap: bad argument");
  if (d->cfg.tp_size > 1 && cap > 0.0f) return dec_fail(B200_ERR_UNSUPPORTED, "b200_decoder_set_logit_soft_cap: one GPU only");
  d->soft_cap = cap;
  for (auto& g : d->graph)  // captured steps hold the old value
    if (g) {
      cudaGraphExecDestroy(g);
      g = nullptr;
    }
  return B200_OK;
}

int b200_decoder_set_positions(b200_decoder* d, const int32_t* h_positions, int batch) {
  if (!d || !h_positions || batch <= 0 || batch > d->cfg.max_batch) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_set_positions: bad argument");
  for (int i = 0; i < batch; ++i)
    if (h_positions[i] < 0 || h_positions[i] >= d->cfg.max_seq) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_set_positions: position out of range");
  DEC_CUDA(cudaMemcpyAsync(d->positions.p, h_positions, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  return B200_OK;
}

int b200_decoder_step(b200_decoder* d, const int32_t* h_tokens, int batch, int32_t* h_next_tokens, float* d_logits) {
  if (!d || !h_tokens || batch <= 0 || batch > d->cfg.max_batch) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_step: bad argument");
  if (d->lm_head.n == 0) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_step: weights not set");
  memcpy(d->h_tokens_pinned, h_tokens, sizeof(int32_t) * batch);
  DEC_CUDA(cudaMemcpyAsync(d->tokens.p, d->h_tokens_pinned, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, d->stream));
  if (d_logits) {
    int rc = enqueue_step(d, batch, d_logits);  // caller-owned logits buffer: not the captured graph
    if (rc) return rc;
  } else {
    int rc = ensure_graph(d, batch);
    if (rc) return rc;
    DEC_CUDA(cudaGraphLaunch(d->graph[batch], d->stream));
  }
  if (h_next_tokens) {
    // tokens and the device status word come back behind the step, one synchronisation for both
    // (the status word's slot in the pinned buffer follows the max_batch token slots)
    int32_t* h_status = d->h_next_pinned + d->cfg.max_batch;
    DEC_CUDA(cudaMemcpyAsync(d->h_next_pinned, d->next_tokens.p, sizeof(int32_t) * batch, cudaMemcpyDeviceToHost, d->stream));
    DEC_CUDA(cudaMemcpyAsync(h_status, d->zero_ws.p, sizeof(int32_t), cudaMemcpyDeviceToHost, d->stream));
    DEC_CUDA(cudaStreamSynchronize(d->stream));
    memcpy(h_next_tokens, d->h_next_pinned, sizeof(int32_t) * batch);
    if (*h_status != 0) {
      const int code = *h_status;
      clear_fault(d);  // this step's results are void; the next call finds a clean workspace
      snprintf(g_dec_error, sizeof(g_dec_error), "b200_decoder_step: a device-side wait ran out (status %d)", code);
      return B200_ERR_KERNEL_TIMEOUT;
    }
  }
  return B200_OK;
}

int b200_decoder_prefill(b200_decoder* d, int seq, const int32_t* h_tokens, int n_tokens, int32_t* h_next_token) {
  if (!d || !h_tokens || seq < 0 || seq >= d->cfg.max_batch || n_tokens <= 0)
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_prefill: bad argument");
  if (d->lm_head.n == 0) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_prefill: weights not set");
  const b200_decoder_config& c = d->cfg;
  if (c.tp_size > 1 && !d->allreduce)
    return dec_fail(B200_ERR_UNSUPPORTED, "b200_decoder_prefill: a tensor-parallel prompt pass sums through the all-reduce (b200_decoder_init_nccl or b200_decoder_set_allreduce)");
  for (int i = 0; i < n_tokens; ++i)
    if (h_tokens[i] < 0 || h_tokens[i] >= c.vocab) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_prefill: token id out of range");
  int rc = ensure_prefill_bufs(d);
  if (rc) return rc;
  int32_t start = 0;
  DEC_CUDA(cudaMemcpyAsync(&start, d->positions.as<int32_t>() + seq, sizeof(int32_t), cudaMemcpyDeviceToHost, d->stream));
  DEC_CUDA(cudaStreamSynchronize(d->stream));
  if ((long long)start + n_tokens > c.max_seq) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_prefill: the prompt does not fit the cache");
  PrefillBufs& f = *d->pf;
  // the per-step launch count and the GEMV trace describe decode steps: a prompt pass leaves them alone
  const int saved_launches = d->launches, saved_trace = d->trace_next;
  d->trace_next = kTraceSlots;
  struct Restore {
    b200_decoder* d;
    int launches, trace;
    ~Restore() {
      d->launches = launches;
      d->trace_next = trace;
    }
  } restore{d, saved_launches, saved_trace};
  for (int done = 0; done < n_tokens;) {
    const int rows = std::min(f.rows, n_tokens - done);
    for (int i = 0; i < rows; ++i) {
      f.h_stage[i] = h_tokens[done + i];
      f.h_stage[f.rows + i] = start + done + i;
    }
    DEC_CUDA(cudaMemcpyAsync(f.tokens.p, f.h_stage, sizeof(int32_t) * rows, cudaMemcpyHostToDevice, d->stream));
    DEC_CUDA(cudaMemcpyAsync(f.positions.p, f.h_stage + f.rows, sizeof(int32_t) * rows, cudaMemcpyHostToDevice, d->stream));
    rc = enqueue_prefill_chunk(d, seq, rows, done + rows == n_tokens);
    if (rc) return rc;
    done += rows;
    DEC_CUDA(cudaStreamSynchronize(d->stream));  // the staging buffer is reused by the next chunk
  }
  const int32_t end = start + n_tokens;
  DEC_CUDA(cudaMemcpy(d->positions.as<int32_t>() + seq, &end, sizeof(int32_t), cudaMemcpyHostToDevice));
  int32_t next = 0;
  DEC_CUDA(cudaMemcpy(&next, d->next_tokens.as<int32_t>() + seq, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (h_next_token) *h_next_token = next;
  int status = 0;
  DEC_CUDA(cudaMemcpy(&status, d->zero_ws.p, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0) {
    clear_fault(d);
    return dec_fail(B200_ERR_KERNEL_TIMEOUT, "b200_decoder_prefill: a device-side wait ran out");
  }
  return B200_OK;
}

int b200_decoder_run(b200_decoder* d, const int32_t* h_first_tokens, int batch, int steps, int32_t* h_next_tokens) {
  if (!d || batch <= 0 || batch > d->cfg.max_batch || steps <= 0) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_run: bad argument");
  int rc = ensure_graph(d, batch);
  if (rc) return rc;
  if (h_first_tokens) {
    memcpy(d->h_tokens_pinned, h_first_tokens, sizeof(int32_t) * batch);
    DEC_CUDA(cudaMemcpyAsync(d->tokens.p, d->h_tokens_pinned, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, d->stream));
  }
  for (int i = 0; i < steps; ++i) {
    if (i > 0 || !h_first_tokens)
      DEC_CUDA(cudaMemcpyAsync(d->tokens.p, d->next_tokens.p, sizeof(int32_t) * batch, cudaMemcpyDeviceToDevice, d->stream));
    DEC_CUDA(cudaGraphLaunch(d->graph[batch], d->stream));
  }
  if (h_next_tokens) {
    DEC_CUDA(cudaMemcpyAsync(d->h_next_pinned, d->next_tokens.p, sizeof(int32_t) * batch, cudaMemcpyDeviceToHost, d->stream));
    DEC_CUDA(cudaStreamSynchronize(d->stream));
    memcpy(h_next_tokens, d->h_next_pinned, sizeof(int32_t) * batch);
  }
  return B200_OK;
}

int b200_decoder_launches_per_step(const b200_decoder* d) { return d ? d->launches : 0; }

int b200_decoder_time_gemv(b200_decoder* d, int batch, int reps, float* ms_per_step, int* launches_per_step) {
  if (!d || !ms_per_step || batch <= 0 || batch > d->cfg.max_batch || reps <= 0)
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_time_gemv: bad argument");
  if (d->lm_head.n == 0) return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_time_gemv: weights not set");
  const int saved_launches = d->launches;
  // the projections of one step, in step order, over whatever the activation buffers hold
  auto enqueue = [&]() -> int {
    for (auto& lp : d->layers) {
      Layer& L = *lp;
      DEC_CUDA(run_fc(d, L.qkv, batch, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(), d->qkv.as<float>()));
      DEC_CUDA(run_fc(d, L.o, batch, d->q_a.as<int8_t>(), d->sc_a.as<float>(), d->zp_a.as<int32_t>(), d->proj));
      DEC_CUDA(run_fc(d, L.gate_up, batch, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(), d->gate_up.as<float>()));
      DEC_CUDA(run_fc(d, L.down, batch, d->q_f.as<int8_t>(), d->sc_f.as<float>(), d->zp_f.as<int32_t>(), d->down_out));
    }
    DEC_CUDA(run_fc(d, d->lm_head, batch, d->q_d.as<int8_t>(), d->sc_d.as<float>(), d->zp_d.as<int32_t>(), d->logits.as<float>()));
    return B200_OK;
  };
  d->launches = 0;
  int rc = enqueue();  // uncaptured once: one-time kernel attribute set-up
  const int n_launch = d->launches;
  d->launches = saved_launches;
  if (rc) return rc;
  cudaGraph_t g = nullptr;
  cudaGraphExec_t ge = nullptr;
  DEC_CUDA(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
  rc = enqueue();
  d->launches = saved_launches;
  cudaError_t e = cudaStreamEndCapture(d->stream, &g);
  if (rc || e != cudaSuccess) {
    if (g) cudaGraphDestroy(g);
    return rc ? rc : dec_fail(B200_ERR_CUDA, "cudaStreamEndCapture", e);
  }
  e = cudaGraphInstantiate(&ge, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return dec_fail(B200_ERR_CUDA, "cudaGraphInstantiate", e);
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  for (int i = 0; i < 2; ++i) cudaGraphLaunch(ge, d->stream);
  cudaEventRecord(a, d->stream);
  for (int i = 0; i < reps; ++i) cudaGraphLaunch(ge, d->stream);
  cudaEventRecord(b, d->stream);
  e = cudaStreamSynchronize(d->stream);
  float ms = 0.0f;
  cudaEventElapsedTime(&ms, a, b);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  cudaGraphExecDestroy(ge);
  if (e != cudaSuccess) return dec_fail(B200_ERR_CUDA, "b200_decoder_time_gemv", e);
  *ms_per_step = ms / (float)reps;
  if (launches_per_step) *launches_per_step = n_launch;
  return B200_OK;
}

int b200_decoder_profile_step(b200_decoder* d, const int32_t* h_tokens, int batch, float* ms_by_class,
                              int* launches_by_class) {
  if (!d || !h_tokens || !ms_by_class || batch <= 0 || batch > d->cfg.max_batch)
    return dec_fail(B200_ERR_INVALID_ARGUMENT, "b200_decoder_profile_step: bad argument");
  memcpy(d->h_tokens_pinned, h_tokens, sizeof(int32_t) * batch);
  DEC_CUDA(cudaMemcpyAsync(d->tokens.p, d->h_tokens_pinned, sizeof(int32_t) * batch, cudaMemcpyHostToDevice, d->stream));
  d->profiling = true;
  d->prof_events.clear();
  d->prof_class.clear();
  int rc = enqueue_step(d, batch, nullptr);
  d->profiling = false;
  cudaError_t e = cudaStreamSynchronize(d->stream);
  for (int c = 0; c < 3; ++c) {
    ms_by_class[c] = 0.0f;
    if (launches_by_class) launches_by_class[c] = 0;
  }
  for (size_t i = 0; i < d->prof_class.size(); ++i) {
    float ms = 0.0f;
    if (e == cudaSuccess) cudaEventElapsedTime(&ms, d->prof_events[2 * i], d->prof_events[2 * i + 1]);
    ms_by_class[d->prof_class[i]] += ms;
    if (launches_by_class) launches_by_class[d->prof_class[i]] += 1;
    cudaEventDestroy(d->prof_events[2 * i]);
    cudaEventDestroy(d->prof_events[2 * i + 1]);
  }
  d->prof_events.clear();
  d->prof_class.clear();
  if (rc) return rc;
  if (e != cudaSuccess) return dec_fail(B200_ERR_CUDA, "b200_decoder_profile_step", e);
  return B200_OK;
}

const char* b200_decoder_last_error(void) { return g_dec_error; }

}  // extern "C"
