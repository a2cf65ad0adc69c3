/*
 * CPU restatement of one decode step of a Gemma-shaped decoder-only graph whose
 * projections are dynamic-range (hybrid) int8 FULLY_CONNECTED ops. TEST
 * INFRASTRUCTURE ONLY (parity arbiter and timed CPU baseline of the decode
 * benchmark).
 *
 * The graph is the one tensor/examples/gemma3/gemma3_graph.cc authors out of
 * TFLite ops (RMS norm, q/k/v projections, rotary embedding as
 * x*cos + rotate_half(x)*sin :150-176, attention, output projection, residual
 * adds, GeGLU feed-forward :118-146, final norm, tied LM head), with the
 * Gemma-1 layout the benchmark names: one KV head (MQA), no q/k norms, no
 * post-norms. Every projection goes through the hybrid kernel restated in
 * oracle.c (orc_fc_hybrid, asymmetric inputs, per-channel scales); the
 * embedding is the hybrid EMBEDDING_LOOKUP (tflite/kernels/embedding_lookup.cc:
 * int8 row times its per-row scale); attention is orc_sdpa_f32 over the cached
 * prefix. `fast` != 0 swaps in the vectorised multi-threaded twins of
 * oracle_fast.c (same formulas) for timing.
 *
 * Tensor-parallel shards: a shard decoder is created with this rank's head and
 * feed-forward counts and given this rank's slices of the weights (q/gate/up by
 * output rows, o/down by input columns). The partial outputs of the two
 * input-sharded projections are summed over ranks by the hook set with
 * orc_decoder_set_reduce before the residual add; the LM head may be limited to
 * a row range of the table (orc_decoder_set_lm_rows), the winner over ranks is
 * then picked by the caller. Each shard quantizes its own slice of the
 * activation row, as a graph with one FULLY_CONNECTED per shard would.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "oracle.h"
#include "oracle_fast.h"

typedef struct {
  int n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, max_seq;
  float rms_eps, rope_base, embed_scale;
} orc_decoder_config;

typedef struct {
  const int8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
  const float *sq, *sk, *sv, *so, *sgate, *sup, *sdown; /* per-output-channel scales */
  const float *norm1, *norm2;                            /* RMS norm gains [d_model] */
} orc_decoder_layer;

typedef struct {
  orc_decoder_config cfg;
  orc_decoder_layer* layers;
  const int8_t* embed; /* [vocab, d_model] */
  const float* embed_scales; /* [vocab] */
  const float* final_norm;
  float* k_cache; /* [layers][batch][max_seq][kvh*hd] */
  float* v_cache;
  int* lengths; /* [batch] */
  int batch;
  int fast;
  void (*reduce)(void* user, float* buf, size_t count); /* in-place sum over ranks, or NULL */
  void* reduce_user;
  int lm_first, lm_rows; /* LM head rows [lm_first, lm_first + lm_rows) of the table */
  int kv_mode;           /* how a row is kept in the cache: 0 float32, 1 rounded to binary16, 2 int8 per token */
} orc_decoder;

static void fc(const orc_decoder* d, int m, int n, int k, const float* x, const int8_t* w, const float* s, float* y) {
  if (d->fast) {
    orcf_fc_hybrid(m, n, k, x, w, s, 1, NULL, 1, ORC_ACT_NONE, NULL, y);
  } else {
    orc_fc_hybrid(m, n, k, x, w, s, 1, NULL, 1, ORC_ACT_NONE, y);
  }
}

/* ---- the stages between the projections, one function each (also called on their own by the
 * per-kernel parity tests) ------------------------------------------------------------------- */

/* Hybrid EMBEDDING_LOOKUP (tflite/kernels/embedding_lookup.cc:EvalHybrid: value * row scale), then the
 * embedding scale the graph applies as a MUL (tensor/examples/gemma3/gemma3_graph.cc). */
void orc_stage_embed(const int32_t* tokens, int rows, const int8_t* table, const float* row_scales, int d,
                     float embed_scale, float* h) {
  for (int b = 0; b < rows; ++b) {
    const int8_t* row = table + (size_t)tokens[b] * d;
    const float s = row_scales[tokens[b]];
    for (int i = 0; i < d; ++i) h[(size_t)b * d + i] = (float)row[i] * s * embed_scale;
  }
}

static void rms_norm(const float* x, const float* gain, int n, float eps, float* y) {
  float ss = 0.0f;
  for (int i = 0; i < n; ++i) ss += x[i] * x[i];
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i) y[i] = x[i] * inv * gain[i];
}

/* h += delta (residual ADD, skipped when delta is NULL); x = rms_norm(h) * gain. */
void orc_stage_add_rmsnorm(float* h, const float* delta, const float* gain, int rows, int d, float eps, float* x) {
  if (delta)
    for (size_t i = 0; i < (size_t)rows * d; ++i) h[i] += delta[i];
  for (int b = 0; b < rows; ++b) rms_norm(h + (size_t)b * d, gain, d, eps, x + (size_t)b * d);
}

/* Rotation angles as the graph's host side prepares them: the cos and sin tensors are INPUTS of the
 * graph (gemma3_graph.cc:150-176 multiplies by them), angle of pair i at position pos =
 * pos * base^(-2i/head_dim). cs[pos][i] = {cos, sin}, i < head_dim / 2. */
void orc_rope_table(int max_seq, int head_dim, float base, float* cs) {
  const int half = head_dim / 2;
  for (int pos = 0; pos < max_seq; ++pos)
    for (int i = 0; i < half; ++i) {
      const float freq = powf(base, -2.0f * (float)i / (float)head_dim);
      const float ang = (float)pos * freq;
      cs[((size_t)pos * half + i) * 2] = cosf(ang);
      cs[((size_t)pos * half + i) * 2 + 1] = sinf(ang);
    }
}

/* x*cos + rotate_half(x)*sin with rotate_half(x) = cat(-x2, x1) */
static void rope(float* x, int head_dim, int pos, float base) {
  const int half = head_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float freq = powf(base, -2.0f * (float)i / (float)head_dim);
    const float ang = (float)pos * freq;
    const float c = cosf(ang), s = sinf(ang);
    const float x1 = x[i], x2 = x[i + half];
    x[i] = x1 * c - x2 * s;
    x[i + half] = x2 * c + x1 * s;
  }
}

/* Rotates `heads` heads per row in place, row r at positions[r]. */
void orc_stage_rope(float* x, int rows, int heads, int head_dim, const int32_t* positions, float base) {
  for (int r = 0; r < rows; ++r)
    for (int hh = 0; hh < heads; ++hh) rope(x + ((size_t)r * heads + hh) * head_dim, head_dim, positions[r], base);
}

static float gelu_tanh(float v) {
  const float k0 = 0.7978845608028654f; /* sqrt(2/pi) */
  return 0.5f * v * (1.0f + tanhf(k0 * (v + 0.044715f * v * v * v)));
}

/* out = gelu_tanh(gate) * up (GELU approximate=true then MUL, gemma3_graph.cc:118-146). */
void orc_stage_geglu(const float* gate, const float* up, size_t count, float* out) {
  for (size_t i = 0; i < count; ++i) out[i] = gelu_tanh(gate[i]) * up[i];
}

/* Logit soft-cap: tanh(x / cap) * cap (litert/vendors/nvidia/trtllm/head_kernels.cu:35-43). */
void orc_stage_softcap(float* logits, size_t count, float cap) {
  const float inv = 1.0f / cap;
  for (size_t i = 0; i < count; ++i) logits[i] = tanhf(logits[i] * inv) * cap;
}

/* Greedy pick per row: the serial scan of the CPU sampler, whose behaviour with NaNs the reference's GPU
 * sampler preserves (litert/vendors/nvidia/dispatch/greedy_sampler_kernel.cu:31-50): a NaN at index 0
 * wins, a NaN anywhere else never does, ties go to the lower index. */
void orc_stage_argmax(const float* logits, int rows, int n, int32_t* out) {
  for (int b = 0; b < rows; ++b) {
    const float* lg = logits + (size_t)b * n;
    int best = 0;
    for (int i = 1; i < n; ++i)
      if (lg[i] > lg[best]) best = i;
    out[b] = best;
  }
}

orc_decoder* orc_decoder_create(const orc_decoder_config* cfg, int batch, int fast) {
  orc_decoder* d = (orc_decoder*)calloc(1, sizeof(orc_decoder));
  d->cfg = *cfg;
  d->batch = batch;
  d->fast = fast;
  d->layers = (orc_decoder_layer*)calloc((size_t)cfg->n_layers, sizeof(orc_decoder_layer));
  const size_t kv = (size_t)cfg->n_layers * batch * cfg->max_seq * cfg->n_kv_heads * cfg->head_dim;
  d->k_cache = (float*)calloc(kv, sizeof(float));
  d->v_cache = (float*)calloc(kv, sizeof(float));
  d->lengths = (int*)calloc((size_t)batch, sizeof(int));
  d->lm_first = 0;
  d->lm_rows = cfg->vocab;
  return d;
}

void orc_decoder_destroy(orc_decoder* d) {
  free(d->layers);
  free(d->k_cache);
  free(d->v_cache);
  free(d->lengths);
  free(d);
}

void orc_decoder_set_layer(orc_decoder* d, int layer, const orc_decoder_layer* w) { d->layers[layer] = *w; }
void orc_decoder_set_embedding(orc_decoder* d, const int8_t* w, const float* scales, const float* final_norm) {
  d->embed = w;
  d->embed_scales = scales;
  d->final_norm = final_norm;
}
void orc_decoder_set_reduce(orc_decoder* d, void (*fn)(void*, float*, size_t), void* user) {
  d->reduce = fn;
  d->reduce_user = user;
}
void orc_decoder_set_lm_rows(orc_decoder* d, int first, int rows) {
  d->lm_first = first;
  d->lm_rows = rows;
}
/* The device keeps its cache in binary16 or int8 (one symmetric scale per token and KV head, scale =
 * max|row| / 127): with kv_mode 1 / 2 the CPU graph stores the same rounded values (as float32). */
void orc_decoder_set_kv_mode(orc_decoder* d, int mode) { d->kv_mode = mode; }

void orc_stage_kv_round(float* row, int n, int mode) {
  if (mode == 1) {
    for (int i = 0; i < n; ++i) row[i] = orc_half_to_float(orc_float_to_half(row[i]));
  } else if (mode == 2) {
    float amax = 0.0f;
    for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(row[i]));
    const float sc = amax > 0.0f ? amax / 127.0f : 1.0f;
    for (int i = 0; i < n; ++i) {
      float q = nearbyintf(row[i] / sc);
      q = q > 127.0f ? 127.0f : (q < -127.0f ? -127.0f : q);
      row[i] = q * sc;
    }
  }
}

/* Declares lengths[b] tokens already cached for sequence b (whatever the cache rows hold): lets the
 * timed CPU baseline step at the same context depth as the device without stepping there first. */
void orc_decoder_set_lengths(orc_decoder* d, const int32_t* lengths) {
  for (int b = 0; b < d->batch; ++b) d->lengths[b] = lengths[b] < d->cfg.max_seq ? lengths[b] : d->cfg.max_seq - 1;
}

void orc_decoder_reset(orc_decoder* d) { memset(d->lengths, 0, sizeof(int) * (size_t)d->batch); }

/* One token per sequence: tokens [batch] -> logits [batch, lm_rows] (may be NULL) and the greedy next
 * token (first index of the maximum, as a row number of the whole table). Appends to the caches. */
void orc_decoder_step(orc_decoder* d, const int32_t* tokens, float* logits_out, int32_t* next_tokens) {
  const orc_decoder_config* c = &d->cfg;
  const int B = d->batch, D = c->d_model, H = c->n_heads, KVH = c->n_kv_heads, HD = c->head_dim, F = c->d_ff;
  float* h = (float*)malloc(sizeof(float) * (size_t)B * D);
  float* x = (float*)malloc(sizeof(float) * (size_t)B * D);
  float* q = (float*)malloc(sizeof(float) * (size_t)B * H * HD);
  float* kk = (float*)malloc(sizeof(float) * (size_t)B * KVH * HD);
  float* vv = (float*)malloc(sizeof(float) * (size_t)B * KVH * HD);
  float* att = (float*)malloc(sizeof(float) * (size_t)B * H * HD);
  float* o = (float*)malloc(sizeof(float) * (size_t)B * D);
  float* gate = (float*)malloc(sizeof(float) * (size_t)B * F);
  float* up = (float*)malloc(sizeof(float) * (size_t)B * F);
  float* logits = logits_out ? logits_out : (float*)malloc(sizeof(float) * (size_t)B * d->lm_rows);

  orc_stage_embed(tokens, B, d->embed, d->embed_scales, D, c->embed_scale, h);
  const size_t per_seq = (size_t)c->max_seq * KVH * HD;
  for (int l = 0; l < c->n_layers; ++l) {
    const orc_decoder_layer* w = &d->layers[l];
    for (int b = 0; b < B; ++b) rms_norm(h + (size_t)b * D, w->norm1, D, c->rms_eps, x + (size_t)b * D);
    fc(d, B, H * HD, D, x, w->wq, w->sq, q);
    fc(d, B, KVH * HD, D, x, w->wk, w->sk, kk);
    fc(d, B, KVH * HD, D, x, w->wv, w->sv, vv);
    float* kc = d->k_cache + (size_t)l * B * per_seq;
    float* vc = d->v_cache + (size_t)l * B * per_seq;
    for (int b = 0; b < B; ++b) {
      const int pos = d->lengths[b];
      for (int hh = 0; hh < H; ++hh) rope(q + ((size_t)b * H + hh) * HD, HD, pos, c->rope_base);
      for (int hh = 0; hh < KVH; ++hh) rope(kk + ((size_t)b * KVH + hh) * HD, HD, pos, c->rope_base);
      memcpy(kc + (size_t)b * per_seq + (size_t)pos * KVH * HD, kk + (size_t)b * KVH * HD, sizeof(float) * KVH * HD);
      memcpy(vc + (size_t)b * per_seq + (size_t)pos * KVH * HD, vv + (size_t)b * KVH * HD, sizeof(float) * KVH * HD);
      if (d->kv_mode)
        for (int hh = 0; hh < KVH; ++hh) {
          orc_stage_kv_round(kc + (size_t)b * per_seq + ((size_t)pos * KVH + hh) * HD, HD, d->kv_mode);
          orc_stage_kv_round(vc + (size_t)b * per_seq + ((size_t)pos * KVH + hh) * HD, HD, d->kv_mode);
        }
      const int len = pos + 1;
      const float scale = 1.0f / sqrtf((float)HD);
      if (d->fast) {
        orcf_sdpa_f32(1, 1, H, KVH, HD, len, q + (size_t)b * H * HD, kc + (size_t)b * per_seq, vc + (size_t)b * per_seq,
                      NULL, NULL, scale, att + (size_t)b * H * HD);
      } else {
        orc_sdpa_f32(1, 1, H, KVH, HD, len, q + (size_t)b * H * HD, kc + (size_t)b * per_seq, vc + (size_t)b * per_seq,
                     NULL, scale, 0.0f, att + (size_t)b * H * HD);
      }
    }
    fc(d, B, D, H * HD, att, w->wo, w->so, o);
    if (d->reduce) d->reduce(d->reduce_user, o, (size_t)B * D);
    for (size_t i = 0; i < (size_t)B * D; ++i) h[i] += o[i];
    for (int b = 0; b < B; ++b) rms_norm(h + (size_t)b * D, w->norm2, D, c->rms_eps, x + (size_t)b * D);
    fc(d, B, F, D, x, w->wgate, w->sgate, gate);
    fc(d, B, F, D, x, w->wup, w->sup, up);
    orc_stage_geglu(gate, up, (size_t)B * F, gate);
    fc(d, B, D, F, gate, w->wdown, w->sdown, o);
    if (d->reduce) d->reduce(d->reduce_user, o, (size_t)B * D);
    for (size_t i = 0; i < (size_t)B * D; ++i) h[i] += o[i];
  }
  for (int b = 0; b < B; ++b) rms_norm(h + (size_t)b * D, d->final_norm, D, c->rms_eps, x + (size_t)b * D);
  fc(d, B, d->lm_rows, D, x, d->embed + (size_t)d->lm_first * D, d->embed_scales + d->lm_first, logits);
  for (int b = 0; b < B; ++b) {
    int32_t best = 0;
    orc_stage_argmax(logits + (size_t)b * d->lm_rows, 1, d->lm_rows, &best);
    if (next_tokens) next_tokens[b] = d->lm_first + best;
    d->lengths[b] += 1;
  }
  free(h); free(x); free(q); free(kk); free(vv); free(att); free(o); free(gate); free(up);
  if (!logits_out) free(logits);
}
