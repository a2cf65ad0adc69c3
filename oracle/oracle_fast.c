/* See oracle_fast.h. TEST INFRASTRUCTURE ONLY. */
#include "oracle_fast.h"

#include <math.h>
#include <pthread.h>
#include <unistd.h>
#include <stdlib.h>
#include <string.h>

#include "oracle.h"

/* Runtime-dispatched SIMD: the compiler vectorises these plain loops once per
 * listed target and picks the best one the host supports when the library is
 * loaded, so one build runs on any x86-64 host. */
#if defined(__x86_64__)
#define ORCF_CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))
#else
#define ORCF_CLONES
#endif


/* ---- a small persistent thread pool (no OpenMP runtime in this image) ---- */
typedef void (*range_fn)(int begin, int end, void* ctx);
#define ORCF_MAX_THREADS 256
static struct {
  pthread_t threads[ORCF_MAX_THREADS];
  int started;      /* worker threads alive */
  int want;         /* threads to use, including the caller */
  pthread_mutex_t mu;
  pthread_cond_t work_cv, done_cv;
  unsigned long generation;
  int pending;
  range_fn fn;
  void* ctx;
  int total, parts;
} g_pool = {.mu = PTHREAD_MUTEX_INITIALIZER, .work_cv = PTHREAD_COND_INITIALIZER,
            .done_cv = PTHREAD_COND_INITIALIZER};

static void run_part(int part) {
  const long long total = g_pool.total, parts = g_pool.parts;
  const int begin = (int)(total * part / parts), end = (int)(total * (part + 1) / parts);
  if (end > begin) g_pool.fn(begin, end, g_pool.ctx);
}

static void* worker_main(void* arg) {
  const int id = (int)(long)arg; /* 1.. */
  unsigned long seen = 0;
  for (;;) {
    pthread_mutex_lock(&g_pool.mu);
    while (g_pool.generation == seen) pthread_cond_wait(&g_pool.work_cv, &g_pool.mu);
    seen = g_pool.generation;
    const int active = id < g_pool.parts;
    pthread_mutex_unlock(&g_pool.mu);
    if (active) {
      run_part(id);
      pthread_mutex_lock(&g_pool.mu);
      if (--g_pool.pending == 0) pthread_cond_signal(&g_pool.done_cv);
      pthread_mutex_unlock(&g_pool.mu);
    }
  }
  return NULL;
}

int orcf_num_threads(void) {
  if (g_pool.want == 0) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    g_pool.want = n < 1 ? 1 : (n > ORCF_MAX_THREADS ? ORCF_MAX_THREADS : (int)n);
  }
  return g_pool.want;
}
void orcf_set_num_threads(int n) { g_pool.want = n < 1 ? 1 : (n > ORCF_MAX_THREADS ? ORCF_MAX_THREADS : n); }

/* Calls fn over [0,total) split into contiguous ranges, one per thread. Not
 * re-entrant: one parallel region at a time (the bench is single-threaded). */
static void parallel_for(int total, range_fn fn, void* ctx) {
  int parts = orcf_num_threads();
  if (parts > total) parts = total;
  if (parts <= 1) {
    if (total > 0) fn(0, total, ctx);
    return;
  }
  pthread_mutex_lock(&g_pool.mu);
  while (g_pool.started < parts - 1) {
    const int id = g_pool.started + 1;
    pthread_create(&g_pool.threads[id], NULL, worker_main, (void*)(long)id);
    pthread_detach(g_pool.threads[id]);
    ++g_pool.started;
  }
  g_pool.fn = fn;
  g_pool.ctx = ctx;
  g_pool.total = total;
  g_pool.parts = parts;
  g_pool.pending = parts - 1;
  ++g_pool.generation;
  pthread_cond_broadcast(&g_pool.work_cv);
  pthread_mutex_unlock(&g_pool.mu);
  run_part(0);
  pthread_mutex_lock(&g_pool.mu);
  while (g_pool.pending != 0) pthread_cond_wait(&g_pool.done_cv, &g_pool.mu);
  pthread_mutex_unlock(&g_pool.mu);
}

ORCF_CLONES
static int32_t dot_s8(const int8_t* restrict a, const int8_t* restrict b, int k) {
  int32_t acc = 0;
  for (int i = 0; i < k; ++i) acc += (int32_t)((int16_t)a[i] * (int16_t)b[i]);
  return acc;
}

ORCF_CLONES
static int32_t sum_s8(const int8_t* restrict a, int k) {
  int32_t acc = 0;
  for (int i = 0; i < k; ++i) acc += a[i];
  return acc;
}

ORCF_CLONES
static float dot_f32(const float* restrict a, const float* restrict b, int k) {
  /* eight partial sums: vector-friendly; SDPA tolerance covers the reorder */
  float p[16] = {0};
  int i = 0;
  for (; i + 16 <= k; i += 16)
    for (int j = 0; j < 16; ++j) p[j] += a[i + j] * b[i + j];
  float acc = 0;
  for (int j = 0; j < 16; ++j) acc += p[j];
  for (; i < k; ++i) acc += a[i] * b[i];
  return acc;
}

ORCF_CLONES
static void axpy_f32(float alpha, const float* restrict x, float* restrict y, int k) {
  for (int i = 0; i < k; ++i) y[i] += alpha * x[i];
}

typedef struct {
  int m, n, k, blocksize, num_blocks, per_channel, asymmetric;
  const int8_t* x8;
  const float* xf;
  const int8_t* w;
  const uint8_t* w4;
  const uint16_t* scales_f16;
  const int32_t* bias_i32;
  const float* bias_f32;
  const float* filter_scales;
  int32_t input_offset, output_offset, act_min, act_max;
  const int32_t* multipliers;
  const int32_t* shifts;
  const int32_t* row_sums_in;
  int32_t* row_sums_out;
  int8_t* q;
  float* scales;
  int32_t* zps;
  int8_t* y8;
  float* yf;
} fc_ctx;

static void row_sums_range(int begin, int end, void* p) {
  fc_ctx* c = (fc_ctx*)p;
  for (int r = begin; r < end; ++r) c->row_sums_out[r] = sum_s8(c->w + (size_t)r * c->k, c->k);
}

void orcf_row_sums(int n, int k, const int8_t* w, int32_t* row_sums) {
  fc_ctx c = {.n = n, .k = k, .w = w, .row_sums_out = row_sums};
  parallel_for(n, row_sums_range, &c);
}

/* Same arithmetic as orc_fc_int8_per_channel with ORC_REQUANT_MBQM:
 * sum w*(x+off) = sum w*x + off*sum w. */
static void fc_int8_range(int begin, int end, void* p) {
  fc_ctx* c = (fc_ctx*)p;
  const int k = c->k;
  for (int ch = begin; ch < end; ++ch) {
    const int8_t* row = c->w + (size_t)ch * k;
    const int32_t rs = sum_s8(row, k);
    for (int b = 0; b < c->m; ++b) {
      int32_t acc = dot_s8(row, c->x8 + (size_t)b * k, k) + c->input_offset * rs;
      if (c->bias_i32) acc += c->bias_i32[ch];
      int32_t v = orc_multiply_by_quantized_multiplier(acc, c->multipliers[ch], c->shifts[ch]) + c->output_offset;
      v = v < c->act_min ? c->act_min : (v > c->act_max ? c->act_max : v);
      c->y8[(size_t)b * c->n + ch] = (int8_t)v;
    }
  }
}

void orcf_fc_int8_per_channel(int m, int n, int k, const int8_t* x, const int8_t* w, const int32_t* bias,
                              int32_t input_offset, int32_t output_offset, const int32_t* multipliers,
                              const int32_t* shifts, int32_t act_min, int32_t act_max, int8_t* y) {
  fc_ctx c = {.m = m, .n = n, .k = k, .x8 = x, .w = w, .bias_i32 = bias, .input_offset = input_offset,
              .output_offset = output_offset, .multipliers = multipliers, .shifts = shifts,
              .act_min = act_min, .act_max = act_max, .y8 = y};
  parallel_for(n, fc_int8_range, &c);
}

static void quantize_range(int begin, int end, void* p) {
  fc_ctx* c = (fc_ctx*)p;
  const int k = c->k;
  for (int b = begin; b < end; ++b) {
    if (c->asymmetric) {
      orc_asymmetric_quantize_floats(c->xf + (size_t)b * k, k, c->q + (size_t)b * k, &c->scales[b], &c->zps[b]);
    } else {
      orc_symmetric_quantize_floats(c->xf + (size_t)b * k, k, c->q + (size_t)b * k, &c->scales[b]);
      c->zps[b] = 0;
    }
    if (!c->per_channel && c->filter_scales) c->scales[b] *= c->filter_scales[0];
  }
}

static void fc_hybrid_range(int begin, int end, void* p) {
  fc_ctx* c = (fc_ctx*)p;
  const int k = c->k;
  for (int r = begin; r < end; ++r) {
    const int8_t* row = c->w + (size_t)r * k;
    const int32_t rs = c->row_sums_in ? c->row_sums_in[r] : sum_s8(row, k);
    for (int b = 0; b < c->m; ++b) {
      float scale = c->scales[b];
      if (c->per_channel) scale *= c->filter_scales[r];
      int32_t dot = dot_s8(row, c->q + (size_t)b * k, k);
      dot -= rs * c->zps[b];
      float out = c->bias_f32 ? c->bias_f32[r] : 0.0f;
      out += (float)dot * scale;
      c->yf[(size_t)b * c->n + r] = out;
    }
  }
}

/* orc_fc_hybrid, weight-stationary. row_sums may be NULL (computed here), or
 * the cached ones, as the reference caches them after the first call. */
void orcf_fc_hybrid(int m, int n, int k, const float* x, const int8_t* w, const float* filter_scales,
                    int per_channel, const float* bias, int asymmetric_inputs, int activation,
                    const int32_t* row_sums, float* y) {
  fc_ctx c = {.m = m, .n = n, .k = k, .xf = x, .w = w, .filter_scales = filter_scales,
              .per_channel = per_channel, .bias_f32 = bias, .asymmetric = asymmetric_inputs,
              .row_sums_in = row_sums, .yf = y};
  c.q = (int8_t*)malloc((size_t)m * k);
  c.scales = (float*)malloc(sizeof(float) * (size_t)m);
  c.zps = (int32_t*)malloc(sizeof(int32_t) * (size_t)m);
  parallel_for(m, quantize_range, &c);
  parallel_for(n, fc_hybrid_range, &c);
  orc_apply_activation(y, (size_t)m * n, activation);
  free(c.q);
  free(c.scales);
  free(c.zps);
}

ORCF_CLONES
static void unpack_row_int4(const uint8_t* restrict src, int k, int8_t* restrict dst) {
  for (int i = 0; i < k / 2; ++i) {
    const uint8_t b = src[i];
    dst[2 * i] = (int8_t)(((b & 0xF) ^ 8) - 8);
    dst[2 * i + 1] = (int8_t)(((b >> 4) ^ 8) - 8);
  }
}

static void fc_w4_range(int begin, int end, void* p) {
  fc_ctx* c = (fc_ctx*)p;
  const int k = c->k, bs = c->blocksize, nb = c->num_blocks;
  const size_t k2 = ((size_t)k + 1) & ~(size_t)1;
  int8_t* row = (int8_t*)malloc((size_t)k + 64);
  float* sc = (float*)malloc(sizeof(float) * (size_t)nb);
  for (int ni = begin; ni < end; ++ni) {
    unpack_row_int4(c->w4 + (size_t)ni * k2 / 2, k, row);
    float kfsum = 0.0f;
    for (int bi = 0; bi < nb; ++bi) {
      sc[bi] = orc_half_to_float(c->scales_f16[(size_t)ni * nb + bi]);
      kfsum += sc[bi] * (float)sum_s8(row + bi * bs, bs);
    }
    for (int mi = 0; mi < c->m; ++mi) {
      float out = 0.0f;
      for (int bi = 0; bi < nb; ++bi) {
        const int32_t acc = dot_s8(row + bi * bs, c->q + (size_t)mi * k + bi * bs, bs);
        out += (float)acc * sc[bi];
      }
      out -= (float)c->zps[mi] * kfsum;
      out *= c->scales[mi];
      if (c->bias_f32) out += c->bias_f32[ni];
      c->yf[(size_t)mi * c->n + ni] = out;
    }
  }
  free(row);
  free(sc);
}

void orcf_fc_blockwise4(int m, int n, int k, int blocksize, const float* x, const uint8_t* w4,
                        const uint16_t* scales_f16, const float* bias, float* y) {
  fc_ctx c = {.m = m, .n = n, .k = k, .blocksize = blocksize, .num_blocks = k / blocksize, .xf = x,
              .w4 = w4, .scales_f16 = scales_f16, .bias_f32 = bias, .asymmetric = 1, .per_channel = 1,
              .yf = y};
  c.q = (int8_t*)malloc((size_t)m * k);
  c.scales = (float*)malloc(sizeof(float) * (size_t)m);
  c.zps = (int32_t*)malloc(sizeof(int32_t) * (size_t)m);
  parallel_for(m, quantize_range, &c);
  parallel_for(n, fc_w4_range, &c);
  free(c.q);
  free(c.scales);
  free(c.zps);
}

typedef struct {
  int b, t, n, nkv, h, s;
  const float *q, *k, *v, *mask;
  const int32_t* lengths;
  float scale;
  float* out;
} sdpa_ctx;

static void sdpa_range(int begin, int end, void* p) {
  sdpa_ctx* c = (sdpa_ctx*)p;
  const int t = c->t, n = c->n, nkv = c->nkv, h = c->h, s = c->s;
  const int group = n / nkv;
  float* logits = (float*)malloc(sizeof(float) * (size_t)s);
  float* qs = (float*)malloc(sizeof(float) * (size_t)h);
  for (int idx = begin; idx < end; ++idx) {
    const int ni = idx % n, ti = (idx / n) % t, bi = idx / (n * t);
    const int kv = ni / group;
    const int len = c->lengths ? c->lengths[bi] : s;
    const float* qp = c->q + (((size_t)bi * t + ti) * n + ni) * h;
    for (int hi = 0; hi < h; ++hi) qs[hi] = qp[hi] * c->scale;
    float mx = -3.402823466e+38f;
    for (int si = 0; si < len; ++si) {
      float acc = dot_f32(qs, c->k + (((size_t)bi * s + si) * nkv + kv) * h, h);
      if (c->mask) acc += c->mask[((size_t)bi * t + ti) * s + si];
      logits[si] = acc;
      mx = acc > mx ? acc : mx;
    }
    float sum = 0.0f;
    for (int si = 0; si < len; ++si) {
      logits[si] = expf(logits[si] - mx);
      sum += logits[si];
    }
    float* op = c->out + (((size_t)bi * t + ti) * n + ni) * h;
    memset(op, 0, sizeof(float) * (size_t)h);
    for (int si = 0; si < len; ++si)
      axpy_f32(logits[si] / sum, c->v + (((size_t)bi * s + si) * nkv + kv) * h, op, h);
  }
  free(logits);
  free(qs);
}

/* orc_sdpa_f32 spread over (batch, query token, head); lengths (optional)
 * bounds the key range per batch entry instead of a mask of large negatives. */
void orcf_sdpa_f32(int b, int t, int n, int nkv, int h, int s, const float* q, const float* k,
                   const float* v, const float* mask, const int32_t* lengths, float scale, float* out) {
  sdpa_ctx c = {b, t, n, nkv, h, s, q, k, v, mask, lengths, scale, out};
  parallel_for(b * t * n, sdpa_range, &c);
}
