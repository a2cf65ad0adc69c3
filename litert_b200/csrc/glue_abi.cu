// C-ABI entry points of the ops between the projections of a decoder layer (declared in
// include/litert_b200.h under "decoder glue ops"): argument checks and launches of the kernels in
// decoder_kernels.cu / sdpa_decode.cu on caller-supplied device tensors. The resident decoder
// (decoder.cu) launches the same kernels.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/litert_b200.h"
#include "common.cuh"
#include "decoder_kernels.h"
#include "kernels.h"
#include "quant.cuh"

namespace {

using namespace b200;

thread_local char g_glue_error[512] = "";

int gfail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_glue_error, sizeof(g_glue_error), fmt, ap);
  va_end(ap);
  return code;
}
int gcuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return B200_OK;
  return gfail(B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

__global__ void untile_rows_kernel(const int8_t* __restrict__ q_tiled, int m, int k, int m_alloc, int8_t* __restrict__ out) {
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < k; i += blockDim.x) out[(size_t)row * k + i] = q_tiled[q_tiled_offset(row, i, m_alloc)];
}

template <typename T>
__global__ void transpose_matrices_kernel(const T* __restrict__ in, T* __restrict__ out, int rows, int cols) {
  __shared__ T tile[32][33];
  const size_t base = (size_t)blockIdx.z * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[base + (size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) out[base + (size_t)c * rows + r] = tile[threadIdx.x][j];
  }
}

void fill_fc_ws(FcParams& p, void* d_zero_ws) {
  uint8_t* z = static_cast<uint8_t*>(d_zero_ws);
  p.status = reinterpret_cast<int*>(z);
  p.ws_count = reinterpret_cast<int32_t*>(z + zero_ws_counter_off());
  p.ws_part = reinterpret_cast<int32_t*>(z + zero_ws_part_off());
}

}  // namespace

extern "C" {

const char* b200_glue_last_error(void) { return g_glue_error; }

size_t b200_tiled_rows_bytes(int m, int k) {
  if (m <= 0 || k <= 0) return 0;
  return (size_t)tiles_k8(k) * m_alloc_for(m) * 128;
}

int b200_untile_rows(const int8_t* d_q_tiled, int m, int k, int8_t* d_q_rowmajor, void* stream) {
  if (!d_q_tiled || !d_q_rowmajor || m <= 0 || k <= 0) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_untile_rows: bad argument");
  untile_rows_kernel<<<m, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_q_tiled, m, k, m_alloc_for(m), d_q_rowmajor);
  return gcuda(cudaGetLastError(), "b200_untile_rows");
}

int b200_transpose_matrices(const void* d_in, void* d_out, int batches, int rows, int cols, int elem_bytes, void* stream) {
  if (!d_in || !d_out || batches <= 0 || rows <= 0 || cols <= 0 || batches > 65535)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_transpose_matrices: bad argument");
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32, batches), block(32, 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (elem_bytes == 1) {
    transpose_matrices_kernel<int8_t><<<grid, block, 0, s>>>(static_cast<const int8_t*>(d_in), static_cast<int8_t*>(d_out), rows, cols);
  } else if (elem_bytes == 4) {
    transpose_matrices_kernel<float><<<grid, block, 0, s>>>(static_cast<const float*>(d_in), static_cast<float*>(d_out), rows, cols);
  } else {
    return gfail(B200_ERR_UNSUPPORTED, "b200_transpose_matrices: element size %d", elem_bytes);
  }
  return gcuda(cudaGetLastError(), "b200_transpose_matrices");
}

int b200_embedding_lookup(const int32_t* d_ids, int rows, const int8_t* d_table, const float* d_row_scales, int vocab,
                          int d, float out_scale, float* d_out, void* stream) {
  if (!d_ids || !d_table || !d_row_scales || !d_out || rows <= 0 || d <= 0 || vocab <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_embedding_lookup: bad argument");
  return gcuda(launch_embed(d_ids, d_table, d_row_scales, rows, vocab, d, out_scale, d_out, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream)),
               "b200_embedding_lookup");
}

int b200_add_rmsnorm_quantize(float* d_h, const float* d_delta, const float* d_gain, int rows, int d, float eps,
                              int8_t* d_q_tiled, float* d_scales, int32_t* d_zero_points, void* stream) {
  if (!d_h || !d_gain || !d_q_tiled || !d_scales || !d_zero_points || rows <= 0 || d <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_add_rmsnorm_quantize: bad argument");
  if (sizeof(float) * (size_t)d > 48 * 1024) return gfail(B200_ERR_UNSUPPORTED, "b200_add_rmsnorm_quantize: rows wider than 12288 elements");
  return gcuda(launch_add_norm_quant(d_h, d_delta, d_gain, rows, d, eps, m_alloc_for(rows), d_q_tiled, d_scales, d_zero_points,
                                     nullptr, static_cast<cudaStream_t>(stream)),
               "b200_add_rmsnorm_quantize");
}

int b200_geglu_quantize(const float* d_gate_up, int rows, int f, int8_t* d_q_tiled, float* d_scales,
                        int32_t* d_zero_points, void* stream) {
  if (!d_gate_up || !d_q_tiled || !d_scales || !d_zero_points || rows <= 0 || f <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_geglu_quantize: bad argument");
  return gcuda(launch_geglu_quant(d_gate_up, rows, f, m_alloc_for(rows), d_q_tiled, d_scales, d_zero_points,
                                  static_cast<cudaStream_t>(stream)),
               "b200_geglu_quantize");
}

int b200_rope_table(float* h_cos_sin, int positions, int head_dim, float base) {
  if (!h_cos_sin || positions <= 0 || head_dim <= 0 || head_dim % 2) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_rope_table: bad argument");
  fill_rope_table(h_cos_sin, positions, head_dim, base);
  return B200_OK;
}

int b200_rope_kv_append(const float* d_qkv, int rows, int heads, int kv_heads, int head_dim, const float* d_cos_sin,
                        const int32_t* d_positions, int max_seq, float* d_q_out, void* d_k_cache, void* d_v_cache,
                        float* d_k_scale, float* d_v_scale, int kv_dtype, int one_sequence, void* stream) {
  if (!d_qkv || !d_cos_sin || !d_positions || !d_q_out || !d_k_cache || !d_v_cache || rows <= 0 || heads <= 0 || kv_heads <= 0 ||
      max_seq <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_rope_kv_append: bad argument");
  if (head_dim <= 0 || head_dim % 2 || head_dim / 2 > 1024) return gfail(B200_ERR_UNSUPPORTED, "b200_rope_kv_append: head size %d", head_dim);
  if (kv_dtype != B200_DTYPE_F16 && kv_dtype != B200_DTYPE_I8) return gfail(B200_ERR_UNSUPPORTED, "b200_rope_kv_append: cache dtype %d", kv_dtype);
  if (kv_dtype == B200_DTYPE_I8 && (!d_k_scale || !d_v_scale)) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_rope_kv_append: int8 cache needs scales");
  return gcuda(launch_rope_cache(d_qkv, rows, heads, kv_heads, head_dim, reinterpret_cast<const float2*>(d_cos_sin), d_positions,
                                 max_seq, d_q_out, d_k_cache, d_v_cache, d_k_scale, d_v_scale, kv_dtype == B200_DTYPE_I8 ? 1 : 0,
                                 one_sequence ? 1 : 0, static_cast<cudaStream_t>(stream)),
               "b200_rope_kv_append");
}

size_t b200_argmax_workspace_bytes(int rows) { return rows > 0 ? (size_t)rows * kArgmaxParts * 8 : 0; }

int b200_argmax_rows(const float* d_logits, int rows, int n, float soft_cap, int32_t* d_out, void* d_workspace,
                     size_t workspace_bytes, void* stream) {
  if (!d_logits || !d_out || !d_workspace || rows <= 0 || n <= 0) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_argmax_rows: bad argument");
  if (workspace_bytes < b200_argmax_workspace_bytes(rows)) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_argmax_rows: workspace too small");
  float* part_val = static_cast<float*>(d_workspace);
  int32_t* part_idx = reinterpret_cast<int32_t*>(part_val + (size_t)rows * kArgmaxParts);
  return gcuda(launch_argmax(d_logits, rows, n, 0, soft_cap, part_val, part_idx, d_out, nullptr, 0, nullptr,
                             static_cast<cudaStream_t>(stream)),
               "b200_argmax_rows");
}

int b200_attention_step_supported(int heads, int kv_heads, int head_dim, int kv_dtype) {
  return attn_step_supported(heads, kv_heads, head_dim, kv_dtype == B200_DTYPE_I8 ? 1 : 0) ? 1 : 0;
}

int b200_attention_step(const float* d_qkv, const int32_t* d_positions, const float* d_cos_sin, void* d_k_cache,
                        void* d_v_cache, float* d_k_scale, float* d_v_scale, int batch, int heads, int head_dim,
                        int max_seq, int kv_dtype, float scale, int8_t* d_q_tiled, float* d_scales,
                        int32_t* d_zero_points, void* stream) {
  if (!d_qkv || !d_positions || !d_cos_sin || !d_k_cache || !d_v_cache || !d_q_tiled || !d_scales || !d_zero_points || batch <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_attention_step: bad argument");
  if (kv_dtype != B200_DTYPE_F16 && kv_dtype != B200_DTYPE_I8) return gfail(B200_ERR_UNSUPPORTED, "b200_attention_step: cache dtype %d", kv_dtype);
  if (kv_dtype == B200_DTYPE_I8 && (!d_k_scale || !d_v_scale)) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_attention_step: int8 cache needs scales");
  if (!attn_step_supported(heads, 1, head_dim, kv_dtype == B200_DTYPE_I8 ? 1 : 0))
    return gfail(B200_ERR_UNSUPPORTED, "b200_attention_step: at most 8 query heads on one KV head, head size 64, 128 or 256");
  AttnStepParams ap;
  memset(&ap, 0, sizeof(ap));
  ap.qkv = d_qkv;
  ap.positions = d_positions;
  ap.k_cache = d_k_cache;
  ap.v_cache = d_v_cache;
  ap.k_scale = d_k_scale;
  ap.v_scale = d_v_scale;
  ap.b = batch;
  ap.n = heads;
  ap.h = head_dim;
  ap.s_max = max_seq;
  ap.kv_dtype = kv_dtype == B200_DTYPE_I8 ? 1 : 0;
  ap.rope_cs = reinterpret_cast<const float2*>(d_cos_sin);
  ap.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)head_dim);
  ap.q_tiled_out = d_q_tiled;
  ap.out_scales = d_scales;
  ap.out_zps = d_zero_points;
  ap.m_alloc = m_alloc_for(batch);
  return gcuda(launch_attn_step(ap, static_cast<cudaStream_t>(stream)), "b200_attention_step");
}

int b200_sdpa_decode_quantized_masked(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                                      const float* d_v_scale, const int32_t* d_lengths, const float* d_mask, int b, int n,
                                      int nkv, int h, int s_max, int q_dtype, int kv_dtype, float scale, float logit_cap,
                                      int8_t* d_q_tiled, float* d_scales, int32_t* d_zero_points, void* d_workspace,
                                      size_t workspace_bytes, void* stream) {
  const char* name = "b200_sdpa_decode_quantized";
  if (!d_q || !d_k || !d_v || !d_q_tiled || !d_scales || !d_zero_points || b <= 0 || n <= 0 || nkv <= 0 || n % nkv || h <= 0 || s_max <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "%s: bad argument", name);
  if (q_dtype != B200_DTYPE_F16 && q_dtype != B200_DTYPE_F32) return gfail(B200_ERR_UNSUPPORTED, "%s: q dtype %d", name, q_dtype);
  if (kv_dtype != B200_DTYPE_F16 && kv_dtype != B200_DTYPE_I8 && kv_dtype != B200_DTYPE_F32)
    return gfail(B200_ERR_UNSUPPORTED, "%s: kv dtype %d", name, kv_dtype);
  if (kv_dtype == B200_DTYPE_I8 && (!d_k_scale || !d_v_scale)) return gfail(B200_ERR_INVALID_ARGUMENT, "%s: int8 cache needs scales", name);
  if (n / nkv > 8 || (h != 64 && h != 128 && h != 256))
    return gfail(B200_ERR_UNSUPPORTED, "%s: at most 8 query heads per KV head, head size 64, 128 or 256", name);
  if (n > 64) return gfail(B200_ERR_UNSUPPORTED, "%s: at most 64 query heads", name);
  if (!d_workspace || workspace_bytes < sdpa_workspace_bytes(b, n, nkv, h, s_max))
    return gfail(B200_ERR_INVALID_ARGUMENT, "%s: workspace too small (b200_sdpa_workspace_bytes)", name);
  SdpaParams p;
  memset(&p, 0, sizeof(p));
  p.q = d_q; p.k = d_k; p.v = d_v; p.k_scale = d_k_scale; p.v_scale = d_v_scale;
  p.lengths = d_lengths;
  p.mask = d_mask;
  p.b = b; p.n = n; p.nkv = nkv; p.h = h; p.s_max = s_max;
  p.q_dtype = q_dtype == B200_DTYPE_F32 ? 1 : 0;
  p.kv_dtype = kv_dtype;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)h);
  p.logit_cap = logit_cap;
  p.q_tiled_out = d_q_tiled;
  p.out_scales = d_scales;
  p.out_zps = d_zero_points;
  p.m_alloc = m_alloc_for(b);
  p.ws = static_cast<float*>(d_workspace);
  p.ws_bytes = workspace_bytes;
  return gcuda(launch_sdpa_decode(p, static_cast<cudaStream_t>(stream)), name);
}

int b200_sdpa_decode_quantized(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                               const float* d_v_scale, const int32_t* d_lengths, int b, int n, int nkv, int h, int s_max,
                               int q_dtype, int kv_dtype, float scale, int8_t* d_q_tiled, float* d_scales,
                               int32_t* d_zero_points, void* d_workspace, size_t workspace_bytes, void* stream) {
  return b200_sdpa_decode_quantized_masked(d_q, d_k, d_v, d_k_scale, d_v_scale, d_lengths, nullptr, b, n, nkv, h, s_max,
                                           q_dtype, kv_dtype, scale, 0.0f, d_q_tiled, d_scales, d_zero_points, d_workspace,
                                           workspace_bytes, stream);
}

int b200_fc_hybrid_quantized(const int8_t* d_q_tiled, const float* d_scales, const int32_t* d_zero_points, int m, int k,
                             const void* d_w_packed, int n, const int32_t* d_row_sums, const float* d_w_scales,
                             int per_channel, const float* d_bias, int activation, float* d_y, void* d_zero_ws,
                             void* stream) {
  if (!d_q_tiled || !d_scales || !d_w_packed || !d_row_sums || !d_w_scales || !d_y || !d_zero_ws || m <= 0 || n <= 0 || k <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_fc_hybrid_quantized: bad argument");
  if (activation < B200_ACT_NONE || activation > B200_ACT_SIGMOID) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_fc_hybrid_quantized: bad activation %d", activation);
  if (reinterpret_cast<uintptr_t>(d_w_packed) % 128 || reinterpret_cast<uintptr_t>(d_q_tiled) % 128 ||
      reinterpret_cast<uintptr_t>(d_zero_ws) % 256)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_fc_hybrid_quantized: packed weights and tiled rows need 128-byte, the workspace 256-byte alignment");
  FcParams p;
  memset(&p, 0, sizeof(p));
  p.w_packed = static_cast<const uint8_t*>(d_w_packed);
  p.q_tiled = d_q_tiled;
  p.m = m; p.n = n; p.k = k;
  p.n_tiles = tiles_n(n); p.k_tiles = tiles_k8(k); p.m_alloc = m_alloc_for(m);
  p.in_scales = d_scales;
  p.in_zps = d_zero_points;
  p.w_scales = d_w_scales; p.per_channel = per_channel;
  p.bias_f32 = d_bias;
  p.row_sums = d_row_sums;
  p.activation = activation;
  p.y = d_y;
  fill_fc_ws(p, d_zero_ws);
  return gcuda(launch_fc_i8_umma(p, kEpiHybridF32, static_cast<cudaStream_t>(stream)), "b200_fc_hybrid_quantized");
}

size_t b200_lm_head_workspace_bytes(int m) { return m > 0 ? (size_t)m * kArgmaxSlots * 8 : 0; }

int b200_lm_head_greedy(const int8_t* d_q_tiled, const float* d_scales, const int32_t* d_zero_points, int m, int k,
                        const void* d_w_packed, int n, const int32_t* d_row_sums, const float* d_w_scales, float soft_cap,
                        float* d_logits, int32_t* d_tokens, void* d_workspace, size_t workspace_bytes, void* d_zero_ws,
                        void* stream) {
  if (!d_q_tiled || !d_scales || !d_w_packed || !d_row_sums || !d_w_scales || !d_tokens || !d_workspace || !d_zero_ws ||
      m <= 0 || n <= 0 || k <= 0)
    return gfail(B200_ERR_INVALID_ARGUMENT, "b200_lm_head_greedy: bad argument");
  if (m > 16) return gfail(B200_ERR_UNSUPPORTED, "b200_lm_head_greedy: at most 16 rows (use b200_fc_hybrid_quantized + b200_argmax_rows)");
  if (workspace_bytes < b200_lm_head_workspace_bytes(m)) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_lm_head_greedy: workspace too small");
  if (!(soft_cap >= 0.0f)) return gfail(B200_ERR_INVALID_ARGUMENT, "b200_lm_head_greedy: soft cap must be >= 0");
  const int parts = fc_argmax_ctas(n);
  if (parts > kArgmaxSlots) return gfail(B200_ERR_UNSUPPORTED, "b200_lm_head_greedy: device with more CTAs than candidate slots");
  float* part_val = static_cast<float*>(d_workspace);
  int32_t* part_idx = reinterpret_cast<int32_t*>(part_val + (size_t)m * kArgmaxSlots);
  FcParams p;
  memset(&p, 0, sizeof(p));
  p.w_packed = static_cast<const uint8_t*>(d_w_packed);
  p.q_tiled = d_q_tiled;
  p.m = m; p.n = n; p.k = k;
  p.n_tiles = tiles_n(n); p.k_tiles = tiles_k8(k); p.m_alloc = m_alloc_for(m);
  p.in_scales = d_scales;
  p.in_zps = d_zero_points;
  p.w_scales = d_w_scales; p.per_channel = 1;
  p.row_sums = d_row_sums;
  p.y = d_logits;
  p.argmax_val = part_val;
  p.argmax_idx = part_idx;
  p.argmax_parts = parts;
  p.soft_cap = soft_cap;
  fill_fc_ws(p, d_zero_ws);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = launch_fc_i8_umma(p, kEpiHybridPick, s);
  if (e != cudaSuccess) return gcuda(e, "b200_lm_head_greedy (projection)");
  return gcuda(launch_argmax_final(part_val, part_idx, m, parts, 0, d_tokens, nullptr, 0, nullptr, s), "b200_lm_head_greedy (pick)");
}

}  // extern "C"
