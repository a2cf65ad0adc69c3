// C-ABI entry points: argument checks, scratch carving, kernel launches.
// Nothing here allocates device memory or synchronises, except where the
// header says so.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/litert_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline size_t zero_ws_counter_off() { return b200::zero_ws_counter_off(); }
inline size_t zero_ws_bytes() { return b200::zero_ws_total_bytes(); }

struct Scratch {
  float* scales;
  int32_t* zps;
  int32_t* x_sums;
  int8_t* q_tiled;
  size_t bytes;
};

// k_tiles8: number of 128-wide activation tiles (twice the 4-bit tile count).
Scratch carve_scratch(void* base, int m, int k_tiles8) {
  const int m_alloc = b200::m_alloc_for(m);
  Scratch s;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  s.scales = reinterpret_cast<float*>(p + off);
  off += align_up(sizeof(float) * m_alloc, 256);
  s.zps = reinterpret_cast<int32_t*>(p + off);
  off += align_up(sizeof(int32_t) * m_alloc, 256);
  s.x_sums = reinterpret_cast<int32_t*>(p + off);
  off += align_up(sizeof(int32_t) * m_alloc, 256);
  s.q_tiled = reinterpret_cast<int8_t*>(p + off);
  off += (size_t)k_tiles8 * m_alloc * 128;
  s.bytes = off;
  return s;
}

cudaError_t run_fc_i8(const b200::FcParams& p, b200::FcEpilogue epi, cudaStream_t s) {
  return b200::launch_fc_i8_umma(p, epi, s);
}

void fill_ws(b200::FcParams& p, void* d_zero_ws) {
  uint8_t* z = static_cast<uint8_t*>(d_zero_ws);
  p.status = reinterpret_cast<int*>(z);
  p.ws_count = reinterpret_cast<int32_t*>(z + zero_ws_counter_off());
  p.ws_part = reinterpret_cast<int32_t*>(z + b200::zero_ws_part_off());
}

}  // namespace

extern "C" {

int b200_abi_version(void) { return 1; }
const char* b200_last_error(void) { return g_error; }

size_t b200_zero_workspace_bytes(void) { return zero_ws_bytes(); }

int b200_zero_workspace_init(void* d_zero_ws, void* stream) {
  if (!d_zero_ws) return fail(B200_ERR_INVALID_ARGUMENT, "zero workspace is null");
  cudaError_t e = cudaMemsetAsync(d_zero_ws, 0, zero_ws_bytes(), static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_zero_workspace_init");
}

int b200_set_wait_budget(void* d_zero_ws, unsigned long long nanoseconds, void* stream) {
  if (!d_zero_ws) return fail(B200_ERR_INVALID_ARGUMENT, "zero workspace is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t*>(d_zero_ws) + 4 * b200::kStatusBudgetWordOffsetInts, &nanoseconds,
                                  sizeof(nanoseconds), cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);  // the source is a stack variable
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_set_wait_budget");
}

int b200_clear_status(void* d_zero_ws, void* stream) {
  if (!d_zero_ws) return fail(B200_ERR_INVALID_ARGUMENT, "zero workspace is null");
  // the status word, and whatever an aborted launch left in the split-K counters and the accumulator
  // slots that must be zero between calls; the wait budget (bytes 8..15) is kept
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* z = static_cast<uint8_t*>(d_zero_ws);
  cudaError_t e = cudaMemsetAsync(z, 0, 8, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(z + 16, 0, b200::zero_ws_part_off() - 16, s);
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_clear_status");
}

size_t b200_fc_scratch_bytes(int m, int k) {
  if (m <= 0 || k <= 0) return 0;
  // sized for either weight format: the 4-bit path keeps the quantized rows as fp16, in tiles 256 wide
  return carve_scratch(nullptr, m, 4 * b200::tiles_k4(k)).bytes;
}

int b200_read_status(void* d_zero_ws, void* stream, int* status_out) {
  if (!d_zero_ws || !status_out) return fail(B200_ERR_INVALID_ARGUMENT, "null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status_out, d_zero_ws, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail(e, "b200_read_status");
  if (*status_out == 201)
    return fail(B200_ERR_INVALID_ARGUMENT, "a key/value cache update ran past the cache's last slot (status 201)");
  if (*status_out != 0) return fail(B200_ERR_KERNEL_TIMEOUT, "device-side wait ran out (status %d)", *status_out);
  return B200_OK;
}

size_t b200_packed_w8_bytes(int n, int k) {
  if (n <= 0 || k <= 0) return 0;
  return (size_t)b200::tiles_n(n) * b200::tiles_k8(k) * b200::kTileBytes;
}

int b200_pack_w8(const int8_t* d_w, int n, int k, void* d_packed, int32_t* d_row_sums, void* stream) {
  if (!d_w || !d_packed || n <= 0 || k <= 0) return fail(B200_ERR_INVALID_ARGUMENT, "b200_pack_w8: bad argument");
  if (reinterpret_cast<uintptr_t>(d_packed) % 128) return fail(B200_ERR_INVALID_ARGUMENT, "packed buffer must be 128-byte aligned");
  cudaError_t e = b200::launch_pack_w8(d_w, n, k, static_cast<uint8_t*>(d_packed), d_row_sums,
                                       static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_pack_w8");
}

size_t b200_packed_w4_bytes(int n, int k) {
  if (n <= 0 || k <= 0) return 0;
  return (size_t)b200::tiles_n(n) * b200::tiles_k4(k) * b200::kTile4Bytes;
}

int b200_pack_w4(const uint8_t* d_w4, const uint16_t* d_scales_f16, int n, int k, int blocksize, void* d_packed,
                 float* d_kfsum, void* stream) {
  if (!d_w4 || !d_scales_f16 || !d_packed || !d_kfsum || n <= 0 || k <= 0)
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_pack_w4: bad argument");
  if (blocksize <= 0 || blocksize % 32 != 0 || k % blocksize != 0)
    return fail(B200_ERR_UNSUPPORTED, "b200_pack_w4: blocksize %d must be a multiple of 32 dividing k=%d", blocksize, k);
  if (reinterpret_cast<uintptr_t>(d_packed) % 128) return fail(B200_ERR_INVALID_ARGUMENT, "packed buffer must be 128-byte aligned");
  cudaError_t e = b200::launch_pack_w4(d_w4, d_scales_f16, n, k, blocksize, static_cast<uint8_t*>(d_packed), d_kfsum,
                                       static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_pack_w4");
}

int b200_quantize_rows(const float* d_x, int m, int k, int asymmetric, int8_t* d_q, float* d_scales,
                       int32_t* d_zero_points, void* stream) {
  if (!d_x || !d_q || !d_scales || m < 0 || k <= 0) return fail(B200_ERR_INVALID_ARGUMENT, "b200_quantize_rows: bad argument");
  if (asymmetric && !d_zero_points) return fail(B200_ERR_INVALID_ARGUMENT, "asymmetric quantization needs zero points");
  const int k_pad = (k + 15) / 16 * 16;
  cudaError_t e = b200::launch_quantize_rows(d_x, m, k, k_pad, 8, asymmetric, nullptr, d_q, d_scales, d_zero_points,
                                             static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_quantize_rows");
}

static int check_fc_common(const char* name, const void* d_x, int m, int k, const void* d_w, int n, const void* d_y,
                           const void* d_zero_ws, const void* d_scratch, size_t scratch_bytes) {
  if (!d_x || !d_w || !d_y || !d_zero_ws || !d_scratch) return fail(B200_ERR_INVALID_ARGUMENT, "%s: null pointer", name);
  if (m < 0 || n <= 0 || k <= 0) return fail(B200_ERR_INVALID_ARGUMENT, "%s: bad shape m=%d n=%d k=%d", name, m, n, k);
  if (scratch_bytes < b200_fc_scratch_bytes(m, k))
    return fail(B200_ERR_INVALID_ARGUMENT, "%s: scratch too small (%zu < %zu)", name, scratch_bytes, b200_fc_scratch_bytes(m, k));
  if (reinterpret_cast<uintptr_t>(d_w) % 128 || reinterpret_cast<uintptr_t>(d_scratch) % 256 ||
      reinterpret_cast<uintptr_t>(d_zero_ws) % 256)
    return fail(B200_ERR_INVALID_ARGUMENT, "%s: packed weights need 128-byte, workspaces 256-byte alignment", name);
  return B200_OK;
}

int b200_fc_int8(const int8_t* d_x, int m, int k, const void* d_w_packed, int n, const int32_t* d_row_sums,
                 const int32_t* d_bias, int32_t input_offset, int32_t filter_offset, int32_t output_offset,
                 const int32_t* d_multipliers, const int32_t* d_shifts, int per_channel, int32_t act_min,
                 int32_t act_max, int8_t* d_y, void* d_zero_ws, void* d_scratch, size_t scratch_bytes, void* stream) {
  int rc = check_fc_common("b200_fc_int8", d_x, m, k, d_w_packed, n, d_y, d_zero_ws, d_scratch, scratch_bytes);
  if (rc) return rc;
  if (!d_multipliers || !d_shifts) return fail(B200_ERR_INVALID_ARGUMENT, "b200_fc_int8: multipliers/shifts are null");
  if (input_offset != 0 && !d_row_sums) return fail(B200_ERR_INVALID_ARGUMENT, "b200_fc_int8: row sums needed with an input offset");
  if (per_channel && filter_offset != 0) return fail(B200_ERR_UNSUPPORTED, "b200_fc_int8: per-channel weights are symmetric");
  if (m == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k_tiles = b200::tiles_k8(k);
  Scratch sc = carve_scratch(d_scratch, m, k_tiles);
  const int m_alloc = b200::m_alloc_for(m);
  cudaError_t e = b200::launch_retile_x8(d_x, m, k, k_tiles * 128, m_alloc, sc.q_tiled,
                                         filter_offset != 0 ? sc.x_sums : nullptr, s);
  if (e != cudaSuccess) return cuda_fail(e, "b200_fc_int8 (retile)");
  b200::FcParams p;
  memset(&p, 0, sizeof(p));
  p.w_packed = static_cast<const uint8_t*>(d_w_packed);
  p.q_tiled = sc.q_tiled;
  p.m = m; p.n = n; p.k = k;
  p.n_tiles = b200::tiles_n(n); p.k_tiles = k_tiles; p.m_alloc = m_alloc;
  p.per_channel = per_channel;
  p.row_sums = d_row_sums;
  p.bias_i32 = d_bias;
  p.multipliers = d_multipliers; p.shifts = d_shifts;
  p.x_sums = filter_offset != 0 ? sc.x_sums : nullptr;
  p.input_offset = input_offset; p.filter_offset = filter_offset; p.output_offset = output_offset;
  p.act_min = act_min; p.act_max = act_max;
  p.y = d_y;
  fill_ws(p, d_zero_ws);
  e = run_fc_i8(p, b200::kEpiRequantI8, s);
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_fc_int8");
}

static int fc_hybrid_impl(const char* name, const float* d_x, int m, int k, const void* d_w_packed, int n,
                          const int32_t* d_row_sums, const float* d_w_scales, int per_channel, const float* d_bias,
                          int asymmetric_inputs, int activation, int float_offset, float* d_y, void* d_zero_ws,
                          void* d_scratch, size_t scratch_bytes, void* stream) {
  int rc = check_fc_common(name, d_x, m, k, d_w_packed, n, d_y, d_zero_ws, d_scratch, scratch_bytes);
  if (rc) return rc;
  if (!d_w_scales) return fail(B200_ERR_INVALID_ARGUMENT, "%s: weight scales are null", name);
  if ((asymmetric_inputs || float_offset) && !d_row_sums) return fail(B200_ERR_INVALID_ARGUMENT, "%s: row sums needed", name);
  if (activation < B200_ACT_NONE || activation > B200_ACT_SIGMOID) return fail(B200_ERR_INVALID_ARGUMENT, "%s: bad activation %d", name, activation);
  if (m == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k_tiles = b200::tiles_k8(k);
  Scratch sc = carve_scratch(d_scratch, m, k_tiles);
  const int m_alloc = b200::m_alloc_for(m);
  cudaError_t e = b200::launch_quantize_rows(d_x, m, k, k_tiles * 128, m_alloc, asymmetric_inputs, sc.q_tiled, nullptr,
                                             sc.scales, sc.zps, s);
  if (e != cudaSuccess) return cuda_fail(e, name);
  b200::FcParams p;
  memset(&p, 0, sizeof(p));
  p.w_packed = static_cast<const uint8_t*>(d_w_packed);
  p.q_tiled = sc.q_tiled;
  p.m = m; p.n = n; p.k = k;
  p.n_tiles = b200::tiles_n(n); p.k_tiles = k_tiles; p.m_alloc = m_alloc;
  p.in_scales = sc.scales;
  p.in_zps = asymmetric_inputs ? sc.zps : nullptr;
  p.w_scales = d_w_scales; p.per_channel = per_channel;
  p.bias_f32 = d_bias;
  p.row_sums = d_row_sums;
  p.activation = activation;
  p.float_offset = float_offset;
  p.y = d_y;
  fill_ws(p, d_zero_ws);
  e = run_fc_i8(p, b200::kEpiHybridF32, s);
  return e == cudaSuccess ? B200_OK : cuda_fail(e, name);
}

int b200_fc_hybrid(const float* d_x, int m, int k, const void* d_w_packed, int n, const int32_t* d_row_sums,
                   const float* d_w_scales, int per_channel, const float* d_bias, int asymmetric_inputs,
                   int activation, float* d_y, void* d_zero_ws, void* d_scratch, size_t scratch_bytes, void* stream) {
  return fc_hybrid_impl("b200_fc_hybrid", d_x, m, k, d_w_packed, n, d_row_sums, d_w_scales, per_channel, d_bias,
                        asymmetric_inputs, activation, 0, d_y, d_zero_ws, d_scratch, scratch_bytes, stream);
}

int b200_bmm_hybrid(const float* d_x, int m, int k, const void* d_w_packed, int n, const int32_t* d_row_sums,
                    const float* d_w_scales, int per_channel, int asymmetric_inputs, float* d_y, void* d_zero_ws,
                    void* d_scratch, size_t scratch_bytes, void* stream) {
  return fc_hybrid_impl("b200_bmm_hybrid", d_x, m, k, d_w_packed, n, d_row_sums, d_w_scales, per_channel, nullptr,
                        asymmetric_inputs, B200_ACT_NONE, 1, d_y, d_zero_ws, d_scratch, scratch_bytes, stream);
}

int b200_fc_w4(const float* d_x, int m, int k, const void* d_w4_packed, int n, int blocksize, const float* d_kfsum,
               const float* d_bias, float* d_y, void* d_zero_ws, void* d_scratch, size_t scratch_bytes, void* stream) {
  int rc = check_fc_common("b200_fc_w4", d_x, m, k, d_w4_packed, n, d_y, d_zero_ws, d_scratch, scratch_bytes);
  if (rc) return rc;
  if (!d_kfsum) return fail(B200_ERR_INVALID_ARGUMENT, "b200_fc_w4: kfsum is null");
  if (blocksize <= 0 || blocksize % 32 != 0 || k % blocksize != 0)
    return fail(B200_ERR_UNSUPPORTED, "b200_fc_w4: blocksize %d must be a multiple of 32 dividing k=%d", blocksize, k);
  if (m == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k_tiles4 = b200::tiles_k4(k);
  b200::FcParams p;
  memset(&p, 0, sizeof(p));
  p.w_packed = static_cast<const uint8_t*>(d_w4_packed);
  p.m = m; p.n = n; p.k = k;
  p.n_tiles = b200::tiles_n(n); p.k_tiles = k_tiles4;
  p.kfsum = d_kfsum; p.bias_f32 = d_bias;
  p.y = d_y;
  fill_ws(p, d_zero_ws);
  if (b200::w4_gemv_supported(m, k)) {
    // decode-sized: one launch, rows quantized inside the kernel
    cudaError_t e = b200::launch_fc_w4_gemv(p, d_x, s);
    return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_fc_w4");
  }
  Scratch sc = carve_scratch(d_scratch, m, 4 * k_tiles4);  // fp16 rows: twice the bytes of the int8 ones
  const int m_alloc = b200::m_alloc_for(m);
  cudaError_t e = b200::launch_quantize_rows(d_x, m, k, k_tiles4 * 256, m_alloc, 1, nullptr, nullptr, sc.scales, sc.zps,
                                             s, sc.q_tiled);
  if (e != cudaSuccess) return cuda_fail(e, "b200_fc_w4 (quantize)");
  p.q_tiled = sc.q_tiled;
  p.m_alloc = m_alloc;
  p.in_scales = sc.scales; p.in_zps = sc.zps;
  e = b200::launch_fc_w4(p, s);
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_fc_w4");
}

// Shapes the split-K attention kernels take (the others run on the one-warp-per-head fallback,
// which needs no workspace but holds all logits of a head in shared memory).
static bool sdpa_fast_shape(int n, int nkv, int h) { return n % nkv == 0 && n / nkv <= 8 && (h == 64 || h == 128 || h == 256); }

size_t b200_sdpa_workspace_bytes(int b, int n, int nkv, int h, int s_max) {
  if (b <= 0 || n <= 0 || nkv <= 0 || h <= 0 || s_max <= 0) return 0;
  return b200::sdpa_workspace_bytes(b, n, nkv, h, s_max);
}

int b200_sdpa_decode(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale, const float* d_v_scale,
                     const int32_t* d_lengths, const float* d_mask, void* d_out, int b, int n, int nkv, int h,
                     int s_max, int q_dtype, int kv_dtype, float scale, float logit_cap, void* d_workspace,
                     size_t workspace_bytes, void* stream) {
  if (!d_q || !d_k || !d_v || !d_out) return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode: null pointer");
  if (b <= 0 || n <= 0 || nkv <= 0 || h <= 0 || s_max <= 0 || n % nkv != 0)
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode: bad shape b=%d n=%d nkv=%d h=%d s=%d", b, n, nkv, h, s_max);
  if (q_dtype != B200_DTYPE_F16 && q_dtype != B200_DTYPE_F32) return fail(B200_ERR_UNSUPPORTED, "b200_sdpa_decode: q dtype %d", q_dtype);
  if (kv_dtype < B200_DTYPE_F16 || kv_dtype > B200_DTYPE_F32) return fail(B200_ERR_UNSUPPORTED, "b200_sdpa_decode: kv dtype %d", kv_dtype);
  if (kv_dtype == B200_DTYPE_I8 && (!d_k_scale || !d_v_scale)) return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode: int8 cache needs scales");
  if (sdpa_fast_shape(n, nkv, h) && (!d_workspace || workspace_bytes < b200::sdpa_workspace_bytes(b, n, nkv, h, s_max)))
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode: workspace too small (%zu < %zu, see b200_sdpa_workspace_bytes)",
                workspace_bytes, b200::sdpa_workspace_bytes(b, n, nkv, h, s_max));
  if (!sdpa_fast_shape(n, nkv, h) && sizeof(float) * ((size_t)h + s_max) > 200 * 1024)
    return fail(B200_ERR_UNSUPPORTED, "b200_sdpa_decode: this head layout runs on the fallback kernel, which holds s_max logits in shared memory (s_max + h <= 51200)");
  b200::SdpaParams p;
  memset(&p, 0, sizeof(p));
  p.q = d_q; p.k = d_k; p.v = d_v; p.k_scale = d_k_scale; p.v_scale = d_v_scale;
  p.lengths = d_lengths; p.mask = d_mask; p.out = d_out;
  p.b = b; p.n = n; p.nkv = nkv; p.h = h; p.s_max = s_max;
  p.q_dtype = q_dtype == B200_DTYPE_F32 ? 1 : 0;
  p.kv_dtype = kv_dtype;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)h);
  p.logit_cap = logit_cap;
  p.ws = static_cast<float*>(d_workspace);
  p.ws_bytes = workspace_bytes;
  cudaError_t e = b200::launch_sdpa_decode(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_sdpa_decode");
}

int b200_sdpa(const void* d_q, const void* d_k, const void* d_v, const float* d_mask, void* d_out, int b, int t, int n,
              int nkv, int h, int s_max, int q_dtype, int kv_dtype, float scale, float logit_cap, void* d_workspace,
              size_t workspace_bytes, void* stream) {
  if (!d_q || !d_k || !d_v || !d_out) return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa: null pointer");
  if (b <= 0 || t <= 0 || n <= 0 || nkv <= 0 || h <= 0 || s_max <= 0 || n % nkv != 0 || (long long)b * t > (1 << 24))
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa: bad shape b=%d t=%d n=%d nkv=%d h=%d s=%d", b, t, n, nkv, h, s_max);
  if (q_dtype != B200_DTYPE_F16 && q_dtype != B200_DTYPE_F32) return fail(B200_ERR_UNSUPPORTED, "b200_sdpa: q dtype %d", q_dtype);
  if (kv_dtype != B200_DTYPE_F16 && kv_dtype != B200_DTYPE_F32) return fail(B200_ERR_UNSUPPORTED, "b200_sdpa: kv dtype %d", kv_dtype);
  if (sdpa_fast_shape(n, nkv, h) && (!d_workspace || workspace_bytes < b200::sdpa_workspace_bytes(b * t, n, nkv, h, s_max)))
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa: workspace too small (b200_sdpa_workspace_bytes(b * t, ...))");
  if (!sdpa_fast_shape(n, nkv, h) && sizeof(float) * ((size_t)h + s_max) > 200 * 1024)
    return fail(B200_ERR_UNSUPPORTED, "b200_sdpa: this head layout runs on the fallback kernel (s_max + h <= 51200)");
  b200::SdpaParams p;
  memset(&p, 0, sizeof(p));
  p.q = d_q; p.k = d_k; p.v = d_v;
  p.mask = d_mask; p.out = d_out;
  p.b = b * t; p.n = n; p.nkv = nkv; p.h = h; p.s_max = s_max;
  p.rows_per_kv = t;
  p.q_dtype = q_dtype == B200_DTYPE_F32 ? 1 : 0;
  p.kv_dtype = kv_dtype;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)h);
  p.logit_cap = logit_cap;
  p.ws = static_cast<float*>(d_workspace);
  p.ws_bytes = workspace_bytes;
  cudaError_t e = b200::launch_sdpa_decode(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_sdpa");
}

size_t b200_sdpa_rows_workspace_bytes(int rows, int n, int nkv, int h, int s_max) {
  if (rows <= 0 || n <= 0 || nkv <= 0 || h <= 0 || s_max <= 0) return 0;
  return b200::sdpa_workspace_bytes(rows, n, nkv, h, s_max, 1);
}

int b200_sdpa_rows(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale, const float* d_v_scale,
                   const int32_t* d_lengths, void* d_out, int rows, int n, int nkv, int h, int s_max, int q_dtype,
                   int kv_dtype, float scale, float logit_cap, void* d_workspace, size_t workspace_bytes, void* stream) {
  if (!d_q || !d_k || !d_v || !d_out || !d_lengths) return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_rows: null pointer");
  if (rows <= 0 || n <= 0 || nkv <= 0 || h <= 0 || s_max <= 0 || n % nkv != 0)
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_rows: bad shape rows=%d n=%d nkv=%d h=%d s=%d", rows, n, nkv, h, s_max);
  if (q_dtype != B200_DTYPE_F16 && q_dtype != B200_DTYPE_F32) return fail(B200_ERR_UNSUPPORTED, "b200_sdpa_rows: q dtype %d", q_dtype);
  if (kv_dtype < B200_DTYPE_F16 || kv_dtype > B200_DTYPE_F32) return fail(B200_ERR_UNSUPPORTED, "b200_sdpa_rows: kv dtype %d", kv_dtype);
  if (kv_dtype == B200_DTYPE_I8 && (!d_k_scale || !d_v_scale)) return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_rows: int8 cache needs scales");
  if (n / nkv > 8 || (h != 64 && h != 128 && h != 256))
    return fail(B200_ERR_UNSUPPORTED, "b200_sdpa_rows: at most 8 query heads per KV head, head size 64, 128 or 256");
  if (!d_workspace || workspace_bytes < b200::sdpa_workspace_bytes(rows, n, nkv, h, s_max, 1))
    return fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_rows: workspace too small (b200_sdpa_rows_workspace_bytes)");
  b200::SdpaParams p;
  memset(&p, 0, sizeof(p));
  p.q = d_q; p.k = d_k; p.v = d_v; p.k_scale = d_k_scale; p.v_scale = d_v_scale;
  p.lengths = d_lengths; p.out = d_out;
  p.b = rows; p.n = n; p.nkv = nkv; p.h = h; p.s_max = s_max;
  p.q_dtype = q_dtype == B200_DTYPE_F32 ? 1 : 0;
  p.kv_dtype = kv_dtype;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)h);
  p.logit_cap = logit_cap;
  p.ws = static_cast<float*>(d_workspace);
  p.ws_bytes = workspace_bytes;
  p.shared_kv = 1;
  cudaError_t e = b200::launch_sdpa_decode(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : cuda_fail(e, "b200_sdpa_rows");
}

}  // extern "C"
