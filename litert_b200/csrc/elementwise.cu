// The float32 builtins a decoder-only graph has around its projections and its attention, as the
// reference's converters author them (tensor/examples/gemma3/gemma3_graph.cc): ADD and MUL with
// broadcasting, GELU, SLICE, CONCATENATION, the odml.rms_norm composite, the odml.update_kv_cache custom
// op on a device-resident cache. None of them is a hot spot: each exists so that a whole decoder graph
// stays inside one delegate partition, with no host round trip between the projections. Plain
// element-per-thread kernels, HBM/L2-bound on a few kilobytes to megabytes.
#include <cstdarg>
#include <cstdio>

#include "../../include/litert_b200.h"
#include "common.cuh"
#include "quant.cuh"

namespace {

using namespace b200;

thread_local char g_ew_error[384] = "";
int efail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_ew_error, sizeof(g_ew_error), fmt, ap);
  va_end(ap);
  return code;
}
int ecuda(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return B200_OK;
  return efail(B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

struct Dims4 {
  int d[4];
};

// out[i0,i1,i2,i3] = a[...] op b[...] with NumPy broadcasting: an operand's dimension of extent 1 has stride 0
// (tflite/kernels/internal/reference/add.h / mul.h, BroadcastAdd4DSlow / BroadcastMul4DSlow).
template <int OP>
__global__ void binary_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, Dims4 od,
                                  Dims4 sa, Dims4 sb, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i;
    const int i3 = (int)(r % od.d[3]);
    r /= od.d[3];
    const int i2 = (int)(r % od.d[2]);
    r /= od.d[2];
    const int i1 = (int)(r % od.d[1]);
    const int i0 = (int)(r / od.d[1]);
    const float x = a[(size_t)i0 * sa.d[0] + (size_t)i1 * sa.d[1] + (size_t)i2 * sa.d[2] + (size_t)i3 * sa.d[3]];
    const float y = b[(size_t)i0 * sb.d[0] + (size_t)i1 * sb.d[1] + (size_t)i2 * sb.d[2] + (size_t)i3 * sb.d[3]];
    out[i] = OP == 0 ? __fadd_rn(x, y) : __fmul_rn(x, y);
  }
}

// GELU, tanh approximation (tflite/kernels/internal/reference/gelu.h:31-45:
// 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))), every product rounded on its own.
__global__ void gelu_f32_kernel(const float* __restrict__ x, float* __restrict__ y, size_t n, int approximate) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i];
    float r;
    if (approximate) {
      const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
      const float th = tanhf(__fmul_rn(0.7978845608028654f, __fadd_rn(v, cube)));
      r = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, th));
    } else {
      r = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, erff(__fmul_rn(v, 0.70710678118654752440f))));
    }
    y[i] = r;
  }
}

// Strided gather of a 4-D box: SLICE, and the pieces of CONCATENATION (dst has its own strides).
template <typename T>
__global__ void box_copy_kernel(const T* __restrict__ src, T* __restrict__ dst, Dims4 box, Dims4 ss, Dims4 ds, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i;
    const int i3 = (int)(r % box.d[3]);
    r /= box.d[3];
    const int i2 = (int)(r % box.d[2]);
    r /= box.d[2];
    const int i1 = (int)(r % box.d[1]);
    const int i0 = (int)(r / box.d[1]);
    dst[(size_t)i0 * ds.d[0] + (size_t)i1 * ds.d[1] + (size_t)i2 * ds.d[2] + (size_t)i3 * ds.d[3]] =
        src[(size_t)i0 * ss.d[0] + (size_t)i1 * ss.d[1] + (size_t)i2 * ss.d[2] + (size_t)i3 * ss.d[3]];
  }
}

// y = x * rsqrt(mean(x^2) + eps) * gain per row (odml.rms_norm: ml_drift_delegate/tflite/convert/convert_rms_norm.cc:40-61).
__global__ void __launch_bounds__(256) rms_norm_f32_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                                           float* __restrict__ y, int d, float eps) {
  __shared__ float red[32];
  const float* xr = x + (size_t)blockIdx.x * d;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_reduce(ss, [](float a, float c) { return a + c; }, 0.0f, red);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    y[(size_t)blockIdx.x * d + i] = gain ? __fmul_rn(__fmul_rn(xr[i], inv), gain[i]) : __fmul_rn(xr[i], inv);
}

// odml.update_kv_cache (tflite/experimental/genai/kvcache.cc:230-340) on device-resident float32 caches
// [max_entries, row]: the t new rows go to slots position .. position + t - 1. A write past the last slot
// (the reference then shifts the whole cache down) is not done here: it raises a status code instead.
__global__ void kv_cache_update_f32_kernel(const long long* __restrict__ position, const float* __restrict__ k,
                                           const float* __restrict__ v, int t, int row, int max_entries,
                                           float* __restrict__ k_cache, float* __restrict__ v_cache, int* status) {
  const long long pos = position[0];
  if (pos < 0 || pos + t > max_entries) {
    if (status && blockIdx.x == 0 && threadIdx.x == 0) atomicCAS(status, 0, 201);
    return;
  }
  const size_t total = (size_t)t * row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    k_cache[(size_t)pos * row + i] = k[i];
    v_cache[(size_t)pos * row + i] = v[i];
  }
}

// The rotary embedding as the graph spells it (tensor/examples/gemma3/gemma3_graph.cc:150-176):
// out = x * cos + concat(-x2, x1) * sin over the last dimension, cos / sin [tokens, h] shared by the heads.
// One kernel for the seven nodes, same roundings (every product and the sum on their own).
__global__ void rope_f32_kernel(const float* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                                float* __restrict__ out, int heads, int h, size_t total) {
  const int half = h / 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % h);
    const size_t token = i / ((size_t)heads * h);
    const float xv = x[i];
    const float rot = d < half ? __fmul_rn(x[i + half], -1.0f) : x[i - half];
    const float c = cs[token * h + d], s = sn[token * h + d];
    out[i] = __fadd_rn(__fmul_rn(xv, c), __fmul_rn(rot, s));
  }
}

// The rotary embedding of a step's query and key rows and odml.update_kv_cache as one launch: three kernels of a
// few kilobytes each in a row cost a decode step three kernel boundaries per layer. q_out = rope(q) (an ordinary
// tensor), rope(k) and v go straight to slots position .. position + t - 1 of the float32 caches; same roundings as
// rope_f32_kernel, same out-of-range rule as kv_cache_update_f32_kernel. Part of a chain of dependent launches:
// resident early, reads and writes only after the kernel before it has finished.
__global__ void __launch_bounds__(256) rope_kv_f32_kernel(const long long* __restrict__ position, const float* __restrict__ q,
                                                          const float* __restrict__ k, const float* __restrict__ v,
                                                          const float* __restrict__ cs, const float* __restrict__ sn,
                                                          float* __restrict__ q_out, float* __restrict__ k_cache,
                                                          float* __restrict__ v_cache, int t, int heads_q, int heads_kv, int h,
                                                          int max_entries, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const long long pos = position[0];
  const bool fits = pos >= 0 && pos + t <= max_entries;
  if (!fits && status && blockIdx.x == 0 && threadIdx.x == 0) atomicCAS(status, 0, 201);
  const int half = h / 2;
  const size_t row = (size_t)heads_kv * h;  // elements per cached token
  const size_t nq = (size_t)t * heads_q * h, nk = (size_t)t * row, total = nq + 2 * nk;
  auto rope = [&](const float* x, size_t i, int heads) {
    const int d = (int)(i % h);
    const size_t token = i / ((size_t)heads * h);
    const float rot = d < half ? __fmul_rn(x[i + half], -1.0f) : x[i - half];
    return __fadd_rn(__fmul_rn(x[i], cs[token * h + d]), __fmul_rn(rot, sn[token * h + d]));
  };
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    if (i < nq) {
      q_out[i] = rope(q, i, heads_q);
    } else if (i < nq + nk) {
      if (fits) k_cache[(size_t)pos * row + (i - nq)] = rope(k, i - nq, heads_kv);
    } else {
      if (fits) v_cache[(size_t)pos * row + (i - nq - nk)] = v[i - nq - nk];
    }
  }
}

__global__ void widen_i32_to_i64_kernel(const int32_t* __restrict__ in, long long* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[i];
}

int grid_for(size_t total) { return (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096); }

// Row-major strides of a 4-D shape, 0 where the operand broadcasts against `out`.
bool broadcast_strides(const int* dims, const int* out, Dims4* s) {
  size_t stride = 1;
  for (int i = 3; i >= 0; --i) {
    if (dims[i] != out[i] && dims[i] != 1) return false;
    s->d[i] = dims[i] == 1 ? 0 : (int)stride;
    stride *= (size_t)dims[i];
  }
  return true;
}

}  // namespace

extern "C" {

const char* b200_elementwise_last_error(void) { return g_ew_error; }

int b200_binary_f32(int op, const float* d_a, const int* a_dims4, const float* d_b, const int* b_dims4, float* d_out,
                    const int* out_dims4, void* stream) {
  if (!d_a || !d_b || !d_out || !a_dims4 || !b_dims4 || !out_dims4 || (op != 0 && op != 1))
    return efail(B200_ERR_INVALID_ARGUMENT, "b200_binary_f32: bad argument");
  Dims4 od, sa, sb;
  size_t total = 1;
  for (int i = 0; i < 4; ++i) {
    od.d[i] = out_dims4[i];
    if (od.d[i] <= 0) return efail(B200_ERR_INVALID_ARGUMENT, "b200_binary_f32: empty dimension");
    total *= (size_t)od.d[i];
  }
  if (!broadcast_strides(a_dims4, out_dims4, &sa) || !broadcast_strides(b_dims4, out_dims4, &sb))
    return efail(B200_ERR_INVALID_ARGUMENT, "b200_binary_f32: shapes do not broadcast");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (op == 0) {
    binary_f32_kernel<0><<<grid_for(total), 256, 0, s>>>(d_a, d_b, d_out, od, sa, sb, total);
  } else {
    binary_f32_kernel<1><<<grid_for(total), 256, 0, s>>>(d_a, d_b, d_out, od, sa, sb, total);
  }
  return ecuda("b200_binary_f32");
}

int b200_gelu_f32(const float* d_x, float* d_y, size_t n, int approximate, void* stream) {
  if (!d_x || !d_y || n == 0) return efail(B200_ERR_INVALID_ARGUMENT, "b200_gelu_f32: bad argument");
  gelu_f32_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_y, n, approximate);
  return ecuda("b200_gelu_f32");
}

int b200_box_copy(const void* d_src, const int* src_dims4, const int* src_begin4, void* d_dst, const int* dst_dims4,
                  const int* dst_begin4, const int* box4, int elem_bytes, void* stream) {
  if (!d_src || !d_dst || !src_dims4 || !src_begin4 || !dst_dims4 || !dst_begin4 || !box4)
    return efail(B200_ERR_INVALID_ARGUMENT, "b200_box_copy: bad argument");
  if (elem_bytes != 1 && elem_bytes != 4) return efail(B200_ERR_UNSUPPORTED, "b200_box_copy: element size %d", elem_bytes);
  Dims4 box, ss, ds;
  size_t total = 1, sstr = 1, dstr = 1, soff = 0, doff = 0;
  for (int i = 3; i >= 0; --i) {
    box.d[i] = box4[i];
    if (box4[i] <= 0 || src_begin4[i] < 0 || dst_begin4[i] < 0 || src_begin4[i] + box4[i] > src_dims4[i] ||
        dst_begin4[i] + box4[i] > dst_dims4[i])
      return efail(B200_ERR_INVALID_ARGUMENT, "b200_box_copy: box outside a tensor (dimension %d)", i);
    total *= (size_t)box4[i];
    ss.d[i] = (int)sstr;
    ds.d[i] = (int)dstr;
    soff += (size_t)src_begin4[i] * sstr;
    doff += (size_t)dst_begin4[i] * dstr;
    sstr *= (size_t)src_dims4[i];
    dstr *= (size_t)dst_dims4[i];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (elem_bytes == 4) {
    box_copy_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(d_src) + soff, static_cast<float*>(d_dst) + doff,
                                                           box, ss, ds, total);
  } else {
    box_copy_kernel<int8_t><<<grid_for(total), 256, 0, s>>>(static_cast<const int8_t*>(d_src) + soff,
                                                            static_cast<int8_t*>(d_dst) + doff, box, ss, ds, total);
  }
  return ecuda("b200_box_copy");
}

int b200_rms_norm_f32(const float* d_x, const float* d_gain, float* d_y, int rows, int d, float eps, void* stream) {
  if (!d_x || !d_y || rows <= 0 || d <= 0) return efail(B200_ERR_INVALID_ARGUMENT, "b200_rms_norm_f32: bad argument");
  rms_norm_f32_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_gain, d_y, d, eps);
  return ecuda("b200_rms_norm_f32");
}

int b200_kv_cache_update_f32(const int64_t* d_position, const float* d_k, const float* d_v, int t, int row_elems,
                             int max_entries, float* d_k_cache, float* d_v_cache, void* d_zero_ws, void* stream) {
  if (!d_position || !d_k || !d_v || !d_k_cache || !d_v_cache || t <= 0 || row_elems <= 0 || max_entries <= 0)
    return efail(B200_ERR_INVALID_ARGUMENT, "b200_kv_cache_update_f32: bad argument");
  kv_cache_update_f32_kernel<<<grid_for((size_t)t * row_elems), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(d_position), d_k, d_v, t, row_elems, max_entries, d_k_cache, d_v_cache,
      static_cast<int*>(d_zero_ws));
  return ecuda("b200_kv_cache_update_f32");
}

int b200_rope_f32(const float* d_x, const float* d_cos, const float* d_sin, float* d_out, int tokens, int heads, int h,
                  void* stream) {
  if (!d_x || !d_cos || !d_sin || !d_out || tokens <= 0 || heads <= 0 || h <= 0 || h % 2)
    return efail(B200_ERR_INVALID_ARGUMENT, "b200_rope_f32: bad argument");
  const size_t total = (size_t)tokens * heads * h;
  rope_f32_kernel<<<grid_for(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_cos, d_sin, d_out, heads, h, total);
  return ecuda("b200_rope_f32");
}

int b200_rope_kv_cache_update_f32(const int64_t* d_position, const float* d_q, const float* d_k, const float* d_v,
                                  const float* d_cos, const float* d_sin, float* d_q_out, int t, int heads_q, int heads_kv,
                                  int h, int max_entries, float* d_k_cache, float* d_v_cache, void* d_zero_ws, void* stream) {
  if (!d_position || !d_q || !d_k || !d_v || !d_cos || !d_sin || !d_q_out || !d_k_cache || !d_v_cache || t <= 0 ||
      heads_q <= 0 || heads_kv <= 0 || h <= 0 || h % 2 || max_entries <= 0)
    return efail(B200_ERR_INVALID_ARGUMENT, "b200_rope_kv_cache_update_f32: bad argument");
  const size_t total = (size_t)t * ((size_t)heads_q + 2 * (size_t)heads_kv) * h;
  const cudaError_t e = launch_chained(rope_kv_f32_kernel, dim3(grid_for(total)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                       reinterpret_cast<const long long*>(d_position), d_q, d_k, d_v, d_cos, d_sin, d_q_out,
                                       d_k_cache, d_v_cache, t, heads_q, heads_kv, h, max_entries, static_cast<int*>(d_zero_ws));
  if (e != cudaSuccess) return efail(B200_ERR_CUDA, "b200_rope_kv_cache_update_f32: %s", cudaGetErrorString(e));
  return ecuda("b200_rope_kv_cache_update_f32");
}

int b200_widen_i32_to_i64(const int32_t* d_in, int64_t* d_out, int n, void* stream) {
  if (!d_in || !d_out || n <= 0) return efail(B200_ERR_INVALID_ARGUMENT, "b200_widen_i32_to_i64: bad argument");
  widen_i32_to_i64_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_in, reinterpret_cast<long long*>(d_out), n);
  return ecuda("b200_widen_i32_to_i64");
}

}  // extern "C"
