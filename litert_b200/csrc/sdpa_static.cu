// b200_sdpa_decode_static: the attention decode step for callers that must not
// allocate device memory.
//
// Who that is: code running where cudaMalloc is off limits -- a real-time
// serving loop that has promised its host never to touch the allocator after
// start-up, a plugin loaded into a process whose memory budget is fixed by
// someone else, or a section of code that is being recorded for later replay,
// where an allocation would be an error. The regular entry point asks such a
// caller for a workspace it has no way to obtain; this one brings its own.
//
// The split-K partial results live in ONE file-scope device array of
// kStaticWorkspaceBytes (8 MiB). Every GPU whose context loads this library
// holds that array until the process exits. All calls on a device share it and
// nothing in it needs clearing between calls (each call writes every record it
// later reads), but two calls that overlap on the GPU -- different streams, or
// two host threads -- would overwrite each other's partials: serialise them.
//
// The array's name is only a host-side stand-in for the device object. The
// address a kernel can use is looked up with cudaGetSymbolAddress, once per
// device, with that device current, by the first call made on that device.
// That first call is therefore a set-up call: make it before any stream
// capture begins.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/litert_b200.h"
#include "kernels.h"

namespace {

constexpr size_t kStaticWorkspaceBytes = 8u << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_sdpa_static_workspace[kStaticWorkspaceBytes];

std::mutex g_mu;
void* g_device_address[kMaxDevices] = {nullptr};

thread_local char g_static_error[256] = "";

int static_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_static_error, sizeof(g_static_error), fmt, ap);
  va_end(ap);
  return code;
}

// Device address of the array on the current device (looked up on first use).
int workspace_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_fail(B200_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return static_fail(B200_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_device_address[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_sdpa_static_workspace);
    if (e != cudaSuccess || !ptr)
      return static_fail(B200_ERR_CUDA, "cudaGetSymbolAddress(static workspace): %s", cudaGetErrorString(e));
    g_device_address[dev] = ptr;
  }
  *out = g_device_address[dev];
  return B200_OK;
}

}  // namespace

extern "C" {

size_t b200_sdpa_static_workspace_limit(void) { return kStaticWorkspaceBytes; }

const char* b200_sdpa_static_last_error(void) { return g_static_error; }

int b200_sdpa_decode_static(const void* d_q, const void* d_k, const void* d_v, const float* d_k_scale,
                            const float* d_v_scale, const int32_t* d_lengths, const float* d_mask, void* d_out, int b,
                            int n, int nkv, int h, int s_max, int q_dtype, int kv_dtype, float scale, float logit_cap,
                            void* stream) {
  if (!d_q || !d_k || !d_v || !d_out) return static_fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode_static: null pointer");
  if (b <= 0 || n <= 0 || nkv <= 0 || h <= 0 || s_max <= 0 || n % nkv != 0)
    return static_fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode_static: bad shape b=%d n=%d nkv=%d h=%d s=%d", b, n,
                       nkv, h, s_max);
  if (q_dtype != B200_DTYPE_F16 && q_dtype != B200_DTYPE_F32)
    return static_fail(B200_ERR_UNSUPPORTED, "b200_sdpa_decode_static: q dtype %d", q_dtype);
  if (kv_dtype < B200_DTYPE_F16 || kv_dtype > B200_DTYPE_F32)
    return static_fail(B200_ERR_UNSUPPORTED, "b200_sdpa_decode_static: kv dtype %d", kv_dtype);
  if (kv_dtype == B200_DTYPE_I8 && (!d_k_scale || !d_v_scale))
    return static_fail(B200_ERR_INVALID_ARGUMENT, "b200_sdpa_decode_static: int8 cache needs scales");
  // only the split-K kernels use the workspace; other head layouts run on a kernel that needs none
  const bool uses_workspace = n / nkv <= 8 && (h == 64 || h == 128 || h == 256);
  const size_t need = uses_workspace ? b200::sdpa_workspace_bytes(b, n, nkv, h, s_max) : 0;
  if (need > kStaticWorkspaceBytes)
    return static_fail(B200_ERR_UNSUPPORTED,
                       "b200_sdpa_decode_static: this shape needs %zu bytes of workspace, the built-in one holds %zu "
                       "(use b200_sdpa_decode with a caller-owned workspace)",
                       need, kStaticWorkspaceBytes);
  // the array's address is that of the CURRENT device: a stream of another device would be handed
  // the wrong GPU's memory
  if (stream) {
    int cur = -1, sdev = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &sdev) == cudaSuccess &&
        sdev != cur)
      return static_fail(B200_ERR_INVALID_ARGUMENT,
                         "b200_sdpa_decode_static: the stream belongs to device %d but device %d is current", sdev, cur);
  }
  void* ws = nullptr;
  const int rc = workspace_for_current_device(&ws);
  if (rc != B200_OK) return rc;
  b200::SdpaParams p;
  memset(&p, 0, sizeof(p));
  p.q = d_q;
  p.k = d_k;
  p.v = d_v;
  p.k_scale = d_k_scale;
  p.v_scale = d_v_scale;
  p.lengths = d_lengths;
  p.mask = d_mask;
  p.out = d_out;
  p.b = b;
  p.n = n;
  p.nkv = nkv;
  p.h = h;
  p.s_max = s_max;
  p.q_dtype = q_dtype == B200_DTYPE_F32 ? 1 : 0;
  p.kv_dtype = kv_dtype;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)h);
  p.logit_cap = logit_cap;
  p.ws = static_cast<float*>(ws);
  p.ws_bytes = kStaticWorkspaceBytes;
  const cudaError_t e = b200::launch_sdpa_decode(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_fail(B200_ERR_CUDA, "b200_sdpa_decode_static: %s", cudaGetErrorString(e));
  return B200_OK;
}

}  // extern "C"
