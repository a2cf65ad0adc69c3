// Measures the int8 tensor-core peak of the device the way the GEMM kernels use the tensor cores:
// one CTA per SM issues tcgen05.mma kind::i8 (M = 128, N = 256, K = 32) back to back on operand
// tiles that stay resident in shared memory, two TMEM accumulators alternating, nothing else going
// on. The figure is the denominator of the prefill GEMM's roofline fraction (the driver-measured
// peaks cover HBM copies and bf16 GEMMs only).
#include <cstdio>

#include "../../include/litert_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace {

using namespace b200;

constexpr int kProbeN = 256;
constexpr int kProbeSmem = kTileBytes + kProbeN * kTileK8 + 1024;

__global__ void __launch_bounds__(128, 1) i8_peak_kernel(int iters, int* sink, int* status) {
  extern __shared__ __align__(1024) uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (kTileBytes + kProbeN * kTileK8) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u * (uint32_t)(i & 3);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads what the threads wrote
  if (tid == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  if (tid == 0) {
    constexpr uint32_t idesc = umma_idesc_s8(kProbeN);
    const uint32_t a_addr = smem_u32(smem), b_addr = a_addr + kTileBytes;
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tmem_base + (uint32_t)(it & 1) * kProbeN;
#pragma unroll
      for (int ks = 0; ks < kTileK8 / 32; ++ks)
        umma_s8(d, umma_smem_desc(a_addr + ks * 32), umma_smem_desc(b_addr + ks * 32), idesc, (it >= 2 || ks > 0) ? 1u : 0u);
    }
    umma_commit(&bar);
    mbar_wait_bounded(&bar, 0, &abort_flag, status, kStatusWaitTimeoutTmem);
  }
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    int r[16];
    tmem_ld16(tmem_base, r);
    tmem_ld_wait();
    if (r[0] == 0x7fffffff && sink) sink[0] = r[1];  // keeps the accumulator observable
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace

extern "C" int b200_measure_int8_tensor_peak(int iters, double* ops_per_second, double* ms_out) {
  if (iters < 16 || iters > (1 << 22) || !ops_per_second) return B200_ERR_INVALID_ARGUMENT;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem) != cudaSuccess) return B200_ERR_CUDA;
    configured[dev] = true;
  }
  const int sms = device_sm_count();
  int* d_misc = nullptr;
  if (cudaMalloc(&d_misc, 256) != cudaSuccess) return B200_ERR_CUDA;
  cudaMemset(d_misc, 0, 256);
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  float best = 0.0f;
  for (int rep = 0; rep < 4; ++rep) {  // the first launch warms up; the best of the others counts
    cudaEventRecord(a, nullptr);
    i8_peak_kernel<<<sms, 128, kProbeSmem>>>(iters, d_misc + 8, d_misc);
    cudaEventRecord(b, nullptr);
    if (cudaEventSynchronize(b) != cudaSuccess) break;
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, a, b);
    if (rep > 0 && (best == 0.0f || ms < best)) best = ms;
  }
  int status = 0;
  const cudaError_t e = cudaMemcpy(&status, d_misc, sizeof(int), cudaMemcpyDeviceToHost);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  cudaFree(d_misc);
  if (e != cudaSuccess || best <= 0.0f) return B200_ERR_CUDA;
  if (status != 0) return B200_ERR_KERNEL_TIMEOUT;
  const double ops = 2.0 * 128 * kProbeN * 32 * (kTileK8 / 32) * (double)iters * sms;
  *ops_per_second = ops / (best * 1e-3);
  if (ms_out) *ms_out = best;
  return B200_OK;
}
