// First-index arg-max with the NaN rule of the reference's sampler, shared by the greedy-pick kernels
// and the fused LM-head epilogue.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

struct BestPick {
  float v;
  int i;
};

// The serial scan `if (x[i] > x[best]) best = i` from best = 0, whatever the order pairs are combined
// in (litert/vendors/nvidia/dispatch/greedy_sampler_kernel.cu:31-50): a NaN at index 0 wins outright,
// a NaN anywhere else never does; otherwise the larger value, ties to the lower index.
__device__ __forceinline__ BestPick better_pick(BestPick a, BestPick b) {
  if (a.i == 0 && isnan(a.v)) return a;
  if (b.i == 0 && isnan(b.v)) return b;
  if (isnan(a.v)) return b;
  if (isnan(b.v)) return a;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// litert/vendors/nvidia/trtllm/head_kernels.cu:35-43: tanh(logit / cap) * cap (cap <= 0: no cap)
__device__ __forceinline__ float soft_capped(float v, float cap) {
  return cap > 0.0f ? __fmul_rn(tanhf(__fmul_rn(v, __fdiv_rn(1.0f, cap))), cap) : v;
}

}  // namespace b200
