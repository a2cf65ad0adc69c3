// Shared device helpers for the sm_100a kernels: mbarrier and bulk-copy PTX
// wrappers with bounded waits, the legacy tensor-core int8/f16 MMA wrappers,
// and the tile geometry of the packed weight layouts.
#pragma once

#include <cstdlib>

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---- packed layouts -------------------------------------------------------
// Weights are repacked once into tiles that one bulk copy moves and that both
// MMA paths read without bank conflicts. A tile covers kTileN output channels
// by kTileK8 reduction bytes: kTileN rows of 128 bytes, in groups of 8 rows
// (1 KiB), and inside a group the 16-byte chunk c of row r sits at chunk
// position c XOR r (swz_chunk_offset below): the K-major layout with 128-byte
// swizzling that tcgen05.mma takes through a shared-memory descriptor, and in
// which a warp of the mma.sync path reading one chunk of 8 rows touches 32
// distinct banks.
constexpr int kTileN = 128;        // output channels per tile
constexpr int kTileK8 = 128;       // int8 reduction elements per tile
constexpr int kTileBytes = kTileN * kTileK8;  // 16 KiB
constexpr int kRowGroups = kTileN / 8;        // 16
constexpr int kChunks8 = kTileK8 / 16;        // 8 chunks of 16 bytes along K

// 4-bit tiles: kTileN rows x 256 reduction elements as four sub-tiles of 64 (the K extent of one
// fp16 operand tile), each 4 KiB of nibbles followed by its 2 x kTileN fp16 block scales: 18 KiB.
constexpr int kTileK4 = 256;
constexpr int kSubBlocks4 = kTileK4 / 32;                     // 8
constexpr int kTile4SubWordBytes = kTileN * 64 / 2;           // 4 KiB of nibbles per sub-tile
constexpr int kTile4SubBytes = kTile4SubWordBytes + kTileN * 2 * 2;  // + 512 B of scales
constexpr int kTile4Bytes = 4 * kTile4SubBytes;               // 18 KiB

// Status word values written by kernels (0 = ok).
enum : int {
  kStatusOk = 0,
  kStatusWaitTimeoutFull = 101,   // consumer gave up waiting for a stage
  kStatusWaitTimeoutEmpty = 102,  // producer gave up waiting for a free stage
  kStatusWaitTimeoutTmem = 103,
  kStatusTimeoutPeer = 104,       // a tensor-parallel peer never signalled its partial result
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in these kernels is bounded. When a wait runs out, the thread
// records why in *status, raises the CTA-wide abort flag and carries on as if
// the wait had succeeded: control flow stays uniform (every barrier is still
// reached, every accumulator still freed), later waits return at once, the
// kernel ends, and the host sees a non-zero status instead of a hung GPU.
// The budget of one wait is one second unless the host wrote another value (nanoseconds, non-zero)
// into the 64-bit word that follows the status word's 8 bytes (b200_set_wait_budget): read on the
// slow path only, after the first polls have failed.
constexpr unsigned long long kWaitBudgetNs = 1000ull * 1000ull * 1000ull;  // one second per wait
constexpr int kStatusBudgetWordOffsetInts = 2;

__device__ __forceinline__ unsigned long long wait_budget_ns(const int* status) {
  if (!status) return kWaitBudgetNs;
  const unsigned long long b =
      *reinterpret_cast<const volatile unsigned long long*>(status + kStatusBudgetWordOffsetInts);
  return b ? b : kWaitBudgetNs;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code) {
  if (*abort_flag) return;
  if (mbar_try_wait(bar, parity)) return;
  const unsigned long long t0 = global_timer_ns();
  const unsigned long long budget = wait_budget_ns(status);
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return;
      if (global_timer_ns() - t0 > budget) break;
    }
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);  // (entry points without a status word still end in bounded time)
}

// Last resort after an abort: waits (10 ms at most, whatever the abort flag says) for a copy that was
// issued towards `bar`, so that a CTA does not exit with copies into its shared memory in flight.
__device__ __forceinline__ void mbar_drain_bounded(uint64_t* bar, uint32_t parity) {
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63u) == 63u && global_timer_ns() - t0 > 10ull * 1000ull * 1000ull) return;
  }
}

// ---- bulk async copy (TMA engine, linear form) ------------------------------
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Same copy for data that is read once (the weight stream): its L2 lines are the first to be
// evicted, so the few MB that every step re-reads (activations, the KV cache, kernel code) stay
// resident in L2 instead of being swept out by gigabytes of weights.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Asks L2 for a range of global memory without any destination (16-byte aligned address, size a
// multiple of 16): used by the GEMV producers for their own weight tiles beyond the shared-memory
// ring while they wait for the kernel that produces their activations, so that HBM keeps streaming
// during the short row kernels between two projections.
__device__ __forceinline__ void prefetch_l2_bulk(const void* gmem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem_src), "r"(bytes) : "memory");
}

// ---- legacy tensor-core MMA -------------------------------------------------
// D(16x8,s32) += A(16x32,s8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Sub-CTA barrier over `count` threads (count a multiple of 32), id 1..15.
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---- fixed-point requantization (int32 accumulator -> int32) --------------
// Same arithmetic as tflite/kernels/internal/common.cc:81-90
// (MultiplyByQuantizedMultiplier, double rounding): x * 2^left, then the
// nearest integer to (that * multiplier) / 2^31 with ties toward +infinity and
// saturation for INT32_MIN^2, then a rounding right shift with ties away from
// zero.
__device__ __forceinline__ int32_t requantize_mbqm(int32_t x, int32_t multiplier, int shift) {
  const int left = shift > 0 ? shift : 0;
  const int right = shift > 0 ? 0 : -shift;
  const int32_t xs = static_cast<int32_t>(static_cast<uint32_t>(x) << left);
  int32_t hi;
  if (xs == INT32_MIN && multiplier == INT32_MIN) {
    hi = INT32_MAX;
  } else {
    const long long ab = static_cast<long long>(xs) * static_cast<long long>(multiplier);
    hi = static_cast<int32_t>((ab + (1ll << 30)) >> 31);
  }
  if (right == 0) return hi;
  const int32_t mask = static_cast<int32_t>((1u << right) - 1u);
  const int32_t rem = hi & mask;
  const int32_t threshold = (mask >> 1) + (hi < 0 ? 1 : 0);
  return (hi >> right) + (rem > threshold ? 1 : 0);
}

// Float fused activations of the hybrid path, numbered like
// TfLiteFusedActivation (tflite/kernels/internal/tensor_utils.h:58-80).
__device__ __forceinline__ float apply_activation(float v, int act) {
  switch (act) {
    case 1: return fmaxf(0.0f, v);
    case 2: return fmaxf(-1.0f, fminf(v, 1.0f));
    case 3: return fmaxf(0.0f, fminf(v, 6.0f));
    case 4: return tanhf(v);
    case 5: return signbit(v) ? 1.0f : 0.0f;
    case 6: return 1.0f / (1.0f + expf(-v));
    default: return v;
  }
}

}  // namespace b200

// ---- tcgen05 (5th-generation tensor cores, TMEM accumulators) ----------------
namespace b200 {

// Operand tiles (weights and quantized activations alike) use the K-major layout with 128-byte
// swizzling that tcgen05.mma reads at full shared-memory bandwidth: rows of 128 reduction bytes,
// groups of 8 rows = 1 KiB, and inside a group the 16-byte chunk c of row r sits at chunk position
// c XOR r. (The plain layout of 8 x 16-byte core matrices costs the tensor core an 8-way bank
// conflict on every operand fetch: measured 0.7 POP/s where this layout is not the limit.)
__host__ __device__ constexpr int swz_chunk_offset(int r, int c) { return r * 128 + ((c ^ r) << 4); }

// Shared-memory matrix descriptor for such a tile: start address (1 KiB aligned tile base plus
// 32 bytes per K step of 32), 1 KiB between 8-row groups, layout type 2 = 128-byte swizzle; the
// leading-dimension offset is unused for this layout (conventionally 1). Bit 46: sm_100 version.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// Instruction descriptor, kind::i8: s8 x s8 -> s32, both operands K-major,
// M = 128 rows of A, N = n columns of B (a multiple of 16 up to 256).
__host__ __device__ constexpr uint32_t umma_idesc_s8(int n) {
  return (2u << 4) /* D = s32 */ | (1u << 7) /* A = s8 */ | (1u << 10) /* B = s8 */ |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// Whole warp. Writes the TMEM base address to *smem_dst.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// One thread. D[tmem] (+)= A[smem] * B[smem]; accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_s8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One thread. The mbarrier gets one arrival when every MMA issued so far by
// this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// Whole warp: lane t receives 16 consecutive 32-bit columns of TMEM lane
// (32 * (warp % 4) + t), starting at the column in taddr.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace b200

// ---- thread-block clusters: barrier and distributed shared memory --------------------
namespace b200 {
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address, in the cluster-wide shared window, of `local` inside CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// Eight bytes to a peer CTA's shared memory that also count as 8 transaction bytes on the peer's
// mbarrier: data and "it has arrived" in one message, no cluster-wide barrier. Both addresses from
// map_to_rank; `addr` 8-byte aligned.
__device__ __forceinline__ void st_async_cluster_f32x2(uint32_t addr, float a, float b, uint32_t remote_bar) {
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(addr), "f"(a),
               "f"(b), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void st_async_cluster_f32(uint32_t addr, float v, uint32_t remote_bar) {  // 4 transaction bytes
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::"r"(addr), "f"(v), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void st_async_cluster_f32x4(uint32_t addr, float4 v, uint32_t remote_bar) {  // 16 bytes, addr 16-byte aligned
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void st_async_cluster_u32(uint32_t addr, int32_t v, uint32_t remote_bar) {  // 4 transaction bytes
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];" ::"r"(addr), "r"(v), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, int32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
}  // namespace b200

// ---- programmatic dependent launch ---------------------------------------------
// Kernels of a dependent chain are launched with programmatic stream
// serialization: a kernel may start while its predecessor is still running, does
// whatever does not depend on it (barrier set-up, TMEM allocation, prefetching
// constant weights), and calls pdl_wait() before touching anything the
// predecessor produces (the wait returns once the predecessor grid has completed
// and its writes are visible). pdl_launch_dependents() lets the successor start.
// Every kernel of a chain calls pdl_wait(), so completion is transitive: when a
// kernel's wait returns, every earlier kernel of the chain has completed. That makes
// it safe to call pdl_launch_dependents() first thing (pdl_enter): several later
// kernels may then be resident early, but before their own wait they only read
// constants. Both are no-ops for a kernel launched the ordinary way.
namespace b200 {
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Entry of a kernel with no work to do ahead of its predecessor: release the successor, then wait.
__device__ __forceinline__ void pdl_enter() {
  pdl_launch_dependents();
  pdl_wait();
}

// Measurement knobs (B200_PDL, B200_FC_*, B200_SDPA_*, B200_DEC_* ...: environment variables that pick a
// kernel variant or leave work out, for A/B timing) exist only in builds made with -DB200_TUNING_KNOBS
// (B200_NVCC_FLAGS=-DB200_TUNING_KNOBS python -m litert_b200.build --force). A regular build reads no
// environment variable on any kernel path: tuning_env() is a constant null pointer there.
inline const char* tuning_env(const char* name) {
#ifdef B200_TUNING_KNOBS
  return getenv(name);
#else
  (void)name;
  return nullptr;
#endif
}

// B200_PDL=0 (tuning builds) turns the attribute off (plain stream order) for A/B measurement.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                  Args... args) {
  cudaLaunchConfig_t cfg;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, with the grid grouped into thread-block clusters of `cluster_x` CTAs (distributed shared
// memory between the CTAs of a cluster).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                                          cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace b200
