/*
 * Entry points of libtflite_b200_delegate.so, the CUDA delegate for the
 * quantized-inference hot path. The library is a TFLite "external delegate"
 * plugin: a host loads it with dlopen and binds the two symbols below, exactly
 * as tflite/delegates/external/external_delegate.cc:39-64 does for
 * `--external_delegate_path`, the kernel test harness
 * (tflite/kernels/test_util.cc:522-560) and Python's
 * tf.lite.experimental.load_delegate (tflite/python/interpreter.py:138-178).
 *
 * TfLiteDelegate is the struct of tflite/core/c/common.h:1442-1493; this
 * header only forward-declares it so that it can be read without the LiteRT
 * tree.
 *
 * Options (string key/value pairs, tflite/delegates/external/external_delegate.h:27-35):
 *   device          CUDA device index (default 0)
 *   buffer_handles  "1": leave outputs on the device and publish buffer handles
 *                   (tensor->buffer_handle, data_is_stale); default copies back in invoke
 *   claim_fc / claim_bmm / claim_sdpa   "0" to leave that op kind to the CPU kernels
 *   fail_on         host-side fault injection for tests: create | init | prepare | invoke | alloc
 *                   (mirrors error_during_* of
 *                   tflite/delegates/utils/dummy_delegate/external_delegate_adaptor.cc:47-66)
 */
#ifndef LITERT_B200_DELEGATE_H_
#define LITERT_B200_DELEGATE_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

struct TfLiteDelegate;

/* Replaces nothing in the reference: it IS the plugin contract of
 * tflite/delegates/external/external_delegate_interface.h:64-73. Returns NULL
 * and calls report_error (when given) on failure. */
__attribute__((visibility("default"))) struct TfLiteDelegate* tflite_plugin_create_delegate(
    const char* const* options_keys, const char* const* options_values, size_t num_options,
    void (*report_error)(const char*));

/* NULL is allowed (external_delegate_interface.h:70-73). */
__attribute__((visibility("default"))) void tflite_plugin_destroy_delegate(struct TfLiteDelegate* delegate);

/* A second library, libLiteRtGpuAccelerator.so (litert_b200/csrc/delegate/litert_accelerator.cc),
 * exports the DATA symbol
 *     extern "C" const LiteRtAcceleratorDef LiteRtAcceleratorImpl;
 * (litert/c/internal/litert_accelerator_def.h:40-66), which the LiteRT environment looks up with dlsym()
 * (litert/runtime/accelerators/gpu_registry.cc:121-134). Its create_delegate calls
 * tflite_plugin_create_delegate above and wraps the result with LiteRtRuntimeContext::wrap_delegate.
 * It is not declared here because its type lives in the LiteRT headers. */

/* Number of graph nodes the last Prepare claimed (what
 * SingleOpModel::CountOpsExecutedByCpuKernel, tflite/kernels/test_util.cc:697-703,
 * lets tests assert from the other side); -1 for NULL. */
__attribute__((visibility("default"))) int b200_delegate_num_claimed_nodes(const struct TfLiteDelegate* delegate);

/* Number of decomposition subgraphs of claimed composites that the last Prepare marked
 * delegation-skippable through tflite::delegates::MarkSubgraphAsDelegationSkippable
 * (tflite/delegates/utils.h:62-93), when the process exports that function; -1 for NULL. */
__attribute__((visibility("default"))) int b200_delegate_num_skippable_subgraphs(const struct TfLiteDelegate* delegate);

/* The delegate's device-arena planner as a pure host function (no CUDA): for n
 * tensors with sizes and [first_use, last_use] op intervals, writes 256-byte
 * aligned offsets and returns the slab size. Same job as ArenaPlanner +
 * SimpleMemoryArena (tflite/arena_planner.cc:204-382,
 * tflite/simple_memory_arena.cc:370-434) do for the host arena. */
__attribute__((visibility("default"))) size_t b200_arena_plan(int n, const size_t* bytes, const int* first_use,
                                                              const int* last_use, int num_ops, size_t* offsets);

#ifdef __cplusplus
}
#endif
#endif /* LITERT_B200_DELEGATE_H_ */
