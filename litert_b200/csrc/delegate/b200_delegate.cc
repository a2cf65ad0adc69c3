// TfLiteDelegate for the B200 kernels: claims FULLY_CONNECTED, BATCH_MATMUL
// (constant right-hand side) and the odml.scaled_dot_product_attention
// composite / custom op, and runs them through the C ABI in
// include/litert_b200.h. Built as an external-delegate plugin
// (tflite/delegates/external/external_delegate_interface.h:64-73).
//
// Contract followed (tflite/core/c/common.h:1442-1493 and
// tflite/core/subgraph.cc:2497-2622): Prepare walks the execution plan, asks
// the runtime to replace the supported node subsets with one delegate kernel
// each; the kernel's init uploads and repacks constant weights once, prepare
// plans the device arena for the partition's tensors, invoke copies the
// partition inputs to the device, enqueues the ops on the delegate's stream
// and brings the outputs back (or publishes buffer handles). There is no CPU
// fallback inside the delegate: an unsupported node is simply not claimed.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_runtime_api.h>
#include <dlfcn.h>

#include "../../../include/litert_b200.h"
#include "../../../include/litert_b200_delegate.h"
#include "device_arena.h"
#include "flex_scale.h"
#include "tflite/builtin_ops.h"
#include "tflite/core/c/builtin_op_data.h"
#include "tflite/core/c/common.h"

namespace {

constexpr char kSdpaName[] = "odml.scaled_dot_product_attention";
constexpr char kDelegateName[] = "B200Delegate";

struct Options {
  int device = 0;
  std::string fail_on;          // "", "init", "prepare", "invoke", "alloc": host-side fault injection
  bool buffer_handles = false;  // publish outputs as buffer handles instead of copying back in invoke
  bool claim_fc = true, claim_bmm = true, claim_sdpa = true;
  bool fuse = true;        // merge op sequences of a decoder graph into the fused kernels (results stay within tolerance)
  bool cuda_graph = true;  // replay a partition's launches as one CUDA graph from its third invocation on
  bool claim_glue = true;  // the float32 ops between a decoder's projections (ADD, MUL, GELU, RESHAPE, SLICE, ...)
  int min_nodes_per_partition = 1;
};

#define CUDA_OK(ctx, expr)                                                             \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) {                                                           \
      TF_LITE_KERNEL_LOG((ctx), "B200 delegate: %s failed: %s", #expr, cudaGetErrorString(_e)); \
      return kTfLiteDelegateError;                                                     \
    }                                                                                  \
  } while (0)

#define B200_OK_OR_RETURN(ctx, expr)                                                   \
  do {                                                                                 \
    int _rc = (expr);                                                                  \
    if (_rc != B200_OK) {                                                              \
      TF_LITE_KERNEL_LOG((ctx), "B200 delegate: %s", b200_last_error());               \
      return kTfLiteDelegateError;                                                     \
    }                                                                                  \
  } while (0)

#define B200_GLUE_OR_RETURN(ctx, expr)                                                 \
  do {                                                                                 \
    int _rc = (expr);                                                                  \
    if (_rc != B200_OK) {                                                              \
      TF_LITE_KERNEL_LOG((ctx), "B200 delegate: %s", b200_glue_last_error());          \
      return kTfLiteDelegateError;                                                     \
    }                                                                                  \
  } while (0)

#define B200_EW_OR_RETURN(ctx, expr)                                                   \
  do {                                                                                 \
    int _rc = (expr);                                                                  \
    if (_rc != B200_OK) {                                                              \
      TF_LITE_KERNEL_LOG((ctx), "B200 delegate: %s", b200_elementwise_last_error());   \
      return kTfLiteDelegateError;                                                     \
    }                                                                                  \
  } while (0)

// ---------------------------------------------------------------- device helpers
struct DeviceMem {
  void* ptr = nullptr;
  size_t bytes = 0;
  ~DeviceMem() { reset(); }
  void reset() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
  }
  bool ensure(size_t n) {
    if (n <= bytes) return true;
    reset();
    if (cudaMalloc(&ptr, n) != cudaSuccess) return false;
    bytes = n;
    return true;
  }
};

struct DelegateState {
  Options options;
  TfLiteDelegate delegate;
  cudaStream_t stream = nullptr;
  DeviceMem zero_ws, scratch, sdpa_ws;
  DeviceMem bmm_lhs, bmm_rhs, bmm_packed, bmm_row_sums;  // BATCH_MATMUL temporaries (transposed operands, run-time RHS)
  bool ready = false;
  // buffer handles: handle id -> (device pointer, bytes)
  std::unordered_map<int, std::pair<const void*, size_t>> handles;
  int next_handle = 1;
  int delegated_nodes = 0, partitions = 0, skippable_marked = 0;

  TfLiteStatus EnsureDevice(TfLiteContext* ctx) {
    CUDA_OK(ctx, cudaSetDevice(options.device));
    if (ready) return kTfLiteOk;
    CUDA_OK(ctx, cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    if (!zero_ws.ensure(b200_zero_workspace_bytes())) {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: cannot allocate the zero workspace");
      return kTfLiteDelegateError;
    }
    B200_OK_OR_RETURN(ctx, b200_zero_workspace_init(zero_ws.ptr, stream));
    ready = true;
    return kTfLiteOk;
  }
};

static void* ArenaAlloc(void* user, size_t bytes) {
  auto* st = static_cast<DelegateState*>(user);
  if (st->options.fail_on == "alloc") return nullptr;
  void* p = nullptr;
  return cudaMalloc(&p, bytes) == cudaSuccess ? p : nullptr;
}
static void ArenaFree(void*, void* p) { cudaFree(p); }

// ---------------------------------------------------------------- node classification
enum class OpKind {
  kNone, kFcInt8, kFcHybrid, kFcW4, kBmmHybrid, kBmmInt8, kSdpa,
  // the ops between a decoder's projections
  kEmbedding, kAdd, kMul, kGelu, kReshape, kSlice, kConcat, kRmsNorm, kKvCache, kArgMax,
  // produced by the fusion pass over a partition's ops (never by Classify)
  kNormQuant,      // odml.rms_norm whose result only feeds hybrid projections: normalised AND quantized once
  kFcQuantized,    // a hybrid projection reading rows another op already quantized
  kSdpaQuant,      // the attention composite (one query token) whose result only feeds a hybrid projection: leaves quantized
  kFcGroup,        // several such projections of the same single row (q, k, v) as one GEMV over the stacked weights
  kGateUpGeglu,    // gate and up projections as one GEMV + GELU x up + quantization for the down projection
  kLmHeadPick,     // the vocabulary projection with ARG_MAX in its epilogue: no logits are written
  kRope,           // SLICE / SLICE / MUL(-1) / CONCATENATION / MUL / MUL / ADD of the rotary embedding as one kernel
  kRopeKv,         // the rotary embeddings of a step's query and key rows and odml.update_kv_cache as one kernel
  kSkipped         // a node whose work a fused op does
};

constexpr char kRmsNormName[] = "odml.rms_norm";
constexpr char kKvCacheName[] = "odml.update_kv_cache";

// A tensor's shape as four dimensions, padded with leading ones; false beyond rank 4.
inline bool Pad4(const TfLiteTensor& t, int out[4]) {
  const int r = t.dims->size;
  if (r > 4) return false;
  for (int i = 0; i < 4; ++i) out[i] = 1;
  for (int i = 0; i < r; ++i) out[4 - r + i] = t.dims->data[i];
  return true;
}

inline bool IsConst(const TfLiteTensor& t) { return t.allocation_type == kTfLiteMmapRo && t.data.raw != nullptr; }

inline int64_t NumElements(const TfLiteTensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.dims->size; ++i) n *= t.dims->data[i];
  return n;
}

inline const TfLiteAffineQuantization* Affine(const TfLiteTensor& t) {
  return t.quantization.type == kTfLiteAffineQuantization
             ? static_cast<const TfLiteAffineQuantization*>(t.quantization.params)
             : nullptr;
}

// Geometry of one BATCH_MATMUL: [.., m, k] x [.., k, n] with up to three broadcast batch dimensions
// (the reference extends both shapes to five, tflite/kernels/internal/reference/batch_matmul.h:
// 118-135). lhs_mats / rhs_mats: matrices held by each operand; out_mats: products computed.
struct BmmGeometry {
  int m = 0, k = 0, n = 0;
  int lhs_batch[3] = {1, 1, 1}, rhs_batch[3] = {1, 1, 1}, out_batch[3] = {1, 1, 1};
  int lhs_mats = 1, rhs_mats = 1, out_mats = 1;
};

bool BmmShapes(const TfLiteTensor& x, const TfLiteTensor& w, bool adj_x, bool adj_y, BmmGeometry* g) {
  const int xr = x.dims->size, wr = w.dims->size;
  if (xr < 2 || xr > 5 || wr < 2 || wr > 5) return false;
  const int xm = x.dims->data[xr - 2], xk = x.dims->data[xr - 1];
  const int wk = w.dims->data[wr - 2], wn = w.dims->data[wr - 1];
  g->m = adj_x ? xk : xm;
  g->k = adj_x ? xm : xk;
  g->n = adj_y ? wk : wn;
  if ((adj_y ? wn : wk) != g->k || g->m <= 0 || g->k <= 0 || g->n <= 0) return false;
  for (int d = 0; d < 3; ++d) {
    const int xi = xr - 3 - (2 - d), wi = wr - 3 - (2 - d);  // right-aligned batch dimensions
    g->lhs_batch[d] = xi >= 0 ? x.dims->data[xi] : 1;
    g->rhs_batch[d] = wi >= 0 ? w.dims->data[wi] : 1;
    const int l = g->lhs_batch[d], r = g->rhs_batch[d];
    if (l <= 0 || r <= 0 || (l != r && l != 1 && r != 1)) return false;
    g->out_batch[d] = l == 1 ? r : l;
  }
  // (the reference's hybrid row sums only cover the two inner batch dimensions of the RHS,
  // batch_matmul.h:151-153: an RHS with an outer one is left to it)
  if (g->rhs_batch[0] != 1) return false;
  g->lhs_mats = g->lhs_batch[0] * g->lhs_batch[1] * g->lhs_batch[2];
  g->rhs_mats = g->rhs_batch[0] * g->rhs_batch[1] * g->rhs_batch[2];
  g->out_mats = g->out_batch[0] * g->out_batch[1] * g->out_batch[2];
  return g->out_mats <= 4096;
}

bool IsSdpaNode(const TfLiteNode* node, const TfLiteRegistration* reg) {
  if (reg->builtin_code == kTfLiteBuiltinStablehloComposite) {
    // tflite/delegates/xnnpack/xnnpack_delegate.cc:3400-3408 recognises the composite by name
    const auto* p = static_cast<const TfLiteStablehloCompositeParams*>(node->builtin_data);
    return p && p->name && strcmp(p->name, kSdpaName) == 0;
  }
  if (reg->builtin_code == kTfLiteBuiltinCustom) {
    return reg->custom_name && strcmp(reg->custom_name, kSdpaName) == 0;  // xnnpack_delegate.cc:3443-3444
  }
  return false;
}


bool IsCompositeNamed(const TfLiteNode* node, const TfLiteRegistration* reg, const char* name) {
  if (reg->builtin_code != kTfLiteBuiltinStablehloComposite) return false;
  const auto* p = static_cast<const TfLiteStablehloCompositeParams*>(node->builtin_data);
  return p && p->name && strcmp(p->name, name) == 0;
}

// The float32 ops a decoder-only graph has between its projections (as
// tensor/examples/gemma3/gemma3_graph.cc authors them), claimed so that the whole graph is one partition.
// Leaves *why empty when the op is simply none of them.
OpKind ClassifyGlue(TfLiteContext* ctx, const TfLiteNode* node, const TfLiteRegistration* reg, std::string* why) {
  const TfLiteTensor* T = ctx->tensors;
  auto in = [&](int i) -> const TfLiteTensor* {
    if (i >= node->inputs->size) return nullptr;
    const int idx = node->inputs->data[i];
    return idx == kTfLiteOptionalTensor ? nullptr : &T[idx];
  };
  if (node->outputs->size < 1) return OpKind::kNone;
  const TfLiteTensor* y = &T[node->outputs->data[0]];
  int d4[4];
  switch (reg->builtin_code) {
    case kTfLiteBuiltinAdd:
    case kTfLiteBuiltinMul: {
      const TfLiteTensor *a = in(0), *b = in(1);
      if (!a || !b || node->inputs->size != 2) return *why = "binary op operands", OpKind::kNone;
      const auto act = reg->builtin_code == kTfLiteBuiltinAdd
                           ? static_cast<const TfLiteAddParams*>(node->builtin_data)->activation
                           : static_cast<const TfLiteMulParams*>(node->builtin_data)->activation;
      if (act != kTfLiteActNone) return *why = "fused activation on a binary op", OpKind::kNone;
      if (a->type != kTfLiteFloat32 || b->type != kTfLiteFloat32 || y->type != kTfLiteFloat32)
        return *why = "binary op is not float32", OpKind::kNone;
      if (IsConst(*a) && IsConst(*b)) return *why = "constant binary op", OpKind::kNone;
      int da[4], db[4];
      if (!Pad4(*a, da) || !Pad4(*b, db) || !Pad4(*y, d4)) return *why = "binary op rank", OpKind::kNone;
      for (int i = 0; i < 4; ++i) {
        const int o = da[i] == 1 ? db[i] : da[i];
        if ((db[i] != 1 && db[i] != o) || d4[i] != o || o <= 0) return *why = "binary op shapes do not broadcast", OpKind::kNone;
      }
      return reg->builtin_code == kTfLiteBuiltinAdd ? OpKind::kAdd : OpKind::kMul;
    }
    case kTfLiteBuiltinGelu: {
      const TfLiteTensor* x = in(0);
      if (!x || x->type != kTfLiteFloat32 || y->type != kTfLiteFloat32 || IsConst(*x) || NumElements(*x) != NumElements(*y))
        return *why = "gelu operands", OpKind::kNone;
      return OpKind::kGelu;
    }
    case kTfLiteBuiltinReshape: {
      const TfLiteTensor* x = in(0);
      if (!x || IsConst(*x) || x->type != y->type || x->bytes != y->bytes || x->bytes == 0) return *why = "reshape operands", OpKind::kNone;
      if (x->type != kTfLiteFloat32 && x->type != kTfLiteInt32 && x->type != kTfLiteInt8) return *why = "reshape type", OpKind::kNone;
      if (node->inputs->size > 1 && in(1) && !IsConst(*in(1))) return *why = "reshape to a run-time shape", OpKind::kNone;
      return OpKind::kReshape;
    }
    case kTfLiteBuiltinSlice: {
      const TfLiteTensor *x = in(0), *b = in(1), *sz = in(2);
      if (!x || !b || !sz || IsConst(*x) || !IsConst(*b) || !IsConst(*sz)) return *why = "slice operands", OpKind::kNone;
      if (x->type != kTfLiteFloat32 || y->type != kTfLiteFloat32 || b->type != kTfLiteInt32 || sz->type != kTfLiteInt32)
        return *why = "slice types", OpKind::kNone;
      const int r = x->dims->size;
      if (r > 4 || r < 1 || NumElements(*b) != r || NumElements(*sz) != r || y->dims->size != r) return *why = "slice rank", OpKind::kNone;
      for (int i = 0; i < r; ++i) {
        const int begin = b->data.i32[i];
        const int size = sz->data.i32[i] < 0 ? x->dims->data[i] - begin : sz->data.i32[i];
        if (begin < 0 || size <= 0 || begin + size > x->dims->data[i] || y->dims->data[i] != size) return *why = "slice box", OpKind::kNone;
      }
      return OpKind::kSlice;
    }
    case kTfLiteBuiltinConcatenation: {
      const auto* p = static_cast<const TfLiteConcatenationParams*>(node->builtin_data);
      if (!p || p->activation != kTfLiteActNone || node->inputs->size < 1) return *why = "concatenation parameters", OpKind::kNone;
      const int r = y->dims->size;
      if (r < 1 || r > 4 || y->type != kTfLiteFloat32) return *why = "concatenation output", OpKind::kNone;
      const int axis = p->axis < 0 ? p->axis + r : p->axis;
      if (axis < 0 || axis >= r) return *why = "concatenation axis", OpKind::kNone;
      int along = 0;
      for (int i = 0; i < node->inputs->size; ++i) {
        const TfLiteTensor* x = in(i);
        if (!x || x->type != kTfLiteFloat32 || x->dims->size != r || IsConst(*x)) return *why = "concatenation operands", OpKind::kNone;
        for (int d = 0; d < r; ++d)
          if (d != axis && x->dims->data[d] != y->dims->data[d]) return *why = "concatenation shapes", OpKind::kNone;
        along += x->dims->data[axis];
      }
      if (along != y->dims->data[axis]) return *why = "concatenation shapes", OpKind::kNone;
      return OpKind::kConcat;
    }
    case kTfLiteBuiltinEmbeddingLookup: {
      // hybrid lookup: int8 table with per-tensor or per-row scales (tflite/kernels/embedding_lookup.cc:307-395)
      const TfLiteTensor *ids = in(0), *table = in(1);
      if (!ids || !table || ids->type != kTfLiteInt32 || IsConst(*ids)) return *why = "embedding ids", OpKind::kNone;
      if (!IsConst(*table) || table->type != kTfLiteInt8 || table->dims->size != 2 || y->type != kTfLiteFloat32)
        return *why = "embedding table is not a constant int8 matrix", OpKind::kNone;
      const auto* q = Affine(*table);
      if (q && q->scale && q->scale->size > 1 && (q->quantized_dimension != 0 || q->scale->size != table->dims->data[0]))
        return *why = "embedding scales must follow the rows", OpKind::kNone;
      if (NumElements(*y) != NumElements(*ids) * table->dims->data[1]) return *why = "embedding output shape", OpKind::kNone;
      return OpKind::kEmbedding;
    }
    case kTfLiteBuiltinArgMax: {
      const TfLiteTensor *x = in(0), *axis = in(1);
      if (!x || !axis || x->type != kTfLiteFloat32 || IsConst(*x) || !IsConst(*axis) || axis->type != kTfLiteInt32)
        return *why = "arg_max operands", OpKind::kNone;
      const int r = x->dims->size;
      const int a = axis->data.i32[0] < 0 ? axis->data.i32[0] + r : axis->data.i32[0];
      if (r < 1 || a != r - 1) return *why = "arg_max over another axis than the last", OpKind::kNone;
      if (y->type != kTfLiteInt32 && y->type != kTfLiteInt64) return *why = "arg_max output type", OpKind::kNone;
      if (NumElements(*y) * x->dims->data[r - 1] != NumElements(*x)) return *why = "arg_max output shape", OpKind::kNone;
      return OpKind::kArgMax;
    }
    default:
      break;
  }
  if (IsCompositeNamed(node, reg, kRmsNormName)) {
    const TfLiteTensor *x = in(0), *g = in(1);
    if (!x || x->type != kTfLiteFloat32 || y->type != kTfLiteFloat32 || IsConst(*x) || x->dims->size < 1 || x->bytes != y->bytes)
      return *why = "rms_norm operands", OpKind::kNone;
    const int d = x->dims->data[x->dims->size - 1];
    if (g && (!IsConst(*g) || g->type != kTfLiteFloat32 || NumElements(*g) != d)) return *why = "rms_norm scale", OpKind::kNone;
    return OpKind::kRmsNorm;
  }
  if (reg->builtin_code == kTfLiteBuiltinCustom && reg->custom_name && strcmp(reg->custom_name, kKvCacheName) == 0) {
    // tflite/experimental/genai/kvcache.cc:78-228: (position, key, value) -> (full keys, full values), float32, batch 1
    const TfLiteTensor *pos = in(0), *k = in(1), *v = in(2);
    if (node->inputs->size != 3 || node->outputs->size != 2 || !pos || !k || !v) return *why = "kv cache operands", OpKind::kNone;
    const TfLiteTensor* y2 = &T[node->outputs->data[1]];
    if (pos->type != kTfLiteInt64 || IsConst(*pos) || IsConst(*k) || IsConst(*v)) return *why = "kv cache operands", OpKind::kNone;
    for (const TfLiteTensor* t : {k, v, y, y2})
      if (t->type != kTfLiteFloat32 || t->dims->size != 4 || t->dims->data[0] != 1) return *why = "kv cache wants float32 [1, t, heads, dim]", OpKind::kNone;
    float cap = 0.0f;
    b200::FlexMapFloat(static_cast<const uint8_t*>(node->custom_initial_data), static_cast<size_t>(node->custom_initial_data_size),
                       "kv_cache_max", &cap);
    const int max_entries = cap > 0.0f ? static_cast<int>(cap) : 2048;  // kDefaultMaxNumCacheEntries
    for (const TfLiteTensor* t : {y, y2})
      if (t->dims->data[1] != max_entries || t->dims->data[2] != k->dims->data[2] || t->dims->data[3] != k->dims->data[3])
        return *why = "kv cache output shape", OpKind::kNone;
    if (v->dims->data[1] != k->dims->data[1] || v->dims->data[2] != k->dims->data[2] || v->dims->data[3] != k->dims->data[3] ||
        k->dims->data[1] > max_entries)
      return *why = "kv cache key / value shapes", OpKind::kNone;
    return OpKind::kKvCache;
  }
  return OpKind::kNone;
}

// Why a node is not claimed is reported through `why` (one line).
OpKind Classify(TfLiteContext* ctx, const TfLiteNode* node, const TfLiteRegistration* reg, const Options& opt,
                std::string* why) {
  const TfLiteTensor* T = ctx->tensors;
  auto in = [&](int i) -> const TfLiteTensor* {
    if (i >= node->inputs->size) return nullptr;
    const int idx = node->inputs->data[i];
    return idx == kTfLiteOptionalTensor ? nullptr : &T[idx];
  };
  if (reg->builtin_code == kTfLiteBuiltinFullyConnected && opt.claim_fc) {
    const auto* p = static_cast<const TfLiteFullyConnectedParams*>(node->builtin_data);
    const TfLiteTensor *x = in(0), *w = in(1), *b = in(2);
    const TfLiteTensor* y = &T[node->outputs->data[0]];
    if (!p || !x || !w) return *why = "missing operands", OpKind::kNone;
    if (p->weights_format != kTfLiteFullyConnectedWeightsFormatDefault) return *why = "shuffled weights", OpKind::kNone;
    if (w->sparsity) return *why = "sparse weights", OpKind::kNone;
    if (!IsConst(*w) || w->dims->size != 2) return *why = "weights not a constant matrix", OpKind::kNone;
    if (b && !IsConst(*b)) return *why = "bias not constant", OpKind::kNone;
    // a constant input would never be uploaded (the arena holds run-time tensors only): leave such a
    // node to the runtime, which folds or evaluates it on the CPU
    if (IsConst(*x)) return *why = "constant input", OpKind::kNone;
    if (x->dims->size < 1 || w->dims->data[1] <= 0 || NumElements(*x) % w->dims->data[1] != 0)
      return *why = "input shape", OpKind::kNone;
    if (b && NumElements(*b) != w->dims->data[0]) return *why = "bias length", OpKind::kNone;
    if (NumElements(*y) != NumElements(*x) / w->dims->data[1] * w->dims->data[0]) return *why = "output shape", OpKind::kNone;
    if (x->type == kTfLiteInt8 && w->type == kTfLiteInt8 && y->type == kTfLiteInt8) {
      const auto* q = Affine(*w);
      if (!q || !q->scale || q->scale->size < 1) return *why = "weights lack affine quantization", OpKind::kNone;
      if (b && b->type != kTfLiteInt32) return *why = "bias type", OpKind::kNone;
      if (q->scale->size > 1 && (q->quantized_dimension != 0 || q->scale->size != w->dims->data[0]))
        return *why = "per-channel axis must be 0", OpKind::kNone;  // fully_connected.cc:539
      if (p->activation != kTfLiteActNone && p->activation != kTfLiteActRelu &&
          p->activation != kTfLiteActReluN1To1 && p->activation != kTfLiteActRelu6)
        return *why = "activation", OpKind::kNone;  // fully_connected.cc:748-753
      return OpKind::kFcInt8;
    }
    if (x->type == kTfLiteFloat32 && w->type == kTfLiteInt8 && y->type == kTfLiteFloat32) {
      if (b && b->type != kTfLiteFloat32) return *why = "bias type", OpKind::kNone;
      const auto* q = Affine(*w);
      if (q && q->scale && q->scale->size > 1 && (q->quantized_dimension != 0 || q->scale->size != w->dims->data[0]))
        return *why = "per-channel axis must be 0", OpKind::kNone;
      return OpKind::kFcHybrid;
    }
    if (x->type == kTfLiteFloat32 && w->type == kTfLiteInt4 && y->type == kTfLiteFloat32 &&
        w->quantization.type == kTfLiteBlockwiseQuantization) {
      const auto* q = static_cast<const TfLiteBlockwiseQuantization*>(w->quantization.params);
      if (!q || q->blocksize != 32) return *why = "blocksize", OpKind::kNone;
      const TfLiteTensor& s = T[q->scale];
      if (!IsConst(s) || s.type != kTfLiteFloat16) return *why = "block scales", OpKind::kNone;
      if (w->dims->data[1] % q->blocksize) return *why = "k not a multiple of the blocksize", OpKind::kNone;
      if (b && b->type != kTfLiteFloat32) return *why = "bias type", OpKind::kNone;
      return OpKind::kFcW4;
    }
    return *why = "tensor types", OpKind::kNone;
  }
  if (reg->builtin_code == kTfLiteBuiltinBatchMatmul && opt.claim_bmm) {
    const auto* p = static_cast<const TfLiteBatchMatMulParams*>(node->builtin_data);
    const TfLiteTensor *x = in(0), *w = in(1);
    const TfLiteTensor* y = &T[node->outputs->data[0]];
    if (!p || !x || !w) return *why = "missing operands", OpKind::kNone;
    if (IsConst(*x)) return *why = "constant lhs", OpKind::kNone;
    if (w->allocation_type == kTfLiteMmapRo && !w->data.raw) return *why = "rhs without data", OpKind::kNone;
    BmmGeometry g;
    if (!BmmShapes(*x, *w, p->adj_x, p->adj_y, &g)) return *why = "batch_matmul shapes", OpKind::kNone;
    if (NumElements(*y) != static_cast<int64_t>(g.out_mats) * g.m * g.n) return *why = "output shape", OpKind::kNone;
    const auto* q = Affine(*w);
    const bool per_channel = q && q->scale && q->scale->size > 1;
    if (x->type == kTfLiteFloat32 && w->type == kTfLiteInt8 && y->type == kTfLiteFloat32) {
      // The reference's hybrid kernel steps through the per-row scales and zero points (and the RHS row
      // sums) by (b0 + b1 + b2) x rows, not by the flattened batch index
      // (tflite/kernels/internal/reference/batch_matmul.h:138-143, 160-186): with one varying batch
      // dimension per operand that is the same thing, with two it reads another batch's parameters.
      // Such graphs are left to it rather than answered differently.
      int lhs_varying = 0, rhs_varying = 0;
      for (int d = 0; d < 3; ++d) {
        lhs_varying += g.lhs_batch[d] > 1;
        rhs_varying += g.rhs_batch[d] > 1;
      }
      if (lhs_varying > 1 || rhs_varying > 1) return *why = "hybrid batch_matmul over several batch dimensions", OpKind::kNone;
      if (per_channel) {
        // the scales follow the output columns: the RHS's N axis (tflite/kernels/batch_matmul.cc:701-708, 487-497)
        const int n_axis = p->adj_y ? w->dims->size - 2 : w->dims->size - 1;
        if (q->quantized_dimension != n_axis || q->scale->size != g.n) return *why = "per-channel rhs axis", OpKind::kNone;
      }
      return OpKind::kBmmHybrid;
    }
    if (x->type == kTfLiteInt8 && w->type == kTfLiteInt8 && y->type == kTfLiteInt8) {
      if (per_channel) return *why = "per-channel int8 rhs", OpKind::kNone;
      return OpKind::kBmmInt8;
    }
    return *why = "tensor types", OpKind::kNone;
  }
  if (opt.claim_sdpa && IsSdpaNode(node, reg)) {
    if (node->inputs->size < 3) return *why = "sdpa operands", OpKind::kNone;
    const TfLiteTensor *q = in(0), *k = in(1), *v = in(2), *m = in(3);
    const TfLiteTensor* y = &T[node->outputs->data[0]];
    if (!q || !k || !v) return *why = "sdpa operands", OpKind::kNone;
    for (const TfLiteTensor* t : {q, k, v, m})
      if (t && IsConst(*t)) return *why = "sdpa with a constant operand", OpKind::kNone;
    // float32 tensors as the reference op and XNNPACK take them (xnnpack_delegate.cc:6404-6433), or all
    // float16 (a graph converted with half-precision activations); the additive mask stays float32
    for (const TfLiteTensor* t : {q, k, v, y})
      if ((t->type != kTfLiteFloat32 && t->type != kTfLiteFloat16) || t->type != q->type || t->dims->size != 4)
        return *why = "sdpa wants 4-D float32 or float16 tensors of one type", OpKind::kNone;
    if (m && (m->type != kTfLiteFloat32 || m->dims->size != 4)) return *why = "sdpa mask", OpKind::kNone;
    const int B = q->dims->data[0], Tq = q->dims->data[1], N = q->dims->data[2], H = q->dims->data[3];
    const int S = k->dims->data[1], Nkv = k->dims->data[2];
    if (B <= 0 || Tq <= 0 || N <= 0 || H <= 0 || S <= 0) return *why = "sdpa shapes", OpKind::kNone;
    if (k->dims->data[0] != B || v->dims->data[0] != B || k->dims->data[3] != H || v->dims->data[3] != H ||
        v->dims->data[1] != S || v->dims->data[2] != Nkv || Nkv <= 0 || N % Nkv != 0)
      return *why = "sdpa shapes", OpKind::kNone;  // xnnpack_delegate.cc:6433-6459
    if (y->dims->data[0] != B || y->dims->data[1] != Tq || y->dims->data[2] != N || y->dims->data[3] != H)
      return *why = "sdpa output shape", OpKind::kNone;
    if (m && (m->dims->data[0] != B || m->dims->data[1] != 1 || m->dims->data[2] != Tq || m->dims->data[3] != S))
      return *why = "sdpa mask shape", OpKind::kNone;
    // head layouts outside the split-K kernels run on a fallback that keeps S logits in shared memory
    if (!(N / Nkv <= 8 && (H == 64 || H == 128 || H == 256)) && (static_cast<int64_t>(S) + H) * 4 > 200 * 1024)
      return *why = "sdpa cache too long for this head layout", OpKind::kNone;
    return OpKind::kSdpa;
  }
  if (opt.claim_glue) {
    const OpKind k = ClassifyGlue(ctx, node, reg, why);
    if (k != OpKind::kNone || !why->empty()) return k;
  }
  return *why = "op not on the hot path", OpKind::kNone;
}

// ---------------------------------------------------------------- delegate kernel
struct OpRecord {
  OpKind kind = OpKind::kNone;
  int node_index = -1;
  int x = -1, y = -1;              // tensor indices (graph numbering)
  int q = -1, k = -1, v = -1, mask = -1;
  int m = 0, n = 0, kdim = 0;
  // constants on the device
  DeviceMem packed, row_sums, w_scales, bias, mult, shift, kfsum;
  bool per_channel = false, asymmetric = false;
  int activation = 0;
  int32_t input_offset = 0, filter_offset = 0, output_offset = 0, act_min = -128, act_max = 127;
  // batch_matmul
  int w = -1;                       // right-hand side tensor (graph numbering)
  bool adj_x = false, adj_y = false, rhs_const = true, fold_lhs = false;
  BmmGeometry g;
  size_t packed_stride = 0;         // bytes between the packed matrices of a batched RHS
  // every tensor the node reads and writes (graph numbering, constants included): the fusion pass's view
  std::vector<int> all_in, all_out;
  // fused ops
  int rows_from = -1;               // kFcQuantized: index (in the partition) of the op that holds its quantized rows
  std::vector<std::pair<int, int>> group_out;  // kFcGroup: (result tensor, first channel in the stacked output)
  DeviceMem q_tiled, q_scales, q_zps, tmp_f32;  // kNormQuant / kGateUpGeglu: the quantized rows they produce
  int heads = 0;
  // glue ops
  std::vector<int> ins;             // operand tensors (graph numbering; -1 = a constant held in const_a / const_b)
  int y2 = -1;                      // second output (kv cache)
  DeviceMem const_a, const_b, ws_small;
  int dims_a[4] = {1, 1, 1, 1}, dims_b[4] = {1, 1, 1, 1}, dims_o[4] = {1, 1, 1, 1}, begin[4] = {0, 0, 0, 0};
  int axis = 0, rows = 0, width = 0, max_entries = 0, approximate = 1, vocab = 0;
  float eps = 0.0f;
  bool out_i64 = false;
  DeviceMem k_cache, v_cache;       // odml.update_kv_cache: the persistent float32 caches
  // sdpa
  int B = 0, T = 1, N = 0, Nkv = 0, H = 0, S = 0;
  int sdpa_dtype = B200_DTYPE_F32;
  float scale = 0.0f, logit_cap = 0.0f;
};

// int32 requantization constants, computed as the reference's Prepare does
// (tflite/kernels/fully_connected.cc:552-582, tflite/kernels/internal/quantization_util.cc:53-104,
// tflite/kernels/kernel_util.cc:354-410).
void QuantizeMultiplier(double m, int32_t* q, int* shift) {
  if (m == 0.) {
    *q = 0;
    *shift = 0;
    return;
  }
  const double f = std::frexp(m, shift);
  int64_t q_fixed = static_cast<int64_t>(std::round(f * (1LL << 31)));
  if (q_fixed == (1LL << 31)) {
    q_fixed /= 2;
    ++*shift;
  }
  if (*shift < -31) {
    *shift = 0;
    q_fixed = 0;
  }
  *q = static_cast<int32_t>(q_fixed);
}

bool ActivationRangeInt8(TfLiteFusedActivation act, float scale, int32_t zp, int32_t* lo, int32_t* hi) {
  auto quant = [&](float f, int32_t* q) {
    const float t = std::round(f / scale);
    if (!(t >= -2147483648.0f && t <= 2147483648.0f)) return false;
    *q = zp + static_cast<int32_t>(t);
    return true;
  };
  *lo = -128;
  *hi = 127;
  int32_t t;
  if (act == kTfLiteActRelu) {
    if (!quant(0.f, &t)) return false;
    *lo = std::max(*lo, t);
  } else if (act == kTfLiteActRelu6) {
    if (!quant(0.f, &t)) return false;
    *lo = std::max(*lo, t);
    if (!quant(6.f, &t)) return false;
    *hi = std::min(*hi, t);
  } else if (act == kTfLiteActReluN1To1) {
    if (!quant(-1.f, &t)) return false;
    *lo = std::max(*lo, t);
    if (!quant(1.f, &t)) return false;
    *hi = std::min(*hi, t);
  }
  return true;
}

class DelegateKernel {
 public:
  explicit DelegateKernel(DelegateState* st) : st_(st), arena_(ArenaAlloc, ArenaFree, st) {}

  TfLiteStatus Init(TfLiteContext* ctx, const TfLiteDelegateParams* params) {
    if (st_->options.fail_on == "init") {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: injected failure in init");
      return kTfLiteDelegateError;
    }
    TF_LITE_ENSURE_STATUS(st_->EnsureDevice(ctx));
    inputs_.assign(params->input_tensors->data, params->input_tensors->data + params->input_tensors->size);
    outputs_.assign(params->output_tensors->data, params->output_tensors->data + params->output_tensors->size);
    ops_.clear();
    for (int i = 0; i < params->nodes_to_replace->size; ++i) {
      const int node_index = params->nodes_to_replace->data[i];
      TfLiteNode* node = nullptr;
      TfLiteRegistration* reg = nullptr;
      TF_LITE_ENSURE_STATUS(ctx->GetNodeAndRegistration(ctx, node_index, &node, &reg));
      std::string why;
      const OpKind kind = Classify(ctx, node, reg, st_->options, &why);
      if (kind == OpKind::kNone) {
        TF_LITE_KERNEL_LOG(ctx, "B200 delegate: node %d handed to the kernel but unsupported (%s)", node_index,
                           why.c_str());
        return kTfLiteDelegateError;
      }
      ops_.emplace_back(new OpRecord());
      OpRecord& op = *ops_.back();
      op.kind = kind;
      op.node_index = node_index;
      for (int j = 0; j < node->inputs->size; ++j) op.all_in.push_back(node->inputs->data[j]);
      for (int j = 0; j < node->outputs->size; ++j) op.all_out.push_back(node->outputs->data[j]);
      TF_LITE_ENSURE_STATUS(BuildOp(ctx, node, reg, &op));
    }
    if (st_->options.fuse) TF_LITE_ENSURE_STATUS(FuseOps(ctx));
    CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));  // staging buffers below go out of scope
    return kTfLiteOk;
  }

  // ---- fusion pass -------------------------------------------------------------------------------------
  // Rewrites op sequences a converter emits for a decoder layer into the fused kernels, wherever every
  // intermediate tensor is consumed inside the pattern and nowhere else (not by another node, not as a
  // partition output). Unfused, the graph is still executed op by op: fusion only removes launches and
  // float32 round trips.
  int Producer(int tensor) const {
    for (size_t i = 0; i < ops_.size(); ++i)
      for (int t : ops_[i]->all_out)
        if (t == tensor && ops_[i]->kind != OpKind::kSkipped) return static_cast<int>(i);
    return -1;
  }
  std::vector<int> Consumers(int tensor) const {
    std::vector<int> c;
    for (size_t i = 0; i < ops_.size(); ++i)
      for (int t : ops_[i]->all_in)
        if (t == tensor) {
          c.push_back(static_cast<int>(i));
          break;
        }
    return c;
  }
  bool IsPartitionOutput(int tensor) const {
    for (int t : outputs_)
      if (t == tensor) return true;
    return false;
  }
  // the only consumer of `tensor`, or -1 (also when it leaves the partition)
  int OnlyConsumer(int tensor) const {
    if (IsPartitionOutput(tensor)) return -1;
    const std::vector<int> c = Consumers(tensor);
    return c.size() == 1 ? c[0] : -1;
  }
  bool AllocRows(TfLiteContext* ctx, OpRecord* op, int m, int k) {
    const size_t per = static_cast<size_t>(std::max(m, 256)) * sizeof(float);
    if (op->q_tiled.ensure(b200_tiled_rows_bytes(m, k)) && op->q_scales.ensure(per) && op->q_zps.ensure(per)) return true;
    TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed (quantized rows)");
    return false;
  }

  TfLiteStatus FuseOps(TfLiteContext* ctx) {
    const TfLiteTensor* T = ctx->tensors;
    const int n_ops = static_cast<int>(ops_.size());
    // (1) rotary embedding: ADD(MUL(x, cos), MUL(CONCAT(MUL(SLICE_hi(x), -1), SLICE_lo(x)), sin))
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& add = *ops_[i];
      if (add.kind != OpKind::kAdd || add.ins[0] < 0 || add.ins[1] < 0) continue;
      const int ma = Producer(add.ins[0]), mb = Producer(add.ins[1]);
      if (ma < 0 || mb < 0 || ops_[ma]->kind != OpKind::kMul || ops_[mb]->kind != OpKind::kMul) continue;
      OpRecord *xc = ops_[ma].get(), *rs = ops_[mb].get();
      if (OnlyConsumer(xc->y) != i || OnlyConsumer(rs->y) != i || xc->ins[0] < 0 || xc->ins[1] < 0 || rs->ins[0] < 0 || rs->ins[1] < 0)
        continue;
      // which MUL is x * cos and which rot * sin: the latter's first operand comes from a CONCATENATION
      auto is_concat = [&](int t) { const int p = Producer(t); return p >= 0 && ops_[p]->kind == OpKind::kConcat; };
      if (is_concat(xc->ins[0])) std::swap(xc, rs);
      if (!is_concat(rs->ins[0])) continue;
      const int x = xc->ins[0], cos_t = xc->ins[1], sin_t = rs->ins[1];
      OpRecord& cat = *ops_[Producer(rs->ins[0])];
      if (cat.ins.size() != 2 || cat.axis != 3 || OnlyConsumer(cat.y) != Producer(rs->y)) continue;
      const int neg_i = Producer(cat.ins[0]), lo_i = Producer(cat.ins[1]);
      if (neg_i < 0 || lo_i < 0 || ops_[neg_i]->kind != OpKind::kMul || ops_[lo_i]->kind != OpKind::kSlice) continue;
      OpRecord &neg = *ops_[neg_i], &lo = *ops_[lo_i];
      if (neg.ins[0] < 0 || neg.ins[1] >= 0 || neg.const_b.bytes != sizeof(float)) continue;  // MUL by a constant scalar
      const TfLiteTensor& scalar = T[neg.all_in[1]];
      if (!IsConst(scalar) || scalar.data.f[0] != -1.0f) continue;
      const int hi_i = Producer(neg.ins[0]);
      if (hi_i < 0 || ops_[hi_i]->kind != OpKind::kSlice) continue;
      OpRecord& hi = *ops_[hi_i];
      const TfLiteTensor& xt = T[x];
      if (xt.dims->size != 4 || hi.ins[0] != x || lo.ins[0] != x) continue;
      const int tokens = xt.dims->data[0] * xt.dims->data[1], heads = xt.dims->data[2], h = xt.dims->data[3];
      if (h % 2 || lo.begin[3] != 0 || hi.begin[3] != h / 2 || lo.dims_o[3] != h / 2 || hi.dims_o[3] != h / 2) continue;
      if (lo.begin[0] || lo.begin[1] || lo.begin[2] || hi.begin[0] || hi.begin[1] || hi.begin[2]) continue;
      if (lo.dims_o[2] != heads || hi.dims_o[2] != heads || lo.dims_o[1] != xt.dims->data[1]) continue;
      if (OnlyConsumer(hi.y) != neg_i || OnlyConsumer(neg.y) != Producer(rs->ins[0]) || OnlyConsumer(lo.y) != Producer(rs->ins[0])) continue;
      const TfLiteTensor &ct = T[cos_t], &st = T[sin_t];
      if (NumElements(ct) != static_cast<int64_t>(tokens) * h || NumElements(st) != NumElements(ct) || IsConst(ct) || IsConst(st)) continue;
      for (OpRecord* dead : {xc, rs, &cat, &neg, &lo, &hi}) dead->kind = OpKind::kSkipped;
      add.kind = OpKind::kRope;
      add.ins = {x, cos_t, sin_t};
      add.rows = tokens;
      add.heads = heads;
      add.width = h;
    }
    // (1b) odml.update_kv_cache whose key rows come from a rotary embedding, with the rotary embedding of the
    // query rows beside it (same cos / sin): one kernel instead of three. It runs at the cache update's place in
    // the plan, so everything that reads the rotated queries must come after that.
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& kv = *ops_[i];
      if (kv.kind != OpKind::kKvCache || kv.ins.size() != 3) continue;
      const int rk_i = Producer(kv.ins[1]);
      if (rk_i < 0 || ops_[rk_i]->kind != OpKind::kRope || OnlyConsumer(ops_[rk_i]->y) != i) continue;
      OpRecord& rk = *ops_[rk_i];
      if (rk.rows != kv.rows || rk.heads * rk.width != kv.width) continue;
      // consumers of the rotated queries (through RESHAPEs, which run nothing) must follow the fused op
      std::function<bool(int)> later = [&](int tensor) {
        if (IsPartitionOutput(tensor)) return false;
        for (int c : Consumers(tensor)) {
          if (ops_[c]->kind == OpKind::kReshape) {
            if (!later(ops_[c]->y)) return false;
          } else if (c <= i) {
            return false;
          }
        }
        return true;
      };
      // every layer's rotations share the graph's cos / sin inputs: this layer's is the nearest one in the plan whose
      // operand exists before the cache update and whose result is only read after it
      int rq_i = -1;
      for (int dist = 1; dist < n_ops && rq_i < 0; ++dist)
        for (int j : {rk_i - dist, rk_i + dist}) {
          if (j < 0 || j >= n_ops || j >= i || rq_i >= 0) continue;
          const OpRecord& c = *ops_[j];
          if (c.kind == OpKind::kRope && c.ins[1] == rk.ins[1] && c.ins[2] == rk.ins[2] && c.rows == rk.rows &&
              c.width == rk.width && later(c.y))
            rq_i = j;
        }
      if (rq_i < 0) continue;
      OpRecord& rq = *ops_[rq_i];
      // operands: position, k, v, cos, sin, q; the rotated queries are listed too, so that the plan gives them a buffer
      kv.ins = {kv.ins[0], rk.ins[0], kv.ins[2], rk.ins[1], rk.ins[2], rq.ins[0], rq.y};
      kv.heads = rq.heads;    // query heads
      kv.B = rk.heads;        // key / value heads
      kv.H = rk.width;
      kv.kind = OpKind::kRopeKv;
      rk.kind = OpKind::kSkipped;
      rq.kind = OpKind::kSkipped;
    }
    // (2) odml.rms_norm feeding only hybrid projections: normalise and quantize once for all of them
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& norm = *ops_[i];
      if (norm.kind != OpKind::kRmsNorm || !norm.const_a.ptr || norm.width > 12288 || IsPartitionOutput(norm.y)) continue;
      const std::vector<int> users = Consumers(norm.y);
      bool ok = !users.empty();
      for (int u : users) ok = ok && ops_[u]->kind == OpKind::kFcHybrid && ops_[u]->asymmetric && ops_[u]->x == norm.y && ops_[u]->kdim == norm.width;
      if (!ok) continue;
      if (!AllocRows(ctx, &norm, norm.rows, norm.width)) return kTfLiteDelegateError;
      norm.kind = OpKind::kNormQuant;
      for (int u : users) {
        ops_[u]->kind = OpKind::kFcQuantized;
        ops_[u]->rows_from = i;
        ops_[u]->m = norm.rows;
      }
    }
    // (3) gate / up projections + GELU x up + the down projection's quantization
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& mul = *ops_[i];
      if (mul.kind != OpKind::kMul || mul.ins[0] < 0 || mul.ins[1] < 0) continue;
      int gelu_i = Producer(mul.ins[0]), up_i = Producer(mul.ins[1]);
      if (gelu_i >= 0 && ops_[gelu_i]->kind != OpKind::kGelu) std::swap(gelu_i, up_i);
      if (gelu_i < 0 || up_i < 0 || ops_[gelu_i]->kind != OpKind::kGelu || !ops_[gelu_i]->approximate) continue;
      const int gate_i = Producer(ops_[gelu_i]->ins[0]);
      if (gate_i < 0) continue;
      OpRecord &gate = *ops_[gate_i], &up = *ops_[up_i], &gelu = *ops_[gelu_i];
      if (gate.kind != OpKind::kFcQuantized || up.kind != OpKind::kFcQuantized || gate.rows_from != up.rows_from) continue;
      if (gate.n != up.n || gate.kdim != up.kdim || !gate.per_channel || !up.per_channel || gate.bias.ptr || up.bias.ptr ||
          gate.activation || up.activation)
        continue;
      const int down_i = OnlyConsumer(mul.y);
      if (down_i < 0 || ops_[down_i]->kind != OpKind::kFcHybrid || !ops_[down_i]->asymmetric || ops_[down_i]->kdim != gate.n) continue;
      if (OnlyConsumer(gate.y) != gelu_i || OnlyConsumer(gelu.y) != i || OnlyConsumer(up.y) != i) continue;
      for (int d = 0; d < 4; ++d)
        if (mul.dims_a[d] != mul.dims_b[d]) gelu_i = -1;  // a broadcasting MUL is something else
      if (gelu_i < 0) continue;
      // one packed matrix [2 f, k]: the gate's rows, then the up projection's
      const TfLiteTensor &wg = T[gate.all_in[1]], &wu = T[up.all_in[1]];
      const int f = gate.n, k = gate.kdim, m = gate.m;
      {
        std::vector<int8_t> both(static_cast<size_t>(2) * f * k);
        memcpy(both.data(), wg.data.int8, static_cast<size_t>(f) * k);
        memcpy(both.data() + static_cast<size_t>(f) * k, wu.data.int8, static_cast<size_t>(f) * k);
        TF_LITE_ENSURE_STATUS(PackInt8(ctx, both.data(), 2 * f, k, false, &mul));
      }
      std::vector<float> scales(static_cast<size_t>(2) * f);
      const auto *qg = Affine(wg), *qu = Affine(wu);
      for (int c = 0; c < f; ++c) {
        scales[c] = qg->scale->data[c];
        scales[f + c] = qu->scale->data[c];
      }
      TF_LITE_ENSURE_STATUS(Upload(ctx, scales, &mul.w_scales));
      if (!mul.tmp_f32.ensure(sizeof(float) * static_cast<size_t>(m) * 2 * f) || !AllocRows(ctx, &mul, m, f)) {
        TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed (gate / up buffer)");
        return kTfLiteDelegateError;
      }
      CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));
      mul.kind = OpKind::kGateUpGeglu;
      mul.rows_from = gate.rows_from;
      mul.m = m;
      mul.n = 2 * f;
      mul.kdim = k;
      mul.per_channel = true;
      gate.packed.reset();
      up.packed.reset();
      gate.kind = up.kind = gelu.kind = OpKind::kSkipped;
      ops_[down_i]->kind = OpKind::kFcQuantized;
      ops_[down_i]->rows_from = i;
      ops_[down_i]->m = m;
    }
    // (3b) what is left of the projections that read the same quantized rows (q, k and v after a norm): with
    // one row per call their results are consecutive slices of one stacked GEMV's output row
    for (int i = 0; i < n_ops; ++i) {
      if (ops_[i]->kind != OpKind::kNormQuant || ops_[i]->rows != 1) continue;
      std::vector<int> sib;
      for (int u = 0; u < n_ops; ++u) {
        const OpRecord& f = *ops_[u];
        if (f.kind == OpKind::kFcQuantized && f.rows_from == i && f.m == 1 && f.per_channel && !f.bias.ptr && !f.activation &&
            f.kdim == ops_[i]->width)
          sib.push_back(u);
      }
      if (sib.size() < 2) continue;
      OpRecord& lead = *ops_[sib[0]];
      const int k = lead.kdim;
      int total = 0;
      for (int u : sib) total += ops_[u]->n;
      std::vector<int8_t> stacked(static_cast<size_t>(total) * k);
      std::vector<float> scales(static_cast<size_t>(total));
      std::vector<std::pair<int, int>> outs;
      int at = 0;
      for (int u : sib) {
        const OpRecord& f = *ops_[u];
        const TfLiteTensor& w = T[f.all_in[1]];
        memcpy(stacked.data() + static_cast<size_t>(at) * k, w.data.int8, static_cast<size_t>(f.n) * k);
        const auto* q = Affine(w);
        for (int c = 0; c < f.n; ++c) scales[at + c] = q->scale->data[c];
        outs.emplace_back(f.y, at);
        at += f.n;
      }
      if (!lead.tmp_f32.ensure(sizeof(float) * static_cast<size_t>(total))) {
        TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed (stacked projections)");
        return kTfLiteDelegateError;
      }
      TF_LITE_ENSURE_STATUS(PackInt8(ctx, stacked.data(), total, k, false, &lead));
      TF_LITE_ENSURE_STATUS(Upload(ctx, scales, &lead.w_scales));
      CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));
      for (size_t j = 1; j < sib.size(); ++j) {
        OpRecord& f = *ops_[sib[j]];
        f.packed.reset();
        f.row_sums.reset();
        f.w_scales.reset();
        f.kind = OpKind::kSkipped;
      }
      lead.kind = OpKind::kFcGroup;
      lead.n = total;
      lead.group_out = outs;
    }
    // (2b) the residual ADD in front of such a norm moves into it: h += delta in place, then normalise and
    // quantize. The sum tensor becomes another name for h's buffer, which no one else may still need.
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& norm = *ops_[i];
      if (norm.kind != OpKind::kNormQuant) continue;
      const int add_i = Producer(norm.ins[0]);
      if (add_i < 0 || ops_[add_i]->kind != OpKind::kAdd) continue;
      OpRecord& add = *ops_[add_i];
      if (add.ins[0] < 0 || add.ins[1] < 0 || IsPartitionOutput(add.y)) continue;
      bool same = true;
      for (int d = 0; d < 4; ++d) same = same && add.dims_a[d] == add.dims_o[d] && add.dims_b[d] == add.dims_o[d];
      if (!same) continue;
      // the residual stream is the operand that dies here; prefer the first, as the graph writes ADD(h, delta)
      int h = add.ins[0], delta = add.ins[1];
      if (OnlyConsumer(h) != add_i) std::swap(h, delta);
      if (OnlyConsumer(h) != add_i || persistent_.count(h) || IsConst(T[h])) continue;
      bool is_input = false;
      for (int t : inputs_) is_input = is_input || t == h;
      if (is_input) continue;  // a partition input keeps its host meaning: do not overwrite its device copy's role
      inplace_alias_[add.y] = h;
      norm.ins = {h, delta};
      add.kind = OpKind::kSkipped;
    }
    // (5) one-token attention read only by a hybrid projection (through RESHAPEs): the merge of the
    // attention partials quantizes the row for that projection, no float result, no separate row kernel
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& at = *ops_[i];
      if (at.kind != OpKind::kSdpa || at.T != 1 || at.sdpa_dtype != B200_DTYPE_F32 || IsPartitionOutput(at.y)) continue;
      if (at.N % at.Nkv || at.N / at.Nkv > 8 || at.N > 64 || (at.H != 64 && at.H != 128 && at.H != 256)) continue;
      int y = at.y, user = OnlyConsumer(y);
      bool through_ok = true;
      for (int hops = 0; hops < 4 && user >= 0 && ops_[user]->kind == OpKind::kReshape; ++hops) {
        if (IsPartitionOutput(ops_[user]->y)) through_ok = false;
        y = ops_[user]->y;
        user = OnlyConsumer(y);
      }
      if (!through_ok || user < 0) continue;
      OpRecord& fc = *ops_[user];
      if (fc.kind != OpKind::kFcHybrid || !fc.asymmetric || fc.x != y || fc.kdim != at.N * at.H) continue;
      if (!AllocRows(ctx, &at, at.B, at.N * at.H)) return kTfLiteDelegateError;
      at.kind = OpKind::kSdpaQuant;
      fc.kind = OpKind::kFcQuantized;
      fc.rows_from = i;
      fc.m = at.B;
    }
    // (4) a projection read only by ARG_MAX (the LM head under greedy sampling): the pick moves into its epilogue
    for (int i = 0; i < n_ops; ++i) {
      OpRecord& am = *ops_[i];
      if (am.kind != OpKind::kArgMax || am.rows > 16) continue;
      const int fc_i = Producer(am.ins[0]);
      if (fc_i < 0 || ops_[fc_i]->kind != OpKind::kFcQuantized || OnlyConsumer(ops_[fc_i]->y) != i) continue;
      OpRecord& fc = *ops_[fc_i];
      if (fc.bias.ptr || fc.activation || !fc.per_channel || fc.n != am.width || fc.m != am.rows) continue;
      const size_t ws = b200_lm_head_workspace_bytes(am.rows) + sizeof(int32_t) * am.rows;
      if (!am.ws_small.ensure(ws)) {
        TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
        return kTfLiteDelegateError;
      }
      am.kind = OpKind::kLmHeadPick;
      am.rows_from = fc.rows_from;
      am.m = fc.m;
      am.n = fc.n;
      am.kdim = fc.kdim;
      am.packed.ptr = fc.packed.ptr;  // the projection's constants move over
      am.packed.bytes = fc.packed.bytes;
      fc.packed.ptr = nullptr;
      fc.packed.bytes = 0;
      std::swap(am.row_sums.ptr, fc.row_sums.ptr);
      std::swap(am.row_sums.bytes, fc.row_sums.bytes);
      std::swap(am.w_scales.ptr, fc.w_scales.ptr);
      std::swap(am.w_scales.bytes, fc.w_scales.bytes);
      fc.kind = OpKind::kSkipped;
    }
    return kTfLiteOk;
  }

  TfLiteStatus Prepare(TfLiteContext* ctx, TfLiteNode*) {
    if (st_->options.fail_on == "prepare") {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: injected failure in prepare");
      return kTfLiteDelegateError;
    }
    CUDA_OK(ctx, cudaSetDevice(st_->options.device));
    if (graph_exec_) {  // a new plan moves tensors: the recorded launches hold the old addresses
      cudaGraphExecDestroy(graph_exec_);
      graph_exec_ = nullptr;
    }
    invocations_ = 0;
    // tensors living on the device for this partition: every op operand that is not a constant
    slot_of_.clear();
    persistent_.clear();
    alias_ = inplace_alias_;  // sums computed in place by a fused norm share the residual stream's buffer
    for (auto& opp : ops_)  // a RESHAPE's result is its operand's bytes: same device buffer, nothing to run
      if (opp->kind == OpKind::kReshape) alias_[opp->y] = opp->ins[0];
    for (auto& opp : ops_)  // (before any touch: a later op's operand may be an earlier op's persistent output)
      if (opp->kind == OpKind::kKvCache || opp->kind == OpKind::kRopeKv) {
        persistent_[opp->y] = opp->k_cache.ptr;
        persistent_[opp->y2] = opp->v_cache.ptr;
      } else if (opp->kind == OpKind::kFcGroup) {
        // the members' results are slices of the group's own output row
        for (const auto& o : opp->group_out) persistent_[o.first] = static_cast<float*>(opp->tmp_f32.ptr) + o.second;
      }
    std::vector<b200::ArenaRequest> req;
    const int num_ops = static_cast<int>(ops_.size());
    auto touch = [&](int tensor, int op_index) {
      if (tensor < 0) return;
      tensor = Canonical(tensor);
      const TfLiteTensor& t = ctx->tensors[tensor];
      if (IsConst(t) || persistent_.count(tensor)) return;
      auto it = slot_of_.find(tensor);
      if (it == slot_of_.end()) {
        slot_of_[tensor] = static_cast<int>(req.size());
        b200::ArenaRequest r;
        r.bytes = t.bytes;
        r.first_use = r.last_use = op_index;
        req.push_back(r);
      } else {
        req[it->second].last_use = op_index;
      }
    };
    size_t scratch = 0, sdpa = 0, bmm_lhs = 0, bmm_rhs = 0, bmm_packed = 0, bmm_rs = 0;
    for (int i = 0; i < num_ops; ++i) {
      OpRecord& op = *ops_[i];
      if (op.kind == OpKind::kSdpaQuant) {
        for (int t : {op.q, op.k, op.v, op.mask}) touch(t, i);
        sdpa = std::max(sdpa, b200_sdpa_workspace_bytes(op.B, op.N, op.Nkv, op.H, op.S));
      } else if (op.kind == OpKind::kSdpa) {
        for (int t : {op.q, op.k, op.v, op.mask, op.y}) touch(t, i);
        sdpa = std::max(sdpa, b200_sdpa_workspace_bytes(op.B * op.T, op.N, op.Nkv, op.H, op.S));
      } else if (op.kind == OpKind::kBmmHybrid || op.kind == OpKind::kBmmInt8) {
        touch(op.x, i);
        touch(op.w, i);  // a run-time right-hand side lives in the arena (a constant one is skipped)
        touch(op.y, i);
        op.m = op.fold_lhs ? op.g.m * op.g.lhs_mats : op.g.m;
        scratch = std::max(scratch, b200_fc_scratch_bytes(op.m, op.kdim));
        if (op.adj_x) bmm_lhs = std::max(bmm_lhs, ctx->tensors[op.x].bytes);
        if (!op.rhs_const) {
          const size_t mats = static_cast<size_t>(op.g.rhs_mats);
          if (!op.adj_y) bmm_rhs = std::max(bmm_rhs, ctx->tensors[op.w].bytes);
          bmm_packed = std::max(bmm_packed, mats * b200_packed_w8_bytes(op.n, op.kdim));
          bmm_rs = std::max(bmm_rs, mats * sizeof(int32_t) * op.n);
        }
      } else if (op.kind == OpKind::kSkipped) {
        continue;
      } else if (op.kind == OpKind::kFcQuantized) {
        touch(op.y, i);
      } else if (op.kind == OpKind::kLmHeadPick) {
        touch(op.y, i);
      } else if (op.kind == OpKind::kGateUpGeglu || op.kind == OpKind::kFcGroup) {
        continue;  // reads another op's quantized rows, writes its own buffer: no arena tensor
      } else if (op.kind >= OpKind::kEmbedding) {
        for (int t : op.ins) touch(t, i);
        if (op.kind == OpKind::kNormQuant) continue;  // its float32 result is never materialised
        if (op.kind == OpKind::kKvCache || op.kind == OpKind::kRopeKv) {
          // the op's outputs ARE its persistent caches: never arena tensors
          persistent_[op.y] = op.k_cache.ptr;
          persistent_[op.y2] = op.v_cache.ptr;
        } else {
          touch(op.y, i);
        }
      } else {
        const TfLiteTensor& x = ctx->tensors[op.x];
        op.m = static_cast<int>(NumElements(x) / op.kdim);  // fully_connected.cc:502
        touch(op.x, i);
        touch(op.y, i);
        scratch = std::max(scratch, b200_fc_scratch_bytes(op.m, op.kdim));
      }
    }
    // partition inputs arrive before the first op and outputs are read after the last one
    for (int t : inputs_) {
      auto it = slot_of_.find(Canonical(t));
      if (it != slot_of_.end()) req[it->second].first_use = 0;
    }
    for (int t : outputs_) {
      auto it = slot_of_.find(Canonical(t));
      if (it != slot_of_.end()) req[it->second].last_use = num_ops - 1;
    }
    if (!arena_.Commit(req, num_ops)) {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device arena allocation of %zu bytes failed", arena_.planned_bytes());
      return kTfLiteDelegateError;
    }
    if (!st_->scratch.ensure(scratch) || !st_->sdpa_ws.ensure(sdpa) || !st_->bmm_lhs.ensure(bmm_lhs) ||
        !st_->bmm_rhs.ensure(bmm_rhs) || !st_->bmm_packed.ensure(bmm_packed) || !st_->bmm_row_sums.ensure(bmm_rs)) {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: workspace allocation failed");
      return kTfLiteDelegateError;
    }
    return kTfLiteOk;
  }

  TfLiteStatus Invoke(TfLiteContext* ctx, TfLiteNode*) {
    if (st_->options.fail_on == "invoke") {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: injected failure in invoke");
      return kTfLiteDelegateError;
    }
    CUDA_OK(ctx, cudaSetDevice(st_->options.device));
    cudaStream_t s = st_->stream;
    // host -> device for the partition's non-constant inputs (tensor data pointers may change
    // between invocations, tflite/delegates/utils/simple_delegate.h:62-63, so read them now)
    for (int t : inputs_) {
      auto it = slot_of_.find(t);
      if (it == slot_of_.end()) continue;
      const TfLiteTensor& tensor = ctx->tensors[t];
      if (!tensor.data.raw) continue;
      CUDA_OK(ctx, cudaMemcpyAsync(arena_.Resolve(it->second), tensor.data.raw, tensor.bytes, cudaMemcpyHostToDevice, s));
    }
    // The partition's launches: eagerly the first time (one-time kernel set-up happens here), recorded into
    // a CUDA graph the second time, replayed from then on: shapes are static and every device address is
    // fixed once the arena is planned, so a partition of hundreds of small kernels costs one launch call.
    ++invocations_;
    if (graph_exec_) {
      CUDA_OK(ctx, cudaGraphLaunch(graph_exec_, s));
    } else if (st_->options.cuda_graph && !graph_failed_ && invocations_ == 2 && ops_.size() > 1) {
      cudaGraph_t g = nullptr;
      TfLiteStatus launched = kTfLiteOk;
      if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        for (auto& opp : ops_)
          if ((launched = Launch(ctx, *opp)) != kTfLiteOk) break;
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (launched == kTfLiteOk && e == cudaSuccess && g && cudaGraphInstantiate(&graph_exec_, g, 0) == cudaSuccess) {
          CUDA_OK(ctx, cudaGraphLaunch(graph_exec_, s));
        } else {
          graph_exec_ = nullptr;
          graph_failed_ = true;  // an op that cannot be recorded: plain launches from now on
          cudaGetLastError();
          for (auto& opp : ops_) TF_LITE_ENSURE_STATUS(Launch(ctx, *opp));
        }
        if (g) cudaGraphDestroy(g);
      } else {
        graph_failed_ = true;
        cudaGetLastError();
        for (auto& opp : ops_) TF_LITE_ENSURE_STATUS(Launch(ctx, *opp));
      }
    } else {
      for (auto& opp : ops_) TF_LITE_ENSURE_STATUS(Launch(ctx, *opp));
    }
    for (int t : outputs_) {
      void* dev = Dev(t);
      if (!dev) continue;
      TfLiteTensor& tensor = ctx->tensors[t];
      if (st_->options.buffer_handles) {
        if (tensor.buffer_handle == kTfLiteNullBufferHandle) tensor.buffer_handle = st_->next_handle++;
        st_->handles[tensor.buffer_handle] = {dev, tensor.bytes};
        tensor.delegate = &st_->delegate;
        tensor.data_is_stale = true;
      } else if (tensor.data.raw) {
        CUDA_OK(ctx, cudaMemcpyAsync(tensor.data.raw, dev, tensor.bytes, cudaMemcpyDeviceToHost, s));
      }
    }
    int status = 0;
    if (b200_read_status(st_->zero_ws.ptr, s, &status) != B200_OK) {  // synchronises the stream
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: %s", b200_last_error());
      // a wait ran out inside a kernel: this invocation's outputs are void; leave the workspace clean
      // so that the next invocation does not inherit the sticky status word or stale split-K counters
      b200_clear_status(st_->zero_ws.ptr, s);
      return kTfLiteDelegateError;
    }
    return kTfLiteOk;
  }

 private:
  // the tensor whose buffer `tensor` shares (chains of RESHAPEs resolved)
  int Canonical(int tensor) const {
    for (int hops = 0; hops < 64; ++hops) {
      auto it = alias_.find(tensor);
      if (it == alias_.end()) break;
      tensor = it->second;
    }
    return tensor;
  }

  void* Dev(int tensor) {
    tensor = Canonical(tensor);
    auto pit = persistent_.find(tensor);
    if (pit != persistent_.end()) return pit->second;
    auto it = slot_of_.find(tensor);
    return it == slot_of_.end() ? nullptr : arena_.Resolve(it->second);
  }

  template <typename T>
  TfLiteStatus Upload(TfLiteContext* ctx, const std::vector<T>& host, DeviceMem* dst) {
    if (host.empty()) return kTfLiteOk;
    if (!dst->ensure(host.size() * sizeof(T))) {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
      return kTfLiteDelegateError;
    }
    CUDA_OK(ctx, cudaMemcpyAsync(dst->ptr, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice, st_->stream));
    // the vector may die before the copy runs from pageable memory: cudaMemcpyAsync from pageable
    // host memory stages the data before returning, so this is safe
    return kTfLiteOk;
  }

  TfLiteStatus UploadRaw(TfLiteContext* ctx, const void* host, size_t bytes, DeviceMem* dst) {
    if (!dst->ensure(bytes)) {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
      return kTfLiteDelegateError;
    }
    CUDA_OK(ctx, cudaMemcpyAsync(dst->ptr, host, bytes, cudaMemcpyHostToDevice, st_->stream));
    return kTfLiteOk;
  }

  // Uploads an int8 weight matrix [n,k] (optionally the transpose of a [k,n] one) and packs it.
  TfLiteStatus PackInt8(TfLiteContext* ctx, const int8_t* host, int n, int k, bool transpose, OpRecord* op) {
    DeviceMem staging;
    if (transpose) {
      std::vector<int8_t> t(static_cast<size_t>(n) * k);
      for (int r = 0; r < k; ++r)
        for (int c = 0; c < n; ++c) t[static_cast<size_t>(c) * k + r] = host[static_cast<size_t>(r) * n + c];
      TF_LITE_ENSURE_STATUS(Upload(ctx, t, &staging));
    } else {
      TF_LITE_ENSURE_STATUS(UploadRaw(ctx, host, static_cast<size_t>(n) * k, &staging));
    }
    if (!op->packed.ensure(b200_packed_w8_bytes(n, k)) || !op->row_sums.ensure(sizeof(int32_t) * n)) {
      TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
      return kTfLiteDelegateError;
    }
    B200_OK_OR_RETURN(ctx, b200_pack_w8(static_cast<const int8_t*>(staging.ptr), n, k, op->packed.ptr,
                                       static_cast<int32_t*>(op->row_sums.ptr), st_->stream));
    CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));  // staging is freed on return
    return kTfLiteOk;
  }

  TfLiteStatus BuildOp(TfLiteContext* ctx, TfLiteNode* node, TfLiteRegistration* reg, OpRecord* op) {
    const TfLiteTensor* T = ctx->tensors;
    auto idx = [&](int i) { return i < node->inputs->size ? node->inputs->data[i] : -1; };
    op->y = node->outputs->data[0];
    switch (op->kind) {
      case OpKind::kFcInt8: {
        const auto* p = static_cast<const TfLiteFullyConnectedParams*>(node->builtin_data);
        op->x = idx(0);
        const TfLiteTensor &x = T[op->x], &w = T[idx(1)], &y = T[op->y];
        const TfLiteTensor* b = idx(2) >= 0 ? &T[idx(2)] : nullptr;
        op->n = w.dims->data[0];
        op->kdim = w.dims->data[1];
        TF_LITE_ENSURE_STATUS(PackInt8(ctx, w.data.int8, op->n, op->kdim, false, op));
        const auto* q = Affine(w);
        op->per_channel = q->scale->size > 1;
        std::vector<int32_t> mult, shift;
        if (op->per_channel) {
          mult.resize(op->n);
          shift.resize(op->n);
          for (int i = 0; i < op->n; ++i) {
            const double eff = static_cast<double>(x.params.scale) * static_cast<double>(q->scale->data[i]) /
                               static_cast<double>(y.params.scale);
            int sh;
            QuantizeMultiplier(eff, &mult[i], &sh);
            shift[i] = sh;
          }
          op->filter_offset = 0;
        } else {
          // tflite/kernels/kernel_util.cc:291-339
          if (b) {
            const double ips = static_cast<double>(x.params.scale) * static_cast<double>(w.params.scale);
            const double diff = std::abs(ips - static_cast<double>(b->params.scale));
            if (!(diff / static_cast<double>(y.params.scale) <= 0.02)) {
              TF_LITE_KERNEL_LOG(ctx, "B200 delegate: bias scale does not match input*filter scale");
              return kTfLiteError;
            }
          }
          const double ips = static_cast<double>(x.params.scale * w.params.scale);
          mult.resize(1);
          shift.resize(1);
          int sh;
          QuantizeMultiplier(ips / static_cast<double>(y.params.scale), &mult[0], &sh);
          shift[0] = sh;
          op->filter_offset = -w.params.zero_point;
        }
        TF_LITE_ENSURE_STATUS(Upload(ctx, mult, &op->mult));
        TF_LITE_ENSURE_STATUS(Upload(ctx, shift, &op->shift));
        if (b) TF_LITE_ENSURE_STATUS(UploadRaw(ctx, b->data.raw, sizeof(int32_t) * op->n, &op->bias));
        op->input_offset = -x.params.zero_point;
        op->output_offset = y.params.zero_point;
        if (!ActivationRangeInt8(p->activation, y.params.scale, y.params.zero_point, &op->act_min, &op->act_max)) {
          TF_LITE_KERNEL_LOG(ctx, "B200 delegate: activation range overflow");
          return kTfLiteError;
        }
        return kTfLiteOk;
      }
      case OpKind::kFcHybrid: {
        op->x = idx(0);
        const TfLiteTensor& w = T[idx(1)];
        const auto* p = static_cast<const TfLiteFullyConnectedParams*>(node->builtin_data);
        op->n = w.dims->data[0];
        op->kdim = w.dims->data[1];
        op->asymmetric = p->asymmetric_quantize_inputs;
        op->activation = p->activation;
        const TfLiteTensor* b = idx(2) >= 0 ? &T[idx(2)] : nullptr;
        TF_LITE_ENSURE_STATUS(PackInt8(ctx, w.data.int8, op->n, op->kdim, false, op));
        const auto* q = Affine(w);
        std::vector<float> scales;
        if (q && q->scale && q->scale->size > 1) {
          scales.assign(q->scale->data, q->scale->data + q->scale->size);
          op->per_channel = true;
        } else {
          scales.assign(1, w.params.scale);  // fully_connected.cc:838-843
          op->per_channel = false;
        }
        TF_LITE_ENSURE_STATUS(Upload(ctx, scales, &op->w_scales));
        if (b) TF_LITE_ENSURE_STATUS(UploadRaw(ctx, b->data.raw, sizeof(float) * op->n, &op->bias));
        return kTfLiteOk;
      }
      case OpKind::kBmmHybrid:
      case OpKind::kBmmInt8: {
        const auto* p = static_cast<const TfLiteBatchMatMulParams*>(node->builtin_data);
        op->x = idx(0);
        op->w = idx(1);
        const TfLiteTensor &x = T[op->x], &w = T[op->w], &y = T[op->y];
        if (!BmmShapes(x, w, p->adj_x, p->adj_y, &op->g)) return kTfLiteDelegateError;
        op->adj_x = p->adj_x;
        op->adj_y = p->adj_y;
        op->n = op->g.n;
        op->kdim = op->g.k;
        op->rhs_const = IsConst(w);
        // one right-hand matrix for every left-hand one: the leading dimensions of the LHS fold into its
        // rows (the reference's own compression, tflite/kernels/batch_matmul.cc:768-788; not with adj_x)
        op->fold_lhs = op->g.rhs_mats == 1 && !op->adj_x;
        op->packed_stride = b200_packed_w8_bytes(op->n, op->kdim);
        if (op->rhs_const) {
          // the reference transposes a constant RHS once and keeps it (batch_matmul.cc:791-798): here it is
          // transposed, uploaded and repacked once, matrix by matrix
          const size_t mat = static_cast<size_t>(op->n) * op->kdim, mats = static_cast<size_t>(op->g.rhs_mats);
          if (!op->packed.ensure(mats * op->packed_stride) || !op->row_sums.ensure(mats * sizeof(int32_t) * op->n)) {
            TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
            return kTfLiteDelegateError;
          }
          DeviceMem staging;
          std::vector<int8_t> t(mat);
          for (size_t i = 0; i < mats; ++i) {
            const int8_t* host = w.data.int8 + i * mat;
            if (!op->adj_y) {
              for (int r = 0; r < op->kdim; ++r)
                for (int c = 0; c < op->n; ++c) t[static_cast<size_t>(c) * op->kdim + r] = host[static_cast<size_t>(r) * op->n + c];
              host = t.data();
            }
            TF_LITE_ENSURE_STATUS(UploadRaw(ctx, host, mat, &staging));
            B200_OK_OR_RETURN(ctx, b200_pack_w8(static_cast<const int8_t*>(staging.ptr), op->n, op->kdim,
                                               static_cast<uint8_t*>(op->packed.ptr) + i * op->packed_stride,
                                               static_cast<int32_t*>(op->row_sums.ptr) + i * op->n, st_->stream));
            CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));  // staging and `t` are reused
          }
        }
        if (op->kind == OpKind::kBmmHybrid) {
          op->asymmetric = p->asymmetric_quantize_inputs;
          const auto* q = Affine(w);
          std::vector<float> scales;
          if (q && q->scale && q->scale->size > 1) {
            scales.assign(q->scale->data, q->scale->data + q->scale->size);
            op->per_channel = true;
          } else {
            scales.assign(1, w.params.scale);  // batch_matmul.cc:498-503
            op->per_channel = false;
          }
          TF_LITE_ENSURE_STATUS(Upload(ctx, scales, &op->w_scales));
        } else {
          // tflite/kernels/batch_matmul.cc:315-331 and 528-556
          const double ips = static_cast<double>(x.params.scale * w.params.scale);
          std::vector<int32_t> mult(1), shift(1);
          int sh;
          QuantizeMultiplier(ips / static_cast<double>(y.params.scale), &mult[0], &sh);
          shift[0] = sh;
          TF_LITE_ENSURE_STATUS(Upload(ctx, mult, &op->mult));
          TF_LITE_ENSURE_STATUS(Upload(ctx, shift, &op->shift));
          op->per_channel = false;
          op->input_offset = -x.params.zero_point;
          op->filter_offset = -w.params.zero_point;
          op->output_offset = y.params.zero_point;
          op->act_min = -128;
          op->act_max = 127;
        }
        return kTfLiteOk;
      }
      case OpKind::kFcW4: {
        op->x = idx(0);
        const TfLiteTensor& w = T[idx(1)];
        const auto* q = static_cast<const TfLiteBlockwiseQuantization*>(w.quantization.params);
        const TfLiteTensor& scale_t = T[q->scale];
        op->n = w.dims->data[0];
        op->kdim = w.dims->data[1];
        DeviceMem w_stage, s_stage;
        const size_t row_bytes = (static_cast<size_t>(op->kdim) + 1) / 2;
        TF_LITE_ENSURE_STATUS(UploadRaw(ctx, w.data.raw, row_bytes * op->n, &w_stage));
        TF_LITE_ENSURE_STATUS(UploadRaw(ctx, scale_t.data.raw, scale_t.bytes, &s_stage));
        if (!op->packed.ensure(b200_packed_w4_bytes(op->n, op->kdim)) || !op->kfsum.ensure(sizeof(float) * op->n)) {
          TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
          return kTfLiteDelegateError;
        }
        B200_OK_OR_RETURN(ctx, b200_pack_w4(static_cast<const uint8_t*>(w_stage.ptr),
                                           static_cast<const uint16_t*>(s_stage.ptr), op->n, op->kdim, q->blocksize,
                                           op->packed.ptr, static_cast<float*>(op->kfsum.ptr), st_->stream));
        if (idx(2) >= 0) TF_LITE_ENSURE_STATUS(UploadRaw(ctx, T[idx(2)].data.raw, sizeof(float) * op->n, &op->bias));
        CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));
        return kTfLiteOk;
      }
      case OpKind::kAdd:
      case OpKind::kMul: {
        const TfLiteTensor &a = T[idx(0)], &b = T[idx(1)];
        Pad4(a, op->dims_a);
        Pad4(b, op->dims_b);
        Pad4(T[op->y], op->dims_o);
        op->ins = {IsConst(a) ? -1 : idx(0), IsConst(b) ? -1 : idx(1)};
        if (IsConst(a)) TF_LITE_ENSURE_STATUS(UploadRaw(ctx, a.data.raw, a.bytes, &op->const_a));
        if (IsConst(b)) TF_LITE_ENSURE_STATUS(UploadRaw(ctx, b.data.raw, b.bytes, &op->const_b));
        return kTfLiteOk;
      }
      case OpKind::kGelu:
        op->ins = {idx(0)};
        op->approximate = static_cast<const TfLiteGeluParams*>(node->builtin_data)->approximate ? 1 : 0;
        return kTfLiteOk;
      case OpKind::kReshape:
        op->ins = {idx(0)};
        return kTfLiteOk;
      case OpKind::kSlice: {
        const TfLiteTensor &x = T[idx(0)], &b = T[idx(1)];
        op->ins = {idx(0)};
        Pad4(x, op->dims_a);
        Pad4(T[op->y], op->dims_o);
        const int r = x.dims->size;
        for (int i = 0; i < r; ++i) op->begin[4 - r + i] = b.data.i32[i];
        return kTfLiteOk;
      }
      case OpKind::kConcat: {
        const auto* p = static_cast<const TfLiteConcatenationParams*>(node->builtin_data);
        const int r = T[op->y].dims->size;
        op->axis = (p->axis < 0 ? p->axis + r : p->axis) + (4 - r);
        Pad4(T[op->y], op->dims_o);
        for (int i = 0; i < node->inputs->size; ++i) op->ins.push_back(idx(i));
        return kTfLiteOk;
      }
      case OpKind::kEmbedding: {
        const TfLiteTensor& table = T[idx(1)];
        op->ins = {idx(0)};
        op->vocab = table.dims->data[0];
        op->width = table.dims->data[1];
        op->rows = static_cast<int>(NumElements(T[idx(0)]));
        TF_LITE_ENSURE_STATUS(UploadRaw(ctx, table.data.raw, table.bytes, &op->const_a));
        const auto* q = Affine(table);
        std::vector<float> scales(op->vocab, table.params.scale);
        if (q && q->scale && q->scale->size > 1) scales.assign(q->scale->data, q->scale->data + q->scale->size);
        TF_LITE_ENSURE_STATUS(Upload(ctx, scales, &op->w_scales));
        CUDA_OK(ctx, cudaStreamSynchronize(st_->stream));
        return kTfLiteOk;
      }
      case OpKind::kArgMax: {
        const TfLiteTensor& x = T[idx(0)];
        op->ins = {idx(0)};
        op->width = x.dims->data[x.dims->size - 1];
        op->rows = static_cast<int>(NumElements(x) / op->width);
        op->out_i64 = T[op->y].type == kTfLiteInt64;
        if (!op->ws_small.ensure(b200_argmax_workspace_bytes(op->rows) + sizeof(int32_t) * op->rows)) {
          TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed");
          return kTfLiteDelegateError;
        }
        return kTfLiteOk;
      }
      case OpKind::kRmsNorm: {
        const TfLiteTensor& x = T[idx(0)];
        op->ins = {idx(0)};
        op->width = x.dims->data[x.dims->size - 1];
        op->rows = static_cast<int>(NumElements(x) / op->width);
        if (idx(1) >= 0) TF_LITE_ENSURE_STATUS(UploadRaw(ctx, T[idx(1)].data.raw, T[idx(1)].bytes, &op->const_a));
        const auto* p = static_cast<const TfLiteStablehloCompositeParams*>(node->builtin_data);
        float eps = 1e-6f;
        b200::FlexMapFloat(p->attributes, p->attributes_size, "epsilon", &eps);
        op->eps = eps;
        return kTfLiteOk;
      }
      case OpKind::kKvCache: {
        const TfLiteTensor& k = T[idx(1)];
        op->ins = {idx(0), idx(1), idx(2)};
        op->y2 = node->outputs->data[1];
        op->rows = k.dims->data[1];                       // new tokens per invocation
        op->width = k.dims->data[2] * k.dims->data[3];    // elements per cached token
        op->max_entries = T[op->y].dims->data[1];
        const size_t bytes = sizeof(float) * static_cast<size_t>(op->max_entries) * op->width;
        if (!op->k_cache.ensure(bytes) || !op->v_cache.ensure(bytes)) {
          TF_LITE_KERNEL_LOG(ctx, "B200 delegate: device allocation failed (kv cache)");
          return kTfLiteDelegateError;
        }
        // a fresh cache holds zeros, like resource::CacheBuffer::Initialize
        CUDA_OK(ctx, cudaMemsetAsync(op->k_cache.ptr, 0, bytes, st_->stream));
        CUDA_OK(ctx, cudaMemsetAsync(op->v_cache.ptr, 0, bytes, st_->stream));
        return kTfLiteOk;
      }
      case OpKind::kSdpa: {
        op->q = idx(0);
        op->k = idx(1);
        op->v = idx(2);
        op->mask = node->inputs->size > 3 ? idx(3) : -1;
        const TfLiteTensor &q = T[op->q], &k = T[op->k];
        op->B = q.dims->data[0];
        op->T = q.dims->data[1];
        op->sdpa_dtype = q.type == kTfLiteFloat16 ? B200_DTYPE_F16 : B200_DTYPE_F32;
        op->N = q.dims->data[2];
        op->H = q.dims->data[3];
        op->S = k.dims->data[1];
        op->Nkv = k.dims->data[2];
        const uint8_t* attr = nullptr;
        size_t attr_size = 0;
        if (reg->builtin_code == kTfLiteBuiltinStablehloComposite) {
          const auto* p = static_cast<const TfLiteStablehloCompositeParams*>(node->builtin_data);
          attr = p->attributes;
          attr_size = p->attributes_size;
        } else {
          attr = static_cast<const uint8_t*>(node->custom_initial_data);
          attr_size = static_cast<size_t>(node->custom_initial_data_size);
        }
        float scale = 0.0f, cap = 0.0f;
        b200::FlexMapFloat(attr, attr_size, "scale", &scale);
        b200::FlexMapFloat(attr, attr_size, "logit_cap", &cap);
        op->scale = scale;  // <= 0 or absent: 1/sqrt(H), tflite/experimental/genai/sdpa.cc:99-105
        op->logit_cap = cap;
        return kTfLiteOk;
      }
      default:
        return kTfLiteDelegateError;
    }
  }

  TfLiteStatus Launch(TfLiteContext* ctx, OpRecord& op) {
    cudaStream_t s = st_->stream;
    switch (op.kind) {
      case OpKind::kFcInt8:
        B200_OK_OR_RETURN(ctx, b200_fc_int8(static_cast<const int8_t*>(Dev(op.x)), op.m, op.kdim, op.packed.ptr, op.n,
                                           static_cast<const int32_t*>(op.row_sums.ptr),
                                           static_cast<const int32_t*>(op.bias.ptr), op.input_offset, op.filter_offset,
                                           op.output_offset, static_cast<const int32_t*>(op.mult.ptr),
                                           static_cast<const int32_t*>(op.shift.ptr), op.per_channel ? 1 : 0,
                                           op.act_min, op.act_max, static_cast<int8_t*>(Dev(op.y)), st_->zero_ws.ptr,
                                           st_->scratch.ptr, st_->scratch.bytes, s));
        return kTfLiteOk;
      case OpKind::kFcHybrid:
        B200_OK_OR_RETURN(ctx, b200_fc_hybrid(static_cast<const float*>(Dev(op.x)), op.m, op.kdim, op.packed.ptr, op.n,
                                             static_cast<const int32_t*>(op.row_sums.ptr),
                                             static_cast<const float*>(op.w_scales.ptr), op.per_channel ? 1 : 0,
                                             static_cast<const float*>(op.bias.ptr), op.asymmetric ? 1 : 0,
                                             op.activation, static_cast<float*>(Dev(op.y)), st_->zero_ws.ptr,
                                             st_->scratch.ptr, st_->scratch.bytes, s));
        return kTfLiteOk;
      case OpKind::kBmmHybrid:
      case OpKind::kBmmInt8:
        return LaunchBmm(ctx, op);
      case OpKind::kFcW4:
        B200_OK_OR_RETURN(ctx, b200_fc_w4(static_cast<const float*>(Dev(op.x)), op.m, op.kdim, op.packed.ptr, op.n, 32,
                                         static_cast<const float*>(op.kfsum.ptr),
                                         static_cast<const float*>(op.bias.ptr), static_cast<float*>(Dev(op.y)),
                                         st_->zero_ws.ptr, st_->scratch.ptr, st_->scratch.bytes, s));
        return kTfLiteOk;
      case OpKind::kAdd:
      case OpKind::kMul: {
        const float* a = op.ins[0] < 0 ? static_cast<const float*>(op.const_a.ptr) : static_cast<const float*>(Dev(op.ins[0]));
        const float* b = op.ins[1] < 0 ? static_cast<const float*>(op.const_b.ptr) : static_cast<const float*>(Dev(op.ins[1]));
        B200_EW_OR_RETURN(ctx, b200_binary_f32(op.kind == OpKind::kAdd ? 0 : 1, a, op.dims_a, b, op.dims_b,
                                              static_cast<float*>(Dev(op.y)), op.dims_o, s));
        return kTfLiteOk;
      }
      case OpKind::kGelu:
        B200_EW_OR_RETURN(ctx, b200_gelu_f32(static_cast<const float*>(Dev(op.ins[0])), static_cast<float*>(Dev(op.y)),
                                            static_cast<size_t>(NumElements(ctx->tensors[op.y])), op.approximate, s));
        return kTfLiteOk;
      case OpKind::kReshape:
        if (Dev(op.y) != Dev(op.ins[0]))
          CUDA_OK(ctx, cudaMemcpyAsync(Dev(op.y), Dev(op.ins[0]), ctx->tensors[op.y].bytes, cudaMemcpyDeviceToDevice, s));
        return kTfLiteOk;
      case OpKind::kSlice: {
        const int zero[4] = {0, 0, 0, 0};
        B200_EW_OR_RETURN(ctx, b200_box_copy(Dev(op.ins[0]), op.dims_a, op.begin, Dev(op.y), op.dims_o, zero, op.dims_o, 4, s));
        return kTfLiteOk;
      }
      case OpKind::kConcat: {
        int at[4] = {0, 0, 0, 0};
        const int zero[4] = {0, 0, 0, 0};
        for (int t : op.ins) {
          int d[4];
          Pad4(ctx->tensors[t], d);
          B200_EW_OR_RETURN(ctx, b200_box_copy(Dev(t), d, zero, Dev(op.y), op.dims_o, at, d, 4, s));
          at[op.axis] += d[op.axis];
        }
        return kTfLiteOk;
      }
      case OpKind::kEmbedding:
        B200_GLUE_OR_RETURN(ctx, b200_embedding_lookup(static_cast<const int32_t*>(Dev(op.ins[0])), op.rows,
                                                      static_cast<const int8_t*>(op.const_a.ptr),
                                                      static_cast<const float*>(op.w_scales.ptr), op.vocab, op.width, 1.0f,
                                                      static_cast<float*>(Dev(op.y)), s));
        return kTfLiteOk;
      case OpKind::kArgMax: {
        uint8_t* ws = static_cast<uint8_t*>(op.ws_small.ptr);
        const size_t ws_bytes = b200_argmax_workspace_bytes(op.rows);
        int32_t* out32 = op.out_i64 ? reinterpret_cast<int32_t*>(ws + ws_bytes) : static_cast<int32_t*>(Dev(op.y));
        B200_GLUE_OR_RETURN(ctx, b200_argmax_rows(static_cast<const float*>(Dev(op.ins[0])), op.rows, op.width, 0.0f, out32, ws,
                                                 ws_bytes, s));
        if (op.out_i64) B200_EW_OR_RETURN(ctx, b200_widen_i32_to_i64(out32, static_cast<int64_t*>(Dev(op.y)), op.rows, s));
        return kTfLiteOk;
      }
      case OpKind::kRmsNorm:
        B200_EW_OR_RETURN(ctx, b200_rms_norm_f32(static_cast<const float*>(Dev(op.ins[0])), static_cast<const float*>(op.const_a.ptr),
                                                static_cast<float*>(Dev(op.y)), op.rows, op.width, op.eps, s));
        return kTfLiteOk;
      case OpKind::kKvCache:
        B200_EW_OR_RETURN(ctx, b200_kv_cache_update_f32(static_cast<const int64_t*>(Dev(op.ins[0])),
                                                       static_cast<const float*>(Dev(op.ins[1])),
                                                       static_cast<const float*>(Dev(op.ins[2])), op.rows, op.width,
                                                       op.max_entries, static_cast<float*>(op.k_cache.ptr),
                                                       static_cast<float*>(op.v_cache.ptr), st_->zero_ws.ptr, s));
        return kTfLiteOk;
      case OpKind::kRopeKv:
        B200_EW_OR_RETURN(ctx, b200_rope_kv_cache_update_f32(
                                   static_cast<const int64_t*>(Dev(op.ins[0])), static_cast<const float*>(Dev(op.ins[5])),
                                   static_cast<const float*>(Dev(op.ins[1])), static_cast<const float*>(Dev(op.ins[2])),
                                   static_cast<const float*>(Dev(op.ins[3])), static_cast<const float*>(Dev(op.ins[4])),
                                   static_cast<float*>(Dev(op.ins[6])), op.rows, op.heads, op.B, op.H, op.max_entries,
                                   static_cast<float*>(op.k_cache.ptr), static_cast<float*>(op.v_cache.ptr), st_->zero_ws.ptr, s));
        return kTfLiteOk;
      case OpKind::kSkipped:
        return kTfLiteOk;
      case OpKind::kRope:
        B200_EW_OR_RETURN(ctx, b200_rope_f32(static_cast<const float*>(Dev(op.ins[0])), static_cast<const float*>(Dev(op.ins[1])),
                                            static_cast<const float*>(Dev(op.ins[2])), static_cast<float*>(Dev(op.y)), op.rows,
                                            op.heads, op.width, s));
        return kTfLiteOk;
      case OpKind::kNormQuant:
        // (with a second operand: the residual ADD in front of the norm, h += delta in place)
        B200_GLUE_OR_RETURN(ctx, b200_add_rmsnorm_quantize(static_cast<float*>(Dev(op.ins[0])),
                                                          op.ins.size() > 1 ? static_cast<const float*>(Dev(op.ins[1])) : nullptr,
                                                          static_cast<const float*>(op.const_a.ptr), op.rows, op.width, op.eps,
                                                          static_cast<int8_t*>(op.q_tiled.ptr), static_cast<float*>(op.q_scales.ptr),
                                                          static_cast<int32_t*>(op.q_zps.ptr), s));
        return kTfLiteOk;
      case OpKind::kFcQuantized: {
        const OpRecord& src = *ops_[op.rows_from];
        B200_GLUE_OR_RETURN(ctx, b200_fc_hybrid_quantized(static_cast<const int8_t*>(src.q_tiled.ptr),
                                                         static_cast<const float*>(src.q_scales.ptr),
                                                         static_cast<const int32_t*>(src.q_zps.ptr), op.m, op.kdim, op.packed.ptr,
                                                         op.n, static_cast<const int32_t*>(op.row_sums.ptr),
                                                         static_cast<const float*>(op.w_scales.ptr), op.per_channel ? 1 : 0,
                                                         static_cast<const float*>(op.bias.ptr), op.activation,
                                                         static_cast<float*>(Dev(op.y)), st_->zero_ws.ptr, s));
        return kTfLiteOk;
      }
      case OpKind::kFcGroup: {
        const OpRecord& src = *ops_[op.rows_from];
        B200_GLUE_OR_RETURN(ctx, b200_fc_hybrid_quantized(static_cast<const int8_t*>(src.q_tiled.ptr),
                                                         static_cast<const float*>(src.q_scales.ptr),
                                                         static_cast<const int32_t*>(src.q_zps.ptr), 1, op.kdim, op.packed.ptr, op.n,
                                                         static_cast<const int32_t*>(op.row_sums.ptr),
                                                         static_cast<const float*>(op.w_scales.ptr), 1, nullptr, 0,
                                                         static_cast<float*>(op.tmp_f32.ptr), st_->zero_ws.ptr, s));
        return kTfLiteOk;
      }
      case OpKind::kLmHeadPick: {
        const OpRecord& src = *ops_[op.rows_from];
        uint8_t* ws = static_cast<uint8_t*>(op.ws_small.ptr);
        const size_t ws_bytes = b200_lm_head_workspace_bytes(op.m);
        int32_t* out32 = op.out_i64 ? reinterpret_cast<int32_t*>(ws + ws_bytes) : static_cast<int32_t*>(Dev(op.y));
        B200_GLUE_OR_RETURN(ctx, b200_lm_head_greedy(static_cast<const int8_t*>(src.q_tiled.ptr),
                                                    static_cast<const float*>(src.q_scales.ptr),
                                                    static_cast<const int32_t*>(src.q_zps.ptr), op.m, op.kdim, op.packed.ptr, op.n,
                                                    static_cast<const int32_t*>(op.row_sums.ptr),
                                                    static_cast<const float*>(op.w_scales.ptr), 0.0f, nullptr, out32, ws, ws_bytes,
                                                    st_->zero_ws.ptr, s));
        if (op.out_i64) B200_EW_OR_RETURN(ctx, b200_widen_i32_to_i64(out32, static_cast<int64_t*>(Dev(op.y)), op.m, s));
        return kTfLiteOk;
      }
      case OpKind::kGateUpGeglu: {
        const OpRecord& src = *ops_[op.rows_from];
        B200_GLUE_OR_RETURN(ctx, b200_fc_hybrid_quantized(static_cast<const int8_t*>(src.q_tiled.ptr),
                                                         static_cast<const float*>(src.q_scales.ptr),
                                                         static_cast<const int32_t*>(src.q_zps.ptr), op.m, op.kdim, op.packed.ptr,
                                                         op.n, static_cast<const int32_t*>(op.row_sums.ptr),
                                                         static_cast<const float*>(op.w_scales.ptr), 1, nullptr, 0,
                                                         static_cast<float*>(op.tmp_f32.ptr), st_->zero_ws.ptr, s));
        B200_GLUE_OR_RETURN(ctx, b200_geglu_quantize(static_cast<const float*>(op.tmp_f32.ptr), op.m, op.n / 2,
                                                    static_cast<int8_t*>(op.q_tiled.ptr), static_cast<float*>(op.q_scales.ptr),
                                                    static_cast<int32_t*>(op.q_zps.ptr), s));
        return kTfLiteOk;
      }
      case OpKind::kSdpaQuant:
        B200_GLUE_OR_RETURN(ctx, b200_sdpa_decode_quantized_masked(
                                     Dev(op.q), Dev(op.k), Dev(op.v), nullptr, nullptr, nullptr,
                                     op.mask >= 0 ? static_cast<const float*>(Dev(op.mask)) : nullptr, op.B, op.N, op.Nkv, op.H,
                                     op.S, op.sdpa_dtype, op.sdpa_dtype, op.scale, op.logit_cap,
                                     static_cast<int8_t*>(op.q_tiled.ptr), static_cast<float*>(op.q_scales.ptr),
                                     static_cast<int32_t*>(op.q_zps.ptr), st_->sdpa_ws.ptr, st_->sdpa_ws.bytes, s));
        return kTfLiteOk;
      case OpKind::kSdpa:
        if (op.T == 1) {
          B200_OK_OR_RETURN(ctx, b200_sdpa_decode(Dev(op.q), Dev(op.k), Dev(op.v), nullptr, nullptr, nullptr,
                                                 op.mask >= 0 ? static_cast<const float*>(Dev(op.mask)) : nullptr,
                                                 Dev(op.y), op.B, op.N, op.Nkv, op.H, op.S, op.sdpa_dtype,
                                                 op.sdpa_dtype, op.scale, op.logit_cap, st_->sdpa_ws.ptr,
                                                 st_->sdpa_ws.bytes, s));
        } else {
          // several query tokens per sequence (a prompt pass): every (sequence, token) pair is one row
          B200_OK_OR_RETURN(ctx, b200_sdpa(Dev(op.q), Dev(op.k), Dev(op.v),
                                          op.mask >= 0 ? static_cast<const float*>(Dev(op.mask)) : nullptr, Dev(op.y),
                                          op.B, op.T, op.N, op.Nkv, op.H, op.S, op.sdpa_dtype, op.sdpa_dtype, op.scale,
                                          op.logit_cap, st_->sdpa_ws.ptr, st_->sdpa_ws.bytes, s));
        }
        return kTfLiteOk;
      default:
        return kTfLiteDelegateError;
    }
  }

  // One BATCH_MATMUL: operands brought to [.., m, k] and packed [n, k] form (transposes as the reference's
  // TransposeRowsColumns, a run-time RHS repacked every invocation), then one product per output matrix
  // with the reference's broadcast rule (tflite/kernels/internal/reference/batch_matmul.h:30-51).
  TfLiteStatus LaunchBmm(TfLiteContext* ctx, OpRecord& op) {
    cudaStream_t s = st_->stream;
    const BmmGeometry& g = op.g;
    const bool hybrid = op.kind == OpKind::kBmmHybrid;
    const size_t elem = hybrid ? sizeof(float) : 1;
    const uint8_t* lhs = static_cast<const uint8_t*>(Dev(op.x));
    if (op.adj_x) {
      B200_GLUE_OR_RETURN(ctx, b200_transpose_matrices(lhs, st_->bmm_lhs.ptr, g.lhs_mats, g.k, g.m, static_cast<int>(elem), s));
      lhs = static_cast<const uint8_t*>(st_->bmm_lhs.ptr);
    }
    const uint8_t* packed = static_cast<const uint8_t*>(op.packed.ptr);
    const int32_t* row_sums = static_cast<const int32_t*>(op.row_sums.ptr);
    if (!op.rhs_const) {
      const int8_t* rhs = static_cast<const int8_t*>(Dev(op.w));
      if (!op.adj_y) {
        B200_GLUE_OR_RETURN(ctx, b200_transpose_matrices(rhs, st_->bmm_rhs.ptr, g.rhs_mats, g.k, g.n, 1, s));
        rhs = static_cast<const int8_t*>(st_->bmm_rhs.ptr);
      }
      for (int i = 0; i < g.rhs_mats; ++i)
        B200_OK_OR_RETURN(ctx, b200_pack_w8(rhs + static_cast<size_t>(i) * op.n * op.kdim, op.n, op.kdim,
                                           static_cast<uint8_t*>(st_->bmm_packed.ptr) + i * op.packed_stride,
                                           static_cast<int32_t*>(st_->bmm_row_sums.ptr) + static_cast<size_t>(i) * op.n, s));
      packed = static_cast<const uint8_t*>(st_->bmm_packed.ptr);
      row_sums = static_cast<const int32_t*>(st_->bmm_row_sums.ptr);
    }
    uint8_t* out = static_cast<uint8_t*>(Dev(op.y));
    const int products = op.fold_lhs ? 1 : g.out_mats;
    for (int o = 0; o < products; ++o) {
      int li = 0, ri = 0;
      if (!op.fold_lhs) {
        const int b2 = o % g.out_batch[2], b1 = (o / g.out_batch[2]) % g.out_batch[1], b0 = o / (g.out_batch[2] * g.out_batch[1]);
        const int b[3] = {b0, b1, b2};
        for (int d = 0; d < 3; ++d) {
          li = li * g.lhs_batch[d] + (g.lhs_batch[d] == 1 ? 0 : b[d]);
          ri = ri * g.rhs_batch[d] + (g.rhs_batch[d] == 1 ? 0 : b[d]);
        }
      }
      const uint8_t* x = lhs + static_cast<size_t>(li) * g.m * g.k * elem;
      const uint8_t* w = packed + static_cast<size_t>(ri) * op.packed_stride;
      const int32_t* rs = row_sums + static_cast<size_t>(ri) * op.n;
      uint8_t* y = out + static_cast<size_t>(o) * g.m * g.n * elem;
      if (hybrid) {
        B200_OK_OR_RETURN(ctx, b200_bmm_hybrid(reinterpret_cast<const float*>(x), op.m, op.kdim, w, op.n, rs,
                                              static_cast<const float*>(op.w_scales.ptr), op.per_channel ? 1 : 0,
                                              op.asymmetric ? 1 : 0, reinterpret_cast<float*>(y), st_->zero_ws.ptr,
                                              st_->scratch.ptr, st_->scratch.bytes, s));
      } else {
        B200_OK_OR_RETURN(ctx, b200_fc_int8(reinterpret_cast<const int8_t*>(x), op.m, op.kdim, w, op.n, rs, nullptr,
                                           op.input_offset, op.filter_offset, op.output_offset,
                                           static_cast<const int32_t*>(op.mult.ptr), static_cast<const int32_t*>(op.shift.ptr),
                                           0, op.act_min, op.act_max, reinterpret_cast<int8_t*>(y), st_->zero_ws.ptr,
                                           st_->scratch.ptr, st_->scratch.bytes, s));
      }
    }
    return kTfLiteOk;
  }

  DelegateState* st_;
  b200::DeviceArena arena_;
  std::vector<int> inputs_, outputs_;
  std::vector<std::unique_ptr<OpRecord>> ops_;
  std::unordered_map<int, int> slot_of_;
  std::unordered_map<int, int> inplace_alias_; // residual sums a fused norm computes in place -> the stream's tensor
  std::unordered_map<int, int> alias_;         // RESHAPE results -> the tensor whose buffer they share
  std::unordered_map<int, void*> persistent_;  // tensors that live outside the arena (the kv-cache op's outputs)
  cudaGraphExec_t graph_exec_ = nullptr;
  bool graph_failed_ = false;
  long long invocations_ = 0;

 public:
  ~DelegateKernel() {
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
  }
};

// ---------------------------------------------------------------- registration glue
void* KernelInit(TfLiteContext* ctx, const char* buffer, size_t) {
  const auto* params = reinterpret_cast<const TfLiteDelegateParams*>(buffer);
  if (!params || !params->delegate) return nullptr;
  auto* st = static_cast<DelegateState*>(params->delegate->data_);
  auto* kernel = new DelegateKernel(st);
  if (kernel->Init(ctx, params) != kTfLiteOk) {
    delete kernel;
    return TfLiteKernelInitFailed();
  }
  return kernel;
}

void KernelFree(TfLiteContext*, void* buffer) {
  if (buffer && buffer != TfLiteKernelInitFailed()) delete static_cast<DelegateKernel*>(buffer);
}

TfLiteStatus KernelPrepare(TfLiteContext* ctx, TfLiteNode* node) {
  if (!node->user_data || node->user_data == TfLiteKernelInitFailed()) return kTfLiteDelegateError;
  return static_cast<DelegateKernel*>(node->user_data)->Prepare(ctx, node);
}

TfLiteStatus KernelInvoke(TfLiteContext* ctx, TfLiteNode* node) {
  if (!node->user_data || node->user_data == TfLiteKernelInitFailed()) return kTfLiteDelegateError;
  return static_cast<DelegateKernel*>(node->user_data)->Invoke(ctx, node);
}

// tflite::delegates::MarkSubgraphAsDelegationSkippable(const TfLiteContext*, int)
// (tflite/delegates/utils.h:62-93) lives in the runtime, not in TfLiteContext's table of function
// pointers: a plugin finds it among the symbols of the process that loaded it, and goes without when
// the runtime does not export it (the composite's decomposition subgraph is then merely unused, as with
// XNNPACK).
using MarkSkippableFn = TfLiteStatus (*)(const TfLiteContext*, int);
MarkSkippableFn FindMarkSkippable() {
  static MarkSkippableFn fn = reinterpret_cast<MarkSkippableFn>(
      dlsym(RTLD_DEFAULT, "_ZN6tflite9delegates33MarkSubgraphAsDelegationSkippableEPK13TfLiteContexti"));
  return fn;
}

TfLiteStatus DelegatePrepare(TfLiteContext* ctx, TfLiteDelegate* delegate) {
  auto* st = static_cast<DelegateState*>(delegate->data_);
  TfLiteIntArray* plan = nullptr;
  TF_LITE_ENSURE_STATUS(ctx->GetExecutionPlan(ctx, &plan));
  // the plan array belongs to the runtime and is invalidated by the next call: copy it
  std::vector<int> nodes(plan->data, plan->data + plan->size);
  std::vector<int> supported;
  for (int node_index : nodes) {
    TfLiteNode* node = nullptr;
    TfLiteRegistration* reg = nullptr;
    TF_LITE_ENSURE_STATUS(ctx->GetNodeAndRegistration(ctx, node_index, &node, &reg));
    std::string why;
    if (Classify(ctx, node, reg, st->options, &why) == OpKind::kNone) continue;
    supported.push_back(node_index);
    // a claimed composite carries its decomposition as another subgraph: tell the runtime that this
    // delegate has taken care of it, so that it is not delegated on its own
    if (reg->builtin_code == kTfLiteBuiltinStablehloComposite) {
      const auto* p = static_cast<const TfLiteStablehloCompositeParams*>(node->builtin_data);
      if (MarkSkippableFn mark = FindMarkSkippable()) {
        if (p && p->subgraph_index > 0 && mark(ctx, p->subgraph_index) == kTfLiteOk) ++st->skippable_marked;
      }
    }
  }
  st->delegated_nodes = static_cast<int>(supported.size());
  if (supported.empty()) return kTfLiteOk;  // nothing to claim is not an error
  TfLiteRegistration reg;
  memset(&reg, 0, sizeof(reg));
  reg.init = KernelInit;
  reg.free = KernelFree;
  reg.prepare = KernelPrepare;
  reg.invoke = KernelInvoke;
  reg.builtin_code = kTfLiteBuiltinDelegate;
  reg.custom_name = kDelegateName;
  reg.version = 1;
  TfLiteIntArray* arr = TfLiteIntArrayCreate(static_cast<int>(supported.size()));
  for (size_t i = 0; i < supported.size(); ++i) arr->data[i] = supported[i];
  const TfLiteStatus status = ctx->ReplaceNodeSubsetsWithDelegateKernels(ctx, reg, arr, delegate);
  TfLiteIntArrayFree(arr);
  return status;
}

TfLiteStatus CopyFromBufferHandle(TfLiteContext* ctx, TfLiteDelegate* delegate, TfLiteBufferHandle handle,
                                  TfLiteTensor* tensor) {
  auto* st = static_cast<DelegateState*>(delegate->data_);
  auto it = st->handles.find(handle);
  if (it == st->handles.end() || !tensor->data.raw) {
    TF_LITE_KERNEL_LOG(ctx, "B200 delegate: unknown buffer handle %d", handle);
    return kTfLiteDelegateError;
  }
  CUDA_OK(ctx, cudaSetDevice(st->options.device));
  const size_t bytes = std::min(it->second.second, tensor->bytes);
  CUDA_OK(ctx, cudaMemcpyAsync(tensor->data.raw, it->second.first, bytes, cudaMemcpyDeviceToHost, st->stream));
  CUDA_OK(ctx, cudaStreamSynchronize(st->stream));
  return kTfLiteOk;
}

void FreeBufferHandle(TfLiteContext*, TfLiteDelegate* delegate, TfLiteBufferHandle* handle) {
  auto* st = static_cast<DelegateState*>(delegate->data_);
  if (handle && *handle != kTfLiteNullBufferHandle) {
    st->handles.erase(*handle);
    *handle = kTfLiteNullBufferHandle;
  }
}

bool ParseBool(const char* v) { return v && (!strcmp(v, "1") || !strcmp(v, "true") || !strcmp(v, "TRUE")); }

}  // namespace

extern "C" {

TfLiteDelegate* tflite_plugin_create_delegate(const char* const* keys, const char* const* values, size_t num_options,
                                              void (*report_error)(const char*)) {
  auto st = std::make_unique<DelegateState>();
  char msg[256];
  for (size_t i = 0; i < num_options; ++i) {
    const char* k = keys ? keys[i] : nullptr;
    const char* v = values ? values[i] : nullptr;
    if (!k || !v) continue;
    if (!strcmp(k, "device")) {
      st->options.device = atoi(v);
    } else if (!strcmp(k, "fail_on")) {
      st->options.fail_on = v;
      if (st->options.fail_on == "create") {
        if (report_error) report_error("B200 delegate: injected failure in create");
        return nullptr;
      }
    } else if (!strcmp(k, "buffer_handles")) {
      st->options.buffer_handles = ParseBool(v);
    } else if (!strcmp(k, "claim_fc")) {
      st->options.claim_fc = ParseBool(v);
    } else if (!strcmp(k, "claim_bmm")) {
      st->options.claim_bmm = ParseBool(v);
    } else if (!strcmp(k, "claim_sdpa")) {
      st->options.claim_sdpa = ParseBool(v);
    } else if (!strcmp(k, "fuse")) {
      st->options.fuse = ParseBool(v);
    } else if (!strcmp(k, "cuda_graph")) {
      st->options.cuda_graph = ParseBool(v);
    } else if (!strcmp(k, "claim_glue")) {
      st->options.claim_glue = ParseBool(v);
    } else {
      snprintf(msg, sizeof(msg), "B200 delegate: unknown option '%s'", k);
      if (report_error) report_error(msg);
      return nullptr;
    }
  }
  if (st->options.device < 0) {
    if (report_error) report_error("B200 delegate: negative device index");
    return nullptr;
  }
  memset(&st->delegate, 0, sizeof(st->delegate));
  st->delegate.data_ = st.get();
  st->delegate.Prepare = DelegatePrepare;
  st->delegate.CopyFromBufferHandle = CopyFromBufferHandle;
  st->delegate.CopyToBufferHandle = nullptr;
  st->delegate.FreeBufferHandle = FreeBufferHandle;
  st->delegate.flags = kTfLiteDelegateFlagsNone;  // static shapes only
  st->delegate.opaque_delegate_builder = nullptr;
  return &st.release()->delegate;
}

void tflite_plugin_destroy_delegate(TfLiteDelegate* delegate) {
  if (!delegate) return;
  auto* st = static_cast<DelegateState*>(delegate->data_);
  if (st->ready) {
    cudaSetDevice(st->options.device);
    if (st->stream) {
      cudaStreamSynchronize(st->stream);
      cudaStreamDestroy(st->stream);
    }
  }
  delete st;
}

size_t b200_arena_plan(int n, const size_t* bytes, const int* first_use, const int* last_use, int num_ops,
                       size_t* offsets) {
  std::vector<b200::ArenaRequest> req(n > 0 ? n : 0);
  for (int i = 0; i < n; ++i) {
    req[i].bytes = bytes[i];
    req[i].first_use = first_use[i];
    req[i].last_use = last_use[i];
  }
  std::vector<size_t> off;
  const size_t total = b200::PlanArena(req, num_ops, &off);
  for (int i = 0; i < n; ++i) offsets[i] = off[i];
  return total;
}

int b200_delegate_num_skippable_subgraphs(const TfLiteDelegate* delegate) {
  return delegate ? static_cast<const DelegateState*>(delegate->data_)->skippable_marked : -1;
}

int b200_delegate_num_claimed_nodes(const TfLiteDelegate* delegate) {
  return delegate ? static_cast<const DelegateState*>(delegate->data_)->delegated_nodes : -1;
}

}  // extern "C"
