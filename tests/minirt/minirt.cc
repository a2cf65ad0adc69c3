// Mini runtime for delegate tests. TEST INFRASTRUCTURE ONLY.
//
// The reference interpreter cannot be built offline (it needs flatbuffers and
// abseil), so this file provides the small part of it a delegate talks to,
// over the reference's real C structs (tflite/core/c/common.h): a TfLiteContext
// with GetExecutionPlan / GetNodeAndRegistration /
// ReplaceNodeSubsetsWithDelegateKernels / ReportError, graph construction by
// hand, and the apply / prepare / invoke sequence of
// Subgraph::ModifyGraphWithDelegateImpl (tflite/core/subgraph.cc:2497-2622)
// and Subgraph::InvokeImpl (:1666-1811), including roll-back to the original
// plan when the delegate fails and CopyFromBufferHandle for stale tensors.
// Nodes that stay on the "CPU" are run by a callback the test provides (it
// calls the oracle); without a callback invoking them is an error.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include <dlfcn.h>

#include "litert/c/internal/litert_accelerator_def.h"
#include "tflite/builtin_ops.h"
#include "tflite/core/c/builtin_op_data.h"
#include "tflite/core/c/common.h"

namespace {

struct NodeRec {
  TfLiteNode node;
  TfLiteRegistration reg;
  std::string custom_name;
  std::string composite_name;
  std::vector<uint8_t> blob;  // attributes / custom initial data
  bool is_delegate = false;
};

typedef int (*CpuCallback)(int node_index);

struct Graph {
  TfLiteContext ctx;
  std::vector<TfLiteTensor> tensors;
  std::vector<std::unique_ptr<NodeRec>> nodes;
  std::vector<int> plan, original_plan;
  std::vector<int> graph_inputs, graph_outputs;
  TfLiteIntArray* plan_array = nullptr;
  std::string error;
  TfLiteDelegate* delegate = nullptr;
  CpuCallback cpu = nullptr;
  int partitions = 0;
  bool replace_called = false;
  std::vector<int> skippable_subgraphs;  // marked by the delegate (MarkSubgraphAsDelegationSkippable)
};

Graph* G(TfLiteContext* ctx) { return static_cast<Graph*>(ctx->impl_); }

void ReportError(TfLiteContext* ctx, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  Graph* g = G(ctx);
  if (!g->error.empty()) g->error += "\n";
  g->error += buf;
}

TfLiteIntArray* MakeArray(const std::vector<int>& v) {
  TfLiteIntArray* a = TfLiteIntArrayCreate(static_cast<int>(v.size()));
  for (size_t i = 0; i < v.size(); ++i) a->data[i] = v[i];
  return a;
}

TfLiteStatus GetExecutionPlan(TfLiteContext* ctx, TfLiteIntArray** plan) {
  Graph* g = G(ctx);
  if (g->plan_array) TfLiteIntArrayFree(g->plan_array);  // invalidated by the next call, as documented
  g->plan_array = MakeArray(g->plan);
  *plan = g->plan_array;
  return kTfLiteOk;
}

TfLiteStatus GetNodeAndRegistration(TfLiteContext* ctx, int node_index, TfLiteNode** node,
                                    TfLiteRegistration** reg) {
  Graph* g = G(ctx);
  if (node_index < 0 || node_index >= static_cast<int>(g->nodes.size())) return kTfLiteError;
  *node = &g->nodes[node_index]->node;
  *reg = &g->nodes[node_index]->reg;
  return kTfLiteOk;
}

bool Contains(const TfLiteIntArray* a, int v) {
  for (int i = 0; i < a->size; ++i)
    if (a->data[i] == v) return true;
  return false;
}

void FreeNode(Graph* g, NodeRec* n) {
  if (n->is_delegate && n->reg.free && n->node.user_data) n->reg.free(&g->ctx, n->node.user_data);
  if (n->node.inputs) TfLiteIntArrayFree(n->node.inputs);
  if (n->node.outputs) TfLiteIntArrayFree(n->node.outputs);
  if (n->node.temporaries) TfLiteIntArrayFree(n->node.temporaries);
  if (n->node.intermediates) TfLiteIntArrayFree(n->node.intermediates);
  if (n->is_delegate && n->node.builtin_data) {
    auto* p = static_cast<TfLiteDelegateParams*>(n->node.builtin_data);
    TfLiteIntArrayFree(p->nodes_to_replace);
    TfLiteIntArrayFree(p->input_tensors);
    TfLiteIntArrayFree(p->output_tensors);
    free(p);
  } else if (n->node.builtin_data) {
    free(n->node.builtin_data);
  }
  n->node = TfLiteNode{};
}

// Partition = maximal run of consecutive plan entries that are all claimed: a
// run of a topological order has no dependency through an outside node.
TfLiteStatus ReplaceNodeSubsets(TfLiteContext* ctx, TfLiteRegistration reg, const TfLiteIntArray* to_replace,
                                TfLiteDelegate* delegate) {
  Graph* g = G(ctx);
  g->replace_called = true;
  std::vector<int> new_plan;
  size_t i = 0;
  while (i < g->plan.size()) {
    if (!Contains(to_replace, g->plan[i])) {
      new_plan.push_back(g->plan[i]);
      ++i;
      continue;
    }
    std::vector<int> subset;
    while (i < g->plan.size() && Contains(to_replace, g->plan[i])) subset.push_back(g->plan[i++]);
    // boundary tensors
    std::vector<int> produced, ins, outs;
    auto has = [](const std::vector<int>& v, int x) {
      for (int e : v)
        if (e == x) return true;
      return false;
    };
    for (int n : subset) {
      const TfLiteNode& nd = g->nodes[n]->node;
      for (int k = 0; k < nd.inputs->size; ++k) {
        const int t = nd.inputs->data[k];
        if (t >= 0 && !has(produced, t) && !has(ins, t)) ins.push_back(t);
      }
      // a blockwise-quantized filter drags its scale tensor along
      for (int k = 0; k < nd.outputs->size; ++k) produced.push_back(nd.outputs->data[k]);
    }
    for (int t : produced) {
      bool external = has(g->graph_outputs, t);
      for (size_t n = 0; n < g->nodes.size() && !external; ++n) {
        if (has(subset, static_cast<int>(n)) || !has(g->plan, static_cast<int>(n))) continue;
        const TfLiteNode& nd = g->nodes[n]->node;
        if (nd.inputs && Contains(nd.inputs, t)) external = true;
      }
      if (external) outs.push_back(t);
    }
    auto* params = static_cast<TfLiteDelegateParams*>(malloc(sizeof(TfLiteDelegateParams)));
    params->delegate = delegate;
    params->nodes_to_replace = MakeArray(subset);
    params->input_tensors = MakeArray(ins);
    params->output_tensors = MakeArray(outs);
    auto rec = std::make_unique<NodeRec>();
    rec->node = TfLiteNode{};
    rec->node.inputs = MakeArray(ins);
    rec->node.outputs = MakeArray(outs);
    rec->node.builtin_data = params;
    rec->node.delegate = delegate;
    rec->reg = reg;
    rec->is_delegate = true;
    const int new_index = static_cast<int>(g->nodes.size());
    g->nodes.push_back(std::move(rec));
    NodeRec* r = g->nodes.back().get();
    r->node.user_data = reg.init ? reg.init(ctx, reinterpret_cast<const char*>(params), 0) : nullptr;
    if (r->node.user_data == TfLiteKernelInitFailed()) {
      r->node.user_data = nullptr;
      return kTfLiteDelegateError;
    }
    for (int t : outs) g->tensors[t].delegate = delegate;
    new_plan.push_back(new_index);
    ++g->partitions;
  }
  g->plan.swap(new_plan);
  return kTfLiteOk;
}

size_t TypeBytes(TfLiteType t, size_t elems) {
  switch (t) {
    case kTfLiteFloat32: case kTfLiteInt32: return 4 * elems;
    case kTfLiteFloat16: case kTfLiteInt16: return 2 * elems;
    case kTfLiteInt8: case kTfLiteUInt8: case kTfLiteBool: return elems;
    case kTfLiteInt64: return 8 * elems;
    case kTfLiteInt4: return (elems + 1) / 2;
    default: return 0;
  }
}

void RemoveDelegates(Graph* g) {
  for (auto& n : g->nodes)
    if (n->is_delegate) FreeNode(g, n.get());
  while (!g->nodes.empty() && g->nodes.back()->is_delegate) g->nodes.pop_back();
  g->plan = g->original_plan;
  g->partitions = 0;
  for (auto& t : g->tensors) {
    if (t.delegate && t.buffer_handle != kTfLiteNullBufferHandle && t.delegate->FreeBufferHandle)
      t.delegate->FreeBufferHandle(&g->ctx, t.delegate, &t.buffer_handle);
    t.delegate = nullptr;
    t.buffer_handle = kTfLiteNullBufferHandle;
    t.data_is_stale = false;
  }
}

TfLiteStatus EnsureReadable(Graph* g, int tensor) {
  TfLiteTensor& t = g->tensors[tensor];
  if (!t.data_is_stale) return kTfLiteOk;
  if (!t.delegate || !t.delegate->CopyFromBufferHandle || t.buffer_handle == kTfLiteNullBufferHandle) return kTfLiteError;
  TfLiteStatus s = t.delegate->CopyFromBufferHandle(&g->ctx, t.delegate, t.buffer_handle, &t);
  if (s == kTfLiteOk) t.data_is_stale = false;
  return s;
}

}  // namespace

extern "C" {
#define MRT_API __attribute__((visibility("default")))

MRT_API void* mrt_create() {
  Graph* g = new Graph();
  memset(&g->ctx, 0, sizeof(g->ctx));
  g->ctx.impl_ = g;
  g->ctx.ReportError = ReportError;
  g->ctx.recommended_num_threads = 1;
  return g;
}

MRT_API void mrt_destroy(void* h) {
  Graph* g = static_cast<Graph*>(h);
  RemoveDelegates(g);
  for (auto& n : g->nodes) FreeNode(g, n.get());
  for (auto& t : g->tensors) {
    if (t.dims) TfLiteIntArrayFree(t.dims);
    if (t.quantization.type == kTfLiteAffineQuantization && t.quantization.params) {
      auto* q = static_cast<TfLiteAffineQuantization*>(t.quantization.params);
      if (q->scale) TfLiteFloatArrayFree(q->scale);
      if (q->zero_point) TfLiteIntArrayFree(q->zero_point);
      free(q);
    } else if (t.quantization.params) {
      free(t.quantization.params);
    }
    if (t.data.raw) free(t.data.raw);
  }
  if (g->plan_array) TfLiteIntArrayFree(g->plan_array);
  delete g;
}

MRT_API const char* mrt_last_error(void* h) { return static_cast<Graph*>(h)->error.c_str(); }
MRT_API void mrt_clear_error(void* h) { static_cast<Graph*>(h)->error.clear(); }

// Adds a tensor; constant tensors (is_const) copy `data` and are marked
// kTfLiteMmapRo like tensors that alias the model file. Returns its index.
MRT_API int mrt_add_tensor(void* h, int type, int rank, const int* dims, int is_const, const void* data, float scale,
                           int zero_point, int num_channel_scales, const float* channel_scales,
                           int quantized_dimension) {
  Graph* g = static_cast<Graph*>(h);
  TfLiteTensor t;
  memset(&t, 0, sizeof(t));
  t.type = static_cast<TfLiteType>(type);
  t.dims = TfLiteIntArrayCreate(rank);
  size_t elems = 1;
  for (int i = 0; i < rank; ++i) {
    t.dims->data[i] = dims[i];
    elems *= static_cast<size_t>(dims[i]);
  }
  t.bytes = TypeBytes(t.type, elems);
  t.data.raw = static_cast<char*>(calloc(t.bytes ? t.bytes : 1, 1));
  if (data) memcpy(t.data.raw, data, t.bytes);
  t.allocation_type = is_const ? kTfLiteMmapRo : kTfLiteArenaRw;
  t.params.scale = scale;
  t.params.zero_point = zero_point;
  t.buffer_handle = kTfLiteNullBufferHandle;
  if (scale != 0.0f || num_channel_scales > 0) {
    auto* q = static_cast<TfLiteAffineQuantization*>(malloc(sizeof(TfLiteAffineQuantization)));
    const int n = num_channel_scales > 0 ? num_channel_scales : 1;
    q->scale = TfLiteFloatArrayCreate(n);
    q->zero_point = TfLiteIntArrayCreate(n);
    for (int i = 0; i < n; ++i) {
      q->scale->data[i] = num_channel_scales > 0 ? channel_scales[i] : scale;
      q->zero_point->data[i] = num_channel_scales > 0 ? 0 : zero_point;
    }
    q->quantized_dimension = quantized_dimension;
    t.quantization.type = kTfLiteAffineQuantization;
    t.quantization.params = q;
  }
  g->tensors.push_back(t);
  g->ctx.tensors = g->tensors.data();
  g->ctx.tensors_size = g->tensors.size();
  return static_cast<int>(g->tensors.size()) - 1;
}

// Marks an int4 tensor as blockwise-quantized with its fp16 scale tensor
// (TfLiteBlockwiseQuantization, tflite/core/c/common.h:390-398).
MRT_API void mrt_set_blockwise(void* h, int tensor, int scale_tensor, int blocksize) {
  Graph* g = static_cast<Graph*>(h);
  auto* q = static_cast<TfLiteBlockwiseQuantization*>(calloc(1, sizeof(TfLiteBlockwiseQuantization)));
  q->scale = scale_tensor;
  q->zero_point = -1;
  q->blocksize = blocksize;
  q->quantized_dimension = 0;
  g->tensors[tensor].quantization.type = kTfLiteBlockwiseQuantization;
  g->tensors[tensor].quantization.params = q;
}

static int AddNode(Graph* g, int builtin_code, const char* custom_name, int n_in, const int* ins, int n_out,
                   const int* outs, void* builtin_data) {
  auto rec = std::make_unique<NodeRec>();
  rec->node = TfLiteNode{};
  rec->node.inputs = TfLiteIntArrayCreate(n_in);
  for (int i = 0; i < n_in; ++i) rec->node.inputs->data[i] = ins[i];
  rec->node.outputs = TfLiteIntArrayCreate(n_out);
  for (int i = 0; i < n_out; ++i) rec->node.outputs->data[i] = outs[i];
  rec->node.builtin_data = builtin_data;
  memset(&rec->reg, 0, sizeof(rec->reg));
  rec->reg.builtin_code = builtin_code;
  if (custom_name) {
    rec->custom_name = custom_name;
    rec->reg.custom_name = rec->custom_name.c_str();
  }
  rec->reg.version = 1;
  g->nodes.push_back(std::move(rec));
  const int idx = static_cast<int>(g->nodes.size()) - 1;
  g->plan.push_back(idx);
  g->original_plan = g->plan;
  return idx;
}

MRT_API int mrt_add_fully_connected(void* h, int x, int w, int bias, int y, int activation, int keep_num_dims,
                                    int asymmetric_quantize_inputs, int weights_format) {
  Graph* g = static_cast<Graph*>(h);
  auto* p = static_cast<TfLiteFullyConnectedParams*>(calloc(1, sizeof(TfLiteFullyConnectedParams)));
  p->activation = static_cast<TfLiteFusedActivation>(activation);
  p->weights_format = static_cast<TfLiteFullyConnectedWeightsFormat>(weights_format);
  p->keep_num_dims = keep_num_dims != 0;
  p->asymmetric_quantize_inputs = asymmetric_quantize_inputs != 0;
  p->quantized_bias_type = kTfLiteNoType;
  const int ins[3] = {x, w, bias};
  return AddNode(g, kTfLiteBuiltinFullyConnected, nullptr, 3, ins, 1, &y, p);
}

MRT_API int mrt_add_batch_matmul(void* h, int x, int y, int out, int adj_x, int adj_y, int asymmetric) {
  Graph* g = static_cast<Graph*>(h);
  auto* p = static_cast<TfLiteBatchMatMulParams*>(calloc(1, sizeof(TfLiteBatchMatMulParams)));
  p->adj_x = adj_x != 0;
  p->adj_y = adj_y != 0;
  p->asymmetric_quantize_inputs = asymmetric != 0;
  const int ins[2] = {x, y};
  return AddNode(g, kTfLiteBuiltinBatchMatmul, nullptr, 2, ins, 1, &out, p);
}

// STABLEHLO_COMPOSITE node (TfLiteStablehloCompositeParams,
// tflite/converter/core/c/builtin_op_data.h:651-657).
MRT_API int mrt_add_composite(void* h, const char* name, const uint8_t* attributes, int attributes_size, int n_in,
                              const int* ins, int out) {
  Graph* g = static_cast<Graph*>(h);
  auto* p = static_cast<TfLiteStablehloCompositeParams*>(calloc(1, sizeof(TfLiteStablehloCompositeParams)));
  const int idx = AddNode(g, kTfLiteBuiltinStablehloComposite, nullptr, n_in, ins, 1, &out, p);
  NodeRec* r = g->nodes[idx].get();
  r->composite_name = name;
  r->blob.assign(attributes, attributes + attributes_size);
  p->name = r->composite_name.c_str();
  p->subgraph_index = 1;
  p->version = 1;
  p->attributes = r->blob.data();
  p->attributes_size = r->blob.size();
  return idx;
}

MRT_API int mrt_add_custom(void* h, const char* custom_name, const uint8_t* init_data, int init_size, int n_in,
                           const int* ins, int out) {
  Graph* g = static_cast<Graph*>(h);
  const int idx = AddNode(g, kTfLiteBuiltinCustom, custom_name, n_in, ins, 1, &out, nullptr);
  NodeRec* r = g->nodes[idx].get();
  r->blob.assign(init_data, init_data + init_size);
  r->node.custom_initial_data = r->blob.data();
  r->node.custom_initial_data_size = init_size;
  return idx;
}

// Any builtin or custom node with several outputs: `params` (may be null) is the op's plain builtin-data
// struct as bytes (TfLiteAddParams, TfLiteGeluParams, ... of tflite/core/c/builtin_op_data.h; copied),
// `init_data` the custom initial data of a custom op (kept alive with the node).
MRT_API int mrt_add_node(void* h, int builtin_code, const char* custom_name, int n_in, const int* ins, int n_out,
                         const int* outs, const void* params, int params_size, const uint8_t* init_data, int init_size) {
  Graph* g = static_cast<Graph*>(h);
  void* data = nullptr;
  if (params && params_size > 0) {
    data = calloc(1, static_cast<size_t>(params_size));
    memcpy(data, params, static_cast<size_t>(params_size));
  }
  const int idx = AddNode(g, builtin_code, custom_name && custom_name[0] ? custom_name : nullptr, n_in, ins, n_out, outs, data);
  NodeRec* r = g->nodes[idx].get();
  if (init_data && init_size > 0) {
    r->blob.assign(init_data, init_data + init_size);
    r->node.custom_initial_data = r->blob.data();
    r->node.custom_initial_data_size = init_size;
  }
  return idx;
}

// Any other builtin (no parameters): stands for ops that stay on the CPU.
MRT_API int mrt_add_other(void* h, int builtin_code, int n_in, const int* ins, int out) {
  return AddNode(static_cast<Graph*>(h), builtin_code, nullptr, n_in, ins, 1, &out, nullptr);
}

MRT_API void mrt_set_io(void* h, int n_in, const int* ins, int n_out, const int* outs) {
  Graph* g = static_cast<Graph*>(h);
  g->graph_inputs.assign(ins, ins + n_in);
  g->graph_outputs.assign(outs, outs + n_out);
}

MRT_API void mrt_set_cpu_callback(void* h, CpuCallback cb) { static_cast<Graph*>(h)->cpu = cb; }

// ModifyGraphWithDelegate: Prepare under the delegate context, then prepare the
// new kernels. Any failure restores the original plan and reports
// kTfLiteDelegateError (tflite/core/subgraph.cc:2508-2517).
MRT_API int mrt_apply_delegate(void* h, TfLiteDelegate* delegate) {
  Graph* g = static_cast<Graph*>(h);
  if (!delegate || !delegate->Prepare) return kTfLiteError;
  g->delegate = delegate;
  g->original_plan = g->plan;
  g->ctx.GetExecutionPlan = GetExecutionPlan;
  g->ctx.GetNodeAndRegistration = GetNodeAndRegistration;
  g->ctx.ReplaceNodeSubsetsWithDelegateKernels = ReplaceNodeSubsets;
  TfLiteStatus s = delegate->Prepare(&g->ctx, delegate);
  g->ctx.GetExecutionPlan = nullptr;  // only valid while the delegate is being applied
  g->ctx.ReplaceNodeSubsetsWithDelegateKernels = nullptr;
  if (s == kTfLiteOk) {
    for (int n : g->plan) {
      NodeRec* r = g->nodes[n].get();
      if (r->is_delegate && r->reg.prepare) {
        s = r->reg.prepare(&g->ctx, &r->node);
        if (s != kTfLiteOk) break;
      }
    }
  }
  if (s != kTfLiteOk) {
    RemoveDelegates(g);
    return kTfLiteDelegateError;
  }
  return kTfLiteOk;
}

MRT_API int mrt_invoke(void* h) {
  Graph* g = static_cast<Graph*>(h);
  for (int n : g->plan) {
    NodeRec* r = g->nodes[n].get();
    // tensors produced on a device by another owner must be readable first (subgraph.cc:1731-1734)
    for (int k = 0; k < r->node.inputs->size; ++k) {
      const int t = r->node.inputs->data[k];
      if (t < 0) continue;
      if (g->tensors[t].data_is_stale && g->tensors[t].delegate != r->node.delegate) {
        if (EnsureReadable(g, t) != kTfLiteOk) return kTfLiteError;
      }
    }
    if (r->is_delegate) {
      const TfLiteStatus s = r->reg.invoke(&g->ctx, &r->node);
      if (s != kTfLiteOk) return s;
    } else {
      if (!g->cpu) {
        ReportError(&g->ctx, "mini runtime: node %d is not delegated and no CPU callback is set", n);
        return kTfLiteError;
      }
      const int s = g->cpu(n);
      if (s != 0) return s;
    }
  }
  for (int t : g->graph_outputs)
    if (EnsureReadable(g, t) != kTfLiteOk) return kTfLiteError;  // interpreter.cc:251-257
  return kTfLiteOk;
}

MRT_API int mrt_num_skippable_subgraphs(void* h) { return static_cast<int>(static_cast<Graph*>(h)->skippable_subgraphs.size()); }
MRT_API void* mrt_tensor_data(void* h, int tensor) { return static_cast<Graph*>(h)->tensors[tensor].data.raw; }
MRT_API size_t mrt_tensor_bytes(void* h, int tensor) { return static_cast<Graph*>(h)->tensors[tensor].bytes; }
MRT_API int mrt_tensor_is_stale(void* h, int tensor) { return static_cast<Graph*>(h)->tensors[tensor].data_is_stale; }
MRT_API int mrt_num_partitions(void* h) { return static_cast<Graph*>(h)->partitions; }
MRT_API int mrt_plan_size(void* h) { return static_cast<int>(static_cast<Graph*>(h)->plan.size()); }
MRT_API int mrt_plan_node(void* h, int i) { return static_cast<Graph*>(h)->plan[i]; }
MRT_API int mrt_node_is_delegate(void* h, int node) { return static_cast<Graph*>(h)->nodes[node]->is_delegate; }
MRT_API int mrt_num_cpu_nodes_in_plan(void* h) {
  Graph* g = static_cast<Graph*>(h);
  int c = 0;
  for (int n : g->plan) c += g->nodes[n]->is_delegate ? 0 : 1;
  return c;
}

// ---- LiteRT accelerator probe ------------------------------------------------------------------
// What the LiteRT environment does with libLiteRtGpuAccelerator.so
// (litert/runtime/accelerators/registration_helper.cc:111-126): dlopen, look the data symbol
// LiteRtAcceleratorImpl up, check its ABI header, ask it for a delegate through a runtime context.
// Only wrap_delegate of the context is live here: it records the delegate and its deleter.
struct WrappedDelegate {
  TfLiteOpaqueDelegate* delegate;
  void (*deleter)(TfLiteOpaqueDelegate*);
};
static LiteRtStatus FakeWrapDelegate(TfLiteOpaqueDelegate* delegate, void (*deleter)(TfLiteOpaqueDelegate*),
                                     LiteRtDelegateWrapper* wrapper) {
  auto* w = new WrappedDelegate{delegate, deleter};
  *wrapper = reinterpret_cast<LiteRtDelegateWrapper>(w);
  return kLiteRtStatusOk;
}

// Returns 0 and fills the outputs, or a negative step number that failed.
MRT_API int mrt_accelerator_probe(const char* path, char* name_out, int name_cap, int* version3, int* hw_set,
                                  int* struct_size, void** wrapped_out, TfLiteDelegate** delegate_out) {
  void* lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!lib) return -1;
  auto* def = static_cast<const LiteRtAcceleratorDef*>(dlsym(lib, "LiteRtAcceleratorImpl"));
  if (!def) return -2;
  *struct_size = def->abi_header.struct_size;
  if (def->abi_header.struct_size != sizeof(LiteRtAcceleratorDefV1) ||
      def->abi_header.major_version != LITERT_ACCELERATOR_DEF_CURRENT_VERSION)
    return -3;
  const char* name = nullptr;
  if (!def->get_name || def->get_name(nullptr, &name) != kLiteRtStatusOk || !name) return -4;
  snprintf(name_out, name_cap, "%s", name);
  LiteRtApiVersion v;
  if (!def->get_version || def->get_version(nullptr, &v) != kLiteRtStatusOk) return -5;
  version3[0] = v.major, version3[1] = v.minor, version3[2] = v.patch;
  LiteRtHwAcceleratorSet hw = 0;
  if (!def->get_hardware_support || def->get_hardware_support(nullptr, &hw) != kLiteRtStatusOk) return -6;
  *hw_set = hw;
  bool jit = false;
  if (!def->is_tflite_delegate_responsible_for_jit_compilation ||
      def->is_tflite_delegate_responsible_for_jit_compilation(nullptr, &jit) != kLiteRtStatusOk)
    return -7;
  if (def->get_name(nullptr, nullptr) == kLiteRtStatusOk) return -8;  // null output must be refused
  LiteRtRuntimeContext ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.abi_header.struct_size = sizeof(ctx);
  ctx.wrap_delegate = FakeWrapDelegate;
  LiteRtDelegateWrapper wrapper = nullptr;
  if (!def->create_delegate || def->create_delegate(&ctx, nullptr, nullptr, nullptr, &wrapper) != kLiteRtStatusOk ||
      !wrapper)
    return -9;
  auto* w = reinterpret_cast<WrappedDelegate*>(wrapper);
  *wrapped_out = w;
  *delegate_out = reinterpret_cast<TfLiteDelegate*>(w->delegate);
  return 0;
}

MRT_API void mrt_accelerator_release(void* wrapped) {
  auto* w = static_cast<WrappedDelegate*>(wrapped);
  if (!w) return;
  if (w->deleter) w->deleter(w->delegate);
  delete w;
}

}  // extern "C"

// What the runtime exports for delegates that absorb other subgraphs
// (tflite/delegates/utils.h:62-93, Subgraph::MarkSubgraphAsDelegationSkippable,
// tflite/core/subgraph.cc:751-757): same name, same signature, same checks (index 0, the primary
// subgraph, is refused), so that a plugin resolving the symbol at run time finds it here.
namespace tflite {
namespace delegates {
MRT_API TfLiteStatus MarkSubgraphAsDelegationSkippable(const TfLiteContext* context, int subgraph_index) {
  if (!context || subgraph_index <= 0) return kTfLiteError;
  static_cast<Graph*>(context->impl_)->skippable_subgraphs.push_back(subgraph_index);
  return kTfLiteOk;
}
}  // namespace delegates
}  // namespace tflite
