// LiteRT accelerator definition for the B200 delegate: the data symbol `LiteRtAcceleratorImpl` that
// the LiteRT environment looks up with dlsym() in libLiteRtGpuAccelerator.so
// (litert/runtime/accelerators/gpu_registry.cc:45-162 -> registration_helper.cc:111-126), with the
// table layout of litert/c/internal/litert_accelerator_def.h:40-66. create_delegate builds the
// TfLiteDelegate of this repository (include/litert_b200_delegate.h) and hands it to the runtime
// through LiteRtRuntimeContext::wrap_delegate, as the reference's own accelerators do
// (litert/runtime/accelerators/xnnpack/xnnpack_accelerator.cc:60-128,
// litert/runtime/accelerators/gpu/ml_drift_cl_accelerator.cc:117-150).
//
// Options: the reference defines no option payload for a CUDA accelerator, so the delegate's
// key/value options are taken from the environment variable B200_DELEGATE_OPTIONS
// ("device:0;buffer_handles:0"), the same strings the external-delegate loader passes.
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../../include/litert_b200_delegate.h"
#include "litert/c/internal/litert_accelerator_def.h"

namespace {

constexpr char kName[] = "B200";

LiteRtStatus GetName(LiteRtAcceleratorConst, const char** name) {
  if (!name) return kLiteRtStatusErrorInvalidArgument;
  *name = kName;
  return kLiteRtStatusOk;
}

LiteRtStatus GetVersion(LiteRtAcceleratorConst, LiteRtApiVersion* version) {
  if (!version) return kLiteRtStatusErrorInvalidArgument;
  version->major = 1;
  version->minor = 0;
  version->patch = 0;
  return kLiteRtStatusOk;
}

LiteRtStatus GetHardwareSupport(LiteRtAcceleratorConst, LiteRtHwAcceleratorSet* supported) {
  if (!supported) return kLiteRtStatusErrorInvalidArgument;
  *supported = kLiteRtHwAcceleratorGpu;
  return kLiteRtStatusOk;
}

// The delegate consumes the model's own weights and needs no compilation step of the runtime's.
LiteRtStatus IsResponsibleForJit(LiteRtAcceleratorConst, bool* does_jit) {
  if (!does_jit) return kLiteRtStatusErrorInvalidArgument;
  *does_jit = true;
  return kLiteRtStatusOk;
}

void DestroyDelegate(TfLiteOpaqueDelegate* d) { tflite_plugin_destroy_delegate(reinterpret_cast<TfLiteDelegate*>(d)); }

LiteRtStatus CreateDelegate(LiteRtRuntimeContext* runtime_context, LiteRtEnvironment, LiteRtAcceleratorConst,
                            LiteRtOptions, LiteRtDelegateWrapper* delegate_wrapper) {
  if (!runtime_context || !delegate_wrapper || !runtime_context->wrap_delegate) return kLiteRtStatusErrorInvalidArgument;
  std::vector<std::string> keys, values;
  if (const char* env = getenv("B200_DELEGATE_OPTIONS")) {
    std::string all(env);
    size_t pos = 0;
    while (pos < all.size()) {
      size_t end = all.find(';', pos);
      if (end == std::string::npos) end = all.size();
      const std::string item = all.substr(pos, end - pos);
      const size_t colon = item.find(':');
      if (colon != std::string::npos && colon > 0) {
        keys.push_back(item.substr(0, colon));
        values.push_back(item.substr(colon + 1));
      }
      pos = end + 1;
    }
  }
  std::vector<const char*> k, v;
  for (size_t i = 0; i < keys.size(); ++i) {
    k.push_back(keys[i].c_str());
    v.push_back(values[i].c_str());
  }
  TfLiteDelegate* d = tflite_plugin_create_delegate(k.empty() ? nullptr : k.data(), v.empty() ? nullptr : v.data(),
                                                    k.size(), nullptr);
  if (!d) return kLiteRtStatusErrorRuntimeFailure;
  const LiteRtStatus st =
      runtime_context->wrap_delegate(reinterpret_cast<TfLiteOpaqueDelegate*>(d), DestroyDelegate, delegate_wrapper);
  if (st != kLiteRtStatusOk) DestroyDelegate(reinterpret_cast<TfLiteOpaqueDelegate*>(d));
  return st;
}

LiteRtAcceleratorDef MakeDef() {
  LiteRtAcceleratorDef def;
  memset(&def, 0, sizeof(def));
  def.abi_header.struct_size = sizeof(LiteRtAcceleratorDefV1);
  def.abi_header.major_version = LITERT_ACCELERATOR_DEF_CURRENT_VERSION;
  def.abi_header.minor_version = 0;
  def.get_name = GetName;
  def.get_version = GetVersion;
  def.get_hardware_support = GetHardwareSupport;
  def.is_tflite_delegate_responsible_for_jit_compilation = IsResponsibleForJit;
  def.create_delegate = CreateDelegate;
  // no metrics collection, no custom tensor-buffer handlers: tensors cross the boundary in host
  // memory (or as delegate buffer handles)
  return def;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const LiteRtAcceleratorDef LiteRtAcceleratorImpl = MakeDef();
