#include "driver_api.h"

#include <dlfcn.h>

namespace b200 {

namespace {

DriverApi bind() {
  DriverApi api = {};
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return api;
  auto sym = [&](const char* name) { return dlsym(lib, name); };
  api.CtxGetCurrent = reinterpret_cast<decltype(api.CtxGetCurrent)>(sym("cuCtxGetCurrent"));
  api.CtxPushCurrent = reinterpret_cast<decltype(api.CtxPushCurrent)>(sym("cuCtxPushCurrent_v2"));
  api.CtxPopCurrent = reinterpret_cast<decltype(api.CtxPopCurrent)>(sym("cuCtxPopCurrent_v2"));
  api.CtxGetId = reinterpret_cast<decltype(api.CtxGetId)>(sym("cuCtxGetId"));
  api.MemGetAddressRange = reinterpret_cast<decltype(api.MemGetAddressRange)>(sym("cuMemGetAddressRange_v2"));
  api.TensorMapEncodeTiled = reinterpret_cast<decltype(api.TensorMapEncodeTiled)>(sym("cuTensorMapEncodeTiled"));
  api.StreamWaitValue32 = reinterpret_cast<decltype(api.StreamWaitValue32)>(sym("cuStreamWaitValue32_v2"));
  api.StreamWriteValue32 = reinterpret_cast<decltype(api.StreamWriteValue32)>(sym("cuStreamWriteValue32_v2"));
  api.ok = api.CtxGetCurrent && api.CtxPushCurrent && api.CtxPopCurrent && api.MemGetAddressRange &&
           api.TensorMapEncodeTiled;
  return api;
}

}  // namespace

const DriverApi& driver_api() {
  static const DriverApi api = bind();
  return api;
}

}  // namespace b200
