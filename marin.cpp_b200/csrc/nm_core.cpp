// Error plumbing and the C ABI basics (nm_version, nm_last_error, nm_device_arch); the role of the reference's
// src/core/core.cpp:40-80 and src/core/capi_core.cpp:12-36.
#include <cuda_runtime.h>

#include <string>

#include "capi_util.hpp"
#include "marincpp/capi.h"

#ifndef NM_BUILD_ID
#define NM_BUILD_ID "b200-fused-ce-dev"
#endif

namespace nm {
namespace {
thread_local std::string g_last_error;
}
void capi_set_error(const std::string& msg) { g_last_error = msg; }
void capi_clear_error() { g_last_error.clear(); }

void fatal(const char* where, const std::string& msg) { throw Fatal(std::string(where) + ": " + msg); }

void cuda_check(int err, const char* expr, const char* where) {
  if (err == 0) return;
  const cudaError_t e = static_cast<cudaError_t>(err);
  const std::string msg = std::string(where) + ": " + expr + " failed: " + cudaGetErrorName(e) + " (" +
                          cudaGetErrorString(e) + ")";
  cudaGetLastError();   // clear the sticky-less error state for the caller's next CUDA call
  throw DeviceError(msg);
}
}  // namespace nm

extern "C" {

const char* nm_version(void) { return NM_BUILD_ID; }

const char* nm_last_error(void) { return nm::g_last_error.c_str(); }

int nm_device_arch(void) {
  int dev = 0, major = 0, minor = 0;
  nm::capi_clear_error();
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (e != cudaSuccess) {
    nm::capi_set_error(std::string("nm_device_arch: ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
    cudaGetLastError();
    return 0;
  }
  return major * 10 + minor;
}

}  // extern "C"
