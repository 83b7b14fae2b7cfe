// The parts every other unit of the library leans on: how failures are raised and reported, the per-device facts the
// launchers ask for, and the three general entry points of the C ABI (nm_version, nm_last_error, nm_device_arch;
// reference include/marincpp/capi.h:23-26).
#include <cuda_runtime.h>

#include <array>
#include <exception>
#include <mutex>
#include <string>

#include "abi_guard.hpp"
#include "device_info.hpp"
#include "marincpp/capi.h"

#ifndef NM_BUILD_ID
#define NM_BUILD_ID "b200-fused-ce-dev"
#endif

namespace nm {

// ------------------------------------------------------------------------------------------------ raising
void fatal(const char* where, const std::string& msg) {
  std::string text(where);
  text += ": ";
  text += msg;
  throw Fatal(text);
}

void cuda_check(int err, const char* expr, const char* where) {
  if (err == int(cudaSuccess)) return;
  const auto code = static_cast<cudaError_t>(err);
  std::string text(where);
  text.append(": CUDA call `").append(expr).append("` returned ").append(cudaGetErrorName(code));
  text.append(": ").append(cudaGetErrorString(code));
  (void)cudaGetLastError();   // a non-sticky error must not be blamed on the caller's next CUDA call
  throw DeviceError(text);
}

// ------------------------------------------------------------------------------------------------ reporting
namespace abi {
namespace {
std::string& slot() {
  thread_local std::string text;
  return text;
}
}  // namespace

void remember_error(const std::string& text) { slot() = text; }
void forget_error() { slot().clear(); }

int status_of_active_exception() noexcept {
  int status = NM_ERR_INTERNAL;
  try {
    try {
      throw;   // the exception the caller's catch block holds
    } catch (const DeviceError& e) {
      status = NM_ERR_DEVICE;
      remember_error(e.what());
    } catch (const Fatal& e) {
      status = NM_ERR_INVALID;
      remember_error(e.what());
    } catch (const std::exception& e) {
      remember_error(std::string("internal error: ") + e.what());
    } catch (...) {
      remember_error("internal error: an exception that is not a std::exception");
    }
  } catch (...) {
    // storing the message itself failed (out of memory): the status still tells the caller what happened
  }
  return status;
}
}  // namespace abi

// ------------------------------------------------------------------------------------------------ device facts
// One record per device ordinal, filled on first use with that device current. The trainer drives one host thread per
// GPU through the same entry points at the same time, so the table is locked while it is read or filled.
const DeviceInfo& current_device_info() {
  static std::mutex guard;
  static std::array<DeviceInfo, kMaxDeviceOrdinals> table{};
  int ordinal = 0;
  NM_CUDA(cudaGetDevice(&ordinal));
  NM_REQUIRE(ordinal >= 0 && ordinal < kMaxDeviceOrdinals, "device ordinal beyond the library's table");
  std::lock_guard<std::mutex> lock(guard);
  DeviceInfo& d = table[size_t(ordinal)];
  if (!d.known) {
    int major = 0, minor = 0, sms = 0;
    NM_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal));
    NM_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, ordinal));
    NM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal));
    d.ordinal = ordinal;
    d.arch = 10 * major + minor;
    d.sm_count = sms;
    d.known = true;
  }
  return d;
}

}  // namespace nm

extern "C" {

const char* nm_version(void) { return NM_BUILD_ID; }

const char* nm_last_error(void) { return nm::abi::slot().c_str(); }

int nm_device_arch(void) {
  return nm::abi::guarded_value<int>(0, [] { return nm::current_device_info().arch; });
}

}  // extern "C"
