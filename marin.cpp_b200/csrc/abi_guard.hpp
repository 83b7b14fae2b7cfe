// The exception boundary of the C ABI. C++ code inside the library reports failures by throwing (nm::Fatal for a
// caller mistake, nm::DeviceError for a CUDA / NCCL failure or a kernel that reported a timed-out wait); no exception
// may cross an extern "C" entry point, so each entry point runs its body inside abi::guarded(), which hands any
// escaping exception to one translator (status_of_active_exception, nm_core.cpp) and returns the NM_* status of
// include/marincpp/capi.h. The text of the failure is kept per host thread and served by nm_last_error().
// The status values and the per-thread message are the reference's convention (include/marincpp/capi.h:14-17).
#pragma once

#include <string>

#include "marincpp/capi.h"
#include "marincpp/core.hpp"

namespace nm::abi {

void remember_error(const std::string& text);   // becomes the calling thread's nm_last_error()
void forget_error();

// Must be called from inside a catch block: rethrows the exception in flight, classifies it, stores its message and
// returns the matching status (DeviceError -> NM_ERR_DEVICE, other Fatal -> NM_ERR_INVALID, the rest NM_ERR_INTERNAL).
int status_of_active_exception() noexcept;

template <class Body>
int guarded(Body&& body) noexcept {
  forget_error();
  try {
    body();
  } catch (...) {
    return status_of_active_exception();
  }
  return NM_OK;
}

// For entry points that return a value instead of a status: `fallback` when the body threw.
template <class R, class Body>
R guarded_value(R fallback, Body&& body) noexcept {
  R out = fallback;
  return guarded([&] { out = body(); }) == NM_OK ? out : fallback;
}

}  // namespace nm::abi
