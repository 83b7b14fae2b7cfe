// Facts about the current CUDA device that launchers need on every call (compute capability, SM count), looked up
// once per device ordinal and kept in a locked table: the library is entered concurrently by one host thread per GPU.
#pragma once

namespace nm {

constexpr int kMaxDeviceOrdinals = 64;

struct DeviceInfo {
  bool known = false;
  int ordinal = -1;
  int arch = 0;        // 10 * major + minor: 100 on a B200
  int sm_count = 0;
};

const DeviceInfo& current_device_info();   // of the calling thread's current device; throws nm::DeviceError

}  // namespace nm
