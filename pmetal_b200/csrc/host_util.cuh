// Host-side helpers shared by every launcher: per-device one-time configuration and the SM count.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace pm {

// ---------------------------------------------------------------- host-side per-device state
// cudaFuncSetAttribute and the SM count belong to one device; a process may drive several.
constexpr int kMaxDevices = 64;
static inline int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return (d < 0 || d >= kMaxDevices) ? 0 : d;
}
struct DeviceOnce {          // "configured on this device yet?"
  bool done[kMaxDevices] = {};
  bool pending() const { return !done[current_device()]; }
  void mark() { done[current_device()] = true; }
};
struct DeviceMax {           // largest value configured so far on this device
  size_t v[kMaxDevices] = {};
  size_t get() const { return v[current_device()]; }
  void set(size_t x) { v[current_device()] = x; }
};
static inline int num_sms() {
  static int n[kMaxDevices] = {};
  const int d = current_device();
  if (!n[d]) cudaDeviceGetAttribute(&n[d], cudaDevAttrMultiProcessorCount, d);
  return n[d] > 0 ? n[d] : 1;
}

}  // namespace pm
