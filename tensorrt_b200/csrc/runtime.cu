// Library identification, status strings and per-device properties.
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace b200q {

namespace {
struct DeviceInfo {
  bool known = false;
  int major = 0;
  int sms = 0;
};
DeviceInfo g_info[64];
std::mutex g_mu;

const DeviceInfo* info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceInfo& d = g_info[dev];
  if (!d.known) {
    if (cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    d.known = true;
  }
  return &d;
}
}  // namespace

int check_arch() {
  const DeviceInfo* d = info();
  if (d == nullptr) return B200Q_ERR_CUDA;
  return d->major == 10 ? B200Q_OK : B200Q_ERR_ARCH;
}

bool pdl_enabled() {
  static const bool v = [] {
    const char* e = std::getenv("B200Q_PDL");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return v;
}

int sm_count() {
  const DeviceInfo* d = info();
  return d == nullptr ? 148 : d->sms;
}

}  // namespace b200q

extern "C" {

int b200q_version(void) { return 100; }

const char* b200q_status_string(int status) {
  switch (status) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_INVALID: return "invalid argument (shape, dtype or null pointer)";
    case B200Q_ERR_ALIGN: return "misaligned pointer or leading dimension";
    case B200Q_ERR_ARCH: return "device is not compute capability 10.x (sm_100a required)";
    case B200Q_ERR_CUDA: return "CUDA runtime or driver call failed";
    case B200Q_ERR_WORKSPACE: return "workspace missing or too small";
    case B200Q_ERR_TIMEOUT: return "device-side bounded wait timed out";
    case B200Q_ERR_TOO_LARGE: return "size exceeds the capacity of the built-in scratch of this entry point";
    default: return "unknown status";
  }
}

}  // extern "C"
