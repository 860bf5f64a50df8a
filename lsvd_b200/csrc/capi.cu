// Status strings, device queries and other host-side plumbing shared by the entry points.
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace lsvd {

static thread_local int g_last_cuda_error = 0;

void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = static_cast<int>(e); }

struct DeviceInfo {
  int sm_count = 0;
  int smem_optin = 0;
};

static std::mutex g_mu;
static std::map<int, DeviceInfo> g_devices;
static std::map<std::pair<int, const void*>, int> g_smem_set;

static const DeviceInfo* current_device_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_devices.find(dev);
  if (it != g_devices.end()) return &it->second;
  DeviceInfo info;
  if (cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
  if (cudaDeviceGetAttribute(&info.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
    return nullptr;
  return &(g_devices[dev] = info);
}

bool chained_launch_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LSVD_CHAINED_LAUNCH");
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}

bool ffn_chain_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LSVD_CHAIN_FFN");
    return chained_launch_enabled() && !(v != nullptr && v[0] == '0');
  }();
  return on;
}

int device_sm_count() {
  const DeviceInfo* d = current_device_info();
  return d ? d->sm_count : 0;
}

int device_max_smem_optin() {
  const DeviceInfo* d = current_device_info();
  return d ? d->smem_optin : 0;
}

cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(g_mu);
  int& have = g_smem_set[{dev, kernel}];
  if (have >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) have = bytes;
  return e;
}

}  // namespace lsvd

extern "C" int lsvd_abi_version(void) { return LSVD_ABI_VERSION; }

extern "C" int lsvd_last_cuda_error(void) { return lsvd::g_last_cuda_error; }

extern "C" const char* lsvd_status_string(int code) {
  switch (code) {
    case LSVD_OK: return "ok";
    case LSVD_ERR_INVALID_ARG: return "invalid argument";
    case LSVD_ERR_UNSUPPORTED: return "unsupported configuration";
    case LSVD_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case LSVD_ERR_CUDA: return "CUDA runtime error";
    case LSVD_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    case LSVD_ERR_BOUNDS: return "device-side index out of range (access skipped)";
    default: return "unknown status";
  }
}
