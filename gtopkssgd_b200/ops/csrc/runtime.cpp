// Host-side runtime shared by all kernels: per-device facts (SM count,
// cooperative-launch support), the launch counter that bench.py reports, and
// size queries for the opaque device structs.
#include <cuda_runtime.h>
#include <atomic>
#include <mutex>
#include <string>
#include "host_api.h"

namespace {
std::atomic<long long> g_launches{0};
std::mutex g_mu;
DeviceInfo g_info[64];
bool g_have[64] = {false};
thread_local std::string g_err;
}  // namespace

extern "C" const DeviceInfo* gtk_device_info(void) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_have[dev]) {
    DeviceInfo di{};
    di.device = dev;
    if (cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    cudaDeviceGetAttribute(&di.coop, cudaDevAttrCooperativeLaunch, dev);
    cudaDeviceGetAttribute(&di.cluster, cudaDevAttrClusterLaunch, dev);
    g_info[dev] = di;
    g_have[dev] = true;
  }
  return &g_info[dev];
}

extern "C" void gtk_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long gtk_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" void gtk_reset_launch_count(void) { g_launches.store(0, std::memory_order_relaxed); }
extern "C" unsigned long long gtk_k1state_bytes(void) { return sizeof(K1State); }

extern "C" const char* gtk_last_cuda_error(void) {
  g_err = cudaGetErrorString(cudaPeekAtLastError());
  return g_err.c_str();
}
