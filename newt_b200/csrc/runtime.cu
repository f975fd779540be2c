// Host-side plumbing shared by every entry point of the library: error text,
// device properties, tuning knobs, and the device status word that kernels
// with bounded waits report into.

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>

#include "sm100.cuh"

namespace nb200 {

namespace {
thread_local char g_error[512] = "";
std::mutex g_mutex;
std::map<std::string, int> g_tuning;
std::map<int, DeviceInfo> g_devices;

// Written by kernels (first error wins), read by nb200_read_status().
__device__ unsigned int g_status[4];
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_check(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  return fail(NB200_E_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

const DeviceInfo& device_info() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_devices.find(dev);
  if (it != g_devices.end()) return it->second;
  DeviceInfo info{dev, 148, 232448};
  cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  return g_devices.emplace(dev, info).first->second;
}

int tuning(const char* key, int dflt) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_tuning.find(key);
  return (it == g_tuning.end() || it->second == 0) ? dflt : it->second;
}

unsigned long long wait_limit_ns() {
  return 1000ull * (unsigned long long)tuning("wait_limit_us", 2000000);
}

unsigned int* device_status_ptr() {
  // the symbol has one instance per device context: resolved once per device
  static std::map<int, unsigned int*> known;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = known.find(dev);
  if (it != known.end()) return it->second;
  unsigned int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status) != cudaSuccess) return nullptr;
  known[dev] = p;
  return p;
}

namespace {
struct KernelKey {
  int device;
  const void* kernel;
  int smem;
  bool operator<(const KernelKey& o) const {
    if (device != o.device) return device < o.device;
    if (kernel != o.kernel) return kernel < o.kernel;
    return smem < o.smem;
  }
};
std::map<KernelKey, int> g_prepared;   // value: cluster capacity, or -1 when not asked yet
}  // namespace

int prepare_kernel(const void* kernel, int smem_bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  const KernelKey key{dev, kernel, smem_bytes};
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_prepared.count(key)) return 0;
  }
  if (cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes))
    return cuda_check(e, "shared-memory attribute");
  std::lock_guard<std::mutex> lock(g_mutex);
  g_prepared.emplace(key, -1);
  return 0;
}

int cluster_capacity(const void* kernel, const cudaLaunchConfig_t* config, int* clusters) {
  int dev = 0;
  cudaGetDevice(&dev);
  const KernelKey key{dev, kernel, (int)config->dynamicSmemBytes};
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_prepared.find(key);
    if (it != g_prepared.end() && it->second >= 0) {
      *clusters = it->second;
      return 0;
    }
  }
  int count = 0;
  if (cudaError_t e = cudaOccupancyMaxActiveClusters(&count, kernel, config))
    return cuda_check(e, "cluster occupancy query");
  std::lock_guard<std::mutex> lock(g_mutex);
  g_prepared[key] = count;
  *clusters = count;
  return 0;
}

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_abi_version(void) { return NB200_ABI_VERSION; }

extern "C" const char* nb200_last_error(void) { return g_error; }

extern "C" int nb200_set_tuning(const char* key, int value) {
  if (!key) return fail(NB200_E_INVALID, "null tuning key");
  std::lock_guard<std::mutex> lock(g_mutex);
  g_tuning[key] = value;
  return 0;
}

namespace nb200 {
namespace {
// One warp, one barrier that nobody arrives on: the bounded wait runs out and reports.
__global__ void wait_timeout_kernel(unsigned int* status, unsigned long long limit_ns,
                                    unsigned int detail) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(sm100::smem_u32(&bar), 1);
    sm100::mbar_init_fence();
  }
  __syncwarp();
  const sm100::WaitCtx ctx{&abort_flag, status, limit_ns};
  sm100::mbar_wait(sm100::smem_u32(&bar), 0, ctx, ST_WAIT_OTHER, detail);
}
}  // namespace
}  // namespace nb200

extern "C" int nb200_selftest_wait_timeout(uint32_t detail, void* stream) {
  unsigned int* status = device_status_ptr();
  if (!status) return fail(NB200_E_CUDA, "selftest: device status word is not addressable");
  wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, wait_limit_ns(), detail);
  return cuda_check(cudaGetLastError(), "selftest launch");
}

extern "C" int nb200_read_status(uint32_t* status, uint32_t* detail) {
  unsigned int host[4] = {0, 0, 0, 0};
  if (int rc = cuda_check(cudaDeviceSynchronize(), "synchronize before status read")) return rc;
  if (int rc = cuda_check(cudaMemcpyFromSymbol(host, g_status, sizeof(host)), "status read"))
    return rc;
  if (host[0] != 0) {
    unsigned int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  if (status) *status = host[0];
  if (detail) *detail = host[1];
  if (host[0] != 0)
    return fail(NB200_E_DEVICE, "a kernel gave up on a bounded wait (code %u, detail 0x%x)", host[0],
                host[1]);
  return 0;
}
