// Entry points that belong to no single kernel: version, error text, the per-device
// status word and the launch counter.
#include <cstring>
#include <map>
#include <mutex>

#include "fo_host.h"

namespace {
thread_local char t_error[512] = "";

// Kernels OR a FO_STATUS_* flag into this word when a bounded wait gives up.  One copy
// exists per device that loads the library; host code reaches it through its device
// address (cudaGetSymbolAddress), never through the host-side symbol.
__device__ int g_device_status = 0;

std::mutex g_status_mutex;
std::map<int, int*> g_status_ptrs;
}  // namespace

namespace fo {

std::atomic<int64_t> g_launch_count{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { t_error[0] = '\0'; }

int* device_status_ptr(int device) {
  std::lock_guard<std::mutex> lock(g_status_mutex);
  auto it = g_status_ptrs.find(device);
  if (it != g_status_ptrs.end()) return it->second;
  DeviceGuard guard(device);
  if (!guard.ok) return nullptr;
  int* ptr = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_device_status) != cudaSuccess) return nullptr;
  g_status_ptrs[device] = ptr;
  return ptr;
}

}  // namespace fo

extern "C" int fo_version(void) { return 100; }

extern "C" const char* fo_last_error(void) { return t_error; }

extern "C" int64_t fo_launch_count(void) { return fo::g_launch_count.load(std::memory_order_relaxed); }

extern "C" int fo_device_status(int device, int* status_out, int reset) {
  fo::clear_error();
  FO_REQUIRE(status_out != nullptr, "status_out is null");
  int* ptr = fo::device_status_ptr(device);
  if (!ptr) return fo::fail(FO_ERR_CUDA, "cannot resolve the status word of device %d", device);
  fo::DeviceGuard guard(device);
  FO_REQUIRE(guard.ok, "cannot make device %d current", device);
  FO_CUDA_CHECK(cudaDeviceSynchronize());
  FO_CUDA_CHECK(cudaMemcpy(status_out, ptr, sizeof(int), cudaMemcpyDeviceToHost));
  if (reset) FO_CUDA_CHECK(cudaMemset(ptr, 0, sizeof(int)));
  return FO_OK;
}
