// Host-side helpers shared by the C-ABI translation units: error text, CUDA call
// checking, the per-device status word and the launch counter.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/fast_ops_b200.h"

namespace fo {

// Stores a printf-style message as this thread's last error and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

// Device-global status word (defined once in capi.cu); kernels OR a non-zero code
// into it when a bounded wait gives up.
int* device_status_ptr(int device);  // device address of the word; nullptr on failure

extern std::atomic<int64_t> g_launch_count;

// Device buffer for the attention kernels' debug timeline (fo_debug_set_attn_trace), or null.
extern unsigned long long* g_attn_trace;

// Options of the attention forward that fo_attn_configure sets (process-wide; -1 / 0 = default).
struct AttnOptions {
  std::atomic<int> impl{0};        // 0 chosen per call, 1 simple, 2 128-key kernel, 3 64-key kernel
  std::atomic<int> ping_pong{1};   // 64-key kernel: the two query tiles alternate on the ex2 units
  std::atomic<int> head_group{0};  // heads scheduled together for L2 reuse; 0 = from the K/V size
};
extern AttnOptions g_attn_options;

// Raises a kernel's dynamic shared-memory limit once per device (the attribute is per device and
// per kernel).  The kernel is a template argument, so that every kernel has once-flags of its own.
template <auto kKernel>
inline cudaError_t ensure_dynamic_smem(int bytes, int device) {
  static std::atomic<uint64_t> done{0};  // bit d: set on device d (devices >= 64 set it every time)
  const uint64_t bit = (device >= 0 && device < 64) ? (1ull << device) : 0;
  if (bit && (done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && bit) done.fetch_or(bit, std::memory_order_release);
  return e;
}

// RAII: make `device` current for the scope, restore the previous one afterwards.
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    if (prev != device && cudaSetDevice(device) != cudaSuccess) return;
    ok = true;
    want = device;
  }
  ~DeviceGuard() {
    if (ok && prev != want) cudaSetDevice(prev);
  }
  int want = -1;
};

}  // namespace fo

#define FO_CUDA_CHECK(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return fo::fail(FO_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                      __FILE__, __LINE__);                                               \
  } while (0)

#define FO_REQUIRE(cond, ...)                                        \
  do {                                                               \
    if (!(cond)) return fo::fail(FO_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

// Status codes written by kernels (bit flags, OR-ed together).
#define FO_STATUS_TIMEOUT_TMA 0x1    // a wait for a TMA load gave up
#define FO_STATUS_TIMEOUT_MMA 0x2    // a wait for a tcgen05.commit gave up
#define FO_STATUS_TIMEOUT_SOFTMAX 0x4  // a wait on a softmax/correction hand-off gave up
#define FO_STATUS_TIMEOUT_EPILOGUE 0x8
#define FO_STATUS_TIMEOUT_SELFTEST 0x10  // the wait of fo_debug_wait_timeout gave up (as it must)
