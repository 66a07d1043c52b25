// Implementation of the allocation-free linear entry point (see linear_noalloc.h).
//
// The split-K scratch is a file-scope __device__ array. In host code the name
// `g_scratch` is only a handle for the runtime, not a device address: the address
// that kernels may use is obtained with cudaGetSymbolAddress, separately on each
// device, and cached.

#include <stdio.h>

#include <atomic>

#include "api.h"
#include "linear_noalloc.h"

namespace {

constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_scratch[AB200_NOALLOC_SCRATCH_BYTES];

// One entry per device, filled on the first call there. Host threads may make that first call
// at the same time: each looks the address up and stores the same value.
std::atomic<void*> g_scratch_addr[kMaxDevices];
thread_local char g_last_error[256] = "";

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_last_error, sizeof(g_last_error), "cannot identify the current device (%s)",
             e == cudaSuccess ? "index out of range" : cudaGetErrorString(e));
    return AB200_ERR_SYMBOL_LOOKUP;
  }
  void* p = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_last_error, sizeof(g_last_error),
               "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return AB200_ERR_SYMBOL_LOOKUP;
    }
    g_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return 0;
}

}  // namespace

extern "C" {

int ab200_linear_bf16_noalloc_fits(int M, int N, int K) {
  return ab200_linear_bf16_workspace_bytes(M, N, K) <= (size_t)AB200_NOALLOC_SCRATCH_BYTES ? 1 : 0;
}

const char* ab200_noalloc_last_error(void) { return g_last_error; }

int ab200_linear_bf16_noalloc(const void* x, long long ldx, const void* w, long long ldw,
                              void* out, long long ldo, int M, int N, int K, const void* bias,
                              const void* residual, long long ldr, int act, int force_splits,
                              int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const size_t need = ab200_linear_bf16_workspace_bytes(M, N, K);
  if (need > (size_t)AB200_NOALLOC_SCRATCH_BYTES) {
    snprintf(g_last_error, sizeof(g_last_error),
             "linear %dx%dx%d may need %zu bytes of split-K scratch; the built-in array holds %u",
             M, N, K, need, (unsigned)AB200_NOALLOC_SCRATCH_BYTES);
    return AB200_ERR_SCRATCH_TOO_SMALL;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  return ab200_linear_bf16(x, ldx, w, ldw, out, ldo, M, N, K, bias, residual, ldr, act, scratch,
                           (size_t)AB200_NOALLOC_SCRATCH_BYTES, force_splits, status, stream);
}

}  // extern "C"
