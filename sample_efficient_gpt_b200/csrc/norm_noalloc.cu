// Allocation-free variant of the add+RMSNorm backward: see noalloc.h for who needs it and for the contract.
// The kernels are the ones of norm.cu; only the home of the gain-gradient partial sums differs: a file-scope
// __device__ array instead of scratch memory handed in by the caller.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "kernels.h"
#include "noalloc.h"

namespace {

// Partial sums of dgain, one row per CTA of the backward kernel.  In host code this name is only a handle for the
// runtime's symbol table, not a device address: the address each device gave its copy comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_dgain_partials[SEGPT_NOALLOC_MAX_PARTIAL_ROWS * SEGPT_NOALLOC_MAX_D];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_mutex;
thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(-10, std::string("cudaGetDevice failed: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(-11, "device index out of range");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_dgain_partials);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(-12, std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = static_cast<float*>(ptr);
  }
  *out = g_scratch_addr[dev];
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int segpt_add_rmsnorm_bwd_noalloc(const void* dy, const float* dres_in, const float* x, const float* gain,
                                             const float* rstd, float* dres, void* dres_lp, float* dgain, int T, int d,
                                             float scale, int bf16, void* stream) {
  if (dy == nullptr || x == nullptr || gain == nullptr || rstd == nullptr || dres == nullptr || dres_lp == nullptr || dgain == nullptr)
    return fail(-1, "null pointer argument");
  if (T < 1 || d < 4 || d % 4 != 0) return fail(-2, "T must be >= 1 and d a positive multiple of 4");
  if (d > SEGPT_NOALLOC_MAX_D)
    return fail(-3, "d = " + std::to_string(d) + " exceeds the built-in scratch (SEGPT_NOALLOC_MAX_D = " +
                        std::to_string(SEGPT_NOALLOC_MAX_D) + ")");
  if (seg::add_rmsnorm_bwd_grid(T) > SEGPT_NOALLOC_MAX_PARTIAL_ROWS) return fail(-4, "kernel grid exceeds the built-in scratch rows");
  if (!aligned16(dy) || !aligned16(x) || !aligned16(gain) || !aligned16(dres) || !aligned16(dres_lp) ||
      (dres_in != nullptr && !aligned16(dres_in)))
    return fail(-5, "matrix arguments must be 16-byte aligned");
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Every CTA writes its whole partial row before the column reduction reads it: nothing needs clearing.
  seg::add_rmsnorm_bwd(dy, dres_in, x, gain, rstd, dres, dres_lp, dgain, scratch, T, d, scale, bf16 != 0,
                       static_cast<cudaStream_t>(stream));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(-20, std::string("kernel launch failed: ") + cudaGetErrorString(e));
  g_last_error.clear();
  return 0;
}

extern "C" const char* segpt_noalloc_last_error(void) { return g_last_error.c_str(); }
