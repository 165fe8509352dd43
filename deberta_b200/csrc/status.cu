// Device-side status word: kernels record here (first error wins) when a bounded wait
// ran out, instead of trapping or spinning forever. The host reads it after a sync.
#include "kernels.h"

#include <cuda_runtime.h>

namespace {
__device__ int g_status_word = 0;
constexpr int kMaxDevices = 16;
int* g_status_addr[kMaxDevices] = {nullptr};
}  // namespace

// Programmatic dependent launch for the kernels that support it (tc05.cuh); on by default.
namespace {
int g_pdl = 1;
}
extern "C" int db200_pdl_enabled(void) { return g_pdl; }
extern "C" int db200_set_pdl(int on) {
  const int old = g_pdl;
  g_pdl = on ? 1 : 0;
  return old;
}

extern "C" int* db200_status_ptr(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!g_status_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_addr[dev] = static_cast<int*>(p);
  }
  return g_status_addr[dev];
}

// Copy the status word into `dst` (device or pinned host int) in stream order, without a synchronisation.
extern "C" int db200_status_snapshot(int* dst, void* stream) {
  int* p = db200_status_ptr();
  if (!p || !dst) return -1;
  return cudaMemcpyAsync(dst, p, sizeof(int), cudaMemcpyDefault, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
             ? 0
             : -2;
}

extern "C" int db200_status_read_and_clear(void) {
  int* p = db200_status_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) {
    int zero = 0;
    cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}
