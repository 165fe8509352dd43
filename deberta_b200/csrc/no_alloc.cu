// Fused vocabulary cross-entropy forward with library-owned scratch (see no_alloc.h).
#include "no_alloc.h"

#include "kernels.h"

#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr long long kScratchFloats = 4ll * DB200_NOALLOC_MAX_PARTIALS + DB200_NOALLOC_MAX_ROWS;

// One array per loaded copy of the library and per GPU; lives until the process exits.
static __device__ __align__(256) float g_ce_scratch[kScratchFloats];

constexpr int kMaxDevices = 16;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device. `g_ce_scratch` itself is only a
// host-side handle; passing it to a kernel would hand the kernel a host address.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!g_scratch_addr[dev]) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_ce_scratch) != cudaSuccess) return nullptr;
    g_scratch_addr[dev] = ptr;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int db200_noalloc_prepare(void) {
  if (!scratch_for_current_device()) return DB200_NOALLOC_NO_DEVICE;
  return db200_gemm_preload_ce() == 0 ? DB200_NOALLOC_OK : DB200_NOALLOC_NO_DEVICE;
}

extern "C" int db200_vocab_ce_forward_noalloc(const void* x, const void* weight, const void* bias,
                                              const long long* labels, const unsigned char* forbidden, int rows,
                                              int vocab, int hidden, float temperature, unsigned long long seed,
                                              float* lse, float* loss_rows, long long* sampled, void* stream) {
  if (rows == 0) return DB200_NOALLOC_OK;
  if (!x || !weight || !labels || !lse || !loss_rows || !sampled || rows < 0 || vocab <= 0 || hidden <= 0 ||
      (hidden % 8) || !(temperature > 0.f) || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(weight) & 15))
    return DB200_NOALLOC_BAD_ARGS;
  const int tile_n = db200_gemm_tile_n(vocab);
  const long long tiles_n = (static_cast<long long>(vocab) + tile_n - 1) / tile_n;
  if (rows > DB200_NOALLOC_MAX_ROWS || tiles_n * rows > DB200_NOALLOC_MAX_PARTIALS) return DB200_NOALLOC_TOO_LARGE;
  float* scratch = scratch_for_current_device();
  if (!scratch) return DB200_NOALLOC_NO_DEVICE;
  float* part = scratch;                                        // [4, tiles_n, rows]
  float* label_logit = scratch + 4ll * DB200_NOALLOC_MAX_PARTIALS;  // [rows]
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Rows whose label is outside the vocabulary never write their label logit: start from zero,
  // not from what the previous call left behind. The partials are fully overwritten.
  if (cudaMemsetAsync(label_logit, 0, static_cast<size_t>(rows) * sizeof(float), st) != cudaSuccess)
    return DB200_NOALLOC_NO_DEVICE;
  GemmArgs a{};
  a.A = x;
  a.B = weight;
  a.bias = bias;
  a.M = rows;
  a.N = vocab;
  a.K = hidden;
  a.batch = 1;
  a.lda = hidden;
  a.ldb = hidden;
  a.alpha = 1.f;
  a.epi = EPI_CE_FWD;
  a.labels = labels;
  a.forbidden = forbidden;
  a.inv_temp = 1.f / temperature;
  a.seed = seed;
  a.ce_part = part;
  a.label_logit = label_logit;
  int rc = db200_gemm_bf16(&a, stream);
  if (rc) return rc;
  return db200_ce_combine(part, label_logit, static_cast<int>(tiles_n), rows, lse, loss_rows, sampled, stream);
}

extern "C" const char* db200_noalloc_strerror(int code) {
  switch (code) {
    case DB200_NOALLOC_OK: return "ok";
    case DB200_NOALLOC_TOO_LARGE:
      return "problem exceeds the built-in scratch (vocabulary tiles x rows > 2^21 or rows > 8192)";
    case DB200_NOALLOC_BAD_ARGS:
      return "bad arguments (null pointer, operand not 16-byte aligned, hidden size not a multiple of 8, "
             "or temperature <= 0)";
    case DB200_NOALLOC_NO_DEVICE: return "could not resolve or clear the scratch array on the current CUDA device";
    default: return "launcher error (see the codes of db200_gemm_bf16)";
  }
}
