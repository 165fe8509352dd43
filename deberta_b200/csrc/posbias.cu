// Position-bias tensors of disentangled attention, in key-indexed form.
//
//   bias[b,h,q,k] = C2P[q, lut_c2p(q-k)] + P2C[k, lut_p2c(q-k)]              (build)
//   dC2P[q, j] = sum_{k : lut_c2p(q-k) = j} dbias[b,h,q,k]                     (scatter, rows = queries)
//   dP2C[k, j] = sum_{q : lut_p2c(q-k) = j} dbias[b,h,q,k]                     (scatter, rows = keys)
//
// Gathering once into a [q, k] layout lets the attention kernels read and write the position
// terms as contiguous 16-byte vectors per query row instead of bucket-indexed 2-byte
// gathers and atomics. All three kernels work on 32x32 (q, k) chunks staged through shared
// memory so that every global access is coalesced; the lookup tables (monotone in q-k) bound
// the bucket window a chunk can touch.
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

constexpr int kChunk = 32;
constexpr int kWin = 2 * kChunk;  // a 32x32 chunk spans 63 consecutive offsets q-k

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// grid (q-chunks, heads, B), 256 threads
__global__ void __launch_bounds__(256)
posbias_build_kernel(const __nv_bfloat16* __restrict__ c2p, const __nv_bfloat16* __restrict__ p2c,
                     const unsigned short* __restrict__ lut_c2p, const unsigned short* __restrict__ lut_p2c,
                     __nv_bfloat16* __restrict__ bias, int S, int ldb, int heads, int span2) {
  extern __shared__ unsigned short lut_smem[];
  __shared__ float cw[kChunk][kWin + 1];
  __shared__ float pw[kChunk][kWin + 1];
  unsigned short* lc = lut_smem;
  unsigned short* lp = lut_smem + 2 * S;
  const int tid = threadIdx.x;
  const int q0 = blockIdx.x * kChunk, h = blockIdx.y, b = blockIdx.z;
  for (int i = tid; i < 2 * S - 1; i += 256) {
    lc[i] = c2p ? lut_c2p[i] : 0;
    lp[i] = p2c ? lut_p2c[i] : 0;
  }
  __syncthreads();
  const long long row_stride = static_cast<long long>(heads) * span2;
  __nv_bfloat16* out = bias + (static_cast<long long>(b) * heads + h) * S * ldb;
  for (int kc = 0; kc < S; kc += kChunk) {
    const int d_lo = clampi(q0 - (kc + kChunk - 1) + S - 1, 0, 2 * S - 2);
    const int d_hi = clampi(q0 + kChunk - 1 - kc + S - 1, 0, 2 * S - 2);
    // lut_c2p grows with q-k, lut_p2c shrinks: the window is bounded by the chunk's corner offsets
    const int c_lo = min(lc[d_lo], lc[d_hi]), p_lo = min(lp[d_lo], lp[d_hi]);
    for (int e = tid; e < kChunk * kWin; e += 256) {
      const int r = e / kWin, j = e % kWin;
      float vc = 0.f, vp = 0.f;
      if (c2p && q0 + r < S && c_lo + j < span2)
        vc = __bfloat162float(c2p[(static_cast<long long>(b) * S + q0 + r) * row_stride + h * span2 + c_lo + j]);
      if (p2c && kc + r < S && p_lo + j < span2)
        vp = __bfloat162float(p2c[(static_cast<long long>(b) * S + kc + r) * row_stride + h * span2 + p_lo + j]);
      cw[r][j] = vc;
      pw[r][j] = vp;
    }
    __syncthreads();
    for (int e = tid; e < kChunk * kChunk; e += 256) {
      const int r = e / kChunk, c = e % kChunk;
      const int q = q0 + r, k = kc + c;
      if (q < S && k < S) {
        const int d = q - k + S - 1;
        const float v = cw[r][clampi(lc[d] - c_lo, 0, kWin - 1)] + pw[c][clampi(lp[d] - p_lo, 0, kWin - 1)];
        out[static_cast<long long>(q) * ldb + k] = __float2bfloat16(v);
      }
    }
    __syncthreads();
  }
}

// grid (row-chunks, heads, B), 256 threads. ROWS_ARE_KEYS = false: rows are queries (dC2P);
// true: rows are keys (dP2C). acc[32][span2] lives in shared memory.
template <bool ROWS_ARE_KEYS>
__global__ void __launch_bounds__(256)
posbias_scatter_kernel(const __nv_bfloat16* __restrict__ dbias, const unsigned short* __restrict__ lut,
                       __nv_bfloat16* __restrict__ dtab, int S, int ldb, int heads, int span2) {
  extern __shared__ float smem_f[];
  float* acc = smem_f;                                           // [32][span2 + 1]
  float* tile = smem_f + kChunk * (span2 + 1);                   // [32][33]
  unsigned short* ls = reinterpret_cast<unsigned short*>(tile + kChunk * (kChunk + 1));  // [2S-1]
  const int tid = threadIdx.x;
  const int r0 = blockIdx.x * kChunk, h = blockIdx.y, b = blockIdx.z;
  const int stride = span2 + 1;
  for (int i = tid; i < kChunk * stride; i += 256) acc[i] = 0.f;
  for (int i = tid; i < 2 * S - 1; i += 256) ls[i] = lut[i];
  __syncthreads();
  const __nv_bfloat16* src = dbias + (static_cast<long long>(b) * heads + h) * S * ldb;
  for (int oc = 0; oc < S; oc += kChunk) {  // the other axis, 32 at a time
    for (int e = tid; e < kChunk * kChunk; e += 256) {
      const int rr = e / kChunk, cc = e % kChunk;  // (row in memory = query, contiguous col = key)
      const int q = ROWS_ARE_KEYS ? oc + rr : r0 + rr;
      const int k = ROWS_ARE_KEYS ? r0 + cc : oc + cc;
      float v = 0.f;
      if (q < S && k < S) v = __bfloat162float(src[static_cast<long long>(q) * ldb + k]);
      tile[rr * (kChunk + 1) + cc] = v;
    }
    __syncthreads();
    for (int e = tid; e < kChunk * kChunk; e += 256) {
      const int rr = e / kChunk, cc = e % kChunk;
      const int q = ROWS_ARE_KEYS ? oc + rr : r0 + rr;
      const int k = ROWS_ARE_KEYS ? r0 + cc : oc + cc;
      const float v = tile[rr * (kChunk + 1) + cc];
      if (v != 0.f && q < S && k < S) {
        const int j = ls[q - k + S - 1];
        atomicAdd(&acc[(ROWS_ARE_KEYS ? cc : rr) * stride + j], v);
      }
    }
    __syncthreads();
  }
  const long long row_stride = static_cast<long long>(heads) * span2;
  for (int e = tid; e < kChunk * span2; e += 256) {
    const int r = e / span2, j = e % span2;
    if (r0 + r < S)
      dtab[(static_cast<long long>(b) * S + r0 + r) * row_stride + h * span2 + j] = __float2bfloat16(acc[r * stride + j]);
  }
}

}  // namespace

extern "C" int db200_posbias_build(const void* c2p, const void* p2c, const void* lut_c2p, const void* lut_p2c, void* bias,
                                   int B, int S, int ldb, int heads, int span2, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  const int smem = 2 * 2 * S * static_cast<int>(sizeof(unsigned short));
  if (smem > 40 * 1024) return -12;
  dim3 grid((S + kChunk - 1) / kChunk, heads, B);
  posbias_build_kernel<<<grid, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(c2p), static_cast<const __nv_bfloat16*>(p2c),
      static_cast<const unsigned short*>(lut_c2p), static_cast<const unsigned short*>(lut_p2c),
      static_cast<__nv_bfloat16*>(bias), S, ldb, heads, span2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_posbias_scatter(const void* dbias, const void* lut, void* dtab, int rows_are_keys, int B, int S,
                                     int ldb, int heads, int span2, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  const int smem = (kChunk * (span2 + 1) + kChunk * (kChunk + 1)) * static_cast<int>(sizeof(float)) +
                   2 * S * static_cast<int>(sizeof(unsigned short));
  if (smem > 200 * 1024) return -12;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((S + kChunk - 1) / kChunk, heads, B);
  auto db = static_cast<const __nv_bfloat16*>(dbias);
  auto lt = static_cast<const unsigned short*>(lut);
  auto dt = static_cast<__nv_bfloat16*>(dtab);
  if (rows_are_keys) {
    static bool cfg = false;
    if (!cfg) {
      if (cudaFuncSetAttribute(posbias_scatter_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return -3;
      cfg = true;
    }
    posbias_scatter_kernel<true><<<grid, 256, smem, st>>>(db, lt, dt, S, ldb, heads, span2);
  } else {
    static bool cfg = false;
    if (!cfg) {
      if (cudaFuncSetAttribute(posbias_scatter_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return -3;
      cfg = true;
    }
    posbias_scatter_kernel<false><<<grid, 256, smem, st>>>(db, lt, dt, S, ldb, heads, span2);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
