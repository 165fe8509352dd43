// Position-bias tensors of disentangled attention, in key-indexed form.
//
//   bias[b,h,q,k] = C2P[q, lut_c2p(q-k)] + P2C[k, lut_p2c(q-k)]              (build)
//   dC2P[q, j] = sum_{k : lut_c2p(q-k) = j} dbias[b,h,q,k]                     (scatter, rows = queries)
//   dP2C[k, j] = sum_{q : lut_p2c(q-k) = j} dbias[b,h,q,k]                     (scatter, rows = keys)
//
// Gathering once into a [q, k] layout lets the attention kernels read and write the position
// terms as contiguous 16-byte vectors per query row instead of bucket-indexed 2-byte
// gathers and atomics. The kernels tile the (q, k) plane and go through shared memory where a
// transposition is needed, so that every global access is a coalesced run of table entries or
// bias columns.
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

constexpr int kT = 64;  // build: (q, k) tile edge

// grid (k-tiles, q-tiles, B*heads), 256 threads. The C2P term is gathered with lanes along k
// (consecutive table entries), the P2C term with lanes along q (again consecutive entries of
// one key's row); the tile is transposed through shared memory in between.
__global__ void __launch_bounds__(256)
posbias_build_kernel(const __nv_bfloat16* __restrict__ c2p, const __nv_bfloat16* __restrict__ p2c,
                     const unsigned short* __restrict__ lut_c2p, const unsigned short* __restrict__ lut_p2c,
                     __nv_bfloat16* __restrict__ bias, int S, int ldb, int heads, int span2) {
  __shared__ float tile[kT][kT + 1];
  const int tid = threadIdx.x;
  const int k0 = blockIdx.x * kT, q0 = blockIdx.y * kT;
  const int b = blockIdx.z / heads, h = blockIdx.z % heads;
  const long long row_stride = static_cast<long long>(heads) * span2;
  const long long base = static_cast<long long>(b) * S * row_stride + static_cast<long long>(h) * span2;
#pragma unroll 4
  for (int e = tid; e < kT * kT; e += 256) {
    const int r = e / kT, c = e % kT;
    const int q = q0 + r, k = k0 + c;
    float v = 0.f;
    if (c2p && q < S && k < S) v = __bfloat162float(c2p[base + q * row_stride + __ldg(lut_c2p + (q - k + S - 1))]);
    tile[r][c] = v;
  }
  __syncthreads();
  if (p2c) {
#pragma unroll 4
    for (int e = tid; e < kT * kT; e += 256) {
      const int c = e / kT, r = e % kT;  // lanes along q
      const int q = q0 + r, k = k0 + c;
      if (q < S && k < S) tile[r][c] += __bfloat162float(p2c[base + k * row_stride + __ldg(lut_p2c + (q - k + S - 1))]);
    }
    __syncthreads();
  }
  __nv_bfloat16* out = bias + static_cast<long long>(blockIdx.z) * S * ldb;
  for (int e = tid; e < kT * kT / 2; e += 256) {
    const int r = e / (kT / 2), c = (e % (kT / 2)) * 2;
    const int q = q0 + r, k = k0 + c;
    if (q < S && k < ldb)
      *reinterpret_cast<__nv_bfloat162*>(out + static_cast<long long>(q) * ldb + k) =
          __floats2bfloat162_rn(tile[r][c], tile[r][c + 1]);
  }
}

constexpr int kRows = 32;    // scatter: table rows (queries or keys) owned by one block
constexpr int kOther = 128;  // scatter: extent of the other axis processed per iteration

// grid (row-chunks, heads, B), 256 threads; acc[32][span2] in shared memory, reduced with
// shared-memory atomics (the only collisions are offsets that share a log bucket).
template <bool ROWS_ARE_KEYS>
__global__ void __launch_bounds__(256)
posbias_scatter_kernel(const __nv_bfloat16* __restrict__ dbias, const unsigned short* __restrict__ lut,
                       __nv_bfloat16* __restrict__ dtab, int S, int ldb, int heads, int span2) {
  extern __shared__ float acc[];  // [32][span2 + 1]
  const int tid = threadIdx.x;
  const int r0 = blockIdx.x * kRows, h = blockIdx.y, b = blockIdx.z;
  const int stride = span2 + 1;
  for (int i = tid; i < kRows * stride; i += 256) acc[i] = 0.f;
  __syncthreads();
  const __nv_bfloat16* src = dbias + (static_cast<long long>(b) * heads + h) * S * ldb;
  if (!ROWS_ARE_KEYS) {
    // rows of dbias are queries: 32 rows x 128 keys per iteration, 16-byte loads along k
    for (int oc = 0; oc < S; oc += kOther) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int rr = tid / 16 + half * 16, c8 = (tid % 16) * 8;
        const int q = r0 + rr, k = oc + c8;
        if (q < S && k < S) {
          const uint4 u = *reinterpret_cast<const uint4*>(src + static_cast<long long>(q) * ldb + k);
          const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float f = __bfloat162float(v[j]);
            if (f != 0.f && k + j < S) atomicAdd(&acc[rr * stride + __ldg(lut + (q - (k + j) + S - 1))], f);
          }
        }
      }
    }
  } else {
    // table rows are keys (32 contiguous columns of dbias): 128 query rows per iteration
    for (int oc = 0; oc < S; oc += kOther) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int rr = tid / 4 + half * 64, c8 = (tid % 4) * 8;
        const int q = oc + rr, k = r0 + c8;
        if (q < S && k < S) {
          const uint4 u = *reinterpret_cast<const uint4*>(src + static_cast<long long>(q) * ldb + k);
          const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float f = __bfloat162float(v[j]);
            if (f != 0.f && k + j < S) atomicAdd(&acc[(c8 + j) * stride + __ldg(lut + (q - (k + j) + S - 1))], f);
          }
        }
      }
    }
  }
  __syncthreads();
  const long long row_stride = static_cast<long long>(heads) * span2;
  for (int e = tid; e < kRows * span2 / 2; e += 256) {
    const int r = e / (span2 / 2), j = (e % (span2 / 2)) * 2;
    if (r0 + r < S)
      *reinterpret_cast<__nv_bfloat162*>(dtab + (static_cast<long long>(b) * S + r0 + r) * row_stride + h * span2 + j) =
          __floats2bfloat162_rn(acc[r * stride + j], acc[r * stride + j + 1]);
  }
}

}  // namespace

extern "C" int db200_posbias_build(const void* c2p, const void* p2c, const void* lut_c2p, const void* lut_p2c, void* bias,
                                   int B, int S, int ldb, int heads, int span2, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if (ldb % 2) return -10;
  dim3 grid((ldb + kT - 1) / kT, (S + kT - 1) / kT, B * heads);
  posbias_build_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(c2p), static_cast<const __nv_bfloat16*>(p2c),
      static_cast<const unsigned short*>(lut_c2p), static_cast<const unsigned short*>(lut_p2c),
      static_cast<__nv_bfloat16*>(bias), S, ldb, heads, span2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_posbias_scatter(const void* dbias, const void* lut, void* dtab, int rows_are_keys, int B, int S,
                                     int ldb, int heads, int span2, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  const int smem = kRows * (span2 + 1) * static_cast<int>(sizeof(float));
  if (smem > 200 * 1024 || (span2 % 2) || (ldb % 8)) return -12;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((S + kRows - 1) / kRows, heads, B);
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
