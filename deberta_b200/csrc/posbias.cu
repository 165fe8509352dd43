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
#include "tc05.cuh"

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


// Interior tiles (all 64 x 64 entries valid), the common case: same data flow as the kernel above with
// the offset -> bucket map of the tile (127 offsets) staged in shared memory and 32-bit index arithmetic.
// grid (S/64, S/64, B*heads), 256 threads; needs S % 64 == 0.
template <bool HAS_C, bool HAS_P>
__global__ void __launch_bounds__(256)
posbias_build_full_kernel(const __nv_bfloat16* __restrict__ c2p, const __nv_bfloat16* __restrict__ p2c,
                          const unsigned short* __restrict__ lut_c2p, const unsigned short* __restrict__ lut_p2c,
                          __nv_bfloat16* __restrict__ bias, int S, int ldb, int heads, int span2) {
  __shared__ float tile[kT][kT + 1];
  __shared__ unsigned short slc[128], slp[128];
  const int tid = threadIdx.x;
  const int k0 = blockIdx.x * kT, q0 = blockIdx.y * kT;
  const int b = blockIdx.z / heads, h = blockIdx.z % heads;
  const int row_stride = heads * span2;
  const long long base = static_cast<long long>(b) * S * row_stride + static_cast<long long>(h) * span2;
  if (tid < 127) {  // offsets q-k of this tile: q0-k0-63 .. q0-k0+63
    const int d = q0 - k0 - 63 + tid + S - 1;
    if (HAS_C) slc[tid] = lut_c2p[d];
    if (HAS_P) slp[tid] = lut_p2c[d];
  }
  __syncthreads();
  const int lane64 = tid & 63, grp = tid >> 6;
  // all 16 bucket indices, then all 16 table reads, then the shared-memory updates: the reads of one
  // thread are independent and stay in flight together
  if (HAS_C) {  // lanes along k: consecutive keys read consecutive table entries of one query row
    const unsigned short* src = reinterpret_cast<const unsigned short*>(c2p + base) + (q0 + grp) * row_stride;
    const unsigned short* l = slc + (grp - lane64 + 63);
    int idx[16];
    unsigned short raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) idx[i] = i * 4 * row_stride + l[4 * i];
#pragma unroll
    for (int i = 0; i < 16; ++i) raw[i] = __ldg(src + idx[i]);
#pragma unroll
    for (int i = 0; i < 16; ++i) tile[grp + 4 * i][lane64] = __uint_as_float(static_cast<unsigned int>(raw[i]) << 16);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) tile[grp + 4 * i][lane64] = 0.f;
  }
  __syncthreads();
  if (HAS_P) {  // lanes along q: consecutive queries read consecutive table entries of one key row
    const unsigned short* src = reinterpret_cast<const unsigned short*>(p2c + base) + (k0 + grp) * row_stride;
    const unsigned short* l = slp + (lane64 - grp + 63);
    int idx[16];
    unsigned short raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) idx[i] = i * 4 * row_stride + l[-4 * i];
#pragma unroll
    for (int i = 0; i < 16; ++i) raw[i] = __ldg(src + idx[i]);
#pragma unroll
    for (int i = 0; i < 16; ++i) tile[lane64][grp + 4 * i] += __uint_as_float(static_cast<unsigned int>(raw[i]) << 16);
    __syncthreads();
  }
  __nv_bfloat16* out = bias + (static_cast<long long>(blockIdx.z) * S + q0) * ldb + k0;
  const int c2 = (tid & 31) * 2, r0 = tid >> 5;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + 8 * i;
    *reinterpret_cast<__nv_bfloat162*>(out + r * ldb + c2) = __floats2bfloat162_rn(tile[r][c2], tile[r][c2 + 1]);
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


// ---- scatter by prefix sums -----------------------------------------------------------------
// When every bucket j collects one contiguous run of offsets  lo[j] <= q-k <= hi[j]  (true for the
// log-bucket maps, which are monotone in q-k), the scatter is a difference of prefix sums along the
// row (keys) or the column (queries) of dbias: no atomics, every element read once.
//
// edges: int[span2 + 2] = {sign, E_0 .. E_span2}. With sign = +1 bucket j collects the offsets E_j <= q-k < E_{j+1},
// with sign = -1 the offsets E_{j+1} <= q-k < E_j (the bucket index falls as q-k grows); an unused bucket has
// E_j = E_{j+1}. Every output is then the difference of the prefix sums at two neighbouring edges, so a thread that
// writes eight consecutive buckets reads nine prefix values and stores 16 bytes.

// eight outputs sign * (g[t+1] - g[t]) (or the reverse for row scans) as one 16-byte store
__device__ __forceinline__ void store_edge_diffs(__nv_bfloat16* dst, const float (&g)[9], float sign) {
  uint4 u;
  __nv_bfloat162 w[4];
#pragma unroll
  for (int t = 0; t < 4; ++t)
    w[t] = __floats2bfloat162_rn(sign * (g[2 * t + 1] - g[2 * t]), sign * (g[2 * t + 2] - g[2 * t + 1]));
  u.x = *reinterpret_cast<uint32_t*>(&w[0]);
  u.y = *reinterpret_cast<uint32_t*>(&w[1]);
  u.z = *reinterpret_cast<uint32_t*>(&w[2]);
  u.w = *reinterpret_cast<uint32_t*>(&w[3]);
  *reinterpret_cast<uint4*>(dst) = u;
}

__device__ __forceinline__ float warp_inclusive_scan(float x, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  return x;
}

// rows of dbias are queries: one warp per query row. grid (ceil(S/8), heads, B), 256 threads.
__global__ void __launch_bounds__(256)
posbias_rowscan_kernel(const __nv_bfloat16* __restrict__ dbias, const int* __restrict__ ranges,
                       __nv_bfloat16* __restrict__ dtab, int S, int ldb, int heads, int span2) {
  extern __shared__ float sm[];
  tc05::pdl_launch_dependents();
  tc05::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stride = (S + 1) + ((S + 1) >> 3) + 1;
  // P[i] = sum of the first i keys, kept at word i + i/8: the lanes of the scan write 8 words apart
  int* edge = reinterpret_cast<int*>(sm);  // E_0 .. E_span2, 16-byte aligned for vector loads
  float* P = sm + ((span2 + 4) & ~3) + warp * stride;
  for (int i = threadIdx.x; i <= span2; i += 256) edge[i] = ranges[i + 1];
  const float sign = ranges[0] >= 0 ? 1.f : -1.f;
  __syncthreads();
  // (batch walked backwards: the attention backward wrote dbias in ascending order and its tail is still in the L2;
  // the column scan that follows walks forwards again and finds this kernel's tail)
  const int q = blockIdx.x * 8 + warp, h = blockIdx.y, b = gridDim.z - 1 - blockIdx.z;
  if (q >= S) return;
  const __nv_bfloat16* src = dbias + ((static_cast<long long>(b) * heads + h) * S + q) * ldb;
  float carry = 0.f;
  if (lane == 0) P[0] = 0.f;
  for (int base = 0; base < S; base += 256) {
    const int k = base + lane * 8;
    float v[8];
    if (k < S) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + k);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (k + j < S) ? __bfloat162float(e[j]) : 0.f;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
#pragma unroll
    for (int j = 1; j < 8; ++j) v[j] += v[j - 1];
    const float incl = warp_inclusive_scan(v[7], lane);
    const float off = carry + incl - v[7];
    if (k < S) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (k + j < S) P[(k + j + 1) + ((k + j + 1) >> 3)] = off + v[j];
    }
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  __syncwarp();
  __nv_bfloat16* dst = dtab + (static_cast<long long>(b) * S + q) * (static_cast<long long>(heads) * span2) + h * span2;
  // keys with offset q-k >= E are the first q-E+1 keys: g = P[clamp(q - E + 1)], and bucket j is sign * (g_j - g_{j+1})
  for (int j = lane * 8; j < span2; j += 256) {
    const int4 e0 = *reinterpret_cast<const int4*>(edge + j), e1 = *reinterpret_cast<const int4*>(edge + j + 4);
    const int e[9] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w, edge[j + 8]};
    float g[9];
#pragma unroll
    for (int t = 0; t < 9; ++t) {
      const int i = min(max(q + 1 - e[t], 0), S);
      g[t] = P[i + (i >> 3)];
    }
    store_edge_diffs(dst + j, g, -sign);
  }
}

// table rows are keys: a block owns kColKeys key columns of dbias and scans them along the queries.
// grid (ceil(S/kColKeys), heads, B), 256 threads; shared: T[kColKeys][stride] (16 keys keep six blocks per SM resident). Prefix i of a key sits at word
// i + (i >> sh) with 2^sh >= ceil(S/32): each lane scans a contiguous run of `per` queries, and the skew
// keeps the 32 lanes on different banks.
constexpr int kColKeys = 16;

template <int PER, int KEYS>  // PER > 0: ceil(S/32) known at compile time (the run of a lane lives in registers); 0: any S
__global__ void __launch_bounds__(256)
posbias_colscan_kernel(const __nv_bfloat16* __restrict__ dbias, const int* __restrict__ ranges,
                       __nv_bfloat16* __restrict__ dtab, int S, int ldb, int heads, int span2, int stride, int per, int sh) {
  extern __shared__ float sm[];
  tc05::pdl_launch_dependents();
  tc05::pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int* edge = reinterpret_cast<int*>(sm);  // E_0 .. E_span2, 16-byte aligned for vector loads
  float* tb = sm + ((span2 + 4) & ~3);     // T[KEYS][stride]
  for (int i = tid; i <= span2; i += 256) edge[i] = ranges[i + 1];
  const float sign = ranges[0] >= 0 ? 1.f : -1.f;
  const int k0 = blockIdx.x * KEYS, h = blockIdx.y, b = blockIdx.z;
  const __nv_bfloat16* src = dbias + (static_cast<long long>(b) * heads + h) * S * ldb + k0;
  constexpr int kGroups = KEYS / 8, kRowsPerPass = 256 / kGroups;
  const int cg = tid % kGroups;  // 8-key group of this thread
  for (int qb = tid / kGroups; qb < S; qb += 4 * kRowsPerPass) {  // four independent 16-byte loads in flight per thread
    uint4 u[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int q = qb + kRowsPerPass * t;
      u[t] = q < S ? *reinterpret_cast<const uint4*>(src + static_cast<long long>(q) * ldb + cg * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int q = qb + kRowsPerPass * t;
      if (q < S) {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[t]);
        const int w = (q + 1) + ((q + 1) >> sh);
#pragma unroll
        for (int j = 0; j < 8; ++j) tb[(cg * 8 + j) * stride + w] = __bfloat162float(e[j]);
      }
    }
  }
  if (tid < KEYS) tb[tid * stride] = 0.f;
  __syncthreads();
  const long long row_stride = static_cast<long long>(heads) * span2;
  for (int kk = warp * (KEYS / 8); kk < (warp + 1) * (KEYS / 8); ++kk) {
    const int k = k0 + kk;
    if (k >= S) break;  // warp-uniform
    float* T = tb + kk * stride;  // T[phys(i)] = sum of the first i queries
    // lane owns prefixes i = lane*per + 1 .. lane*per + per
    const int first = lane * per + 1;
    if (PER > 0) {
      float x[PER > 0 ? PER : 1];
#pragma unroll
      for (int o = 0; o < PER; ++o) {
        const int i = first + o;
        x[o] = (i <= S) ? T[i + (i >> sh)] : 0.f;
      }
#pragma unroll
      for (int o = 1; o < PER; ++o) x[o] += x[o - 1];
      const float run = x[PER > 0 ? PER - 1 : 0];
      const float off = warp_inclusive_scan(run, lane) - run;
#pragma unroll
      for (int o = 0; o < PER; ++o) {
        const int i = first + o;
        if (i <= S) T[i + (i >> sh)] = x[o] + off;
      }
    } else {
      float run = 0.f;
      for (int o = 0; o < per; ++o) {
        const int i = first + o;
        if (i <= S) {
          run += T[i + (i >> sh)];
          T[i + (i >> sh)] = run;
        }
      }
      const float off = warp_inclusive_scan(run, lane) - run;
      for (int o = 0; o < per; ++o) {
        const int i = first + o;
        if (i <= S) T[i + (i >> sh)] += off;
      }
    }
    __syncwarp();
    __nv_bfloat16* dst = dtab + (static_cast<long long>(b) * S + k) * row_stride + h * span2;
    // queries with offset q-k < E are the first k+E queries: g = T[clamp(k + E)], and bucket j is sign * (g_{j+1} - g_j)
    for (int j = lane * 8; j < span2; j += 256) {
      const int4 e0 = *reinterpret_cast<const int4*>(edge + j), e1 = *reinterpret_cast<const int4*>(edge + j + 4);
      const int e[9] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w, edge[j + 8]};
      float g[9];
#pragma unroll
      for (int t = 0; t < 9; ++t) {
        const int i = min(max(k + e[t], 0), S);
        g[t] = T[i + (i >> sh)];
      }
      store_edge_diffs(dst + j, g, sign);
    }
  }
}

}  // namespace

extern "C" int db200_posbias_build(const void* c2p, const void* p2c, const void* lut_c2p, const void* lut_p2c, void* bias,
                                   int B, int S, int ldb, int heads, int span2, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if (ldb % 2) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto c = static_cast<const __nv_bfloat16*>(c2p);
  auto pp = static_cast<const __nv_bfloat16*>(p2c);
  auto lc = static_cast<const unsigned short*>(lut_c2p);
  auto lp = static_cast<const unsigned short*>(lut_p2c);
  auto o = static_cast<__nv_bfloat16*>(bias);
  if (S % kT == 0 && ldb == S && static_cast<long long>(S) * heads * span2 < (1ll << 30)) {
    dim3 grid(S / kT, S / kT, B * heads);
    if (c && pp)
      posbias_build_full_kernel<true, true><<<grid, 256, 0, st>>>(c, pp, lc, lp, o, S, ldb, heads, span2);
    else if (c)
      posbias_build_full_kernel<true, false><<<grid, 256, 0, st>>>(c, pp, lc, lp, o, S, ldb, heads, span2);
    else
      posbias_build_full_kernel<false, true><<<grid, 256, 0, st>>>(c, pp, lc, lp, o, S, ldb, heads, span2);
  } else {
    dim3 grid((ldb + kT - 1) / kT, (S + kT - 1) / kT, B * heads);
    posbias_build_kernel<<<grid, 256, 0, st>>>(c, pp, lc, lp, o, S, ldb, heads, span2);
  }
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

extern "C" int db200_posbias_scatter_ranges(const void* dbias, const void* ranges, void* dtab, int rows_are_keys, int B,
                                            int S, int ldb, int heads, int span2, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if ((span2 % 8) || (ldb % 8) || ldb < S) return -12;  // eight buckets per 16-byte store
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto db = static_cast<const __nv_bfloat16*>(dbias);
  auto rg = static_cast<const int*>(ranges);
  auto dt = static_cast<__nv_bfloat16*>(dtab);
  constexpr int kMaxSmem = 200 * 1024;
  if (rows_are_keys) {
    if (ldb % kColKeys) return -12;  // key groups are read with 16-byte loads up to the padded width
    const int per = (S + 31) / 32;
    int sh = 0;
    while ((1 << sh) < per) ++sh;
    int stride = (S + 1) + ((S + 1) >> sh) + 1;
    stride |= 1;  // odd: the 32 key rows start on different banks
    const int smem = kColKeys * stride * 4 + 2 * span2 * 4;
    if (smem > kMaxSmem) return -12;
    // 16 keys per block measured fastest (228 us against 253 / 492 us for 32 / 64 keys at B=32, S=512, 12 heads)
    auto kern = posbias_colscan_kernel<0, kColKeys>;
    if (per == 16) kern = posbias_colscan_kernel<16, kColKeys>;
    else if (per == 8) kern = posbias_colscan_kernel<8, kColKeys>;
    else if (per == 32) kern = posbias_colscan_kernel<32, kColKeys>;
    else if (per == 4) kern = posbias_colscan_kernel<4, kColKeys>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem) != cudaSuccess) return -3;
    tc05::launch_pdl(kern, dim3((S + kColKeys - 1) / kColKeys, heads, B), dim3(256), smem, st, db, rg, dt, S, ldb, heads, span2,
                     stride, per, sh);
  } else {
    const int smem = 8 * ((S + 1) + ((S + 1) >> 3) + 1) * 4 + 2 * span2 * 4;
    if (smem > kMaxSmem) return -12;
    static bool cfg = false;
    if (!cfg) {
      if (cudaFuncSetAttribute(posbias_rowscan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem) != cudaSuccess)
        return -3;
      cfg = true;
    }
    tc05::launch_pdl(posbias_rowscan_kernel, dim3((S + 7) / 8, heads, B), dim3(256), smem, st, db, rg, dt, S, ldb, heads, span2);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
