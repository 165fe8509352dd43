// LayerNorm / RMSNorm forward and backward for bf16 activations, fp32 statistics.
// One warp owns one row; the row lives in registers (16-byte vector loads), so every
// element is read once and written once. Backward accumulates the weight / bias
// gradients in registers across the rows a warp visits and flushes them once per block
// with fp32 atomics (directly into the optimizer's fp32 gradient buffer when given).
#include "kernels.h"
#include "tc05.cuh"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

constexpr int kWarpsPerBlock = 8;

// V = number of 8-element vectors each lane holds: covers H <= 256 * V.
template <int V, bool RMS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, const unsigned char* __restrict__ row_keep,
                __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                int H, float eps) {
  tc05::pdl_launch_dependents();
  tc05::pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  for (long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + warp; row < rows;
       row += static_cast<long long>(gridDim.x) * kWarpsPerBlock) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    float v[V][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        unpack8(xr[c], v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      }
    }
    float mean = 0.f;
    if (!RMS) mean = warp_sum(s) / H;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[i][j] - mean;
          ss += d * d;
        }
      }
    }
    const float var = warp_sum(ss) / H;
    const float rstd = rsqrtf(var + eps);
    const float keep = (row_keep == nullptr || row_keep[row]) ? 1.f : 0.f;
    uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float g[8], b[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(gamma)[c], g);
        if (!RMS && beta) unpack8(reinterpret_cast<const uint4*>(beta)[c], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float t = (v[i][j] - mean) * rstd * g[j];
          if (!RMS && beta) t += b[j];
          o[j] = t * keep;
        }
        yr[c] = pack8(o);
      }
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
  }
}

template <int V, bool RMS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (V <= 2) ? 2 : 1)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const unsigned char* __restrict__ row_keep,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int H) {
  __shared__ float red[kWarpsPerBlock][32 * 8 + 1];
  tc05::pdl_launch_dependents();
  tc05::pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  uint4 gq[V];  // gamma stays packed (bf16): the registers go to the next row's loads
  float dg[V][8], db[V][8];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = lane + i * 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; }
    gq[i] = c < nvec ? reinterpret_cast<const uint4*>(gamma)[c] : make_uint4(0, 0, 0, 0);
  }
  // The rows of a warp are processed one after the other and each needs two row reductions before it can be written,
  // so the loads of the NEXT row are issued before the current row's arithmetic: their latency hides behind it.
  const long long row_step = static_cast<long long>(gridDim.x) * kWarpsPerBlock;
  long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + warp;
  uint4 xq[V], dq[V];  // raw bf16 vectors of the current row
  float keep = 0.f, mean = 0.f, rstd = 0.f;
  auto fetch = [&](long long r, uint4 (&xo)[V], uint4 (&dout)[V], float& k, float& m, float& rs) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * H);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + r * H);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        xo[i] = xr[c];
        dout[i] = dyr[c];
      }
    }
    k = (row_keep == nullptr || row_keep[r]) ? 1.f : 0.f;
    m = RMS ? 0.f : mean_in[r];
    rs = rstd_in[r];
  };
  if (row < rows) fetch(row, xq, dq, keep, mean, rstd);
  for (; row < rows; row += row_step) {
    uint4 xn[V], dn[V];
    float keep_n = 0.f, mean_n = 0.f, rstd_n = 0.f;
    constexpr bool kAhead = V <= 4;  // (wider rows have no registers to spare: they fetch at the bottom of the loop)
    if (kAhead && row + row_step < rows) fetch(row + row_step, xn, dn, keep_n, mean_n, rstd_n);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float xh[8], dyv[8], g[8];
        unpack8(xq[i], xh);
        unpack8(dq[i], dyv);
        unpack8(gq[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xn_ = (xh[j] - mean) * rstd;
          const float d = dyv[j] * keep;
          const float dxh = d * g[j];
          s1 += dxh;
          s2 += dxh * xn_;
          dg[i][j] += d * xn_;
          db[i][j] += d;
        }
      }
    }
    s1 = RMS ? 0.f : warp_sum(s1) / H;
    s2 = warp_sum(s2) / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float xh[8], dyv[8], g[8], o[8];
        unpack8(xq[i], xh);  // (unpacked again rather than kept: the registers hold the next row's loads instead)
        unpack8(dq[i], dyv);
        unpack8(gq[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          o[j] = rstd * (dyv[j] * keep * g[j] - s1 - (xh[j] - mean) * rstd * s2);
        dxr[c] = pack8(o);
      }
    }
    if (!kAhead && row + row_step < rows) fetch(row + row_step, xn, dn, keep_n, mean_n, rstd_n);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      xq[i] = xn[i];
      dq[i] = dn[i];
    }
    keep = keep_n;
    mean = mean_n;
    rstd = rstd_n;
  }
  // block-level reduction of the parameter gradients, one vector slot at a time
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = lane + i * 32;
    for (int pass = 0; pass < 2; ++pass) {
      if (pass == 1 && (RMS || dbeta == nullptr)) break;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = pass == 0 ? dg[i][j] : db[i][j];
      __syncthreads();
      for (int e = threadIdx.x; e < 256; e += blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerBlock; ++w) acc += red[w][e];
        const int col = (i * 32 + (e >> 3)) * 8 + (e & 7);
        if (col < H && acc != 0.f) atomicAdd((pass == 0 ? dgamma : dbeta) + col, acc);
      }
    }
    (void)c;
  }
}

template <bool RMS>
int launch_fwd(const void* x, const void* g, const void* b, const void* keep, void* y, float* mean, float* rstd,
               int rows, int H, float eps, cudaStream_t st) {
  const int blocks = min((rows + kWarpsPerBlock - 1) / kWarpsPerBlock, 148 * 8);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(g);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto K = static_cast<const unsigned char*>(keep);
  auto Y = static_cast<__nv_bfloat16*>(y);
  if (H <= 256) tc05::launch_pdl(norm_fwd_kernel<1, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, X, G, B, K, Y, mean, rstd, rows, H, eps);
  else if (H <= 1024) tc05::launch_pdl(norm_fwd_kernel<4, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, X, G, B, K, Y, mean, rstd, rows, H, eps);
  else if (H <= 2048) tc05::launch_pdl(norm_fwd_kernel<8, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, X, G, B, K, Y, mean, rstd, rows, H, eps);
  else return -12;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <bool RMS>
int launch_bwd(const void* dy, const void* x, const void* g, const float* mean, const float* rstd, const void* keep,
               void* dx, float* dgamma, float* dbeta, int rows, int H, cudaStream_t st) {
  // one resident block per SM from 768 columns on (the parameter-gradient accumulators and the next row's loads
  // take about 150 registers per thread, and spilling them costs more than the second block brings), two below
  const int blocks = min((rows + kWarpsPerBlock - 1) / kWarpsPerBlock, 148 * (H <= 512 ? 2 : 1));
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(g);
  auto K = static_cast<const unsigned char*>(keep);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  if (H <= 256) tc05::launch_pdl(norm_bwd_kernel<1, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, DY, X, G, mean, rstd, K, DX, dgamma, dbeta, rows, H);
  else if (H <= 512) tc05::launch_pdl(norm_bwd_kernel<2, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, DY, X, G, mean, rstd, K, DX, dgamma, dbeta, rows, H);
  else if (H <= 768) tc05::launch_pdl(norm_bwd_kernel<3, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, DY, X, G, mean, rstd, K, DX, dgamma, dbeta, rows, H);
  else if (H <= 1024) tc05::launch_pdl(norm_bwd_kernel<4, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, DY, X, G, mean, rstd, K, DX, dgamma, dbeta, rows, H);
  else if (H <= 2048) tc05::launch_pdl(norm_bwd_kernel<8, RMS>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, st, DY, X, G, mean, rstd, K, DX, dgamma, dbeta, rows, H);
  else return -12;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace

extern "C" int db200_norm_fwd(const void* x, const void* gamma, const void* beta, const void* row_keep, void* y,
                              float* mean, float* rstd, int rows, int H, float eps, int rms, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return rms ? launch_fwd<true>(x, gamma, beta, row_keep, y, mean, rstd, rows, H, eps, st)
             : launch_fwd<false>(x, gamma, beta, row_keep, y, mean, rstd, rows, H, eps, st);
}

extern "C" int db200_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                              const void* row_keep, void* dx, float* dgamma, float* dbeta, int rows, int H, int rms,
                              void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return rms ? launch_bwd<true>(dy, x, gamma, mean, rstd, row_keep, dx, dgamma, dbeta, rows, H, st)
             : launch_bwd<false>(dy, x, gamma, mean, rstd, row_keep, dx, dgamma, dbeta, rows, H, st);
}
