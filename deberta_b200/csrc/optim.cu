// Optimizer kernels over the engine's flat fp32 buffers.
//   db200_sumsq  : sum of squares of a gradient range, accumulated into one device float
//   db200_adamw  : AdamW on a contiguous range; the clip coefficient is derived on the device
//                  from the (already reduced) squared gradient norm, a non-finite norm (or a
//                  device-side gate of 0) turns the launch into a no-op, and the bf16 compute
//                  copy of every parameter is rewritten in the same pass.
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      const float4 v = *reinterpret_cast<const float4*>(g + i);
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      for (long long j = i; j < n; ++j) acc += g[j] * g[j];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float warp_acc[8];
  if ((threadIdx.x & 31) == 0) warp_acc[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += warp_acc[w];
    atomicAdd(out, t);
  }
}

struct AdamArgs {
  float lr, wd, b1, b2, eps, inv_bc1, inv_sqrt_bc2, max_norm, grad_scale;
};

__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ shadow, long long n, AdamArgs a, const float* __restrict__ norm_sq,
             const float* __restrict__ gate) {
  if (gate != nullptr && !(*gate > 0.f)) return;  // the caller switched this update off on the device
  float coef = a.grad_scale;
  if (norm_sq != nullptr) {
    const float norm = sqrtf(*norm_sq) * a.grad_scale;
    if (!isfinite(norm)) return;  // skipped step: parameters and moments stay untouched
    if (a.max_norm > 0.f) coef *= fminf(1.f, a.max_norm / (norm + 1e-6f));
  }
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    float pv[4], gv[4], mv[4], vv[4];
    const int cnt = (i + 3 < n) ? 4 : static_cast<int>(n - i);
    if (cnt == 4) {
      *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(p + i);
      *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(g + i);
      *reinterpret_cast<float4*>(mv) = *reinterpret_cast<const float4*>(m + i);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + i);
    } else {
      for (int j = 0; j < cnt; ++j) { pv[j] = p[i + j]; gv[j] = g[i + j]; mv[j] = m[i + j]; vv[j] = v[i + j]; }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < cnt) {
        const float gj = gv[j] * coef;
        pv[j] *= (1.f - a.lr * a.wd);
        mv[j] = mv[j] + (gj - mv[j]) * (1.f - a.b1);
        vv[j] = vv[j] * a.b2 + gj * gj * (1.f - a.b2);
        const float denom = sqrtf(vv[j]) * a.inv_sqrt_bc2 + a.eps;
        pv[j] -= a.lr * a.inv_bc1 * mv[j] / denom;
      }
    }
    if (cnt == 4) {
      *reinterpret_cast<float4*>(p + i) = *reinterpret_cast<float4*>(pv);
      *reinterpret_cast<float4*>(m + i) = *reinterpret_cast<float4*>(mv);
      *reinterpret_cast<float4*>(v + i) = *reinterpret_cast<float4*>(vv);
      if (shadow) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(pv[0], pv[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(pv[2], pv[3]);
        uint2 u;
        u.x = *reinterpret_cast<unsigned int*>(&lo);
        u.y = *reinterpret_cast<unsigned int*>(&hi);
        *reinterpret_cast<uint2*>(shadow + i) = u;
      }
    } else {
      for (int j = 0; j < cnt; ++j) {
        p[i + j] = pv[j]; m[i + j] = mv[j]; v[i + j] = vv[j];
        if (shadow) shadow[i + j] = __float2bfloat16(pv[j]);
      }
    }
  }
}

int grid_for(long long n) {
  long long blocks = (n / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return static_cast<int>(blocks);
}

}  // namespace

extern "C" int db200_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) & 15) return -10;
  sumsq_kernel<<<grid_for(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(g, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_adamw(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr,
                           float wd, float b1, float b2, float eps, float inv_bc1, float inv_sqrt_bc2,
                           const float* norm_sq, float max_norm, float grad_scale, const float* gate, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -10;
  if (shadow_bf16 && (reinterpret_cast<uintptr_t>(shadow_bf16) & 7)) return -10;
  AdamArgs a{lr, wd, b1, b2, eps, inv_bc1, inv_sqrt_bc2, max_norm, grad_scale};
  adamw_kernel<<<grid_for(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, g, m, v, static_cast<__nv_bfloat16*>(shadow_bf16), n, a, norm_sq, gate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
