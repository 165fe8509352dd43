// Column sums of a bf16 matrix accumulated into an fp32 vector (bias gradients).
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

// block (32, 8): 32 threads x 8 columns = 256 columns, 8 row lanes; grid (col blocks, row splits)
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N, float* __restrict__ out) {
  __shared__ float red[8][257];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = (blockIdx.x * 32 + tx) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < N) {
    const bool vec = (col + 8 <= N);
#pragma unroll 4
    for (int r = blockIdx.y * 8 + ty; r < M; r += gridDim.y * 8) {
      const __nv_bfloat16* src = x + static_cast<long long>(r) * ld + col;
      if (vec) {
        const uint4 u = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(v[j]);
      } else {
        for (int j = 0; j < 8 && col + j < N; ++j) acc[j] += __bfloat162float(src[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[ty][tx * 8 + j] = acc[j];
  __syncthreads();
  const int t = ty * 32 + tx;  // 256 threads -> 256 columns of this block
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) s += red[w][t];
  const int c = blockIdx.x * 256 + t;
  if (c < N && s != 0.f) atomicAdd(out + c, s);
}

}  // namespace

extern "C" int db200_colsum_bf16(const void* x, long long ld, int M, int N, float* out_accum, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((ld % 8) || (reinterpret_cast<uintptr_t>(x) & 15)) return -10;
  // enough blocks to keep every SM's memory pipeline full: about 64 rows per block, at most ~1200 blocks
  int splits = (M + 63) / 64;
  const int col_blocks = (N + 255) / 256;
  const int max_splits = (1184 + col_blocks - 1) / col_blocks;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  dim3 grid((N + 255) / 256, splits), block(32, 8);
  colsum_kernel<<<grid, block, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), ld, M, N,
                                                                          out_accum);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
