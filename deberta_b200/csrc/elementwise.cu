// Fused elementwise kernels of the RoPE backbone.
//   db200_rotary_bf16 : interleaved-pair rotary embedding on the first `rotary_dim` features of every head of q and k
//                       in one pass (forward, or the inverse rotation for the backward pass); may run in place
//   db200_swiglu_fwd  : out = silu(gate) * up           with [gate | up] the two halves of one row
//   db200_swiglu_bwd  : d[gate | up] from d(out)         (silu'(g) = s * (1 + g * (1 - s)), s = sigmoid(g))
#include "kernels.h"
#include "tc05.cuh"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

__device__ __forceinline__ float lo_f(unsigned int w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(unsigned int w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ unsigned int pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned int*>(&v);
}

// One thread rotates 4 pairs (8 features, 16 bytes). cos/sin: fp32 [S, rotary_dim] with every frequency stored twice
// (entries 2i and 2i+1 equal), as the rotary cache of the model keeps them.
__global__ void __launch_bounds__(256)
rotary_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long ldx, long long ldy,  // y may be x (in place)
              const float* __restrict__ cos_t, const float* __restrict__ sin_t, long long tokens, int S, int heads,
              int head_dim, int rotary_dim, float sign) {
  const int vec_per_head = head_dim / 8;
  const long long vecs = tokens * heads * vec_per_head;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const int s = static_cast<int>(t % S);
    const int f0 = v * 8;
    uint4 u = *reinterpret_cast<const uint4*>(x + t * ldx + h * head_dim + f0);
    if (f0 < rotary_dim) {
      unsigned int w[4] = {u.x, u.y, u.z, u.w};
      const float* c = cos_t + static_cast<long long>(s) * rotary_dim + f0;
      const float* sn = sin_t + static_cast<long long>(s) * rotary_dim + f0;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        if (f0 + 2 * p < rotary_dim) {
          const float a = lo_f(w[p]), b = hi_f(w[p]);
          const float cc = c[2 * p], ss = sn[2 * p] * sign;
          w[p] = pack2(a * cc - b * ss, b * cc + a * ss);
        }
      }
      u = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(y + t * ldy + h * head_dim + f0) = u;
  }
}

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ld_in, __nv_bfloat16* __restrict__ out, long long ld_out,
                  long long rows, int F) {
  const int vec_per_row = F / 8;
  const long long vecs = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld_in + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ld_in + F + c);
    const unsigned int gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    unsigned int o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float g0 = lo_f(gw[p]), g1 = hi_f(gw[p]);
      const float s0 = g0 / (1.f + __expf(-g0)), s1 = g1 / (1.f + __expf(-g1));
      // the product is formed from the bf16-rounded silu, as the unfused composition does
      o[p] = pack2(__bfloat162float(__float2bfloat16(s0)) * lo_f(uw[p]), __bfloat162float(__float2bfloat16(s1)) * hi_f(uw[p]));
    }
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ld_in, const __nv_bfloat16* __restrict__ dout,
                  long long ld_do, __nv_bfloat16* __restrict__ dgu, long long ld_dg, long long rows, int F) {
  const int vec_per_row = F / 8;
  const long long vecs = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld_in + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ld_in + F + c);
    const uint4 d = *reinterpret_cast<const uint4*>(dout + r * ld_do + c);
    const unsigned int gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w}, dw[4] = {d.x, d.y, d.z, d.w};
    unsigned int og[4], ou[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float gv[2] = {lo_f(gw[p]), hi_f(gw[p])}, uv[2] = {lo_f(uw[p]), hi_f(uw[p])}, dv[2] = {lo_f(dw[p]), hi_f(dw[p])};
      float dg[2], du[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float sig = 1.f / (1.f + __expf(-gv[e]));
        const float silu = gv[e] * sig;
        du[e] = dv[e] * silu;
        dg[e] = dv[e] * uv[e] * sig * (1.f + gv[e] * (1.f - sig));
      }
      og[p] = pack2(dg[0], dg[1]);
      ou[p] = pack2(du[0], du[1]);
    }
    *reinterpret_cast<uint4*>(dgu + r * ld_dg + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + r * ld_dg + F + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// y[r, c] = bf16(x[r, c]) for a dense fp32 matrix and a row-strided bf16 destination: 8 values per thread
// (two 16-byte loads, one 16-byte store), grid-stride over rows * cols / 8 vectors.
__global__ void __launch_bounds__(256)
cast_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long ld_y, long long rows, int cols) {
  tc05::pdl_launch_dependents();
  tc05::pdl_wait();
  const int vpr = cols / 8;
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * 256) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    const float4 a = *reinterpret_cast<const float4*>(x + r * cols + c);
    const float4 b = *reinterpret_cast<const float4*>(x + r * cols + c + 4);
    *reinterpret_cast<uint4*>(y + r * ld_y + c) = make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
  }
}

// Masked-row gather: out[n, :] = x[idx[n], :] (16 bytes per thread), and inv[idx[n]] = n for the backward pass.
__global__ void __launch_bounds__(256)
rows_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ld_x, const long long* __restrict__ idx,
                   __nv_bfloat16* __restrict__ out, int* __restrict__ inv, long long n_rows, int cols) {
  const int vpr = cols / 8;
  const long long total = n_rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * 256) {
    const long long n = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    const long long src = idx[n];
    *reinterpret_cast<uint4*>(out + n * cols + c) = *reinterpret_cast<const uint4*>(x + src * ld_x + c);
    if (c == 0 && inv) inv[src] = static_cast<int>(n);
  }
}

// Its gradient: dx[m, :] = dout[inv[m], :] for selected rows and 0 elsewhere; every row of dx is written once, so the
// destination needs no clearing pass.
__global__ void __launch_bounds__(256)
rows_scatter_kernel(const __nv_bfloat16* __restrict__ dout, long long ld_do, const int* __restrict__ inv,
                    __nv_bfloat16* __restrict__ dx, long long m_rows, int cols) {
  const int vpr = cols / 8;
  const long long total = m_rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * 256) {
    const long long m = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    const int n = inv[m];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n >= 0) v = *reinterpret_cast<const uint4*>(dout + static_cast<long long>(n) * ld_do + c);
    *reinterpret_cast<uint4*>(dx + m * cols + c) = v;
  }
}

int ew_grid(long long vecs) {
  long long blocks = (vecs + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}
bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int db200_rotary_bf16(const void* x, void* y, long long ldx, long long ldy, const float* cos_t,
                                 const float* sin_t, long long tokens, int S, int heads, int head_dim, int rotary_dim,
                                 int inverse, void* stream) {
  if (tokens <= 0) return 0;
  if (!al16(x) || !al16(y) || (ldx % 8) || (ldy % 8) || (head_dim % 8) || (rotary_dim % 2) || rotary_dim > head_dim || S <= 0)
    return -10;
  const long long vecs = tokens * heads * (head_dim / 8);
  rotary_kernel<<<ew_grid(vecs), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), ldx, ldy, cos_t, sin_t, tokens, S, heads,
      head_dim, rotary_dim, inverse ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_cast_f32_bf16(const float* x, void* y, long long ld_y, long long rows, int cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (!al16(x) || !al16(y) || (ld_y % 8) || (cols % 8) || ld_y < cols) return -10;
  tc05::launch_pdl(cast_rows_kernel, dim3(ew_grid(rows * (cols / 8))), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                   x, static_cast<__nv_bfloat16*>(y), ld_y, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_swiglu_fwd(const void* gate_up, long long ld_in, void* out, long long ld_out, long long rows, int F,
                                void* stream) {
  if (rows <= 0) return 0;
  if (!al16(gate_up) || !al16(out) || (ld_in % 8) || (ld_out % 8) || (F % 8)) return -10;
  swiglu_fwd_kernel<<<ew_grid(rows * (F / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), ld_in, static_cast<__nv_bfloat16*>(out), ld_out, rows, F);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_swiglu_bwd(const void* gate_up, long long ld_in, const void* dout, long long ld_do, void* d_gate_up,
                                long long ld_dg, long long rows, int F, void* stream) {
  if (rows <= 0) return 0;
  if (!al16(gate_up) || !al16(dout) || !al16(d_gate_up) || (ld_in % 8) || (ld_do % 8) || (ld_dg % 8) || (F % 8)) return -10;
  swiglu_bwd_kernel<<<ew_grid(rows * (F / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), ld_in, static_cast<const __nv_bfloat16*>(dout), ld_do,
      static_cast<__nv_bfloat16*>(d_gate_up), ld_dg, rows, F);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---- embedding lookup (+ optional second table) and its gradient ----------------------------------------------------
//   db200_embed_fwd : out[t, :] = table[id[t], :] (+ delta[id[t], :])         one warp per token, 16-byte accesses
//   db200_embed_bwd : grad[id[t], :] += dout[t, :] (fp32, red.add.v4), tokens whose id equals padding_idx are skipped.
//                     Rows that many tokens share are summed in an order that varies from run to run.
namespace {

__global__ void __launch_bounds__(256)
embed_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                 const __nv_bfloat16* __restrict__ delta, __nv_bfloat16* __restrict__ out, long long tokens, int H,
                 long long vocab) {
  const int lane = threadIdx.x & 31;
  const int vecs = H / 8;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < tokens;
       t += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // out-of-range ids are clamped, never dereferenced as given
    const uint4* src = reinterpret_cast<const uint4*>(table + id * H);
    const uint4* dsrc = delta ? reinterpret_cast<const uint4*>(delta + id * H) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(out + t * H);
    for (int v = lane; v < vecs; v += 32) {
      uint4 a = __ldg(src + v);
      if (dsrc) {
        const uint4 b = __ldg(dsrc + v);
        a.x = pack2(lo_f(a.x) + lo_f(b.x), hi_f(a.x) + hi_f(b.x));
        a.y = pack2(lo_f(a.y) + lo_f(b.y), hi_f(a.y) + hi_f(b.y));
        a.z = pack2(lo_f(a.z) + lo_f(b.z), hi_f(a.z) + hi_f(b.z));
        a.w = pack2(lo_f(a.w) + lo_f(b.w), hi_f(a.w) + hi_f(b.w));
      }
      dst[v] = a;
    }
  }
}

__global__ void __launch_bounds__(256)
embed_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout, long long ld_do,
                 float* __restrict__ grad, long long tokens, int H, long long vocab, long long padding_idx) {
  const int lane = threadIdx.x & 31;
  const int vecs = H / 8;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < tokens;
       t += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const long long id = ids[t];
    if (id < 0 || id >= vocab || id == padding_idx) continue;  // warp-uniform
    const uint4* src = reinterpret_cast<const uint4*>(dout + t * ld_do);
    float* dst = grad + id * H;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 a = src[v];
      float* d = dst + v * 8;
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(lo_f(a.x)), "f"(hi_f(a.x)),
                   "f"(lo_f(a.y)), "f"(hi_f(a.y)) : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + 4), "f"(lo_f(a.z)), "f"(hi_f(a.z)),
                   "f"(lo_f(a.w)), "f"(hi_f(a.w)) : "memory");
    }
  }
}

}  // namespace

extern "C" int db200_embed_fwd(const long long* ids, const void* table, const void* delta, void* out, long long tokens,
                               int H, long long vocab, void* stream) {
  if (tokens <= 0) return 0;
  if (!al16(table) || !al16(out) || (delta && !al16(delta)) || (H % 8) || vocab <= 0) return -10;
  embed_fwd_kernel<<<ew_grid(tokens * 32), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<const __nv_bfloat16*>(delta),
      static_cast<__nv_bfloat16*>(out), tokens, H, vocab);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_embed_bwd(const long long* ids, const void* dout, long long ld_do, float* grad, long long tokens,
                               int H, long long vocab, long long padding_idx, void* stream) {
  if (tokens <= 0) return 0;
  if (!al16(dout) || !al16(grad) || (H % 8) || (ld_do % 8) || vocab <= 0) return -10;
  embed_bwd_kernel<<<ew_grid(tokens * 32), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(dout), ld_do, grad, tokens, H, vocab, padding_idx);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---- replaced-token-detection head: classifier dot product + masked BCE-with-logits + counts ----------------------------
//   db200_rtd_tail_fwd : logit[t] = a[t,:] . w + b ;  stats += {sum of BCE over active tokens, correct, active, positive}
//   db200_rtd_tail_bwd : dz[t] = (sigmoid(logit) - y) * active * gscale ;  d_pre[t,:] = dz * w * gelu'(pre[t,:]) (or dz * w
//                        when pre is null) ;  dw += sum_t dz * a[t,:] ;  db += sum_t dz        (gscale = *grad / max(count,1))
// One warp per token row; H <= 1024 (multiple of 8).
namespace {

constexpr int kTailVec = 4;  // 16-byte vectors per lane: H <= 1024

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float dgelu_exact(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

__global__ void __launch_bounds__(256)
rtd_tail_fwd_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const __nv_bfloat16* __restrict__ w,
                    const __nv_bfloat16* __restrict__ bias, const long long* __restrict__ labels,
                    const unsigned char* __restrict__ active, float* __restrict__ logits, float* __restrict__ stats,
                    long long tokens, int H) {
  __shared__ float part[8][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vecs = H / 8;
  float wv[kTailVec][8];
#pragma unroll
  for (int i = 0; i < kTailVec; ++i) {
    const int v = lane + 32 * i;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (v < vecs) u = __ldg(reinterpret_cast<const uint4*>(w) + v);
    const unsigned int uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { wv[i][2 * e] = lo_f(uw[e]); wv[i][2 * e + 1] = hi_f(uw[e]); }
  }
  const float b = bias ? __bfloat162float(bias[0]) : 0.f;
  float s_loss = 0.f, s_correct = 0.f, s_count = 0.f, s_pos = 0.f;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < tokens;
       t += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const uint4* row = reinterpret_cast<const uint4*>(a + t * lda);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kTailVec; ++i) {
      const int v = lane + 32 * i;
      if (v < vecs) {
        const uint4 u = row[v];
        const unsigned int uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) acc += lo_f(uw[e]) * wv[i][2 * e] + hi_f(uw[e]) * wv[i][2 * e + 1];
      }
    }
    // the reference rounds the logit to the activation dtype before the loss
    const float z = __bfloat162float(__float2bfloat16(warp_sum_f(acc) + b));
    if (lane == 0) {
      logits[t] = z;
      if (active[t]) {
        const float y = labels[t] > 0 ? 1.f : 0.f;
        s_loss += fmaxf(z, 0.f) - z * y + log1pf(__expf(-fabsf(z)));
        s_correct += ((z > 0.f) == (y > 0.5f)) ? 1.f : 0.f;
        s_count += 1.f;
        s_pos += y;
      }
    }
  }
  if (lane == 0) { part[warp][0] = s_loss; part[warp][1] = s_correct; part[warp][2] = s_count; part[warp][3] = s_pos; }
  __syncthreads();
  if (threadIdx.x < 4) {
    float s = 0.f;
    for (int k = 0; k < 8; ++k) s += part[k][threadIdx.x];
    if (s != 0.f) atomicAdd(stats + threadIdx.x, s);
  }
}

__global__ void __launch_bounds__(256)
rtd_tail_bwd_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const __nv_bfloat16* __restrict__ pre,
                    long long ldp, const __nv_bfloat16* __restrict__ w, const float* __restrict__ logits,
                    const long long* __restrict__ labels, const unsigned char* __restrict__ active,
                    const float* __restrict__ grad, const float* __restrict__ stats, __nv_bfloat16* __restrict__ d_pre,
                    long long ldd, float* __restrict__ dw, float* __restrict__ db, long long tokens, int H) {
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vecs = H / 8;
  const float gscale = grad[0] / fmaxf(stats[2], 1.f);
  float wv[kTailVec][8], dwv[kTailVec][8];
#pragma unroll
  for (int i = 0; i < kTailVec; ++i) {
    const int v = lane + 32 * i;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (v < vecs) u = __ldg(reinterpret_cast<const uint4*>(w) + v);
    const unsigned int uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { wv[i][2 * e] = lo_f(uw[e]); wv[i][2 * e + 1] = hi_f(uw[e]); }
#pragma unroll
    for (int e = 0; e < 8; ++e) dwv[i][e] = 0.f;
  }
  float dbv = 0.f;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < tokens;
       t += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    float dz = 0.f;
    if (active[t]) {
      const float z = logits[t];
      const float y = labels[t] > 0 ? 1.f : 0.f;
      dz = (1.f / (1.f + __expf(-z)) - y) * gscale;
    }
    dz = __bfloat162float(__float2bfloat16(dz));  // the logit gradient reaches the classifier in the activation dtype
    dbv += dz;
    const uint4* arow = reinterpret_cast<const uint4*>(a + t * lda);
    const uint4* prow = pre ? reinterpret_cast<const uint4*>(pre + t * ldp) : nullptr;
    uint4* drow = reinterpret_cast<uint4*>(d_pre + t * ldd);
#pragma unroll
    for (int i = 0; i < kTailVec; ++i) {
      const int v = lane + 32 * i;
      if (v < vecs) {
        const uint4 ua = arow[v];
        const unsigned int aw[4] = {ua.x, ua.y, ua.z, ua.w};
        float g[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          dwv[i][2 * e] += dz * lo_f(aw[e]);
          dwv[i][2 * e + 1] += dz * hi_f(aw[e]);
          g[2 * e] = dz * wv[i][2 * e];
          g[2 * e + 1] = dz * wv[i][2 * e + 1];
        }
        if (prow) {
          const uint4 up = prow[v];
          const unsigned int pw[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            g[2 * e] *= dgelu_exact(lo_f(pw[e]));
            g[2 * e + 1] *= dgelu_exact(hi_f(pw[e]));
          }
        }
        drow[v] = make_uint4(pack2(g[0], g[1]), pack2(g[2], g[3]), pack2(g[4], g[5]), pack2(g[6], g[7]));
      }
    }
  }
  // block reduction of the classifier gradient: one 8-feature vector slot at a time
#pragma unroll
  for (int i = 0; i < kTailVec; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      red[warp][lane] = dwv[i][e];
      __syncthreads();
      if (warp == 0) {
        float s = 0.f;
        for (int k = 0; k < 8; ++k) s += red[k][lane];
        const int v = lane + 32 * i;
        if (v < vecs && s != 0.f) atomicAdd(dw + v * 8 + e, s);
      }
      __syncthreads();
    }
  }
  dbv = (lane == 0) ? dbv : 0.f;  // every lane of a warp carries the same dz
  red[warp][lane] = dbv;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int k = 0; k < 8; ++k) s += red[k][0];
    if (s != 0.f) atomicAdd(db, s);
  }
}

}  // namespace

extern "C" int db200_rtd_tail_fwd(const void* a, long long lda, const void* w, const void* bias, const long long* labels,
                                  const unsigned char* active, float* logits, float* stats, long long tokens, int H,
                                  void* stream) {
  if (tokens <= 0) return 0;
  if (!al16(a) || !al16(w) || (lda % 8) || (H % 8) || H > 1024) return -10;
  int blocks = static_cast<int>((tokens + 7) / 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  rtd_tail_fwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), lda, static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(bias), labels, active, logits, stats, tokens, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_rtd_tail_bwd(const void* a, long long lda, const void* pre, long long ldp, const void* w,
                                  const float* logits, const long long* labels, const unsigned char* active,
                                  const float* grad, const float* stats, void* d_pre, long long ldd, float* dw, float* db,
                                  long long tokens, int H, void* stream) {
  if (tokens <= 0) return 0;
  if (!al16(a) || !al16(w) || !al16(d_pre) || (pre && !al16(pre)) || (lda % 8) || (ldp % 8) || (ldd % 8) || (H % 8) || H > 1024)
    return -10;
  int blocks = static_cast<int>((tokens + 7) / 8);
  if (blocks > 148 * 2) blocks = 148 * 2;  // few blocks: each ends with a reduction of the classifier gradient
  rtd_tail_bwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), lda, static_cast<const __nv_bfloat16*>(pre), ldp,
      static_cast<const __nv_bfloat16*>(w), logits, labels, active, grad, stats, static_cast<__nv_bfloat16*>(d_pre), ldd, dw,
      db, tokens, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_rows_gather(const void* x, long long ld_x, const long long* idx, void* out, int* inv, long long m_rows,
                                 long long n_rows, int cols, void* stream) {
  if (cols <= 0 || (cols % 8) || (ld_x % 8) || !al16(x) || !al16(out)) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (inv && m_rows > 0 && cudaMemsetAsync(inv, 0xFF, static_cast<size_t>(m_rows) * sizeof(int), st) != cudaSuccess) return -4;
  if (n_rows <= 0) return 0;
  rows_gather_kernel<<<ew_grid(n_rows * (cols / 8)), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ld_x, idx,
                                                                    static_cast<__nv_bfloat16*>(out), inv, n_rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_rows_scatter(const void* dout, long long ld_do, const int* inv, void* dx, long long m_rows, int cols,
                                  void* stream) {
  if (m_rows <= 0) return 0;
  if (cols <= 0 || (cols % 8) || (ld_do % 8) || !al16(dout) || !al16(dx) || !inv) return -10;
  rows_scatter_kernel<<<ew_grid(m_rows * (cols / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), ld_do, inv, static_cast<__nv_bfloat16*>(dx), m_rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
