// Gradient reduction and parameter update fused with their collectives over NVLink peer memory.
//
// Every rank (one process per GPU) holds the same flat layout: an fp32 gradient buffer, a bf16
// parameter buffer and a small "pad" of flags, all allocated symmetrically so that each rank has
// a mapped pointer to every peer's copy (and, where the fabric offers it, one multicast address
// that reaches all copies through the switch). The kernels below replace
//
//   reduce-scatter -> scale -> sum of squares -> all-reduce(norm) -> AdamW -> all-gather
//
// with two launches per optimizer step, and an all-reduce with one:
//
//   db200_comm_reduce     mode 0: this rank sums its slab over all peers (peer loads, or one
//                         multimem.ld_reduce per 16 bytes), scales, stores the result locally and
//                         publishes its share of the squared norm to every peer's pad.
//                         mode 1: the same, but the reduced slab is stored into every peer's
//                         buffer (all-reduce) and the kernel returns the full squared norm.
//   db200_comm_adamw      waits for every peer's squared-norm share, derives the clip coefficient
//                         (or skips on a non-finite norm), runs AdamW on the slab and stores the
//                         bf16 parameters into every peer's parameter buffer (peer stores or
//                         multimem.st); returns once every peer's slab has landed here.
//   db200_comm_vector_sum small vectors (token counts, flags, metrics): every rank pushes its
//                         vector into every pad, then sums the pads in rank order.
//
// Ordering between ranks uses per-source flags in the pads that carry a call counter ("epoch")
// supplied by the host; the host passes the same strictly increasing epochs on every rank. A wait
// gives up after `timeout_ns` of the global timer and records kErrPeerWait in the status word. The
// kernel then runs to completion (all addresses stay valid) but fails safe: a reduction whose peers
// did not show up publishes an infinite squared-norm share, so that no rank applies an update to
// partially reduced gradients; the update kernel treats a missing share the same way; a vector sum
// returns NaN. The host reads the status word with the step's outcome and raises.
//
// These kernels spin on flags written by other GPUs: ranks must be on different GPUs.
#include "kernels.h"
#include "tc05.cuh"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

using tc05::kErrPeerWait;
using tc05::pack_bf16;

constexpr int kMaxWorld = DB200_COMM_MAX_WORLD;
constexpr int kChStart = 0, kChNorm = 1, kChDone = 2, kChVec = 3;
// pad layout in 32-bit words
constexpr int kPadFlags = 0;                    // [4 channels][kMaxWorld sources]
constexpr int kPadNorm = 4 * kMaxWorld;         // [kMaxWorld] float: squared-norm share of each source
constexpr int kPadTicket = kPadNorm + kMaxWorld;  // local: CTAs finished
constexpr int kPadAcc = kPadTicket + 1;           // local: float accumulator of this rank's share
constexpr int kPadVec = 64;                       // [kMaxWorld][DB200_COMM_VEC_MAX] float
static_assert(kPadAcc < kPadVec, "pad header overflows");
static_assert(kPadVec + kMaxWorld * DB200_COMM_VEC_MAX <= DB200_COMM_PAD_WORDS, "pad too small");

struct CommDev {
  int world, rank;
  float* grads[kMaxWorld];
  __nv_bfloat16* params[kMaxWorld];
  uint32_t* pads[kMaxWorld];
  float* mc_grads;
  __nv_bfloat16* mc_params;
  unsigned long long timeout_ns;
  int* status;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_sys_v4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_v4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Tell every peer that this rank reached `epoch` on `channel` (idempotent: any CTA may do it).
__device__ __forceinline__ void signal_peers(const CommDev& c, int channel, uint32_t epoch) {
  if (threadIdx.x < c.world) st_release_sys(c.pads[threadIdx.x] + kPadFlags + channel * kMaxWorld + c.rank, epoch);
}

// Threads 0..world-1 wait for their source's flag; false (block-uniform after the barrier) on a timeout.
__device__ __forceinline__ bool wait_peers(const CommDev& c, int channel, uint32_t epoch, int* smem_flag) {
  if (threadIdx.x == 0) *smem_flag = 0;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const uint32_t* f = c.pads[c.rank] + kPadFlags + channel * kMaxWorld + threadIdx.x;
    const unsigned long long t0 = global_ns();
    bool seen = false;
    for (;;) {
      if (static_cast<int>(ld_acquire_sys(f) - epoch) >= 0) { seen = true; break; }
      if (global_ns() - t0 > c.timeout_ns) break;
      __nanosleep(64);
    }
    if (!seen) {
      atomicCAS(c.status, 0, kErrPeerWait | (channel << 8) | (static_cast<int>(threadIdx.x) << 16));
      *smem_flag = 1;
    }
  }
  __syncthreads();
  return *smem_flag == 0;
}

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x == 0)
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t += smem[w];
  return t;  // valid on thread 0
}

// True on exactly one thread of the grid: thread 0 of the last CTA to get here.
__device__ __forceinline__ bool last_block_done(uint32_t* ticket) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t t = atomicAdd(ticket, 1u);
    is_last = (t == gridDim.x - 1);
    if (is_last) *ticket = 0;
  }
  __syncthreads();
  if (is_last) __threadfence_system();  // order the other CTAs' (fenced) writes before what this CTA signals
  return is_last != 0;
}

template <bool kToAll>
__global__ void __launch_bounds__(256)
comm_reduce_kernel(const CommDev c, long long off, long long n, float scale, uint32_t epoch, const float* extra_share,
                   float* norm_sq_out) {
  __shared__ int wait_flag;
  __shared__ float red[8];
  uint32_t* pad = c.pads[c.rank];
  __threadfence_system();
  signal_peers(c, kChStart, epoch);
  const bool peers_here = wait_peers(c, kChStart, epoch, &wait_flag);

  float ss = peers_here ? 0.f : INFINITY;  // a peer never arrived: its gradients may be missing from the sum
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    float4 a;
    if (c.mc_grads) {
      a = multimem_ld_reduce_v4(c.mc_grads + off + i);
    } else {
      a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int r = 0; r < c.world; ++r) {
        const float4 v = ld_sys_v4(c.grads[r] + off + i);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
    }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    if (!kToAll) {
      *reinterpret_cast<float4*>(c.grads[c.rank] + off + i) = a;
    } else if (c.mc_grads) {
      multimem_st_v4(c.mc_grads + off + i, a);
    } else {
      for (int r = 0; r < c.world; ++r) *reinterpret_cast<float4*>(c.grads[r] + off + i) = a;
    }
  }
  const float bs = block_sum(ss, red);
  if (threadIdx.x == 0) atomicAdd(reinterpret_cast<float*>(pad + kPadAcc), bs);
  if (!last_block_done(pad + kPadTicket)) return;

  // last CTA: publish this rank's share of the squared norm
  __shared__ float share;
  if (threadIdx.x == 0) share = atomicExch(reinterpret_cast<float*>(pad + kPadAcc), 0.f) + (extra_share ? *extra_share : 0.f);
  __syncthreads();
  if (threadIdx.x < c.world) {
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(c.pads[threadIdx.x] + kPadNorm + c.rank), "f"(share) : "memory");
    __threadfence_system();
  }
  signal_peers(c, kChNorm, epoch);
  if (kToAll) {
    // every peer's slab has landed here once its flag is up; then the norm is complete too
    const bool all_in = wait_peers(c, kChNorm, epoch, &wait_flag);
    if (threadIdx.x == 0 && norm_sq_out) {
      float t = all_in ? 0.f : INFINITY;
      for (int r = 0; r < c.world; ++r) t += __uint_as_float(ld_acquire_sys(pad + kPadNorm + r));
      *norm_sq_out = t;
    }
  }
}

struct AdamSeg {
  long long begin, end;  // relative to the slab, multiples of 8
  float lr, wd;
};
struct AdamDev {
  AdamSeg seg[4];
  int nseg;
  float b1, b2, eps, inv_bc1, inv_sqrt_bc2, max_norm;
};

__global__ void __launch_bounds__(256)
comm_adamw_kernel(const CommDev c, long long off, float* __restrict__ master, float* __restrict__ m,
                  float* __restrict__ v, const AdamDev a, uint32_t epoch, float* norm_sq_out,
                  const float* __restrict__ gate, __nv_bfloat16* __restrict__ local_params) {
  __shared__ int wait_flag;
  uint32_t* pad = c.pads[c.rank];
  const bool shares_in = wait_peers(c, kChNorm, epoch, &wait_flag);
  float norm_sq = shares_in ? 0.f : INFINITY;  // a missing share: skip the update like a non-finite norm
  for (int r = 0; r < c.world; ++r) norm_sq += __uint_as_float(ld_acquire_sys(pad + kPadNorm + r));
  if (blockIdx.x == 0 && threadIdx.x == 0 && norm_sq_out) *norm_sq_out = norm_sq;
  const float norm = sqrtf(norm_sq);
  // same values on every rank: all of them skip together (the gate is a sum over ranks computed earlier)
  const bool skip = !isfinite(norm) || (gate != nullptr && !(*gate > 0.f));
  const float coef = (a.max_norm > 0.f) ? fminf(1.f, a.max_norm / (norm + 1e-6f)) : 1.f;
  const float* g = c.grads[c.rank] + off;

  if (!skip) {
    for (int s = 0; s < a.nseg; ++s) {
      const float lr = a.seg[s].lr, decay = 1.f - a.seg[s].lr * a.seg[s].wd;
      const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
      for (long long i = a.seg[s].begin + (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
           i < a.seg[s].end; i += stride) {
        float pv[8], gv[8], mv[8], vv[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          *reinterpret_cast<float4*>(pv + 4 * h) = *reinterpret_cast<const float4*>(master + i + 4 * h);
          *reinterpret_cast<float4*>(gv + 4 * h) = *reinterpret_cast<const float4*>(g + i + 4 * h);
          *reinterpret_cast<float4*>(mv + 4 * h) = *reinterpret_cast<const float4*>(m + i + 4 * h);
          *reinterpret_cast<float4*>(vv + 4 * h) = *reinterpret_cast<const float4*>(v + i + 4 * h);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gj = gv[j] * coef;
          pv[j] *= decay;
          mv[j] = mv[j] + (gj - mv[j]) * (1.f - a.b1);
          vv[j] = vv[j] * a.b2 + gj * gj * (1.f - a.b2);
          pv[j] -= lr * a.inv_bc1 * mv[j] / (sqrtf(vv[j]) * a.inv_sqrt_bc2 + a.eps);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          *reinterpret_cast<float4*>(master + i + 4 * h) = *reinterpret_cast<float4*>(pv + 4 * h);
          *reinterpret_cast<float4*>(m + i + 4 * h) = *reinterpret_cast<float4*>(mv + 4 * h);
          *reinterpret_cast<float4*>(v + i + 4 * h) = *reinterpret_cast<float4*>(vv + 4 * h);
        }
        float4 packed;
        packed.x = __uint_as_float(pack_bf16(pv[0], pv[1]));
        packed.y = __uint_as_float(pack_bf16(pv[2], pv[3]));
        packed.z = __uint_as_float(pack_bf16(pv[4], pv[5]));
        packed.w = __uint_as_float(pack_bf16(pv[6], pv[7]));
        if (local_params) {  // parameters stay sharded: only this rank keeps the slab (peers fetch it per layer)
          *reinterpret_cast<float4*>(local_params + i) = packed;
        } else if (c.mc_params) {
          multimem_st_v4(c.mc_params + off + i, packed);
        } else {
          for (int r = 0; r < c.world; ++r) *reinterpret_cast<float4*>(c.params[r] + off + i) = packed;
        }
      }
    }
  }
  if (!last_block_done(pad + kPadTicket)) return;
  signal_peers(c, kChDone, epoch);
  wait_peers(c, kChDone, epoch, &wait_flag);  // all slabs of the parameter buffer are in place
}

__global__ void __launch_bounds__(DB200_COMM_VEC_MAX)
comm_vector_sum_kernel(const CommDev c, const float* __restrict__ in, float* __restrict__ out, int n, uint32_t epoch) {
  __shared__ int wait_flag;
  const int t = threadIdx.x;
  if (t < n) {
    const float x = in[t];
    for (int r = 0; r < c.world; ++r)
      asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(c.pads[r] + kPadVec + c.rank * DB200_COMM_VEC_MAX + t), "f"(x)
                   : "memory");
  }
  __threadfence_system();
  __syncthreads();
  signal_peers(c, kChVec, epoch);
  const bool all_in = wait_peers(c, kChVec, epoch, &wait_flag);
  if (t < n) {
    float s = all_in ? 0.f : NAN;
    for (int r = 0; r < c.world; ++r)
      s += __uint_as_float(ld_acquire_sys(c.pads[c.rank] + kPadVec + r * DB200_COMM_VEC_MAX + t));
    out[t] = s;
  }
  // a peer may start its next vector sum only after this rank has read the current one
  __syncthreads();
  signal_peers(c, kChStart, epoch);
  wait_peers(c, kChStart, epoch, &wait_flag);
}

// Gather of sharded parameters: up to kMaxPieces contiguous byte ranges, each read from memory that may belong to a
// peer GPU (plain 16-byte loads through the peer mapping) and written to this GPU's memory. One launch per layer
// unit; ordering against the owners' optimizer kernels is the caller's (stream events after the kernels' own
// all-rank barrier).
constexpr int kMaxPieces = 2 * kMaxWorld;
struct PieceList {
  const uint4* src[kMaxPieces];
  uint4* dst[kMaxPieces];
  long long n16[kMaxPieces];  // 16-byte units
  int count;
};
__global__ void __launch_bounds__(256) copy_pieces_kernel(const PieceList p) {
  for (int k = 0; k < p.count; ++k) {
    const uint4* __restrict__ s = p.src[k];
    uint4* __restrict__ d = p.dst[k];
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n16[k]; i += stride) {
      uint4 v;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(s + i) : "memory");
      d[i] = v;
    }
  }
}

int make_dev(const Db200CommCtx* h, CommDev* d) {
  if (!h || h->world < 2 || h->world > kMaxWorld || h->rank < 0 || h->rank >= h->world) return -10;
  d->world = h->world;
  d->rank = h->rank;
  for (int r = 0; r < kMaxWorld; ++r) {
    d->grads[r] = r < h->world ? static_cast<float*>(h->grads[r]) : nullptr;
    d->params[r] = r < h->world ? static_cast<__nv_bfloat16*>(h->params[r]) : nullptr;
    d->pads[r] = r < h->world ? static_cast<uint32_t*>(h->pads[r]) : nullptr;
    if (r < h->world && !d->pads[r]) return -10;
  }
  d->mc_grads = static_cast<float*>(h->mc_grads);
  d->mc_params = static_cast<__nv_bfloat16*>(h->mc_params);
  d->timeout_ns = h->timeout_ns ? h->timeout_ns : 20ull * 1000 * 1000 * 1000;
  d->status = db200_status_ptr();
  return d->status ? 0 : -3;
}

int comm_grid(long long n, int per_thread) {
  long long blocks = (n / per_thread + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  return static_cast<int>(blocks);
}

}  // namespace

extern "C" int db200_comm_reduce(const Db200CommCtx* ctx, long long offset, long long count, float scale,
                                 int to_all, unsigned epoch, const float* extra_share, float* norm_sq_out, void* stream) {
  CommDev d;
  if (int rc = make_dev(ctx, &d)) return rc;
  if (count <= 0 || (count % 4) || (offset % 4)) return -10;
  for (int r = 0; r < d.world; ++r)
    if (!d.grads[r] || (reinterpret_cast<uintptr_t>(d.grads[r]) & 15)) return -10;
  if (d.mc_grads && (reinterpret_cast<uintptr_t>(d.mc_grads) & 15)) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = comm_grid(count, 4);
  if (to_all)
    comm_reduce_kernel<true><<<grid, 256, 0, st>>>(d, offset, count, scale, epoch, extra_share, norm_sq_out);
  else
    comm_reduce_kernel<false><<<grid, 256, 0, st>>>(d, offset, count, scale, epoch, extra_share, norm_sq_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_comm_adamw(const Db200CommCtx* ctx, long long offset, long long count, float* master, float* exp_avg,
                                float* exp_avg_sq, const Db200AdamSegment* segs, int nseg, float b1, float b2, float eps,
                                float inv_bc1, float inv_sqrt_bc2, float max_norm, unsigned epoch, float* norm_sq_out,
                                const float* gate, void* local_params, void* stream) {
  CommDev d;
  if (int rc = make_dev(ctx, &d)) return rc;
  if (count <= 0 || (count % 8) || (offset % 8) || nseg < 0 || nseg > 4) return -10;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(exp_avg) | reinterpret_cast<uintptr_t>(exp_avg_sq) |
       reinterpret_cast<uintptr_t>(local_params)) & 15)
    return -10;
  for (int r = 0; r < d.world; ++r)
    if ((!local_params && (!d.params[r] || (reinterpret_cast<uintptr_t>(d.params[r]) & 15))) || !d.grads[r]) return -10;
  AdamDev a{};
  a.nseg = nseg;
  for (int s = 0; s < nseg; ++s) {
    if (segs[s].begin < 0 || segs[s].end > count || (segs[s].begin % 8) || (segs[s].end % 8)) return -10;
    a.seg[s] = AdamSeg{segs[s].begin, segs[s].end, segs[s].lr, segs[s].weight_decay};
  }
  a.b1 = b1; a.b2 = b2; a.eps = eps; a.inv_bc1 = inv_bc1; a.inv_sqrt_bc2 = inv_sqrt_bc2; a.max_norm = max_norm;
  comm_adamw_kernel<<<comm_grid(count, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      d, offset, master, exp_avg, exp_avg_sq, a, epoch, norm_sq_out, gate, static_cast<__nv_bfloat16*>(local_params));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_comm_vector_sum(const Db200CommCtx* ctx, const float* in, float* out, int n, unsigned epoch,
                                     void* stream) {
  CommDev d;
  if (int rc = make_dev(ctx, &d)) return rc;
  if (n <= 0 || n > DB200_COMM_VEC_MAX) return -10;
  comm_vector_sum_kernel<<<1, DB200_COMM_VEC_MAX, 0, reinterpret_cast<cudaStream_t>(stream)>>>(d, in, out, n, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_comm_copy_pieces(const void* const* src, void* const* dst, const long long* bytes, int count,
                                      void* stream) {
  if (count <= 0) return 0;
  if (count > kMaxPieces) return -10;
  PieceList p{};
  long long total = 0;
  for (int k = 0; k < count; ++k) {
    if (!src[k] || !dst[k] || bytes[k] < 0 || (bytes[k] % 16) || (reinterpret_cast<uintptr_t>(src[k]) & 15) ||
        (reinterpret_cast<uintptr_t>(dst[k]) & 15))
      return -10;
    p.src[k] = static_cast<const uint4*>(src[k]);
    p.dst[k] = static_cast<uint4*>(dst[k]);
    p.n16[k] = bytes[k] / 16;
    total += p.n16[k];
  }
  p.count = count;
  if (total == 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;  // a copy that shares the GPU with compute kernels: a third of the SMs' slots
  copy_pieces_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
