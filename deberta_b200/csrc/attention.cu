// Flash-style attention for sm_100a with DeBERTa's disentangled position terms.
//
//   score[q,k] = ( Q[q]·K[k] + C2P[q, lut_c2p(q-k)] + P2C[k, lut_p2c(q-k)] ) / scale
//
// Q, K, V are token-major [B*S, ld] bf16 tensors (a head is a 64-column slice), read by TMA
// into 128B-swizzled shared memory. Both GEMMs of a tile (Q·Kᵀ and P·V) run on tcgen05 with
// accumulators in TMEM; one thread owns one query row (TMEM lane), so the softmax needs no
// shuffles and the position gathers are plain per-row loads. C2P / P2C are the per-head
// products of queries / keys with the projected relative-position table, computed once per
// layer by the GEMM kernel; they are read through L1/L2 with the bucket lookup tables held in
// shared memory. Masking: optional key-padding flags or packed-document ids; inactive queries
// produce zero rows. With document ids and a per-tile table of the ids' range, a CTA only visits the
// tiles whose range meets its own (block-diagonal skipping for packed sequences).
// The position terms are optional, which gives plain (rotary) attention.
//
// Forward : grid (q-tiles, heads, batch), 512 threads: four threads share a query row so that
//           16 warps hide the latency of the softmax arithmetic.
// Backward: grid (k-tiles, heads, batch); dK/dV accumulate in TMEM, dQ and the gradients of
//           C2P / P2C are reduced into fp32 buffers with red.global.add.
#include "tc05.cuh"

#include <type_traits>
#include "kernels.h"

namespace {

using namespace tc05;

constexpr int kTile = 128;   // query rows and key rows per tile
constexpr int kD = 64;       // head dimension
constexpr int kTileBytes = kTile * kD * 2;  // 16 KB

struct AttnDev {
  int B, S, heads;
  int span2;              // rows of the position tables (2 * att_span); 0 = no position terms
  float scale_log2;       // log2(e) / scale
  float inv_scale;        // 1 / scale
  const __nv_bfloat16* c2p;   // [B*S, heads, span2] or null
  const __nv_bfloat16* p2c;   // [B*S, heads, span2] or null
  const unsigned short* lut_c2p;  // [2S-1], index q-k+S-1
  const unsigned short* lut_p2c;
  const unsigned char* key_keep;  // [B*S] or null
  const int* doc_ids;             // [B*S] or null
  const int* doc_tiles;           // [B, tiles, 2]: smallest / largest non-zero id of each 128-token tile, or null
  const __nv_bfloat16* bias;      // [B, heads, S, ldb] pre-gathered position bias (unscaled) or null
  long long ldb;
  __nv_bfloat16* out;   // [B*S, ldo]
  long long ldo;
  float* lse;           // [B, heads, S] log2-domain log-sum-exp of the scaled scores
  int* status;
};

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Tiles whose document-id range [lo, hi] meets that of tile `self`: first such tile and the length of the
// run up to the last one (tiles inside the run that do not meet it are still visited and fully masked).
// A tile without live tokens has lo > hi and meets nothing; a CTA always visits at least one tile.
// Called by whole warps (32 tiles per ballot); without a table every tile is visited.
__device__ __forceinline__ void doc_tile_run(const int* tiles, int b, int ntiles, int self, int lane, int& first,
                                             int& count) {
  first = 0;
  count = ntiles;
  if (tiles == nullptr) return;
  const int* t = tiles + static_cast<long long>(b) * ntiles * 2;
  const int slo = t[2 * self], shi = t[2 * self + 1];
  int lo_tile = -1, hi_tile = -1;
  for (int base = 0; base < ntiles; base += 32) {
    const int i = base + lane;
    bool hit = false;
    if (i < ntiles) {
      const int lo = t[2 * i], hi = t[2 * i + 1];
      hit = lo <= hi && slo <= shi && lo <= shi && hi >= slo;
    }
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (m != 0) {
      if (lo_tile < 0) lo_tile = base + __ffs(m) - 1;
      hi_tile = base + 31 - __clz(m);
    }
  }
  if (lo_tile < 0) {
    count = 1;
  } else {
    first = lo_tile;
    count = hi_tile - lo_tile + 1;
  }
}

// 16 packed bf16 (32 contiguous bytes) of one row: one 256-bit store when aligned, else two 128-bit ones.
__device__ __forceinline__ void store_bf16x16(__nv_bfloat16* dst, const uint32_t* w) {
  if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
    st_global_32B(dst, w);
  } else {
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}


// --------------------------------------------------------------------------------------------
// forward
// --------------------------------------------------------------------------------------------
// KT = keys per tile. 128: one CTA of 512 threads per SM. 64: 256 threads and ~67 KB, so two CTAs share an SM and
// each one's barrier, TMEM and TMA latencies hide behind the other's arithmetic (short sequences give a CTA only a
// few key tiles to pipeline over).
template <int KT>
struct FwdSmem {
  static constexpr int kKVBytes = KT * kD * 2;        // one K or V tile
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;          // 2 buffers
  static constexpr int kV = kK + 2 * kKVBytes;        // 2 buffers
  static constexpr int kP = kV + 2 * kKVBytes;        // 128 x KT bf16 in 64-key blocks of 16 KB
  static constexpr int kBar = kP + (KT / 64) * kTileBytes;
  static constexpr int kMeta = kBar + 128;            // KT ints of key metadata
  static constexpr int kRed = kMeta + KT * 4;         // (KT / 32) x 128 floats: per column-group row statistics
  static constexpr int kLut = kRed + (KT / 32) * 512; // 2 * (2S-1) uint16
  static int total(int S, bool pos) { return kLut + (pos ? 2 * (2 * S) * 2 : 0) + 1024; }
};

// warp w owns the rows of TMEM lane quadrant (w & 3) and the key columns 32 * (w >> 2) .. of a tile
template <int KT>
constexpr int fwd_threads() { return KT * 4; }


__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Four threads share a query row (one per 32-key column group of the tile); the row maximum is
// exchanged through shared memory, the running sum stays per thread until the end.
// MASK: 0 = no mask (only the sequence end), 1 = key padding, 2 = document ids.
// POS: 0 = content scores only, 1 = key-indexed bias tensor, 2 = gathers from the bucket-indexed tables.
template <int MASK, int POS, int KT>
__global__ void __launch_bounds__(KT * 4, KT == 64 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = FwdSmem<KT>;
  constexpr int kThreads = KT * 4;
  constexpr int kParts = KT / 32;          // column groups of a tile = threads per query row
  constexpr int kOCols = kD / kParts;      // output columns a thread rescales and stores
  constexpr int kKV = L::kKVBytes;
  constexpr uint32_t kTmemCols = KT == 64 ? 128 : 256;
  uint8_t* sQ = smem + L::kQ;
  uint8_t* sK = smem + L::kK;
  uint8_t* sV = smem + L::kV;
  uint8_t* sP = smem + L::kP;
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* bar_k = bar_q + 1;  // [2]
  uint64_t* bar_v = bar_q + 3;  // [2]
  uint64_t* bar_s = bar_q + 5;
  uint64_t* bar_o = bar_q + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* kmeta = reinterpret_cast<int*>(smem + L::kMeta);
  float* red = reinterpret_cast<float*>(smem + L::kRed);  // [kParts][128] row maxima / sums per column group
  unsigned short* lutc = reinterpret_cast<unsigned short*>(smem + L::kLut);
  unsigned short* lutp = lutc + 2 * p.S;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int quad = warp & 3;
  const int part = warp >> 2;       // which 32 keys of the tile
  const int row = quad * 32 + lane; // query row inside the tile
  const int q0 = blockIdx.x * kTile;
  const int h = blockIdx.y;
  // The bias tensor was written batch by batch just before this launch and is larger than the L2 at training sizes:
  // walking the batch backwards starts with the part that is still cached.
  const int b = POS == 1 ? static_cast<int>(gridDim.z - 1 - blockIdx.z) : static_cast<int>(blockIdx.z);
  const int S = p.S;
  pdl_launch_dependents();

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(&bar_k[0], 1);
    mbar_init(&bar_k[1], 1);
    mbar_init(&bar_v[0], 1);
    mbar_init(&bar_v[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  pdl_wait();  // shared memory, barriers and TMEM are set up; everything below may touch global memory
  int jb = 0, nkt = (S + kTile - 1) / kTile;  // first key tile and number of key tiles this CTA visits
  if (MASK == 2) doc_tile_run(p.doc_tiles, b, nkt, blockIdx.x, lane, jb, nkt);  // in 128-token tiles
  if (KT == 64) {
    jb *= 2;
    nkt = min(nkt * 2, (S + KT - 1) / KT - jb);
  }
  if (POS == 2) {
    for (int i = tid; i < 2 * S - 1; i += kThreads) {
      lutc[i] = p.lut_c2p[i];
      lutp[i] = p.lut_p2c[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base;          // KT columns: scores
  const uint32_t t_o = tmem_base + KT;     // 64 columns: output accumulator
  const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;

  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    mbar_expect_tx(bar_q, kTileBytes);
    tma_load_3d(sQ, &tm_q, bar_q, h * kD, q0, b);
    mbar_expect_tx(&bar_k[0], kKV);
    tma_load_3d(sK, &tm_k, &bar_k[0], h * kD, jb * KT, b);
    mbar_expect_tx(&bar_v[0], kKV);
    tma_load_3d(sV, &tm_v, &bar_v[0], h * kD, jb * KT, b);
    if (nkt > 1) {  // second tile of K and V straight away: both buffers start empty
      mbar_expect_tx(&bar_k[1], kKV);
      tma_load_3d(sK + kKV, &tm_k, &bar_k[1], h * kD, (jb + 1) * KT, b);
      mbar_expect_tx(&bar_v[1], kKV);
      tma_load_3d(sV + kKV, &tm_v, &bar_v[1], h * kD, (jb + 1) * KT, b);
    }
  }

  const int q = q0 + row;
  const bool q_valid = q < S;
  const long long tq = static_cast<long long>(b) * S + (q_valid ? q : 0);
  int q_doc = 1;
  bool q_live = q_valid;
  if (MASK == 1 && q_valid) q_live = p.key_keep[tq] != 0;
  if (MASK == 2 && q_valid) {
    q_doc = p.doc_ids[tq];
    q_live = q_doc != 0;
  }
  const long long pos_row = static_cast<long long>(p.heads) * p.span2;
  const __nv_bfloat16* c2p_row = (POS == 2 && p.c2p) ? p.c2p + tq * pos_row + static_cast<long long>(h) * p.span2 : nullptr;
  const uint4* bias_row = POS == 1 ? reinterpret_cast<const uint4*>(
                                         p.bias + ((static_cast<long long>(b) * p.heads + h) * S + (q_valid ? q : 0)) * p.ldb)
                                   : nullptr;

  constexpr uint32_t idesc_s = make_idesc_bf16(128, KT, false, false);
  constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, false, true);
  bool ok = true;

  if (tid == 0) {  // first score tile
    ok = mbar_wait(bar_q, 0, abort_flag, p.status, kErrFullWait) &&
         mbar_wait(&bar_k[0], 0, abort_flag, p.status, kErrFullWait);
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(t_s, make_smem_desc(smem_u32(sQ) + ks * 32, 16, 1024), make_smem_desc(smem_u32(sK) + ks * 32, 16, 1024),
                  idesc_s, ks > 0);
    }
    umma_commit(bar_s);
  }

  float m_run = -INFINITY, l_part = 0.f;
  // bias of this thread's 32 keys, fetched one tile ahead so that the L2 round trip overlaps the previous tile's math
  uint4 bias_pf[4] = {};
  if (POS == 1) {
#pragma unroll
    for (int g = 0; g < 4; ++g) bias_pf[g] = __ldg(bias_row + ((jb * KT + part * 32) >> 3) + g);
  }
  for (int j = 0; j < nkt; ++j) {  // j counts visited tiles (buffers and barrier phases follow it)
    const int k0 = (jb + j) * KT;
    bool tile_all_keep = false;
    if (MASK != 0) {
      int tile_meta = 1;
      if (tid < KT) {  // key metadata of this tile: 0 = masked, otherwise doc id (or 1)
        const int kk = k0 + tid;
        int meta = 0;
        if (kk < S) {
          const long long tk = static_cast<long long>(b) * S + kk;
          meta = MASK == 1 ? (p.key_keep[tk] ? 1 : 0) : p.doc_ids[tk];
        }
        kmeta[tid] = meta;
        tile_meta = meta;
      }
      // padding masks are all-ones for most tiles: those skip the per-element selects
      tile_all_keep = __syncthreads_and(MASK == 1 && tile_meta != 0) != 0;
    }
    // A wait that ran out must not let this thread leave the loop alone (the others would meet it at different
    // barriers): its answer is combined at the next block barrier and the whole block leaves together.
    const bool got_s = mbar_wait(bar_s, j & 1, abort_flag, p.status, kErrAccFullWait);
    tc_fence_after();

    float s[32];  // unscaled scores of this thread's 32 keys
    {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_s + lane_addr + part * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]);
    }
    float tmax = -INFINITY;
    const int kb = k0 + part * 32;  // first key of this thread's column group
    if (POS == 1) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 bvec = bias_pf[g];
        const uint32_t w[4] = {bvec.x, bvec.y, bvec.z, bvec.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[g * 8 + 2 * e] += __uint_as_float(w[e] << 16);
          s[g * 8 + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
        }
      }
      if (j + 1 < nkt) {
#pragma unroll
        for (int g = 0; g < 4; ++g) bias_pf[g] = __ldg(bias_row + ((kb + KT) >> 3) + g);
      }
    } else if (POS == 2) {
      const int dbase = q - kb + S - 1;  // lut index for the first key
      const __nv_bfloat16* p2c_base =
          p.p2c ? p.p2c + (static_cast<long long>(b) * S + kb) * pos_row + static_cast<long long>(h) * p.span2 : nullptr;
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        if (q_valid && kb + k < S) {
          const int di = dbase - k;
          if (c2p_row) s[k] += __bfloat162float(c2p_row[lutc[di]]);
          if (p2c_base) s[k] += __bfloat162float(p2c_base[static_cast<long long>(k) * pos_row + lutp[di]]);
        }
      }
    }
    if (MASK == 0) {
      if (k0 + KT > S) {  // last, partial tile (block-uniform)
#pragma unroll
        for (int k = 0; k < 32; ++k) s[k] = (kb + k < S) ? s[k] : -INFINITY;
      }
    } else if (!tile_all_keep) {
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const int meta = kmeta[part * 32 + k];
        const bool keep = MASK == 1 ? (meta != 0) : (meta != 0 && meta == q_doc);
        s[k] = keep ? s[k] : -INFINITY;
      }
    }
#pragma unroll
    for (int k = 0; k < 32; ++k) tmax = fmaxf(tmax, s[k]);
    red[part * kTile + row] = tmax;
    tc_fence_before();
    // every thread has read its scores of tile j: the score accumulator is free again
    if (!__syncthreads_and(got_s)) { ok = false; break; }
    if (tid == 0 && j + 1 < nkt) {  // scores of the next tile run on the tensor core during this tile's softmax
      const int nb = (j + 1) & 1;
      if (mbar_wait(&bar_k[nb], ((j + 1) >> 1) & 1, abort_flag, p.status, kErrFullWait)) {
        tc_fence_after();
        const uint32_t kb2 = smem_u32(sK + nb * kKV);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16(t_s, make_smem_desc(smem_u32(sQ) + ks * 32, 16, 1024), make_smem_desc(kb2 + ks * 32, 16, 1024),
                    idesc_s, ks > 0);
      }
      umma_commit(bar_s);
    }
    tmax = fmaxf(red[row], red[kTile + row]);
    if (kParts == 4) tmax = fmaxf(tmax, fmaxf(red[2 * kTile + row], red[3 * kTile + row]));
    const float m_new = fmaxf(m_run, tmax);  // running maximum of the unscaled scores
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = (m_run == -INFINITY) ? 0.f : ex2((m_run - m_use) * p.scale_log2);
    const float neg_ms = -m_use * p.scale_log2;
    float lsum = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      s[k] = ex2(fmaf(s[k], p.scale_log2, neg_ms));
      lsum += s[k];
    }
    l_part = l_part * alpha + lsum;
    m_run = m_new;

    bool got_o = true;
    if (j > 0) {
      got_o = __all_sync(0xffffffffu, mbar_wait(bar_o, (j - 1) & 1, abort_flag, p.status, kErrAccFullWait));
      tc_fence_after();
      // rescale the running output (this thread's share of its 64 columns) when a row of this warp raised its maximum
      if (got_o && __any_sync(0xffffffffu, alpha != 1.f)) {
        uint32_t r[kOCols];
        if constexpr (kOCols == 16) tmem_ld_32x32b_x16(t_o + lane_addr + part * kOCols, r);
        else tmem_ld_32x32b_x32(t_o + lane_addr + part * kOCols, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < kOCols; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        if constexpr (kOCols == 16) tmem_st_32x32b_x16(t_o + lane_addr + part * kOCols, r);
        else tmem_st_32x32b_x32(t_o + lane_addr + part * kOCols, r);
        tmem_st_wait();
      }
    }
    if (tid == 0 && j > 0 && j + 1 < nkt) {
      // P·V of tile j-1 and the scores of tile j have retired: buffer (j+1)&1 of V and of K is free for tile j+1
      const int nb = (j + 1) & 1;
      mbar_expect_tx(&bar_v[nb], kKV);
      tma_load_3d(sV + nb * kKV, &tm_v, &bar_v[nb], h * kD, k0 + KT, b);
    }
    // this thread's 32 probabilities: 4 chunks of 8 bf16 in 64-key block (part >> 1)
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) {
      uint4 u;
      u.x = pack_bf16(s[g4 * 8 + 0], s[g4 * 8 + 1]);
      u.y = pack_bf16(s[g4 * 8 + 2], s[g4 * 8 + 3]);
      u.z = pack_bf16(s[g4 * 8 + 4], s[g4 * 8 + 5]);
      u.w = pack_bf16(s[g4 * 8 + 6], s[g4 * 8 + 7]);
      *reinterpret_cast<uint4*>(sP + (part >> 1) * kTileBytes + swz128(row, (part & 1) * 4 + g4)) = u;
    }
    fence_proxy_async();
    tc_fence_before();
    if (!__syncthreads_and(got_o)) { ok = false; break; }
    if (tid == 0) {
      const bool v_ok = mbar_wait(&bar_v[j & 1], (j >> 1) & 1, abort_flag, p.status, kErrFullWait);
      tc_fence_after();
      const uint32_t pv = smem_u32(sV + (j & 1) * kKV);
#pragma unroll
      for (int ks = 0; ks < KT / 16; ++ks) {
        if (!v_ok) break;
        umma_bf16(t_o, make_smem_desc(smem_u32(sP) + (ks >> 2) * kTileBytes + (ks & 3) * 32, 16, 1024),
                  make_smem_desc(pv + ks * 2048, 8192, 1024), idesc_o, (j > 0) || (ks > 0));
      }
      umma_commit(bar_o);
      if (j + 2 < nkt) {  // K buffer j&1 was read by the scores of tile j (retired before this tile's softmax ended)
        mbar_expect_tx(&bar_k[j & 1], kKV);
        tma_load_3d(sK + (j & 1) * kKV, &tm_k, &bar_k[j & 1], h * kD, k0 + 2 * KT, b);
      }
    }
  }

  // row sums: combine the four column groups
  __syncthreads();
  red[part * kTile + row] = l_part;
  __syncthreads();
  float l_run = red[row] + red[kTile + row];
  if (kParts == 4) l_run += red[2 * kTile + row] + red[3 * kTile + row];
  if (ok && mbar_wait(bar_o, (nkt - 1) & 1, abort_flag, p.status, kErrAccFullWait)) {
    tc_fence_after();
    const float inv = (q_live && l_run > 0.f) ? 1.f / l_run : 0.f;
    __nv_bfloat16* o = p.out + tq * p.ldo + h * kD + part * kOCols;
    uint32_t r[kOCols];
    if constexpr (kOCols == 16) tmem_ld_32x32b_x16(t_o + lane_addr + part * kOCols, r);
    else tmem_ld_32x32b_x32(t_o + lane_addr + part * kOCols, r);
    tmem_ld_wait();
    if (q_valid) {
      uint32_t w[kOCols / 2];
#pragma unroll
      for (int g = 0; g < kOCols / 2; ++g)
        w[g] = pack_bf16(__uint_as_float(r[2 * g]) * inv, __uint_as_float(r[2 * g + 1]) * inv);
      store_bf16x16(o, w);
      if constexpr (kOCols == 32) store_bf16x16(o + 16, w + 8);
    }
    if (q_valid && part == 0 && p.lse)
      p.lse[(static_cast<long long>(b) * p.heads + h) * S + q] =
          (q_live && l_run > 0.f) ? (m_run * p.scale_log2 + log2f(l_run)) : INFINITY;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------------------------
// forward, warp-specialised (64 keys per tile, no document ids, no in-kernel table gathers)
// --------------------------------------------------------------------------------------------
// Same arithmetic as attn_fwd_kernel<MASK, POS, 64>, different choreography. A ninth warp owns every TMA load and
// every MMA; the eight softmax warps never meet at a block-wide barrier inside the loop. What orders them:
//   bar_s[2]      (tcgen05.commit)  scores of a tile are in TMEM buffer j & 1 (two buffers: the next tile's scores are
//                                   computed while this tile's are still being read)
//   bar_sfree[2]  (8 warp arrivals) every softmax warp has copied its scores of that buffer into registers
//   bar_pair[4]   (2 warp arrivals) the two warps that share query rows have published their partial row maxima
//   bar_p         (8 warp arrivals) P of the tile is in shared memory and the running output has been rescaled
//   bar_o         (tcgen05.commit)  P·V of a tile has retired: P may be overwritten, O may be rescaled or read
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, which ends every other role's waits too.
struct FwdWsSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;       // 2 x 8 KB
  static constexpr int kV = kK + kTileBytes;       // 2 x 8 KB
  static constexpr int kP = kV + kTileBytes;       // 128 x 64 bf16
  static constexpr int kBar = kP + kTileBytes;     // 16 barriers + TMEM slot + abort flag
  static constexpr int kRed = kBar + 256;          // [2 tiles][2 column groups][128 rows] floats
  static constexpr int kTotal = kRed + 2048 + 1024;
};
constexpr int kFwdWsThreads = 288;  // warps 0-7: softmax (quadrant w & 3, 32-key column group w >> 2); warp 8: TMA + MMA

template <int MASK, int POS>  // MASK 0 | 1, POS 0 | 1
__global__ void __launch_bounds__(kFwdWsThreads, 2)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const AttnDev p) {
  constexpr int KT = 64;
  constexpr int kKV = KT * kD * 2;
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + FwdWsSmem::kQ;
  uint8_t* sK = smem + FwdWsSmem::kK;
  uint8_t* sV = smem + FwdWsSmem::kV;
  uint8_t* sP = smem + FwdWsSmem::kP;
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + FwdWsSmem::kBar);
  uint64_t* bar_k = bar_q + 1;      // [2]
  uint64_t* bar_v = bar_q + 3;      // [2]
  uint64_t* bar_s = bar_q + 5;      // [2]
  uint64_t* bar_sfree = bar_q + 7;  // [2]
  uint64_t* bar_pair = bar_q + 9;   // [4]
  uint64_t* bar_p = bar_q + 13;
  uint64_t* bar_o = bar_q + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(smem + FwdWsSmem::kRed);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int q0 = blockIdx.x * kTile;
  const int h = blockIdx.y;
  const int b = POS == 1 ? static_cast<int>(gridDim.z - 1 - blockIdx.z) : static_cast<int>(blockIdx.z);  // see attn_fwd_kernel
  const int S = p.S;
  const int nkt = (S + KT - 1) / KT;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_k[i], 1);
      mbar_init(&bar_v[i], 1);
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_sfree[i], 8);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&bar_pair[i], 2);
    mbar_init(bar_p, 8);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_o = tmem_base + 128;  // scores: columns [0, 64) and [64, 128)

  if (warp == 8) {
    // ------------------------------------ TMA + MMA ------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, KT, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, false, true);
      auto issue_scores = [&](int buf) {
        const uint32_t kaddr = smem_u32(sK + buf * kKV);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16(tmem_base + buf * KT, make_smem_desc(smem_u32(sQ) + ks * 32, 16, 1024),
                    make_smem_desc(kaddr + ks * 32, 16, 1024), idesc_s, ks > 0);
        umma_commit(&bar_s[buf]);
      };
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(bar_q, kTileBytes);
      tma_load_3d(sQ, &tm_q, bar_q, h * kD, q0, b);
      for (int t = 0; t < 2 && t < nkt; ++t) {
        mbar_expect_tx(&bar_k[t], kKV);
        tma_load_3d(sK + t * kKV, &tm_k, &bar_k[t], h * kD, t * KT, b);
        mbar_expect_tx(&bar_v[t], kKV);
        tma_load_3d(sV + t * kKV, &tm_v, &bar_v[t], h * kD, t * KT, b);
      }
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, kErrFullWait) &&
                mbar_wait(&bar_k[0], 0, abort_flag, p.status, kErrFullWait);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
        if (nkt > 1) {
          ok = mbar_wait(&bar_k[1], 0, abort_flag, p.status, kErrFullWait);
          if (ok) {
            tc_fence_after();
            issue_scores(1);
          }
        }
      }
      for (int j = 0; j < nkt && ok; ++j) {
        const int sb = j & 1;
        const uint32_t use = (j >> 1) & 1;  // parity of the j-th tile's use of a double-buffered resource
        if (j + 2 < nkt) {  // K buffer sb is free once the scores of tile j have retired
          ok = mbar_wait(&bar_s[sb], use, abort_flag, p.status, kErrAccFullWait);
          if (!ok) break;
          mbar_expect_tx(&bar_k[sb], kKV);
          tma_load_3d(sK + sb * kKV, &tm_k, &bar_k[sb], h * kD, (j + 2) * KT, b);
        }
        if (j >= 1 && j + 1 < nkt) {  // V buffer (j+1) & 1 held tile j-1: free once its P·V has retired
          ok = mbar_wait(bar_o, (j - 1) & 1, abort_flag, p.status, kErrAccFullWait);
          if (!ok) break;
          const int vb = (j + 1) & 1;
          mbar_expect_tx(&bar_v[vb], kKV);
          tma_load_3d(sV + vb * kKV, &tm_v, &bar_v[vb], h * kD, (j + 1) * KT, b);
        }
        ok = mbar_wait(bar_p, j & 1, abort_flag, p.status, kErrAccEmptyWait) &&
             mbar_wait(&bar_v[sb], use, abort_flag, p.status, kErrFullWait);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t pv = smem_u32(sV + sb * kKV);
#pragma unroll
          for (int ks = 0; ks < KT / 16; ++ks)
            umma_bf16(t_o, make_smem_desc(smem_u32(sP) + ks * 32, 16, 1024), make_smem_desc(pv + ks * 2048, 8192, 1024),
                      idesc_o, (j > 0) || (ks > 0));
          umma_commit(bar_o);
        }
        if (j + 2 < nkt) {  // scores of tile j+2 into the buffer every softmax warp has emptied
          ok = mbar_wait(&bar_k[sb], ((j + 2) >> 1) & 1, abort_flag, p.status, kErrFullWait) &&
               mbar_wait(&bar_sfree[sb], use, abort_flag, p.status, kErrAccEmptyWait);
          if (!ok) break;
          tc_fence_after();
          issue_scores(sb);
        }
      }
    }
  } else {
    // ------------------------------------ softmax ------------------------------------
    const int quad = warp & 3;
    const int part = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int q = q0 + row;
    const bool q_valid = q < S;
    const long long tq = static_cast<long long>(b) * S + (q_valid ? q : 0);
    bool q_live = q_valid;
    if (MASK == 1 && q_valid) q_live = p.key_keep[tq] != 0;
    const uint4* bias_row = POS == 1 ? reinterpret_cast<const uint4*>(
                                           p.bias + ((static_cast<long long>(b) * p.heads + h) * S + (q_valid ? q : 0)) * p.ldb)
                                     : nullptr;
    float m_run = -INFINITY, l_part = 0.f;
    uint4 bias_pf[4] = {};
    if (POS == 1) {
#pragma unroll
      for (int g = 0; g < 4; ++g) bias_pf[g] = __ldg(bias_row + ((part * 32) >> 3) + g);
    }
    // a wait's answer is agreed by the whole warp: the TMEM loads, votes and arrivals below are warp-collective
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int err) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, p.status, err)) != 0;
    };
    bool ok = true;
    for (int j = 0; j < nkt; ++j) {
      const int sb = j & 1;
      const int kb = j * KT + part * 32;  // first key of this thread's column group
      uint4 keep_lo = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u), keep_hi = keep_lo;
      if (MASK == 1) {  // this thread's 32 keep bytes (keys past the end read as dropped)
        const unsigned char* kp = p.key_keep + static_cast<long long>(b) * S + kb;
        if (kb + 32 <= S && ((reinterpret_cast<uintptr_t>(kp) & 15) == 0)) {
          keep_lo = __ldg(reinterpret_cast<const uint4*>(kp));
          keep_hi = __ldg(reinterpret_cast<const uint4*>(kp) + 1);
        } else {
          unsigned int w[8] = {};
          for (int k = 0; k < 32; ++k)
            if (kb + k < S && kp[k]) w[k >> 2] |= 1u << (8 * (k & 3));
          keep_lo = make_uint4(w[0], w[1], w[2], w[3]);
          keep_hi = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      if (!wait_all(&bar_s[sb], (j >> 1) & 1, kErrAccFullWait)) { ok = false; break; }
      tc_fence_after();
      float s[32];
      {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + sb * KT + lane_addr + part * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_sfree[sb]);
      if (POS == 1) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4 bvec = bias_pf[g];
          const uint32_t w[4] = {bvec.x, bvec.y, bvec.z, bvec.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[g * 8 + 2 * e] += __uint_as_float(w[e] << 16);
            s[g * 8 + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
        if (j + 1 < nkt) {
#pragma unroll
          for (int g = 0; g < 4; ++g) bias_pf[g] = __ldg(bias_row + ((kb + KT) >> 3) + g);
        }
        // a 64-key tile is too short to hide a DRAM access behind: the 64 bytes of the tile after the next one are
        // asked into the L2 already
        if (j + 2 < nkt) asm volatile("prefetch.global.L2 [%0];" ::"l"(bias_row + ((kb + 2 * KT) >> 3)));
      }
      if (MASK == 0) {
        if (j * KT + KT > S) {
#pragma unroll
          for (int k = 0; k < 32; ++k) s[k] = (kb + k < S) ? s[k] : -INFINITY;
        }
      } else {
        // every lane of the warp looks at the same 32 keys, so "all of them kept" (the usual case: packed batches carry
        // a mask of ones) is a warp-uniform test that skips the per-score selects
        const bool all_kept = kb + 32 <= S &&
                              (keep_lo.x & keep_lo.y & keep_lo.z & keep_lo.w & keep_hi.x & keep_hi.y & keep_hi.z & keep_hi.w) ==
                                  0x01010101u &&
                              (keep_lo.x | keep_lo.y | keep_lo.z | keep_lo.w | keep_hi.x | keep_hi.y | keep_hi.z | keep_hi.w) ==
                                  0x01010101u;
        if (!all_kept) {
          const uint32_t kw[8] = {keep_lo.x, keep_lo.y, keep_lo.z, keep_lo.w, keep_hi.x, keep_hi.y, keep_hi.z, keep_hi.w};
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const bool keep = ((kw[k >> 2] >> (8 * (k & 3))) & 0xffu) != 0 && (kb + k < S);
            s[k] = keep ? s[k] : -INFINITY;
          }
        }
      }
      float tmax = -INFINITY;
#pragma unroll
      for (int k = 0; k < 32; ++k) tmax = fmaxf(tmax, s[k]);
      float* red_t = red + sb * 256;  // per-tile-parity copy: the partner may still be reading the previous tile's
      red_t[part * kTile + row] = tmax;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_pair[quad]);
      if (!wait_all(&bar_pair[quad], j & 1, kErrGeneric)) { ok = false; break; }
      tmax = fmaxf(red_t[row], red_t[kTile + row]);
      const float m_new = fmaxf(m_run, tmax);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : ex2((m_run - m_use) * p.scale_log2);
      const float neg_ms = -m_use * p.scale_log2;
      float lsum = 0.f;
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        s[k] = ex2(fmaf(s[k], p.scale_log2, neg_ms));
        lsum += s[k];
      }
      l_part = l_part * alpha + lsum;
      m_run = m_new;
      if (j > 0) {  // P·V of the previous tile retired: its P is consumed and O is stable
        if (!wait_all(bar_o, (j - 1) & 1, kErrAccFullWait)) { ok = false; break; }
        tc_fence_after();
      }
      // P first, then the rescaling of O: the 32 probabilities are dead before the 32 accumulator values arrive, so
      // the two sets never hold registers at the same time
#pragma unroll
      for (int g4 = 0; g4 < 4; ++g4) {
        uint4 u;
        u.x = pack_bf16(s[g4 * 8 + 0], s[g4 * 8 + 1]);
        u.y = pack_bf16(s[g4 * 8 + 2], s[g4 * 8 + 3]);
        u.z = pack_bf16(s[g4 * 8 + 4], s[g4 * 8 + 5]);
        u.w = pack_bf16(s[g4 * 8 + 6], s[g4 * 8 + 7]);
        *reinterpret_cast<uint4*>(sP + swz128(row, part * 4 + g4)) = u;
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_o + lane_addr + part * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st_32x32b_x32(t_o + lane_addr + part * 32, r);
        tmem_st_wait();
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
    }
    // row sums of the two column groups, then the output
    if (ok) {
      float* red_t = red + (nkt & 1) * 256;
      red_t[part * kTile + row] = l_part;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_pair[quad]);
      ok = wait_all(&bar_pair[quad], nkt & 1, kErrGeneric);
      const float l_run = red_t[row] + red_t[kTile + row];
      if (ok && wait_all(bar_o, (nkt - 1) & 1, kErrAccFullWait)) {
        tc_fence_after();
        const float inv = (q_live && l_run > 0.f) ? 1.f / l_run : 0.f;
        __nv_bfloat16* o = p.out + tq * p.ldo + h * kD + part * 32;
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_o + lane_addr + part * 32, r);
        tmem_ld_wait();
        if (q_valid) {
          uint32_t w[16];
#pragma unroll
          for (int g = 0; g < 16; ++g) w[g] = pack_bf16(__uint_as_float(r[2 * g]) * inv, __uint_as_float(r[2 * g + 1]) * inv);
          store_bf16x16(o, w);
          store_bf16x16(o + 16, w + 8);
        }
        if (q_valid && part == 0 && p.lse)
          p.lse[(static_cast<long long>(b) * p.heads + h) * S + q] =
              (q_live && l_run > 0.f) ? (m_run * p.scale_log2 + log2f(l_run)) : INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// --------------------------------------------------------------------------------------------
// backward
// --------------------------------------------------------------------------------------------
struct AttnBwdDev {
  int B, S, heads, span2;
  float scale_log2, inv_scale;
  const __nv_bfloat16* c2p;
  const __nv_bfloat16* p2c;
  const unsigned short* lut_c2p;
  const unsigned short* lut_p2c;
  const unsigned char* key_keep;
  const int* doc_ids;
  const int* doc_tiles;       // as in the forward kernel
  const __nv_bfloat16* bias;  // [B, heads, S, ldb] or null
  __nv_bfloat16* dbias;       // [B, heads, S, ldb] gradient of the bias (written when bias is given)
  long long ldb;
  const float* lse;     // [B, heads, S] (log2 domain)
  const float* delta;   // [B, heads, S] rowsum(dO * O)
  float* dq_acc;        // [B*S, heads*64] fp32, zero-initialised
  __nv_bfloat16* dk;    // [B*S, ldk]
  __nv_bfloat16* dv;
  long long ldk, ldv;
  float* d_c2p;         // [B*S, heads, span2] fp32, zero-initialised (or null)
  float* d_p2c;
  int* status;
};

struct BwdSmem {
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kQ = kV + kTileBytes;           // 3 buffers
  static constexpr int kdO = kQ + 3 * kTileBytes;      // 3 buffers
  static constexpr int kP = kdO + 3 * kTileBytes;      // 128x128 bf16
  static constexpr int kdS = kP + 2 * kTileBytes;      // 128x128 bf16
  static constexpr int kBar = kdS + 2 * kTileBytes;
  static constexpr int kMeta = kBar + 128;
  static constexpr int kLut = kMeta + 512;
  static int total(int S, bool pos) { return kLut + (pos ? 2 * (2 * S) * 2 : 0) + 1024; }
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

constexpr int kBwdThreads = 512;  // warp w: TMEM lane quadrant (w & 3), 32-key column group (w >> 2)

template <int MASK, int POS>  // as in the forward kernel
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const AttnBwdDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + BwdSmem::kK;
  uint8_t* sV = smem + BwdSmem::kV;
  uint8_t* sQ = smem + BwdSmem::kQ;
  uint8_t* sdO = smem + BwdSmem::kdO;
  uint8_t* sP = smem + BwdSmem::kP;
  uint8_t* sdS = smem + BwdSmem::kdS;
  uint64_t* bar_kv = reinterpret_cast<uint64_t*>(smem + BwdSmem::kBar);
  uint64_t* bar_qd = bar_kv + 1;  // [3]
  uint64_t* bar_s = bar_kv + 4;
  uint64_t* bar_g = bar_kv + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_kv + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* kmeta = reinterpret_cast<int*>(smem + BwdSmem::kMeta);
  unsigned short* lutc = reinterpret_cast<unsigned short*>(smem + BwdSmem::kLut);
  unsigned short* lutp = lutc + 2 * p.S;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int quad = warp & 3;
  const int part = warp >> 2;
  const int row = quad * 32 + lane;  // row of the tile this thread works on (query row, or key row at the end)
  const int S = p.S;
  // Work items are (batch, head, key tile) triples, key tile fastest. A CTA takes items blockIdx.x, blockIdx.x +
  // gridDim.x, ...: the launcher starts one CTA per item where items differ in length (document ids) and one per SM
  // otherwise, so that barriers, tensor memory and the lookup tables are set up once and the loads of the next item
  // fly while the gradients of the current one leave the tensor memory.
  const int nkt_all = (S + kTile - 1) / kTile;
  const int n_items = nkt_all * p.heads * p.B;
  pdl_launch_dependents();

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(&bar_qd[0], 1);
    mbar_init(&bar_qd[1], 1);
    mbar_init(&bar_qd[2], 1);
    // One thread gets a 64- or 128-column MMA out only every 70-100 clocks (about twice what the tensor core needs for
    // it), and it is blocked while it does. The score MMAs are therefore issued by two threads of different warps and
    // the gradient MMAs by three, each committing its own: a phase of these barriers takes 2 resp. 3 arrivals.
    mbar_init(bar_s, 2);
    mbar_init(bar_g, 3);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  pdl_wait();  // set-up done; everything below may touch global memory
  if (POS == 2) {
    for (int i = tid; i < 2 * S - 1; i += kBwdThreads) {
      lutc[i] = p.lut_c2p[i];
      lutp[i] = p.lut_p2c[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 320,
                 t_dq = tmem_base + 384;
  const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
  const long long pos_row = static_cast<long long>(p.heads) * p.span2;

  constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);    // Q·Kᵀ, dO·Vᵀ
  constexpr uint32_t idesc_t = make_idesc_bf16(128, 64, true, true);       // Pᵀ·dO, dSᵀ·Q
  constexpr uint32_t idesc_q = make_idesc_bf16(128, 64, false, true);      // dS·K

  const bool issuer_s = tid == 0, issuer_dp = tid == 32;  // (also: dV and dK; thread 64 issues dQ)
  auto issue_scores = [&](int buf) {  // called by both issuers, each for its own product
    if (issuer_s) {
      const uint32_t q = smem_u32(sQ + buf * kTileBytes);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(t_s, make_smem_desc(q + ks * 32, 16, 1024), make_smem_desc(smem_u32(sK) + ks * 32, 16, 1024), idesc_s,
                  ks > 0);
    } else {
      const uint32_t d = smem_u32(sdO + buf * kTileBytes);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(t_dp, make_smem_desc(d + ks * 32, 16, 1024), make_smem_desc(smem_u32(sV) + ks * 32, 16, 1024), idesc_s,
                  ks > 0);
    }
    umma_commit(bar_s);
  };

  // K, V and the first two (Q, dO) tiles of an item; `g` is the running count of query tiles this CTA has visited,
  // which names the ring slot (g % 3) and the barrier phase ((g / 3) & 1) of a tile
  auto issue_item_loads = [&](int b_, int h_, int k0_, int ib_, int nqt_, int g) {
    mbar_expect_tx(bar_kv, 2 * kTileBytes);
    tma_load_3d(sK, &tm_k, bar_kv, h_ * kD, k0_, b_);
    tma_load_3d(sV, &tm_v, bar_kv, h_ * kD, k0_, b_);
    for (int t = 0; t < 2 && t < nqt_; ++t) {
      const int slot = (g + t) % 3;
      mbar_expect_tx(&bar_qd[slot], 2 * kTileBytes);
      tma_load_3d(sQ + slot * kTileBytes, &tm_q, &bar_qd[slot], h_ * kD, (ib_ + t) * kTile, b_);
      tma_load_3d(sdO + slot * kTileBytes, &tm_do, &bar_qd[slot], h_ * kD, (ib_ + t) * kTile, b_);
    }
  };
  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
  }

  bool ok = true;
  int g0 = 0;       // query tiles visited by this CTA before the current item
  int n_done = 0;   // items finished by this CTA (phase of bar_kv)
  bool loads_issued = false;  // the previous item already asked for this item's operands
  for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
  const int k0 = (w % nkt_all) * kTile;
  const int h = (w / nkt_all) % p.heads;
  const int b = w / (nkt_all * p.heads);
  int ib = 0, nqt = nkt_all;  // first query tile and number of query tiles of this item
  if (MASK == 2) doc_tile_run(p.doc_tiles, b, nkt_all, w % nkt_all, lane, ib, nqt);
  if (tid == 0 && !loads_issued) issue_item_loads(b, h, k0, ib, nqt, g0);
  int cta_meta = 1;
  if (MASK != 0 && tid < kTile) {
    const int kk = k0 + tid;
    int meta = 0;
    if (kk < S) {
      const long long tk = static_cast<long long>(b) * S + kk;
      meta = MASK == 1 ? (p.key_keep[tk] ? 1 : 0) : p.doc_ids[tk];
    }
    kmeta[tid] = meta;
    cta_meta = meta;
  }
  const bool tile_all_keep = __syncthreads_and(MASK == 1 && cta_meta != 0) != 0;  // all 128 keys of this item are kept
  if (issuer_s || issuer_dp) {
    if (mbar_wait(bar_kv, n_done & 1, abort_flag, p.status, kErrFullWait) &&
        mbar_wait(&bar_qd[g0 % 3], (g0 / 3) & 1, abort_flag, p.status, kErrFullWait)) {
      tc_fence_after();
      issue_scores(g0 % 3);
    } else {
      umma_commit(bar_s);
    }
  }

  auto flush_dq = [&](int qt) {  // dQ of q-tile `qt` from TMEM into the fp32 accumulator (16 columns per thread)
    const int q = qt * kTile + row;
    uint32_t r[16];
    tmem_ld_32x32b_x16(t_dq + lane_addr + part * 16, r);
    tmem_ld_wait();
    if (q < S) {
      float* dst = p.dq_acc + (static_cast<long long>(b) * S + q) * (static_cast<long long>(p.heads) * kD) + h * kD + part * 16;
#pragma unroll
      for (int g = 0; g < 4; ++g)
        red_add_v4(dst + g * 4, __uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]), __uint_as_float(r[g * 4 + 2]),
                   __uint_as_float(r[g * 4 + 3]));
    }
  };

  for (int i = 0; i < nqt; ++i) {  // i counts the visited tiles of this item; buffers and barrier phases follow g
    const int g = g0 + i;
    const int buf = g % 3;
    const int q0 = (ib + i) * kTile;
    // per-row inputs that do not depend on the scores are requested before the wait: their latency hides behind the MMAs
    const int q = q0 + row;
    const bool q_valid = q < S;
    const long long stat = (static_cast<long long>(b) * p.heads + h) * S + (q_valid ? q : 0);
    const float lse = q_valid ? p.lse[stat] : INFINITY;
    const float delta = q_valid ? p.delta[stat] : 0.f;
    const long long brow_off = ((static_cast<long long>(b) * p.heads + h) * S + (q_valid ? q : 0)) * p.ldb + k0;
    const uint4* bias_row = POS == 1 ? reinterpret_cast<const uint4*>(p.bias + brow_off) : nullptr;
    uint4 bias_cur[4] = {};
    if (POS == 1) {
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) bias_cur[g8] = __ldg(bias_row + part * 4 + g8);
      // the same 64 bytes of the next query tile's row: fetched into the L2 now (no registers to spare for a
      // tile-ahead copy here), so that the next iteration's load does not wait for DRAM
      if (i + 1 < nqt && q + kTile < S)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.bias + brow_off + static_cast<long long>(kTile) * p.ldb + part * 32));
    }
    bool got_g = true;
    // (a wait that ran out is reported at the next block barrier, where the whole block leaves the loop together)
    const bool got_s = mbar_wait(bar_s, g & 1, abort_flag, p.status, kErrAccFullWait);
    tc_fence_after();
    uint32_t rs[32], rd[32];  // this thread's 32 scores and 32 dP values of tile i
    tmem_ld_32x32b_x32(t_s + lane_addr + part * 32, rs);
    tmem_ld_32x32b_x32(t_dp + lane_addr + part * 32, rd);
    tmem_ld_wait();
    tc_fence_before();
    // both accumulators are in registers: the tensor core may start on tile i+1
    if (!__syncthreads_and(got_s)) { ok = false; break; }
    if ((issuer_s || issuer_dp) && i + 1 < nqt) {
      const int nb = (g + 1) % 3;
      if (mbar_wait(&bar_qd[nb], ((g + 1) / 3) & 1, abort_flag, p.status, kErrFullWait)) {
        tc_fence_after();
        issue_scores(nb);
      } else {
        umma_commit(bar_s);
      }
    }

    const long long tq = static_cast<long long>(b) * S + (q_valid ? q : 0);
    int q_doc = 1;
    if (MASK == 2 && q_valid) q_doc = p.doc_ids[tq];
    const __nv_bfloat16* c2p_row = (POS == 2 && p.c2p) ? p.c2p + tq * pos_row + static_cast<long long>(h) * p.span2 : nullptr;
    float* dc2p_row = (POS == 2 && p.d_c2p) ? p.d_c2p + tq * pos_row + static_cast<long long>(h) * p.span2 : nullptr;
    const long long kbase = (static_cast<long long>(b) * S + k0) * pos_row + static_cast<long long>(h) * p.span2;
    const int dbase = q - k0 + S - 1;
    uint4* dbias_row = (POS == 1 && q_valid) ? reinterpret_cast<uint4*>(p.dbias + brow_off) : nullptr;

    {
      const int c = part;  // this thread's 32 keys of the tile
      float pv[32], gv[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) pv[e] = __uint_as_float(rs[e]);
      if (POS == 1) {
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          const uint4 bvec = bias_cur[g8];
          const uint32_t w[4] = {bvec.x, bvec.y, bvec.z, bvec.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pv[g8 * 8 + 2 * e] += __uint_as_float(w[e] << 16);
            pv[g8 * 8 + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
      const float delta_s = delta * p.inv_scale;
      // Two copies of the loop, chosen by a block-uniform test: tiles whose 128 keys are all kept (every full tile of
      // an unmasked input, and of a padding mask of ones) carry no per-score select and no metadata reads.
      auto score_loop = [&](auto masked_tag) {
      constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int k = c * 32 + e;
        bool keep = true;
        if (kMasked) {
          if (MASK == 0) {
            keep = k0 + k < S;  // last, partial key tile
          } else {
            const int meta = kmeta[k];
            keep = MASK == 1 ? (meta != 0) : (meta != 0 && meta == q_doc);
          }
        }
        float v = pv[e];
        int ic = 0, ip = 0;
        if (POS == 2 && keep && q_valid) {
          const int di = dbase - k;
          ic = lutc[di];
          ip = lutp[di];
          if (c2p_row) v += __bfloat162float(c2p_row[ic]);
          if (p.p2c) v += __bfloat162float(p.p2c[kbase + static_cast<long long>(k) * pos_row + ip]);
        }
        // rows past the sequence end and dead queries carry lse = +inf: their probabilities are exactly 0
        const float prob = keep ? ex2(fmaf(v, p.scale_log2, -lse)) : 0.f;
        const float g = prob * fmaf(__uint_as_float(rd[e]), p.inv_scale, -delta_s);
        pv[e] = prob;
        gv[e] = g;
        if (POS == 2 && keep && q_valid && g != 0.f) {
          if (dc2p_row) atomicAdd(dc2p_row + ic, g);
          if (p.d_p2c) atomicAdd(p.d_p2c + kbase + static_cast<long long>(k) * pos_row + ip, g);
        }
      }
      };
      if (MASK == 0 ? (k0 + kTile > S) : !tile_all_keep) {
        score_loop(std::true_type{});
      } else {
        score_loop(std::false_type{});
      }
      // the previous tile's gradient MMAs must retire before its P / dS tiles and dQ accumulator are reused
      if (i > 0) {
        got_g = __all_sync(0xffffffffu, mbar_wait(bar_g, (g - 1) & 1, abort_flag, p.status, kErrAccFullWait));
        tc_fence_after();
        if (tid == 0 && got_g && i + 2 < nqt) {  // slot (g+2)%3 held tile g-1
          const int nb = (g + 2) % 3;
          mbar_expect_tx(&bar_qd[nb], 2 * kTileBytes);
          tma_load_3d(sQ + nb * kTileBytes, &tm_q, &bar_qd[nb], h * kD, q0 + 2 * kTile, b);
          tma_load_3d(sdO + nb * kTileBytes, &tm_do, &bar_qd[nb], h * kD, q0 + 2 * kTile, b);
        }
        if (got_g) flush_dq(ib + i - 1);
      } else if (tid == 0 && nqt > 2) {  // the item's third tile: its slot is free (every earlier MMA has retired)
        const int nb = (g + 2) % 3;
        mbar_expect_tx(&bar_qd[nb], 2 * kTileBytes);
        tma_load_3d(sQ + nb * kTileBytes, &tm_q, &bar_qd[nb], h * kD, (ib + 2) * kTile, b);
        tma_load_3d(sdO + nb * kTileBytes, &tm_do, &bar_qd[nb], h * kD, (ib + 2) * kTile, b);
      }
      // rows of P and dS for these 32 keys: 4 chunks of 8 bf16 inside 64-key block (c >> 1)
      uint32_t dsw[16];
#pragma unroll
      for (int g4 = 0; g4 < 4; ++g4) {
        const int chunk = (c & 1) * 4 + g4;
        const uint32_t off = (c >> 1) * kTileBytes + swz128(row, chunk);
        uint4 u;
        u.x = pack_bf16(pv[g4 * 8 + 0], pv[g4 * 8 + 1]);
        u.y = pack_bf16(pv[g4 * 8 + 2], pv[g4 * 8 + 3]);
        u.z = pack_bf16(pv[g4 * 8 + 4], pv[g4 * 8 + 5]);
        u.w = pack_bf16(pv[g4 * 8 + 6], pv[g4 * 8 + 7]);
        *reinterpret_cast<uint4*>(sP + off) = u;
        u.x = pack_bf16(gv[g4 * 8 + 0], gv[g4 * 8 + 1]);
        u.y = pack_bf16(gv[g4 * 8 + 2], gv[g4 * 8 + 3]);
        u.z = pack_bf16(gv[g4 * 8 + 4], gv[g4 * 8 + 5]);
        u.w = pack_bf16(gv[g4 * 8 + 6], gv[g4 * 8 + 7]);
        *reinterpret_cast<uint4*>(sdS + off) = u;
        dsw[g4 * 4] = u.x; dsw[g4 * 4 + 1] = u.y; dsw[g4 * 4 + 2] = u.z; dsw[g4 * 4 + 3] = u.w;
      }
      if (dbias_row) {  // 64 contiguous bytes of this query's row
        st_global_32B(dbias_row + c * 4, dsw);
        st_global_32B(dbias_row + c * 4 + 2, dsw + 8);
      }
    }
    fence_proxy_async();
    tc_fence_before();
    if (!__syncthreads_and(got_g)) { ok = false; break; }
    if (tid == 0 || tid == 32 || tid == 64) {  // one product each
      tc_fence_after();
      const uint32_t sp = smem_u32(sP), sds = smem_u32(sdS), sq = smem_u32(sQ + buf * kTileBytes),
                     sdo = smem_u32(sdO + buf * kTileBytes), sk = smem_u32(sK);
      if (tid == 0) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)  // dV[k,d] += sum_q P[q,k] dO[q,d]
          umma_bf16(t_dv, make_smem_desc(sp + ks * 2048, kTileBytes, 1024), make_smem_desc(sdo + ks * 2048, 8192, 1024),
                    idesc_t, (i > 0) || (ks > 0));
      } else if (tid == 32) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)  // dK[k,d] += sum_q dS[q,k] Q[q,d]
          umma_bf16(t_dk, make_smem_desc(sds + ks * 2048, kTileBytes, 1024), make_smem_desc(sq + ks * 2048, 8192, 1024),
                    idesc_t, (i > 0) || (ks > 0));
      } else {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)  // dQ[q,d] = sum_k dS[q,k] K[k,d]
          umma_bf16(t_dq, make_smem_desc(sds + (ks >> 2) * kTileBytes + (ks & 3) * 32, 16, 1024),
                    make_smem_desc(sk + ks * 2048, 8192, 1024), idesc_q, ks > 0);
      }
      umma_commit(bar_g);
    }
  }

  if (!ok) break;
  const bool fin = mbar_wait(bar_g, (g0 + nqt - 1) & 1, abort_flag, p.status, kErrAccFullWait);
  tc_fence_after();
  g0 += nqt;
  ++n_done;
  loads_issued = false;
  if (MASK != 2) {
    // every MMA of this item has retired: K, V and the (Q, dO) ring are free, and the next item's operands can
    // travel while this item's gradients are read out of the tensor memory
    const int wn = w + gridDim.x;
    if (wn < n_items) {
      loads_issued = true;
      if (tid == 0 && fin)
        issue_item_loads(wn / (nkt_all * p.heads), (wn / nkt_all) % p.heads, (wn % nkt_all) * kTile, 0, nkt_all, g0);
    }
  }
  if (fin) {
    flush_dq(ib + nqt - 1);
    const int kk = k0 + row;
    const long long tk = static_cast<long long>(b) * S + kk;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = (which == 0 ? p.dv + tk * p.ldv : p.dk + tk * p.ldk) + h * kD + part * 16;
      uint32_t r[16];
      tmem_ld_32x32b_x16((which == 0 ? t_dv : t_dk) + lane_addr + part * 16, r);
      tmem_ld_wait();
      if (kk < S) {
        uint32_t pk[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) pk[e] = pack_bf16(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
        store_bf16x16(dst, pk);
      }
    }
  }
  // the next item's first gradient MMAs (and its key metadata) may only follow once every thread is done here;
  // a wait that ran out ends the CTA for all threads together
  tc_fence_before();
  if (!__syncthreads_and(fin)) ok = false;
  tc_fence_after();
  }  // work items

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}



// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d] (fp32), the row term of the softmax gradient.
// Eight lanes share one (token, head): 16 bytes of dO and of O each.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, long long ld_do, const __nv_bfloat16* __restrict__ out,
                  long long ldo, float* __restrict__ delta, float* __restrict__ zero_f32, int B, int S, int heads) {
  pdl_launch_dependents();
  pdl_wait();
  const long long gid = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  // the dQ accumulator of the backward kernel that follows has exactly 8 floats per thread of this grid
  // ([tokens, heads * 64]): clearing it here saves a fill launch per layer
  if (zero_f32 && gid < static_cast<long long>(B) * S * heads * 8) {
    float4* z = reinterpret_cast<float4*>(zero_f32 + gid * 8);
    z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const long long pair = gid >> 3;  // (token, head)
  const int sub = static_cast<int>(gid & 7);
  const long long total = static_cast<long long>(B) * S * heads;
  float acc = 0.f;
  long long token = 0;
  int h = 0;
  if (pair < total) {
    token = pair / heads;
    h = static_cast<int>(pair % heads);
    const uint4 a = *reinterpret_cast<const uint4*>(dout + token * ld_do + h * kD + sub * 8);
    const uint4 o = *reinterpret_cast<const uint4*>(out + token * ldo + h * kD + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      acc += __uint_as_float(aw[e] << 16) * __uint_as_float(ow[e] << 16) +
             __uint_as_float(aw[e] & 0xffff0000u) * __uint_as_float(ow[e] & 0xffff0000u);
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (pair < total && sub == 0) {
    const long long bb = token / S, ss = token % S;
    delta[(bb * heads + h) * S + ss] = acc;
  }
}

// tiles[b, t] = (smallest, largest) non-zero document id among tokens [128 t, 128 t + 128) of row b;
// (INT_MAX, -1) when the tile holds padding only. One block of 128 threads per tile.
__global__ void __launch_bounds__(kTile)
attn_doc_tiles_kernel(const int* __restrict__ doc_ids, int* __restrict__ tiles, int S) {
  __shared__ int s_lo[4], s_hi[4];
  const int t = blockIdx.x, b = blockIdx.y;
  const int pos = t * kTile + threadIdx.x;
  const int id = pos < S ? doc_ids[static_cast<long long>(b) * S + pos] : 0;
  int lo = id != 0 ? id : 2147483647, hi = id != 0 ? id : -1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0) {
    s_lo[threadIdx.x >> 5] = lo;
    s_hi[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int* dst = tiles + (static_cast<long long>(b) * gridDim.x + t) * 2;
    dst[0] = min(min(s_lo[0], s_lo[1]), min(s_lo[2], s_lo[3]));
    dst[1] = max(max(s_hi[0], s_hi[1]), max(s_hi[2], s_hi[3]));
  }
}

int make_head_map(CUtensorMap* m, const void* ptr, const AttnArgs* a, long long ld, int box_rows = kTile) {
  return db200_make_tmap_bf16(m, ptr, static_cast<long long>(a->heads) * kD, a->S, a->B, ld,
                              static_cast<long long>(a->S) * ld, box_rows);
}

// Keys per tile of the forward kernel: 64 (two 256-thread CTAs per SM) or 128 (one 512-thread CTA).
int g_fwd_key_tile = 64;
// With 64-key tiles and neither document ids nor in-kernel table gathers: the warp-specialised kernel (a dedicated
// TMA/MMA warp, mbarriers instead of block-wide barriers).
int g_fwd_specialised = 1;
// backward: 1 = one CTA per SM walks the (batch, head, key tile) items; 0 = one CTA per item; n > 1 = at most n CTAs
// (tests: several items per CTA on small inputs)
int g_bwd_persistent = 1;

int sm_count() {  // per device: a process may drive more than one GPU
  static int count[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev >= 0 && dev < 16) ? dev : 0;
  if (count[dev] == 0) {
    cudaDeviceGetAttribute(&count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (count[dev] <= 0) count[dev] = 148;
  }
  return count[dev];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int db200_attn_fwd(const AttnArgs* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a->B <= 0 || a->S <= 0 || a->heads <= 0) return 0;
  const bool pos = a->span2 > 0;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out) || (a->ldq % 8) || (a->ldk % 8) ||
      (a->ldv % 8) || (a->ldo % 8))
    return -10;
  if (pos && (a->S > 4096 || a->span2 > 65535 || !a->lut_c2p || !a->lut_p2c)) return -12;
  CUtensorMap tq, tk, tv;
  int rc;
  const int kt = g_fwd_key_tile == 128 ? 128 : 64;
  if ((rc = make_head_map(&tq, a->q, a, a->ldq))) return rc;
  if ((rc = make_head_map(&tk, a->k, a, a->ldk, kt))) return rc;
  if ((rc = make_head_map(&tv, a->v, a, a->ldv, kt))) return rc;
  AttnDev d{};
  d.B = a->B; d.S = a->S; d.heads = a->heads; d.span2 = a->span2;
  d.scale_log2 = 1.4426950408889634f / a->scale;
  d.inv_scale = 1.f / a->scale;
  d.c2p = static_cast<const __nv_bfloat16*>(a->c2p);
  d.p2c = static_cast<const __nv_bfloat16*>(a->p2c);
  d.lut_c2p = static_cast<const unsigned short*>(a->lut_c2p);
  d.lut_p2c = static_cast<const unsigned short*>(a->lut_p2c);
  d.key_keep = static_cast<const unsigned char*>(a->key_keep);
  d.doc_ids = static_cast<const int*>(a->doc_ids);
  d.doc_tiles = d.doc_ids ? static_cast<const int*>(a->doc_tiles) : nullptr;
  d.bias = static_cast<const __nv_bfloat16*>(a->bias);
  d.ldb = a->ldb;
  if (d.bias && ((a->ldb % 128) || !aligned16(a->bias))) return -10;
  d.out = static_cast<__nv_bfloat16*>(a->out);
  d.ldo = a->ldo;
  d.lse = a->lse;
  d.status = db200_status_ptr();
  const int pos_mode = d.bias ? 1 : (pos ? 2 : 0);
  const int mask_mode = d.doc_ids ? 2 : (d.key_keep ? 1 : 0);
  if (kt == 64 && g_fwd_specialised && mask_mode != 2 && pos_mode != 2) {
    using WsKernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, AttnDev);
    static const WsKernel ws[2][2] = {{attn_fwd_ws_kernel<0, 0>, attn_fwd_ws_kernel<0, 1>},
                                      {attn_fwd_ws_kernel<1, 0>, attn_fwd_ws_kernel<1, 1>}};
    static bool ws_configured[16][2][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev >= 0 && dev < 16) ? dev : 0;
    const WsKernel kern = ws[mask_mode][pos_mode];
    if (!ws_configured[dev][mask_mode][pos_mode]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdWsSmem::kTotal) != cudaSuccess) return -3;
      ws_configured[dev][mask_mode][pos_mode] = true;
    }
    dim3 grid((a->S + kTile - 1) / kTile, a->heads, a->B);
    return launch_pdl(kern, grid, dim3(kFwdWsThreads), FwdWsSmem::kTotal, stream, tq, tk, tv, d) == cudaSuccess ? 0 : -4;
  }
  const int wide = kt == 128 ? 1 : 0;
  const int smem = wide ? FwdSmem<128>::total(a->S, pos_mode == 2) : FwdSmem<64>::total(a->S, pos_mode == 2);
  using FwdKernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, AttnDev);
  static const FwdKernel kernels[2][3][3] = {
      {{attn_fwd_kernel<0, 0, 64>, attn_fwd_kernel<0, 1, 64>, attn_fwd_kernel<0, 2, 64>},
       {attn_fwd_kernel<1, 0, 64>, attn_fwd_kernel<1, 1, 64>, attn_fwd_kernel<1, 2, 64>},
       {attn_fwd_kernel<2, 0, 64>, attn_fwd_kernel<2, 1, 64>, attn_fwd_kernel<2, 2, 64>}},
      {{attn_fwd_kernel<0, 0, 128>, attn_fwd_kernel<0, 1, 128>, attn_fwd_kernel<0, 2, 128>},
       {attn_fwd_kernel<1, 0, 128>, attn_fwd_kernel<1, 1, 128>, attn_fwd_kernel<1, 2, 128>},
       {attn_fwd_kernel<2, 0, 128>, attn_fwd_kernel<2, 1, 128>, attn_fwd_kernel<2, 2, 128>}}};
  static int configured[16][2][3][3] = {};  // per device: the opt-in to large shared memory is a per-device attribute
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev >= 0 && dev < 16) ? dev : 0;
  const FwdKernel kern = kernels[wide][mask_mode][pos_mode];
  if (configured[dev][wide][mask_mode][pos_mode] < smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
    configured[dev][wide][mask_mode][pos_mode] = smem;
  }
  dim3 grid((a->S + kTile - 1) / kTile, a->heads, a->B);
  return launch_pdl(kern, grid, dim3(kt * 4), smem, stream, tq, tk, tv, d) == cudaSuccess ? 0 : -4;
}

extern "C" int db200_attn_bwd(const AttnArgs* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a->B <= 0 || a->S <= 0 || a->heads <= 0) return 0;
  const bool pos = a->span2 > 0;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->dout) || !aligned16(a->dk) ||
      !aligned16(a->dv) || !aligned16(a->dq_acc) || (a->ldq % 8) || (a->ldk % 8) || (a->ldv % 8) || (a->ld_do % 8) ||
      (a->ld_dk % 8) || (a->ld_dv % 8))
    return -10;
  if (pos && (a->S > 4096 || a->span2 > 65535 || !a->lut_c2p || !a->lut_p2c)) return -12;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_head_map(&tq, a->q, a, a->ldq))) return rc;
  if ((rc = make_head_map(&tk, a->k, a, a->ldk))) return rc;
  if ((rc = make_head_map(&tv, a->v, a, a->ldv))) return rc;
  if ((rc = make_head_map(&tdo, a->dout, a, a->ld_do))) return rc;
  AttnBwdDev d{};
  d.B = a->B; d.S = a->S; d.heads = a->heads; d.span2 = a->span2;
  d.scale_log2 = 1.4426950408889634f / a->scale;
  d.inv_scale = 1.f / a->scale;
  d.c2p = static_cast<const __nv_bfloat16*>(a->c2p);
  d.p2c = static_cast<const __nv_bfloat16*>(a->p2c);
  d.lut_c2p = static_cast<const unsigned short*>(a->lut_c2p);
  d.lut_p2c = static_cast<const unsigned short*>(a->lut_p2c);
  d.key_keep = static_cast<const unsigned char*>(a->key_keep);
  d.doc_ids = static_cast<const int*>(a->doc_ids);
  d.doc_tiles = d.doc_ids ? static_cast<const int*>(a->doc_tiles) : nullptr;
  d.bias = static_cast<const __nv_bfloat16*>(a->bias);
  d.dbias = static_cast<__nv_bfloat16*>(a->dbias);
  d.ldb = a->ldb;
  if (d.bias && ((a->ldb % 128) || !aligned16(a->bias) || !d.dbias || (reinterpret_cast<uintptr_t>(a->dbias) & 31))) return -10;
  d.lse = a->lse;
  d.delta = a->delta;
  d.dq_acc = a->dq_acc;
  d.dk = static_cast<__nv_bfloat16*>(a->dk);
  d.dv = static_cast<__nv_bfloat16*>(a->dv);
  d.ldk = a->ld_dk; d.ldv = a->ld_dv;
  d.d_c2p = a->d_c2p;
  d.d_p2c = a->d_p2c;
  d.status = db200_status_ptr();
  const int pos_mode = d.bias ? 1 : (pos ? 2 : 0);
  const int mask_mode = d.doc_ids ? 2 : (d.key_keep ? 1 : 0);
  const int smem = BwdSmem::total(a->S, pos_mode == 2);
  using BwdKernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, AttnBwdDev);
  static const BwdKernel kernels[3][3] = {
      {attn_bwd_kernel<0, 0>, attn_bwd_kernel<0, 1>, attn_bwd_kernel<0, 2>},
      {attn_bwd_kernel<1, 0>, attn_bwd_kernel<1, 1>, attn_bwd_kernel<1, 2>},
      {attn_bwd_kernel<2, 0>, attn_bwd_kernel<2, 1>, attn_bwd_kernel<2, 2>}};
  static int configured[16][3][3] = {};  // per device, as in the forward launcher
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev >= 0 && dev < 16) ? dev : 0;
  const BwdKernel kern = kernels[mask_mode][pos_mode];
  if (configured[dev][mask_mode][pos_mode] < smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
    configured[dev][mask_mode][pos_mode] = smem;
  }
  // one CTA per SM walks the work items; items of different lengths (document ids) get a CTA each, which the
  // hardware hands out as SMs become free
  const long long items = static_cast<long long>((a->S + kTile - 1) / kTile) * a->heads * a->B;
  if (items > 0x7fffffffLL) return -12;
  const bool persistent = g_bwd_persistent && mask_mode != 2;
  const int max_ctas = g_bwd_persistent > 1 && g_bwd_persistent < sm_count() ? g_bwd_persistent : sm_count();
  dim3 grid(static_cast<unsigned>(persistent && items > max_ctas ? max_ctas : items));
  if (launch_pdl(kern, grid, dim3(kBwdThreads), smem, stream, tq, tk, tv, tdo, d) != cudaSuccess) return -4;
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_attn_delta(const void* dout, long long ld_do, const void* out, long long ldo, float* delta,
                                float* zero_f32, int B, int S, int heads, void* stream) {
  if (B <= 0 || S <= 0 || heads <= 0) return 0;
  if (!aligned16(dout) || !aligned16(out) || (ld_do % 8) || (ldo % 8) || !aligned16(zero_f32)) return -10;
  const long long threads = static_cast<long long>(B) * S * heads * 8;
  return launch_pdl(attn_delta_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0,
                    reinterpret_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(dout), ld_do,
                    static_cast<const __nv_bfloat16*>(out), ldo, delta, zero_f32, B, S, heads) == cudaSuccess ? 0 : -4;
}

extern "C" int db200_attn_doc_tiles(const void* doc_ids, void* tiles, int B, int S, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if (!doc_ids || !tiles) return -10;
  dim3 grid((S + kTile - 1) / kTile, B);
  attn_doc_tiles_kernel<<<grid, kTile, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const int*>(doc_ids),
                                                                                   static_cast<int*>(tiles), S);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Backward kernel: 1 = one CTA per SM loops over the work items (default), 0 = one CTA per item, n > 1 = at most n
// CTAs; returns the previous value (A/B comparisons, tests).
extern "C" int db200_attn_set_bwd_persistent(int on) {
  const int old = g_bwd_persistent;
  g_bwd_persistent = on < 0 ? 0 : on;
  return old;
}

// 64 or 128 keys per tile in the forward kernel (anything else selects 64); returns the previous value.
// 65 selects 64-key tiles on the kernel without warp specialisation (A/B comparisons, tests).
extern "C" int db200_attn_set_fwd_key_tile(int keys) {
  const int old = g_fwd_key_tile == 128 ? 128 : (g_fwd_specialised ? 64 : 65);
  g_fwd_key_tile = keys == 128 ? 128 : 64;
  g_fwd_specialised = keys == 65 ? 0 : 1;
  return old;
}
