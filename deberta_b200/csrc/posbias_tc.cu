// Position terms of disentangled attention on the tensor cores, one 128 x 128 (query, key) tile at a time.
//
//   bias[b,h,q,k] = Q[q]·PosK[lut_c2p(q-k)] + K[k]·PosQ[lut_p2c(q-k)]                         (forward)
//
//   G = d loss / d bias:   dQ[q]    += sum_k G[q,k] PosK[lut_c2p(q-k)]      dPosK[w] += sum_{lut_c2p(q-k)=w} G[q,k] Q[q]
//                          dK[k]    += sum_q G[q,k] PosQ[lut_p2c(q-k)]      dPosQ[w] += sum_{lut_p2c(q-k)=w} G[q,k] K[k]
//
// The bucket index is monotone in q-k, so one tile only touches a window of at most 256 consecutive rows of the
// projected position tables. Forward: the two window products Q_tile·PosK_winᵀ and K_tile·PosQ_winᵀ (128 x 256
// each) run as tcgen05 MMAs into TMEM, are drained as bf16 into shared memory, and every (q, k) entry picks its
// two values with the bucket lookup table. Backward: the tile of G is folded onto the bucket axis in shared
// memory (row sums over the keys, or the queries, that share a bucket), and the folded 128 x 256 tile is the
// operand of two MMAs per side: one for the gradient of the content rows (dQ or dK), one for the gradient of the
// position table, which stays in TMEM for all tiles of a (batch, head) and is added to global memory once.
// Neither the [tokens, heads, 2·span] score tables nor their gradients exist in global memory.
//
// Shared with attention.cu: token-major bf16 operands [B*S, ld] (a head is a 64-column slice), 128B-swizzled TMA
// tiles, bounded waits that report through the status word.
#include "tc05.cuh"
#include "kernels.h"

namespace {

using namespace tc05;

constexpr int kTile = 128;
constexpr int kD = 64;
constexpr int kTileBytes = kTile * kD * 2;    // 16 KB: 128 rows of one head
constexpr int kWin = 256;                     // rows of a position-table window
constexpr int kWinBytes = kWin * kD * 2;      // 32 KB
constexpr int kMaxDiag = 64;                  // tile diagonals i - j the window tables can describe (S <= 4096)
// One CTA fills an SM (shared memory), so the warps of that one CTA have to hide the latencies
// of TMEM loads, shared-memory gathers and the barriers between phases. Warp w owns TMEM lane quadrant (w & 3)
// and "part" (w >> 2) of whatever a row is split into.
#ifndef DB200_POS_PARTS
#define DB200_POS_PARTS 4
#endif
constexpr int kParts = DB200_POS_PARTS;       // threads per tile row (4 or 8)
constexpr int kThreads = 128 * kParts;
constexpr int kPer = kTile / kParts;          // (q, k) entries of a row one thread handles
constexpr int kDrain = kWin / kParts;         // window columns one thread drains
constexpr int kAccCols = kD / kParts;         // accumulator columns one thread reads back

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
static_assert(kParts == 4 || kParts == 8, "a tile row is shared by 4 or 8 threads");

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// --------------------------------------------------------------------------------------------
// forward
// --------------------------------------------------------------------------------------------
struct PosFwdDev {
  int B, S, heads, nt;
  const unsigned short* lut_c2p;  // [2S-1], index q-k+S-1
  const unsigned short* lut_p2c;
  __nv_bfloat16* bias;            // [B, heads, S, ldb]
  long long ldb;
  unsigned char win_c[kMaxDiag];  // first 128-row block of the PosK window of tile diagonal i-j+nt-1
  unsigned char win_p[kMaxDiag];  // the same for PosQ
  int* status;
};

// Staging rows are 256 bf16 + 2 of padding = 129 words: at the gather the 32 lanes of a warp read 32 different rows
// at (nearly) the same column, and an odd word stride puts those on different banks. The drain therefore stores
// 32-bit words (rows are only 4-byte aligned).
constexpr int kStageLd = kWin + 2;
constexpr int kStageBytes = kTile * kStageLd * 2;

struct FwdSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;
  static constexpr int kPK = kK + kTileBytes;
  static constexpr int kPQ = kPK + kWinBytes;
  static constexpr int kStage = kPQ + kWinBytes;
  static constexpr int kBar = kStage + kStageBytes;
  static constexpr int kLut = kBar + 128;
  static int total(int nt) { return kLut + 2 * (2 * nt * kTile) * 2 + 1024; }
};

// grid (q-tiles, heads, B), 128·kParts threads: warp w owns the TMEM lanes of quadrant (w & 3) and share (w >> 2) of the
// window columns; at the gather a thread owns one query row and kPer keys of the tile.
template <bool HAS_C, bool HAS_P>
__global__ void __launch_bounds__(kThreads, 1)
posbias_tc_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_pk, const __grid_constant__ CUtensorMap tm_pq,
                      const PosFwdDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + FwdSmem::kQ;
  uint8_t* sK = smem + FwdSmem::kK;
  uint8_t* sPK = smem + FwdSmem::kPK;
  uint8_t* sPQ = smem + FwdSmem::kPQ;
  __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + FwdSmem::kStage);
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + FwdSmem::kBar);
  uint64_t* bar_ld = bar_q + 1;
  uint64_t* bar_mma = bar_q + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // lookup tables over x = q - k + nt*128 - 1 for every (q, k) of the padded tile grid (edge values repeated)
  const int nt = p.nt, S = p.S;
  const int lut_len = 2 * nt * kTile;
  unsigned short* lutc = reinterpret_cast<unsigned short*>(smem + FwdSmem::kLut);
  unsigned short* lutp = lutc + lut_len;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int quad = warp & 3, part = warp >> 2;
  const int row = quad * 32 + lane;
  const int ti = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = ti * kTile;
  pdl_launch_dependents();

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_ld, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  for (int x = tid; x < lut_len - 1; x += kThreads) {
    const int d = min(max(x - (nt * kTile - 1) + (S - 1), 0), 2 * S - 2);
    if (HAS_C) lutc[x] = p.lut_c2p[d];  // (the bucket maps are written once, when the model is built)
    if (HAS_P) lutp[x] = p.lut_p2c[d];
  }
  pdl_wait();  // set-up done; Q, K, the position tables and the bias are touched only from here on
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_c = tmem_base, t_p = tmem_base + kWin;
  const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
  constexpr uint32_t idesc = make_idesc_bf16(128, kWin, false, false);
  constexpr uint32_t kLoadBytes = (HAS_P ? kTileBytes : 0) + (HAS_C ? kWinBytes : 0) + (HAS_P ? kWinBytes : 0);

  auto issue_loads = [&](int tj) {  // operands of tile pair (ti, tj): K tile and the two table windows
    const int diag = ti - tj + nt - 1;
    mbar_expect_tx(bar_ld, kLoadBytes);
    if (HAS_P) tma_load_3d(sK, &tm_k, bar_ld, h * kD, tj * kTile, b);
    if (HAS_C) {
      tma_load_3d(sPK, &tm_pk, bar_ld, h * kD, p.win_c[diag] * kTile, 0);
      tma_load_3d(sPK + kTileBytes, &tm_pk, bar_ld, h * kD, (p.win_c[diag] + 1) * kTile, 0);
    }
    if (HAS_P) {
      tma_load_3d(sPQ, &tm_pq, bar_ld, h * kD, p.win_p[diag] * kTile, 0);
      tma_load_3d(sPQ + kTileBytes, &tm_pq, bar_ld, h * kD, (p.win_p[diag] + 1) * kTile, 0);
    }
  };
  auto issue_mmas = [&]() {
    if (HAS_C) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(t_c, make_smem_desc(smem_u32(sQ) + ks * 32, 16, 1024), make_smem_desc(smem_u32(sPK) + ks * 32, 16, 1024),
                  idesc, ks > 0);
    }
    if (HAS_P) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(t_p, make_smem_desc(smem_u32(sK) + ks * 32, 16, 1024), make_smem_desc(smem_u32(sPQ) + ks * 32, 16, 1024),
                  idesc, ks > 0);
    }
  };

  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_pk);
    tma_prefetch_desc(&tm_pq);
    mbar_expect_tx(bar_q, kTileBytes);
    tma_load_3d(sQ, &tm_q, bar_q, h * kD, q0, b);
    issue_loads(0);
    if (mbar_wait(bar_q, 0, abort_flag, p.status, kErrFullWait) &&
        mbar_wait(bar_ld, 0, abort_flag, p.status, kErrFullWait)) {
      tc_fence_after();
      issue_mmas();
    }
    umma_commit(bar_mma);
  }

  const int qg = q0 + row;
  const uint32_t stage_row = static_cast<uint32_t>(row) * kStageLd;

  auto drain = [&](uint32_t t_src) {  // this thread's columns of the window product, as bf16, into its staging row
#pragma unroll
    for (int c = 0; c < kDrain / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_src + lane_addr + part * kDrain + c * 32, r);
      tmem_ld_wait();
      uint32_t* dst = reinterpret_cast<uint32_t*>(stage + stage_row + part * kDrain + c * 32);
#pragma unroll
      for (int g = 0; g < 16; ++g) dst[g] = pack_bf16(__uint_as_float(r[2 * g]), __uint_as_float(r[2 * g + 1]));
    }
  };

  for (int tj = 0; tj < nt; ++tj) {
    // one thread polls the barrier (a spinning CTA would burn the issue slots the working warps need); the block
    // barrier hands its answer to everybody and also ends the previous tile's reads of the staging buffer
    const bool got = tid != 0 || mbar_wait(bar_mma, tj & 1, abort_flag, p.status, kErrAccFullWait);
    if (!__syncthreads_and(got)) break;
    tc_fence_after();
    const bool more = tj + 1 < nt;
    if (tid == 0 && more) issue_loads(tj + 1);  // the MMAs that read these buffers have retired
    const int diag = ti - tj + nt - 1;
    const int k0 = tj * kTile;
    const int xbase = qg - (k0 + part * kPer) + nt * kTile - 1;  // lookup index of this thread's first key
    float acc[kPer];
#pragma unroll
    for (int e = 0; e < kPer; ++e) acc[e] = 0.f;

    if (HAS_C) {
      drain(t_c);
      __syncthreads();
      const unsigned short* l = lutc + xbase;
      const __nv_bfloat16* src = stage + stage_row - p.win_c[diag] * kTile;
#pragma unroll
      for (int e = 0; e < kPer; ++e) acc[e] = __bfloat162float(src[l[-e]]);
    }
    if (HAS_P) {
      if (HAS_C) __syncthreads();  // the gather above is done with the staging buffer
      drain(t_p);
    }
    tc_fence_before();
    __syncthreads();  // both accumulators are drained
    if (tid == 0 && more) {
      if (mbar_wait(bar_ld, (tj + 1) & 1, abort_flag, p.status, kErrFullWait)) {
        tc_fence_after();
        issue_mmas();
      }
      umma_commit(bar_mma);
    }
    if (HAS_P) {
      const unsigned short* l = lutp + xbase;
      const __nv_bfloat16* src = stage + static_cast<uint32_t>(part * kPer) * kStageLd - p.win_p[diag] * kTile;
#pragma unroll
      for (int e = 0; e < kPer; ++e) acc[e] += __bfloat162float(src[e * kStageLd + l[-e]]);
    }
    if (qg < S) {
      uint32_t w[kPer / 2];
#pragma unroll
      for (int e = 0; e < kPer / 2; ++e) w[e] = pack_bf16(acc[2 * e], acc[2 * e + 1]);
      __nv_bfloat16* dst = p.bias + ((static_cast<long long>(b) * p.heads + h) * S + qg) * p.ldb + k0 + part * kPer;
#pragma unroll
      for (int v = 0; v < kPer / 16; ++v) st_global_32B(dst + v * 16, w + v * 8);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// First 128-row block of the window of table rows a tile diagonal touches; -1 when the rows do not fit 256.
// `lut` is the host copy of the lookup table over q-k+S-1; edge values stand in for the padded part of the grid.
int window_block(const unsigned short* lut, int S, int nt, int diag) {
  const int centre = (diag - (nt - 1)) * kTile;  // q0 - k0
  int lo = 1 << 30, hi = -1;
  for (int rel = centre - (kTile - 1); rel <= centre + (kTile - 1); ++rel) {
    const int d = rel + S - 1 < 0 ? 0 : (rel + S - 1 > 2 * S - 2 ? 2 * S - 2 : rel + S - 1);
    lo = lut[d] < lo ? lut[d] : lo;
    hi = lut[d] > hi ? lut[d] : hi;
  }
  const int blk = lo / kTile;
  return (hi < blk * kTile + kWin && blk < 255) ? blk : -1;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int head_map(CUtensorMap* m, const void* ptr, int heads, int S, int B, long long ld) {
  return db200_make_tmap_bf16(m, ptr, static_cast<long long>(heads) * kD, S, B, ld, static_cast<long long>(S) * ld, kTile);
}

}  // namespace

extern "C" int db200_posbias_tc_fwd(const PosBiasArgs* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a->B <= 0 || a->S <= 0 || a->heads <= 0) return 0;
  const bool has_c = a->pos_k != nullptr, has_p = a->pos_q != nullptr;
  if (!has_c && !has_p) return -10;
  const int nt = (a->S + kTile - 1) / kTile;
  if (2 * nt - 1 > kMaxDiag || a->span2 <= 0 || a->span2 > 32767) return -12;
  if (!aligned16(a->q) || !aligned16(a->k) || (a->ldq % 8) || (a->ldk % 8) || (a->ld_pos % 8) || !a->bias ||
      (reinterpret_cast<uintptr_t>(a->bias) & 31) || (a->ldb % kTile) || a->ldb < nt * kTile ||
      (has_c && (!aligned16(a->pos_k) || !a->lut_c2p_host || !a->lut_c2p)) ||
      (has_p && (!aligned16(a->pos_q) || !a->lut_p2c_host || !a->lut_p2c)))
    return -10;
  PosFwdDev d{};
  d.B = a->B; d.S = a->S; d.heads = a->heads; d.nt = nt;
  d.lut_c2p = static_cast<const unsigned short*>(a->lut_c2p);
  d.lut_p2c = static_cast<const unsigned short*>(a->lut_p2c);
  d.bias = static_cast<__nv_bfloat16*>(a->bias);
  d.ldb = a->ldb;
  d.status = db200_status_ptr();
  for (int diag = 0; diag < 2 * nt - 1; ++diag) {
    const int wc = has_c ? window_block(static_cast<const unsigned short*>(a->lut_c2p_host), a->S, nt, diag) : 0;
    const int wp = has_p ? window_block(static_cast<const unsigned short*>(a->lut_p2c_host), a->S, nt, diag) : 0;
    if (wc < 0 || wp < 0) return -13;  // a tile needs more than 256 table rows: the caller takes another path
    d.win_c[diag] = static_cast<unsigned char>(wc);
    d.win_p[diag] = static_cast<unsigned char>(wp);
  }
  CUtensorMap tq, tk, tpk, tpq;
  int rc;
  if ((rc = head_map(&tq, has_c ? a->q : a->k, a->heads, a->S, a->B, has_c ? a->ldq : a->ldk))) return rc;
  if ((rc = head_map(&tk, has_p ? a->k : a->q, a->heads, a->S, a->B, has_p ? a->ldk : a->ldq))) return rc;
  const void* pk = has_c ? a->pos_k : a->pos_q;
  const void* pq = has_p ? a->pos_q : a->pos_k;
  if ((rc = head_map(&tpk, pk, a->heads, a->span2, 1, a->ld_pos))) return rc;
  if ((rc = head_map(&tpq, pq, a->heads, a->span2, 1, a->ld_pos))) return rc;
  const int smem = FwdSmem::total(nt);
  using Kernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, PosFwdDev);
  const Kernel kern = has_c ? (has_p ? posbias_tc_fwd_kernel<true, true> : posbias_tc_fwd_kernel<true, false>)
                            : posbias_tc_fwd_kernel<false, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
  dim3 grid(nt, a->heads, a->B);
  return launch_pdl(kern, grid, dim3(kThreads), smem, stream, tq, tk, tpk, tpq, d) == cudaSuccess ? 0 : -4;
}


// --------------------------------------------------------------------------------------------
// backward
// --------------------------------------------------------------------------------------------
namespace {

constexpr int kMaxBlocks = 4;  // 128-row blocks of a position table whose gradient fits TMEM beside the row gradient

struct PosBwdDev {
  int B, S, heads, nt, span2, nblk;
  const unsigned short* lut[2];  // c2p (rows are queries), p2c (rows are keys)
  float* dq_acc;                 // fp32 [B*S, heads*64]
  __nv_bfloat16* dk;             // bf16 [B*S, ld_dk]
  long long ld_dk;
  float* d_pos[2];               // fp32 [span2, heads*64]
  unsigned char win[2][kMaxDiag];
  unsigned touched[2];           // bit blk: some tile of this side writes block blk of the table gradient
  int has[2];
  int* status;
};

struct BwdSmem {
  static constexpr int kTab = 0;                                  // the head's position table, 4 blocks of 128 rows
  static constexpr int kRow = kTab + kMaxBlocks * kTileBytes;     // Q tile (c2p side) or K tile (p2c side)
  static constexpr int kG = kRow + kTileBytes;                    // 2 buffers of 128 x 128 bf16 (two 64-key halves)
  static constexpr int kF = kG + 4 * kTileBytes;                  // folded tile: 128 rows x 256 buckets (four chunks)
  static constexpr int kBar = kF + 4 * kTileBytes;
  static constexpr int kLut = kBar + 128;
  static int total(int nt) { return kLut + (2 * nt * kTile) * 2 + 1024; }
};

// One CTA per (side, head, batch row). SIDE 0: rows are queries, the outer loop runs over query tiles and the
// inner one over key tiles; SIDE 1: rows are keys, outer loop over key tiles. Thread = (row, kPer entries of the
// other axis) during the fold, (TMEM lane, kAccCols columns) when accumulators are read.
template <int SIDE>
__device__ __forceinline__ void posbias_bwd_body(const CUtensorMap& tm_row, const CUtensorMap& tm_tab,
                                                  const CUtensorMap& tm_g, const PosBwdDev& p, uint8_t* smem) {
  uint8_t* sTab = smem + BwdSmem::kTab;
  uint8_t* sRow = smem + BwdSmem::kRow;
  uint8_t* sG = smem + BwdSmem::kG;
  uint8_t* sF = smem + BwdSmem::kF;
  uint64_t* bar_tab = reinterpret_cast<uint64_t*>(smem + BwdSmem::kBar);
  uint64_t* bar_row = bar_tab + 1;
  uint64_t* bar_g = bar_tab + 2;  // [2]
  uint64_t* bar_f = bar_tab + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tab + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned short* lut = reinterpret_cast<unsigned short*>(smem + BwdSmem::kLut);

  const int nt = p.nt, S = p.S;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int quad = warp & 3, part = warp >> 2;
  const int row = quad * 32 + lane;
  const int h = blockIdx.y, b = blockIdx.z;
  const int npairs = nt * nt;
  const long long H = static_cast<long long>(p.heads) * kD;

  if (tid == 0) {
    mbar_init(bar_tab, 1);
    mbar_init(bar_row, 1);
    mbar_init(&bar_g[0], 1);
    mbar_init(&bar_g[1], 1);
    mbar_init(bar_f, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  const int lut_len = 2 * nt * kTile;
  for (int x = tid; x < lut_len - 1; x += kThreads)
    lut[x] = p.lut[SIDE][min(max(x - (nt * kTile - 1) + (S - 1), 0), 2 * S - 2)];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_row = tmem_base;        // 64 columns: gradient of the current row tile (dQ or dK part)
  const uint32_t t_pos = tmem_base + 64;   // 64 columns per 128-row block of the table gradient
  const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
  constexpr uint32_t idesc_row = make_idesc_bf16(128, 64, false, true);  // F · Tab_window
  constexpr uint32_t idesc_pos = make_idesc_bf16(128, 64, true, true);   // Fᵀ · Row

  auto load_g = [&](int n) {  // bias-gradient tile of pair n into buffer n & 1
    const int outer = n / nt, inner = n % nt;
    const int ti = SIDE == 0 ? outer : inner, tj = SIDE == 0 ? inner : outer;
    uint8_t* dst = sG + (n & 1) * 2 * kTileBytes;
    mbar_expect_tx(&bar_g[n & 1], 2 * kTileBytes);
    tma_load_3d(dst, &tm_g, &bar_g[n & 1], tj * kTile, ti * kTile, b * p.heads + h);
    tma_load_3d(dst + kTileBytes, &tm_g, &bar_g[n & 1], tj * kTile + 64, ti * kTile, b * p.heads + h);
  };
  auto load_row = [&](int outer) {
    mbar_expect_tx(bar_row, kTileBytes);
    tma_load_3d(sRow, &tm_row, bar_row, h * kD, outer * kTile, b);
  };
  // gradient of the row tile `outer` out of TMEM: kAccCols columns per thread
  auto flush_row = [&](int outer) {
    const int g = outer * kTile + row;
#pragma unroll
    for (int c = 0; c < kAccCols / 8; ++c) {
      uint32_t r[8];
      tmem_ld8(t_row + lane_addr + part * kAccCols + c * 8, r);
      tmem_ld_wait();
      if (g >= S) continue;
      if (SIDE == 0) {
        float* dst = p.dq_acc + (static_cast<long long>(b) * S + g) * H + h * kD + part * kAccCols + c * 8;
#pragma unroll
        for (int v = 0; v < 2; ++v)
          red_add_v4(dst + v * 4, __uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]), __uint_as_float(r[v * 4 + 2]),
                     __uint_as_float(r[v * 4 + 3]));
      } else {
        uint4* dst = reinterpret_cast<uint4*>(p.dk + (static_cast<long long>(b) * S + g) * p.ld_dk + h * kD +
                                              part * kAccCols + c * 8);
        const uint4 old = *dst;
        const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
        uint32_t nw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          nw[e] = pack_bf16(bf16_lo(ow[e]) + __uint_as_float(r[2 * e]), bf16_hi(ow[e]) + __uint_as_float(r[2 * e + 1]));
        *dst = make_uint4(nw[0], nw[1], nw[2], nw[3]);
      }
    }
  };

  bool pend_g0 = false, pend_g1 = false;  // thread 0: a G load is in flight into that buffer
  if (tid == 0) {
    tma_prefetch_desc(&tm_row);
    tma_prefetch_desc(&tm_tab);
    tma_prefetch_desc(&tm_g);
    mbar_expect_tx(bar_tab, p.nblk * kTileBytes);
    for (int blk = 0; blk < p.nblk; ++blk) tma_load_3d(sTab + blk * kTileBytes, &tm_tab, bar_tab, h * kD, blk * kTile, 0);
    load_row(0);
    load_g(0);
    pend_g0 = true;
    if (npairs > 1) {
      load_g(1);
      pend_g1 = true;
    }
  }

  unsigned touched = 0;  // thread 0: blocks of the table gradient that hold data
  bool failed = false;
  int fail_n = 0;
  for (int n = 0; n < npairs; ++n) {
    const int outer = n / nt, inner = n % nt;
    const int ti = SIDE == 0 ? outer : inner, tj = SIDE == 0 ? inner : outer;
    const int wb = p.win[SIDE][ti - tj + nt - 1];          // first table block of this pair's window
    const int nwb = min(2, p.nblk - wb);                   // blocks in the window
    // thread 0 polls: the folded tile is free and the accumulators are current (MMAs of pair n-1 retired), and this
    // pair's tile of G has landed; the block barrier hands the answer to everybody
    bool got = true;
    if (tid == 0) {
      if (n > 0) got = mbar_wait(bar_f, (n - 1) & 1, abort_flag, p.status, kErrAccFullWait);
      got = got && mbar_wait(&bar_g[n & 1], (n >> 1) & 1, abort_flag, p.status, kErrFullWait);
    }
    if (!__syncthreads_and(got)) {
      failed = true;
      fail_n = n;
      break;
    }
    tc_fence_after();
    if (n > 0 && inner == 0) flush_row(outer - 1);
    {  // clear the folded tile (only the chunks this window uses)
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int i = tid; i < nwb * 2 * kTileBytes / 16; i += kThreads) reinterpret_cast<uint4*>(sF)[i] = z;
    }
    tc_fence_before();
    __syncthreads();  // cleared before the scattered stores of the fold; accumulator reads done before the next MMAs
    if (tid == 0) {
      if (n & 1) pend_g1 = false; else pend_g0 = false;
      if (inner == 0 && n > 0) load_row(outer);  // the MMAs that read the previous row tile have retired
    }

    // ---- fold: F[row][w - 128 wb] = sum of G over this thread's run of entries that share bucket w ----
    {
      const uint8_t* g_tile = sG + (n & 1) * 2 * kTileBytes;
      const int o0 = part * kPer;
      float g[kPer];
      int xb;
      if (SIDE == 0) {  // row = query, entries = keys o0 .. o0+kPer-1: one contiguous stretch of the row
        xb = (ti * kTile + row) - (tj * kTile + o0) + nt * kTile - 1;
        const uint8_t* src = g_tile + (o0 >> 6) * kTileBytes + row * 128;
#pragma unroll
        for (int c = 0; c < kPer / 8; ++c) {
          const uint4 u = *reinterpret_cast<const uint4*>(src + (((((o0 & 63) >> 3) + c) ^ (row & 7)) << 4));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            g[c * 8 + 2 * e] = bf16_lo(w[e]);
            g[c * 8 + 2 * e + 1] = bf16_hi(w[e]);
          }
        }
      } else {          // row = key, entries = queries o0 .. o0+kPer-1: one column of the tile
        xb = (ti * kTile + o0) - (tj * kTile + row) + nt * kTile - 1;
        const uint8_t* src = g_tile + (row >> 6) * kTileBytes + o0 * 128 + (row & 7) * 2;
        const int ck = (row & 63) >> 3;
#pragma unroll
        for (int e = 0; e < kPer; ++e)
          g[e] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src + e * 128 + ((ck ^ (e & 7)) << 4)));
      }
      constexpr int dir = SIDE == 0 ? -1 : 1;  // the lookup index falls (rises) along the entries
      const unsigned short* l = lut + xb;
      const int wbase = wb * kTile;
      uint8_t* f_row = sF + row * 128;
      const uint32_t f_xor = static_cast<uint32_t>(row & 7) << 4;
      auto f_store = [&](int w, float v) {
        const uint32_t wl = static_cast<uint32_t>(w - wbase);
        *reinterpret_cast<__nv_bfloat16*>(f_row + ((((wl >> 6) << 14) | ((wl & 63) << 1)) ^ f_xor)) = __float2bfloat16(v);
      };
      // entries that continue the previous part's run belong to the thread that started it
      int wcur = part > 0 ? static_cast<int>(l[-dir]) : -1;
      bool mine = part == 0;
      float run = 0.f;
#pragma unroll
      for (int e = 0; e < kPer; ++e) {
        const int w = l[dir * e];
        if (w != wcur) {
          if (mine && wcur >= 0) f_store(wcur, run);
          mine = true;
          wcur = w;
          run = 0.f;
        }
        run += g[e];
      }
      if (mine) {
        for (int o = o0 + kPer; o < kTile && l[dir * (o - o0)] == wcur; ++o) {  // the run goes on in the next part
          const uint8_t* src = SIDE == 0 ? g_tile + (o >> 6) * kTileBytes + row * 128 + ((((o & 63) >> 3) ^ (row & 7)) << 4) + (o & 7) * 2
                                         : g_tile + (row >> 6) * kTileBytes + o * 128 + ((((row & 63) >> 3) ^ (o & 7)) << 4) + (row & 7) * 2;
          run += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src));
        }
        f_store(wcur, run);
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();

    if (tid == 0) {
      if (n + 2 < npairs) {  // every thread is done with this buffer of G
        load_g(n + 2);
        if (n & 1) pend_g1 = true; else pend_g0 = true;
      }
      bool ready = true;
      if (n == 0) ready = mbar_wait(bar_tab, 0, abort_flag, p.status, kErrFullWait);
      if (ready && inner == 0) ready = mbar_wait(bar_row, outer & 1, abort_flag, p.status, kErrFullWait);
      if (ready) {
        tc_fence_after();
        const uint32_t f = smem_u32(sF), tab = smem_u32(sTab) + wb * kTileBytes, rw = smem_u32(sRow);
        for (int ks = 0; ks < nwb * 8; ++ks)  // row gradient += F[:, 16 buckets] · Tab[16 rows]
          umma_bf16(t_row, make_smem_desc(f + (ks >> 2) * kTileBytes + (ks & 3) * 32, 16, 1024),
                    make_smem_desc(tab + ks * 2048, 8192, 1024), idesc_row, (inner > 0) || (ks > 0));
        for (int wk = 0; wk < nwb; ++wk) {    // table gradient block += F[:, block]ᵀ · Row
          const int blk = wb + wk;
          const bool acc = (touched >> blk) & 1u;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16(t_pos + blk * 64, make_smem_desc(f + wk * 2 * kTileBytes + ks * 2048, kTileBytes, 1024),
                      make_smem_desc(rw + ks * 2048, 8192, 1024), idesc_pos, acc || (ks > 0));
          touched |= 1u << blk;
        }
      }
      umma_commit(bar_f);
    }
  }

  if (!failed) {
    const bool got = tid != 0 || mbar_wait(bar_f, (npairs - 1) & 1, abort_flag, p.status, kErrAccFullWait);
    if (__syncthreads_and(got)) {
      tc_fence_after();
      flush_row(nt - 1);
      for (int blk = 0; blk < p.nblk; ++blk) {
        if (!((p.touched[SIDE] >> blk) & 1u)) continue;
        const int w = blk * kTile + row;
#pragma unroll
        for (int c = 0; c < kAccCols / 8; ++c) {
          uint32_t r[8];
          tmem_ld8(t_pos + blk * 64 + lane_addr + part * kAccCols + c * 8, r);
          tmem_ld_wait();
          if (w >= p.span2) continue;
          float* dst = p.d_pos[SIDE] + static_cast<long long>(w) * H + h * kD + part * kAccCols + c * 8;
#pragma unroll
          for (int v = 0; v < 2; ++v)
            red_add_v4(dst + v * 4, __uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                       __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
        }
      }
    }
  } else if (tid == 0) {  // leave no bulk copy in flight behind this CTA: tiles fail_n and fail_n + 1 may still land
    for (int m = fail_n; m < min(fail_n + 2, npairs); ++m) {
      if (!((m & 1) ? pend_g1 : pend_g0)) continue;
      for (uint32_t i = 0; i < kSpinLimit && !mbar_try_wait(&bar_g[m & 1], (m >> 1) & 1); ++i) {
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// grid (2 sides, heads, B), 128·kParts threads
__global__ void __launch_bounds__(kThreads, 1)
posbias_tc_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_pk, const __grid_constant__ CUtensorMap tm_pq,
                      const __grid_constant__ CUtensorMap tm_g, const PosBwdDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (!p.has[blockIdx.x]) return;
  if (blockIdx.x == 0) posbias_bwd_body<0>(tm_q, tm_pk, tm_g, p, smem);
  else posbias_bwd_body<1>(tm_k, tm_pq, tm_g, p, smem);
}

}  // namespace

extern "C" int db200_posbias_tc_bwd(const PosBiasArgs* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a->B <= 0 || a->S <= 0 || a->heads <= 0) return 0;
  const bool has_c = a->pos_k != nullptr, has_p = a->pos_q != nullptr;
  if (!has_c && !has_p) return -10;
  const int nt = (a->S + kTile - 1) / kTile;
  const int nblk = (a->span2 + kTile - 1) / kTile;
  if (2 * nt - 1 > kMaxDiag || a->span2 <= 0) return -12;
  if (nblk > kMaxBlocks || nt > 8) return -13;
  if (!aligned16(a->q) || !aligned16(a->k) || (a->ldq % 8) || (a->ldk % 8) || (a->ld_pos % 8) || !a->dbias ||
      !aligned16(a->dbias) || (a->ldb % kTile) || a->ldb < nt * kTile ||
      (has_c && (!aligned16(a->pos_k) || !a->lut_c2p_host || !a->lut_c2p || !a->dq_acc || !aligned16(a->dq_acc) || !a->d_pos_k ||
                 !aligned16(a->d_pos_k))) ||
      (has_p && (!aligned16(a->pos_q) || !a->lut_p2c_host || !a->lut_p2c || !a->dk || !aligned16(a->dk) || (a->ld_dk % 8) ||
                 !a->d_pos_q || !aligned16(a->d_pos_q))))
    return -10;
  PosBwdDev d{};
  d.B = a->B; d.S = a->S; d.heads = a->heads; d.nt = nt; d.span2 = a->span2; d.nblk = nblk;
  d.lut[0] = static_cast<const unsigned short*>(a->lut_c2p);
  d.lut[1] = static_cast<const unsigned short*>(a->lut_p2c);
  d.dq_acc = a->dq_acc;
  d.dk = static_cast<__nv_bfloat16*>(a->dk);
  d.ld_dk = a->ld_dk;
  d.d_pos[0] = a->d_pos_k;
  d.d_pos[1] = a->d_pos_q;
  d.has[0] = has_c; d.has[1] = has_p;
  d.status = db200_status_ptr();
  for (int side = 0; side < 2; ++side) {
    if (!d.has[side]) continue;
    const unsigned short* lut = static_cast<const unsigned short*>(side == 0 ? a->lut_c2p_host : a->lut_p2c_host);
    for (int diag = 0; diag < 2 * nt - 1; ++diag) {
      int w = window_block(lut, a->S, nt, diag);
      if (w < 0) return -13;
      if (nblk >= 2 && w > nblk - 2) w = nblk - 2;  // keep both blocks of the window inside the table
      d.win[side][diag] = static_cast<unsigned char>(w);
      for (int wk = 0; wk < 2 && w + wk < nblk; ++wk) d.touched[side] |= 1u << (w + wk);
    }
  }
  CUtensorMap tq, tk, tpk, tpq, tg;
  int rc;
  if ((rc = head_map(&tq, has_c ? a->q : a->k, a->heads, a->S, a->B, has_c ? a->ldq : a->ldk))) return rc;
  if ((rc = head_map(&tk, has_p ? a->k : a->q, a->heads, a->S, a->B, has_p ? a->ldk : a->ldq))) return rc;
  if ((rc = head_map(&tpk, has_c ? a->pos_k : a->pos_q, a->heads, a->span2, 1, a->ld_pos))) return rc;
  if ((rc = head_map(&tpq, has_p ? a->pos_q : a->pos_k, a->heads, a->span2, 1, a->ld_pos))) return rc;
  if ((rc = db200_make_tmap_bf16(&tg, a->dbias, a->ldb, a->S, static_cast<long long>(a->B) * a->heads, a->ldb,
                                 static_cast<long long>(a->S) * a->ldb, kTile)))
    return rc;
  const int smem = BwdSmem::total(nt);
  if (cudaFuncSetAttribute(posbias_tc_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
  dim3 grid(2, a->heads, a->B);
  posbias_tc_bwd_kernel<<<grid, kThreads, smem, stream>>>(tq, tk, tpk, tpq, tg, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
