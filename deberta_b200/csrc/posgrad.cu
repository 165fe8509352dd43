// Both products of one side of the position-term gradient in ONE pass over the folded gradient table.
//
// The scans of posbias.cu leave G[token, head, w] = d loss / d (content row · position row w) for w in [0, W),
// W = 2·span table rows. Two things are owed per side and head:
//
//     rows[t, :]  += sum_w G[t, w] · Tab[w, :]        (the query rows for c2p, the key rows for p2c)
//     dTab[w, :]  += sum_t G[t, w] · X[t, :]          (X = Q for c2p, K for p2c)
//
// As two batched GEMMs each of them reads G (tokens x heads x W bf16: 201 MB at 16 384 tokens, 12 heads, W = 512)
// from HBM, and that read is all they wait for. Here a 128-token tile of G lands in shared memory once and feeds
// both: as the K-major A operand of  G·Tab  (accumulator: 128 tokens x 64) and, the same bytes read M-major, as the
// A operand of  Gᵀ·X  (accumulator: W x 64, kept in tensor memory for all token tiles of the CTA and added to
// global memory once). Structure as in gemm.cu: one TMA warp, one MMA warp, eight epilogue warps; bounded waits
// that report through the status word.
//
// Reference semantics: the gradient of the c2p / p2c score gathers, src/deberta/modeling/deberta_v2_native.py:564-652.
#include "tc05.cuh"
#include "kernels.h"

namespace {

using namespace tc05;

constexpr int kTok = 128;                    // tokens per tile
constexpr int kD = 64;                       // head dimension
constexpr int kStepW = 128;                  // table rows per load step (one 128-row block of the table gradient)
constexpr int kStages = 4;                   // one stage per 128-row block of a 512-row table
constexpr int kBoxBytes = kTok * 64 * 2;     // 16 KB: 128 rows x 64 bf16, 128B swizzle
constexpr int kStageBytes = 2 * kBoxBytes;   // 32 KB: 128 tokens x 128 table rows
constexpr int kTabBytes = 512 * kD * 2;      // 64 KB: the head's slice of the position table (up to 512 rows)
constexpr int kThreads = 320;

struct Smem {
  static constexpr int kTab = 0;
  static constexpr int kG = kTab + kTabBytes;          // four stages: table rows [128 s, 128 s + 128) of a tile
  static constexpr int kX = kG + kStages * kStageBytes;  // two token tiles of X
  static constexpr int kBar = kX + 2 * kBoxBytes;
  static constexpr int kTotal = kBar + 256 + 1024;
};
static_assert(Smem::kTotal <= 227 * 1024, "shared memory of one CTA");

struct Dev {
  int T, heads, W, steps;       // steps = W / 128 (2 or 4)
  int tiles, tiles_per_cta;
  float* out_f32;               // [T, ld_of] fp32, += (red.add), or null
  __nv_bfloat16* out_bf16;      // [T, ld_ob] bf16 (every element has one owner), or null: = acc_in + result when
                                // acc_in is given, else += result (read-modify-write)
  const float* acc_in;          // [T, ld_ai] fp32 or null
  long long ld_of, ld_ob, ld_ai;
  float* d_tab;                 // [W, ld_dt] fp32, +=
  long long ld_dt;
  int* status;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// grid (chunks, heads): CTA (c, h) owns token tiles [c * tiles_per_cta, (c + 1) * tiles_per_cta) of head h.
__global__ void __launch_bounds__(kThreads, 1)
posgrad_dual_kernel(const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_tab,
                    const __grid_constant__ CUtensorMap tm_x, const Dev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sTab = smem + Smem::kTab;
  uint8_t* sG = smem + Smem::kG;
  uint8_t* sX = smem + Smem::kX;
  uint64_t* full_g = reinterpret_cast<uint64_t*>(smem + Smem::kBar);  // [4]
  uint64_t* empty_g = full_g + 4;                                     // [4]
  uint64_t* acc_full = full_g + 8;                                    // [2]
  uint64_t* acc_empty = full_g + 10;                                  // [2]
  uint64_t* tab_full = full_g + 12;
  uint64_t* pos_full = full_g + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(full_g + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int tile0 = blockIdx.x * p.tiles_per_cta;
  const int ntile = min(p.tiles_per_cta, p.tiles - tile0);  // >= 1 by the launcher's grid
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_g[s], 1);
      mbar_init(&empty_g[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 8);  // one arrival per epilogue warp
    }
    mbar_init(tab_full, 1);
    mbar_init(pos_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_rows = tmem_base;        // 2 x 64 columns: G·Tab of the current / next token tile
  const uint32_t t_pos = tmem_base + 128;   // 4 x 64 columns: Gᵀ·X, one 128-row block of the table per 64 columns
  pdl_wait();  // set-up done; from here on global memory is touched

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tm_g);
      tma_prefetch_desc(&tm_tab);
      tma_prefetch_desc(&tm_x);
      mbar_expect_tx(tab_full, p.steps * (kStepW * kD * 2));
      for (int hf = 0; hf < p.steps; ++hf)
        tma_load_3d(sTab + hf * (kStepW * kD * 2), &tm_tab, tab_full, h * kD, hf * kStepW, 0);
      bool ok = true;
      for (int t = 0; t < ntile && ok; ++t) {
        const int tok0 = (tile0 + t) * kTok;
        for (int hf = 0; hf < p.steps; ++hf) {
          // stage hf holds table rows [hf * 128, hf * 128 + 128) of every tile: its k-th use is tile k. A stage is
          // asked for again as soon as the MMAs that read it have retired, so up to three are in flight at a time.
          if (!mbar_wait(&empty_g[hf], (t & 1) ^ 1, abort_flag, p.status, kErrEmptyWait)) { ok = false; break; }
          uint8_t* dst = sG + hf * kStageBytes;
          mbar_expect_tx(&full_g[hf], kStageBytes + (hf == 0 ? kBoxBytes : 0));
          if (hf == 0) tma_load_3d(sX + (t & 1) * kBoxBytes, &tm_x, &full_g[0], h * kD, tok0, 0);
#pragma unroll
          for (int bx = 0; bx < 2; ++bx)
            tma_load_3d(dst + bx * kBoxBytes, &tm_g, &full_g[hf], h * p.W + hf * kStepW + bx * 64, tok0, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_rows = make_idesc_bf16(128, 64, false, true);  // G (K-major) · Tab (N-major)
      constexpr uint32_t idesc_pos = make_idesc_bf16(128, 64, true, true);    // Gᵀ (M-major) · X (N-major)
      bool ok = mbar_wait(tab_full, 0, abort_flag, p.status, kErrFullWait);
      for (int t = 0; t < ntile && ok; ++t) {
        const int a = t & 1;
        if (!mbar_wait(&acc_empty[a], ((t >> 1) & 1) ^ 1, abort_flag, p.status, kErrAccEmptyWait)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sx = smem_u32(sX + a * kBoxBytes);
        for (int hf = 0; hf < p.steps; ++hf) {
          if (!mbar_wait(&full_g[hf], t & 1, abort_flag, p.status, kErrFullWait)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sg = smem_u32(sG + hf * kStageBytes);
          const uint32_t st = smem_u32(sTab + hf * (kStepW * kD * 2));
          // rows[128 tokens, 64] += G[128, 128] · Tab[128, 64]: 8 steps of 16 table rows; a step is 32 bytes inside
          // the 128-byte row of one of the two 64-column boxes
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16(t_rows + a * 64, make_smem_desc(sg + (ks >> 2) * kBoxBytes + (ks & 3) * 32, 16, 1024),
                      make_smem_desc(st + ks * 2048, 8192, 1024), idesc_rows, (hf > 0) || (ks > 0));
          // dTab[128 table rows, 64] += Gᵀ[128, 128 tokens] · X[128 tokens, 64]: 8 steps of 16 tokens (2048 bytes
          // down the box); the block's two 64-column boxes are 16 KB apart
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16(t_pos + hf * 64, make_smem_desc(sg + ks * 2048, kBoxBytes, 1024),
                      make_smem_desc(sx + ks * 2048, 8192, 1024), idesc_pos, (t > 0) || (ks > 0));
          umma_commit(&empty_g[hf]);  // frees the stage (and, after the last step, this tile's X buffer)
        }
        if (!ok) break;
        umma_commit(&acc_full[a]);
      }
      umma_commit(pos_full);  // (also on the error path: the epilogue's bounded wait then ends at once)
    }
  } else {
    // ------------------------------- epilogue -----------------------------------
    const int quad = warp & 3;          // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;   // which 32 of the 64 columns
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (int t = 0; t < ntile; ++t) {
      const int a = t & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[a], (t >> 1) & 1, abort_flag, p.status, kErrAccFullWait)) != 0;
      if (!ok) break;
      tc_fence_after();
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_rows + a * 64 + lane_addr + part * 32, r);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
      const long long tok = static_cast<long long>(tile0 + t) * kTok + row;
      if (tok < p.T) {
        if (p.out_f32) {
          float* dst = p.out_f32 + tok * p.ld_of + h * kD + part * 32;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            red_add_v4(dst + q * 4, __uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                       __uint_as_float(r[q * 4 + 3]));
        } else {
          uint4* dst = reinterpret_cast<uint4*>(p.out_bf16 + tok * p.ld_ob + h * kD + part * 32);
          if (p.acc_in) {  // fp32 partial result of another kernel + this one, rounded once
            const float4* src = reinterpret_cast<const float4*>(p.acc_in + tok * p.ld_ai + h * kD + part * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 a0 = src[2 * q], a1 = src[2 * q + 1];
              dst[q] = make_uint4(pack_bf16(a0.x + __uint_as_float(r[q * 8]), a0.y + __uint_as_float(r[q * 8 + 1])),
                                  pack_bf16(a0.z + __uint_as_float(r[q * 8 + 2]), a0.w + __uint_as_float(r[q * 8 + 3])),
                                  pack_bf16(a1.x + __uint_as_float(r[q * 8 + 4]), a1.y + __uint_as_float(r[q * 8 + 5])),
                                  pack_bf16(a1.z + __uint_as_float(r[q * 8 + 6]), a1.w + __uint_as_float(r[q * 8 + 7])));
            }
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 old = dst[q];
              const uint32_t o[4] = {old.x, old.y, old.z, old.w};
              uint32_t n[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                n[e] = pack_bf16(bf16_lo(o[e]) + __uint_as_float(r[q * 8 + 2 * e]),
                                 bf16_hi(o[e]) + __uint_as_float(r[q * 8 + 2 * e + 1]));
              dst[q] = make_uint4(n[0], n[1], n[2], n[3]);
            }
          }
        }
      }
    }
    // the table gradient of this CTA's tokens, once
    if (ok && __all_sync(0xffffffffu, mbar_wait(pos_full, 0, abort_flag, p.status, kErrAccFullWait)) != 0) {
      tc_fence_after();
      for (int blk = 0; blk < p.steps; ++blk) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_pos + blk * 64 + lane_addr + part * 32, r);
        tmem_ld_wait();
        float* dst = p.d_tab + static_cast<long long>(blk * 128 + row) * p.ld_dt + h * kD + part * 32;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          red_add_v4(dst + q * 4, __uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                     __uint_as_float(r[q * 4 + 3]));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// rows += G·Tab (fp32 red.add into `out_f32`, or bf16 read-modify-write into `out_bf16`; exactly one of the two; with
// `acc_in` the bf16 rows are acc_in + G·Tab instead, rounded once) and d_tab += Gᵀ·X, per head. g: [T, heads*W] bf16 (row stride ld_g), tab: [W, heads*64] bf16, x: [T, >= heads*64] bf16,
// d_tab: [W, heads*64] fp32. W must be 256 or 512. Returns -13 when the shape is not covered (the caller then uses
// the two GEMMs).
extern "C" int db200_posgrad_dual(const void* g, long long ld_g, const void* tab, long long ld_tab, const void* x,
                                  long long ld_x, float* out_f32, long long ld_of, void* out_bf16, long long ld_ob,
                                  const float* acc_in, long long ld_ai, float* d_tab, long long ld_dt, int T, int heads,
                                  int W, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || heads <= 0) return 0;
  if (W != 256 && W != 512) return -13;
  if (!g || !tab || !x || !d_tab || ((out_f32 == nullptr) == (out_bf16 == nullptr))) return -10;
  if (!aligned16(g) || !aligned16(tab) || !aligned16(x) || !aligned16(d_tab) || (ld_g % 8) || (ld_tab % 8) || (ld_x % 8) ||
      (ld_dt % 4) || (out_f32 && (!aligned16(out_f32) || (ld_of % 4))) || (out_bf16 && (!aligned16(out_bf16) || (ld_ob % 8))) ||
      (acc_in && (!out_bf16 || !aligned16(acc_in) || (ld_ai % 4))))
    return -10;
  CUtensorMap tg, tt, tx;
  int rc;
  if ((rc = db200_make_tmap_bf16(&tg, g, static_cast<long long>(heads) * W, T, 1, ld_g, 0, kTok))) return rc;
  if ((rc = db200_make_tmap_bf16(&tt, tab, static_cast<long long>(heads) * kD, W, 1, ld_tab, 0, kStepW))) return rc;
  if ((rc = db200_make_tmap_bf16(&tx, x, static_cast<long long>(heads) * kD, T, 1, ld_x, 0, kTok))) return rc;
  Dev d{};
  d.T = T; d.heads = heads; d.W = W; d.steps = W / kStepW;
  d.tiles = (T + kTok - 1) / kTok;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  int chunks = sms / heads;
  if (chunks < 1) chunks = 1;
  if (chunks > d.tiles) chunks = d.tiles;
  d.tiles_per_cta = (d.tiles + chunks - 1) / chunks;
  chunks = (d.tiles + d.tiles_per_cta - 1) / d.tiles_per_cta;  // no empty CTA
  d.out_f32 = out_f32; d.ld_of = ld_of;
  d.out_bf16 = static_cast<__nv_bfloat16*>(out_bf16); d.ld_ob = ld_ob;
  d.acc_in = acc_in; d.ld_ai = ld_ai;
  d.d_tab = d_tab; d.ld_dt = ld_dt;
  d.status = db200_status_ptr();
  static bool configured[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  dev = (dev >= 0 && dev < 16) ? dev : 0;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(posgrad_dual_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) != cudaSuccess)
      return -3;
    configured[dev] = true;
  }
  return launch_pdl(posgrad_dual_kernel, dim3(chunks, heads), dim3(kThreads), Smem::kTotal, stream, tg, tt, tx, d) == cudaSuccess
             ? 0
             : -4;
}
