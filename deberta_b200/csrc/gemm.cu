// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] = alpha * sum_k A[m,k] * B[n,k]   (fp32 accumulation in TMEM)
//
// Roles inside one 320-thread CTA (one CTA per SM, static round-robin over tiles):
//   warp 0      : TMA producer  (cp.async.bulk.tensor -> 128B-swizzled smem ring)
//   warp 1      : tcgen05.mma issuer + TMEM owner (two accumulator buffers)
//   warps 2..9  : epilogue (tcgen05.ld -> bias / GELU / residual / dGELU -> global); two warps per
//                 TMEM lane quadrant split the tile's columns so the epilogue is not latency-bound
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Operand layouts (all bf16, row-major in global memory, leading dims in elements):
//   a_mn = 0 : A is [M, K]  (K contiguous)      a_mn = 1 : A is [K, M]  (M contiguous)
//   b_mn = 0 : B is [N, K]  (K contiguous)      b_mn = 1 : B is [K, N]  (N contiguous)
// which covers forward (0,0), data-gradient (0,1) and weight-gradient (1,1) of a
// linear layer without any transposed copies.
#include "tc05.cuh"
#include "kernels.h"

#include <mutex>
#include <unordered_map>

namespace {

using namespace tc05;

constexpr int BM = 128;
constexpr int BK = 64;
// Epilogue warps per CTA: a warp may read only its own TMEM lane quadrant (warp id mod 4), so the warps come in sets
// of four and each set owns an equal share of the tile's columns. Two sets cover every epilogue that hides behind the
// MMAs; the ones that do real arithmetic per element (cross-entropy with sampling, GELU with two outputs) and would
// otherwise set the kernel's pace with two warps per scheduler get four sets on the wide tile.
template <int BN, int MODE>
__host__ __device__ constexpr int epilogue_warps() { return (BN == 256 && (MODE == 4 || MODE == 5 || MODE == 6)) ? 16 : 8; }
template <int BN, int MODE>
__host__ __device__ constexpr int gemm_threads() { return 64 + 32 * epilogue_warps<BN, MODE>(); }

template <int BN, int MODE>
struct SmemLayout {
  static constexpr int kEpilogueWarps = epilogue_warps<BN, MODE>();
  // the cross-entropy epilogues write from registers and need no staging tiles (2 KB stay for alignment's sake)
  static constexpr bool kStaging = !(MODE == 4 || MODE == 5);
  static constexpr int kStagingBytes = 32 * 128;  // per epilogue warp: 32 rows x 64 bf16, 128B swizzle
  static constexpr int kStagingTotal = kStaging ? kEpilogueWarps * kStagingBytes : 2048;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // 16 staging tiles leave room for three operand stages of the wide tile
  static constexpr int kStages = (BN == 256) ? ((kStaging && kEpilogueWarps == 16) ? 3 : 4) : 6;
  static constexpr int kStagingOffset = kStages * kStageBytes;          // 1024-byte aligned
  static constexpr int kBarOffset = kStagingOffset + kStagingTotal;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // barriers + alignment slack
  static_assert(kTotal <= 227 * 1024, "shared memory of one CTA");
};

struct DevParams {
  int M, N, K;
  int tiles_m, tiles_n, batch, splits;
  int kb_total;
  float alpha;
  int epi;
  int out_f32;      // 1: fp32 output
  int tma_out;      // 1: bf16 outputs leave through shared memory and TMA stores (tmap_out / tmap_out2)
  int accumulate;   // 1: out += result (fp32 output only, uses red.add)
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* aux;
  void* out;
  __nv_bfloat16* out2;
  long long ldo, ldr, ldaux, ldo2;
  long long bs_out, bs_res, bs_aux, bs_out2, bs_bias;
  int* status;
  // vocabulary cross-entropy epilogues (EPI_CE_FWD / EPI_CE_BWD)
  const long long* labels;          // [M]
  const unsigned char* forbidden;   // [N] ids that may not be sampled, or null
  float inv_temp;                   // 1 / sampling temperature
  unsigned long long seed;
  float* ce_part;                   // [4, tiles_n, M]: tile max, tile sum-exp, largest sampling key, its candidate id
  float* label_logit;               // [M]
  const float* row_lse;             // [M] natural-log log-sum-exp (backward)
  float gscale;                     // dLoss/dlogit scale (backward)
  const float* gscale_ptr;          // optional device scalar multiplied into gscale
  float* a_sum;                     // [M] fp32 or null: += sum_k A[m,k] (fp32 output with M-major A: bias gradients)
  int half_n;                       // SwiGLU epilogues: F, the width of the gate (and of the up) half
};

// Counter-based uniform in (0,1) from (seed, row, column): 32-bit multiply-xorshift mixing (two rounds), the seed's
// halves entering before and between the rounds; ~10 integer operations. The sampler draws two per 32 logits.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned int row, unsigned int col) {
  unsigned int x = (col * 0x9E3779B1u) ^ (row * 0x85EBCA77u) ^ static_cast<unsigned int>(seed);
  x ^= x >> 16; x *= 0x7FEB352Du;
  x ^= x >> 15; x ^= static_cast<unsigned int>(seed >> 32);
  x *= 0x846CA68Bu; x ^= x >> 16;
  return (static_cast<float>(x >> 9) + 0.5f) * (1.0f / 8388608.0f);  // 23 bits + 1/2: exact in fp32, inside (0,1)
}

// Normal CDF and density through one exponential: erf by Abramowitz-Stegun 7.1.26 (|error| < 1.5e-7, far below
// bf16 resolution) shares exp(-x^2/2) with the density, so GELU and its derivative cost one ex2 and one
// reciprocal per element instead of an erff plus an expf.
__device__ __forceinline__ void normal_cdf_pdf(float x, float& cdf, float& pdf) {
  const float ax = fabsf(x) * 0.70710678118654752f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.0f)));
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * x * -0.72134752044448170f));  // exp(-x^2/2)
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float half_erfc = 0.5f * poly * t * e;  // 0.5 * erfc(|x|/sqrt 2)
  cdf = x >= 0.f ? 1.0f - half_erfc : half_erfc;
  pdf = 0.3989422804014327f * e;
}
__device__ __forceinline__ float gelu_erf(float x) {
  float cdf, pdf;
  normal_cdf_pdf(x, cdf, pdf);
  return x * cdf;
}
__device__ __forceinline__ float dgelu_erf(float x) {
  float cdf, pdf;
  normal_cdf_pdf(x, cdf, pdf);
  return fmaf(x, pdf, cdf);
}

// MODE selects the epilogue at compile time (one lean code path per instantiation):
// 0 bf16 output (+bias, +residual), 1 GELU (two outputs), 2 GELU derivative, 3 fp32 output (store / accumulate /
// split-K), 4 cross-entropy forward, 5 cross-entropy backward, 6 GELU with its derivative as the first output,
// 7 product with a stored operand (the backward partner of 6: no transcendental in the epilogue),
// 8 SwiGLU forward (a tile = 128 gate columns and the 128 up columns that go with them; three outputs' worth of
// stores), 9 SwiGLU backward.
template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(gemm_threads<BN, MODE>(), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_out2,
            const DevParams p) {
  using L = SmemLayout<BN, MODE>;
  constexpr int kEpilogueWarps = L::kEpilogueWarps;
  constexpr int kThreads = gemm_threads<BN, MODE>();
  constexpr int kParts = kEpilogueWarps / 4;  // column shares of a tile (one per set of four warps)
  constexpr int kEpi = MODE == 1 ? EPI_GELU : MODE == 2 ? EPI_DGELU : MODE == 4 ? EPI_CE_FWD : MODE == 5 ? EPI_CE_BWD
                       : MODE == 6 ? EPI_GELU_GRAD : MODE == 7 ? EPI_MUL : MODE == 8 ? EPI_SWIGLU
                       : MODE == 9 ? EPI_SWIGLU_BWD : EPI_NONE;
  constexpr bool kSwigluFwd = MODE == 8;  // needs BN == 256 and a K-major B (instantiated only that way)
  constexpr bool kTwoOut = kEpi == EPI_GELU || kEpi == EPI_GELU_GRAD;  // second output: gelu of the pre-activation
  constexpr bool kAuxMul = kEpi == EPI_DGELU || kEpi == EPI_MUL;       // accumulator times a function of `aux`
  constexpr bool kOutF32 = MODE == 3;
  // Row sums of A on the tensor cores (the bias gradient of a linear layer inside its weight-gradient GEMM): the
  // work items of the first column tile multiply every A tile by a 16-column tile of ones as well, into 16 spare
  // TMEM columns. With BN = 256 the two accumulator buffers fill the tensor memory, so such a launch runs on one
  // buffer (weight gradients are split along K into about one work item per CTA, so nothing is lost).
  constexpr bool kRowSum = kOutF32 && A_MN;
  constexpr uint32_t kSumCol = 256;
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* acc_full = empty_bar + L::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = kRowSum ? 512 : 2 * BN;  // 256 or 512: powers of two
  const bool want_sum = kRowSum && p.a_sum != nullptr;
  const int acc_stages = (want_sum && BN == 256) ? 1 : 2;
  if (want_sum) {  // bf16 ones: identical under every swizzle, so the tile needs no layout
    uint32_t* ones = reinterpret_cast<uint32_t*>(smem + L::kStagingOffset);
    for (int i = threadIdx.x; i < 512; i += kThreads) ones[i] = 0x3F803F80u;
    fence_proxy_async();
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], kEpilogueWarps);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // set-up done; from here on global memory is touched

  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int total_work = tiles_per_batch * p.batch * p.splits;
  const int kb_per_split = (p.kb_total + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w % p.splits;
        const int t = w / p.splits;
        const int z = t / tiles_per_batch;
        const int tt = t % tiles_per_batch;
        const int m0 = (tt % p.tiles_m) * BM;
        const int n0 = (tt / p.tiles_m) * BN;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrEmptyWait)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          if (!A_MN) {
            tma_load_3d(sa, &tmap_a, &full_bar[stage], kb * BK, m0, z);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(sa + c * (BK * 128), &tmap_a, &full_bar[stage], m0 + c * 64, kb * BK, z);
          }
          if (!B_MN) {
            if (kSwigluFwd) {  // 128 gate rows of W12 and the 128 up rows of the same hidden columns
              tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * BK, n0 / 2, z);
              tma_load_3d(sb + 128 * 128, &tmap_b, &full_bar[stage], kb * BK, p.half_n + n0 / 2, z);
            } else if (BN == 256) {
              tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * BK, n0, z);
              tma_load_3d(sb + 128 * 128, &tmap_b, &full_bar[stage], kb * BK, n0 + 128, z);
            } else {
              tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * BK, n0, z);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sb + c * (BK * 128), &tmap_b, &full_bar[stage], n0 + c * 64, kb * BK, z);
          }
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      constexpr uint32_t idesc_sum = make_idesc_bf16(BM, 16, A_MN, false);
      const uint64_t d_ones = make_smem_desc(smem_u32(smem + L::kStagingOffset), 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w % p.splits;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, kErrAccEmptyWait)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const bool do_sum = want_sum && ((w / p.splits) % tiles_per_batch) / p.tiles_m == 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrFullWait)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 16 bf16 of K = 32 bytes inside the 128-byte swizzled row.
            // MN-major: 16 rows of K = two 1024-byte swizzle atoms.
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > kb0) || (k > 0));
            if (kRowSum && do_sum) umma_bf16(tmem_base + kSumCol + acc * 16, da, d_ones, idesc_sum, (kb > kb0) || (k > 0));
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------- epilogue -----------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which share of the tile's columns (a half with two sets of warps)
    constexpr int kChunksPerHalf = BN / (32 * kParts);  // 32-column chunks of one share
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // TMA-store path: a warp collects 64 columns (two chunks) of its 32 rows in a swizzled staging tile and
    // hands it to the TMA unit, which writes whole lines and clips rows >= M and columns >= N.
    uint8_t* stg = smem + L::kStagingOffset + (warp - 2) * L::kStagingBytes;
    bool stg_busy = false;  // a bulk store may still be reading the staging tile (warp-uniform)
    auto stage_words = [&](const uint32_t* wds, int sub) {  // 16 packed words = 32 columns of this lane's row
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int chunk = (sub * 4 + q4) ^ (lane & 7);
        *reinterpret_cast<uint4*>(stg + lane * 128 + chunk * 16) =
            make_uint4(wds[q4 * 4], wds[q4 * 4 + 1], wds[q4 * 4 + 2], wds[q4 * 4 + 3]);
      }
    };
    auto stage_acquire = [&]() {  // before the first write of a new 64-column group
      if (stg_busy) {
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        stg_busy = false;
      }
    };
    auto stage_flush = [&](const CUtensorMap* tm, int x, int y, int zz) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        tma_store_3d(tm, stg, x, y, zz);
        tma_store_commit();
      }
      stg_busy = true;
    };
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const int t = w / p.splits;
      const int z = t / tiles_per_batch;
      const int tt = t % tiles_per_batch;
      const int m0 = (tt % p.tiles_m) * BM;
      const int n0 = (tt / p.tiles_m) * BN;
      const int split = w % p.splits;
      const bool empty_split = split * kb_per_split >= p.kb_total;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, kErrAccFullWait)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const __nv_bfloat16* bias = p.bias ? p.bias + z * p.bs_bias : nullptr;
      if constexpr (kEpi == EPI_CE_FWD || kEpi == EPI_CE_BWD) {
        // One thread owns one row of logits. Forward: tile-local max / sum-exp / label logit and the
        // sampling candidate (an id drawn inside each 32-column chunk, the chunks competing through Gumbel-max
        // keys over their masses; forbidden ids excluded); partial results of every vocabulary tile are
        // combined by a second small kernel, which keeps the candidate with the largest key. Backward: softmax
        // minus one-hot.
        const long long label = row_ok ? p.labels[row] : -1;
        const float lse = (kEpi == EPI_CE_BWD && row_ok) ? p.row_lse[row] : 0.f;
        const float gs = p.gscale * ((kEpi == EPI_CE_BWD && p.gscale_ptr) ? *p.gscale_ptr : 1.f);
        float t_max = -INFINITY, t_sum = 0.f, best = -INFINITY;
        int best_idx = 0;
#pragma unroll 1
        for (int c = half * kChunksPerHalf; c < (half + 1) * kChunksPerHalf; ++c) {
          const int nc = n0 + c * 32;
          if (nc >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          tmem_ld_wait();
          const bool label_here = kEpi == EPI_CE_FWD && __any_sync(0xffffffffu, label >= nc && label < nc + 32);
          if (!row_ok) continue;
          float v[32];
          float cmax = -INFINITY;
          const bool full_chunk = nc + 32 <= p.N;  // warp-uniform
          if (full_chunk && (bias == nullptr || ((reinterpret_cast<uintptr_t>(bias + nc) & 15) == 0))) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            if (bias) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias + nc) + q4);
                const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  v[q4 * 8 + 2 * e] += bf16_lo(bw[e]);
                  v[q4 * 8 + 2 * e + 1] += bf16_hi(bw[e]);
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) cmax = fmaxf(cmax, v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = nc + j;
              float x = __uint_as_float(r[j]);
              if (n < p.N) {
                if (bias) x += __bfloat162float(bias[n]);
              } else {
                x = -INFINITY;
              }
              v[j] = x;
              cmax = fmaxf(cmax, x);
            }
          }
          if (kEpi == EPI_CE_FWD) {
            // forbidden-id flags of the chunk as one bit mask (two 16-byte loads when the chunk is complete);
            // every lane sees the same columns, so the mask is warp-uniform
            unsigned int ban_mask = 0;
            if (p.forbidden) {
              if (nc + 32 <= p.N && ((reinterpret_cast<uintptr_t>(p.forbidden) + nc) & 15) == 0) {
                const uint4 f0 = __ldg(reinterpret_cast<const uint4*>(p.forbidden + nc));
                const uint4 f1 = __ldg(reinterpret_cast<const uint4*>(p.forbidden + nc) + 1);
                const unsigned int fw[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                if ((f0.x | f0.y | f0.z | f0.w | f1.x | f1.y | f1.z | f1.w) != 0u) {  // few chunks hold a forbidden id
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    ban_mask |= ((fw[j >> 2] >> ((j & 3) * 8)) & 0xffu) ? (1u << j) : 0u;
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (nc + j < p.N && p.forbidden[nc + j]) ban_mask |= 1u << j;
              }
            }
            if (label_here) {  // some row of this warp has its label in this chunk (about one chunk in a hundred)
              const long long label_off = label - nc;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (label_off == j) p.label_logit[row] = v[j];
            }
            // Sampling from softmax(logits / T) over the allowed ids, exactly, with two uniforms per chunk instead of
            // one per logit: the chunk competes with the others through a Gumbel-max key over its total mass
            // (ln of the sum of exp(logit/T) plus Gumbel noise), and the id inside the chunk is drawn by inverting
            // the running sum of the same terms. Columns past N hold -inf and weigh nothing.
            constexpr float kLog2e = 1.4426950408889634f;
            const bool unit_temp = p.inv_temp == 1.f;
            const float c_l2 = cmax * kLog2e;
            float s_all = 0.f;  // sum over the chunk of exp(logit - cmax): the loss's share
            if (unit_temp) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = ex2_approx(fmaf(v[j], kLog2e, -c_l2));
              if (ban_mask) {
#pragma unroll
                for (int j = 0; j < 32; ++j) s_all += v[j];
              }
            } else {
              const float c1 = p.inv_temp * kLog2e;
              const float c_t = cmax * c1;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                s_all += ex2_approx(fmaf(v[j], kLog2e, -c_l2));
                v[j] = ex2_approx(fmaf(v[j], c1, -c_t));
              }
            }
            if (ban_mask) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if ((ban_mask >> j) & 1u) v[j] = 0.f;
            }
            // running sums in place; the last one is the mass of the chunk
#pragma unroll
            for (int j = 1; j < 32; ++j) v[j] += v[j - 1];
            const float mass = v[31];
            if (unit_temp && !ban_mask) s_all = mass;
            if (mass > 0.f) {
              // u is an odd multiple of 2^-24: never 0 or 1, so every logarithm below is finite
              const float u_in = hash_uniform(p.seed, static_cast<unsigned int>(row), static_cast<unsigned int>(nc));
              const float u_key = hash_uniform(p.seed, static_cast<unsigned int>(row), static_cast<unsigned int>(nc) + 1u);
              // strictly below the total: the count of partial sums <= target is then at most 31, and the chosen
              // column is one whose term moved the sum, i.e. an allowed id with non-zero weight
              const float target = fminf(u_in * mass, __uint_as_float(__float_as_uint(mass) - 1u));
              int pick = 0;
#pragma unroll
              for (int j = 0; j < 32; ++j) pick += v[j] <= target ? 1 : 0;
              // ln(sum_j exp(logit_j / T)) - ln(-ln u): lg2 is one MUFU each
              const float key = fmaf(cmax, p.inv_temp, 0.69314718f * lg2_approx(mass)) -
                                0.69314718f * lg2_approx(-0.69314718f * lg2_approx(u_key));
              if (key > best) { best = key; best_idx = nc + pick; }
            }
            const float m_new = fmaxf(t_max, cmax);
            t_sum = t_sum * __expf(t_max - m_new) + s_all * __expf(cmax - m_new);
            t_max = m_new;
          } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + nc;
            const bool vec = (nc + 32 <= p.N) && (p.ldo % 8 == 0);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = (__expf(v[j] - lse) - ((nc + j) == label ? 1.f : 0.f)) * gs;
            if (vec) {
              store_bf16x32(o, v);
            } else {
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) o[j] = __float2bfloat16(v[j]);
            }
          }
        }
        if (kEpi == EPI_CE_FWD && row_ok && (n0 + half * (BN / kParts) < p.N)) {
          // partial results are kept per column share of a tile (64 columns): ceil(N / 64) entries per row
          static_assert(kEpi != EPI_CE_FWD || BN / kParts == 64, "db200_gemm_tile_n");
          const long long tn = (n0 / BN) * kParts + half;
          const long long plane = static_cast<long long>((p.N + BN / kParts - 1) / (BN / kParts)) * p.M;
          float* dst = p.ce_part + tn * p.M + row;
          dst[0] = t_max;
          dst[plane] = t_sum;
          dst[2 * plane] = best;
          dst[3 * plane] = __int_as_float(best_idx);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      } else if constexpr (kEpi == EPI_SWIGLU) {
        // accumulator columns [0, 128) = gate, [128, 256) = up of hidden columns j0 .. j0 + 127; a warp takes two
        // 32-column chunks of both halves
        const int j0 = n0 / 2;
        __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo;
        __nv_bfloat16* hrow = p.out2 + static_cast<long long>(row) * p.ldo2;
#pragma unroll 1
        for (int cc = half * 2; cc < half * 2 + 2; ++cc) {
          const int jc = j0 + cc * 32;
          if (jc >= p.half_n) continue;  // warp-uniform
          uint32_t rg[32], ru[32];
          tmem_ld_32x32b_x32(t_row + cc * 32, rg);
          tmem_ld_32x32b_x32(t_row + 128 + cc * 32, ru);
          tmem_ld_wait();
          if (!row_ok) continue;
          const bool full = jc + 32 <= p.half_n;
          float g[32], u[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            g[j] = __uint_as_float(rg[j]) * p.alpha;
            u[j] = __uint_as_float(ru[j]) * p.alpha;
          }
          if (bias) {
            for (int j = 0; j < 32; ++j) {
              if (jc + j < p.half_n) {
                g[j] += __bfloat162float(bias[jc + j]);
                u[j] += __bfloat162float(bias[p.half_n + jc + j]);
              }
            }
          }
          float hv[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {  // from the bf16-rounded halves, as a separate activation pass would see them
            const float gr = __bfloat162float(__float2bfloat16(g[j])), ur = __bfloat162float(__float2bfloat16(u[j]));
            float sig;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(sig) : "f"(1.0f + ex2_approx(gr * -1.4426950408889634f)));
            hv[j] = gr * sig * ur;
          }
          const bool vec = full && (p.ldo % 8 == 0) && (p.half_n % 8 == 0) && (p.ldo2 % 8 == 0);
          if (vec) {
            store_bf16x32(gu + jc, g);
            store_bf16x32(gu + p.half_n + jc, u);
            store_bf16x32(hrow + jc, hv);
          } else {
            for (int j = 0; j < 32; ++j) {
              if (jc + j < p.half_n) {
                gu[jc + j] = __float2bfloat16(g[j]);
                gu[p.half_n + jc + j] = __float2bfloat16(u[j]);
                hrow[jc + j] = __float2bfloat16(hv[j]);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }
      } else if constexpr (kEpi == EPI_SWIGLU_BWD) {
        const __nv_bfloat16* gu = p.aux + static_cast<long long>(row) * p.ldaux;
        __nv_bfloat16* dgu = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo;
#pragma unroll 1
        for (int c = half * kChunksPerHalf; c < (half + 1) * kChunksPerHalf; ++c) {
          const int nc = n0 + c * 32;
          if (nc >= p.N) continue;  // warp-uniform (N = F here)
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          const bool full = nc + 32 <= p.N;
          const bool vec = full && row_ok && (p.ldaux % 8 == 0) && (p.ldo % 8 == 0) && (p.half_n % 8 == 0);
          uint32_t gw[16], uw[16];
          if (vec) {
            load_bf16x32(gu + nc, gw);
            load_bf16x32(gu + p.half_n + nc, uw);
          }
          tmem_ld_wait();
          if (!row_ok) continue;
          float dg[32], du[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float gate, up;
            if (vec) {
              gate = (j & 1) ? bf16_hi(gw[j >> 1]) : bf16_lo(gw[j >> 1]);
              up = (j & 1) ? bf16_hi(uw[j >> 1]) : bf16_lo(uw[j >> 1]);
            } else {
              const bool in = nc + j < p.N;
              gate = in ? __bfloat162float(gu[nc + j]) : 0.f;
              up = in ? __bfloat162float(gu[p.half_n + nc + j]) : 0.f;
            }
            const float dh = __uint_as_float(r[j]) * p.alpha;
            float sig;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(sig) : "f"(1.0f + ex2_approx(gate * -1.4426950408889634f)));
            dg[j] = dh * up * sig * fmaf(gate, 1.0f - sig, 1.0f);
            du[j] = dh * gate * sig;
          }
          if (vec) {
            store_bf16x32(dgu + nc, dg);
            store_bf16x32(dgu + p.half_n + nc, du);
          } else {
            for (int j = 0; j < 32; ++j) {
              if (nc + j < p.N) {
                dgu[nc + j] = __float2bfloat16(dg[j]);
                dgu[p.half_n + nc + j] = __float2bfloat16(du[j]);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }
      } else {
#pragma unroll 1
      for (int cp = half * (kChunksPerHalf / 2); cp < (half + 1) * (kChunksPerHalf / 2); ++cp) {
      // GELU-derivative operand of both chunks of the group: one round trip instead of two
      uint32_t auxp[2][16];
      bool auxv[2] = {false, false};
      if (kAuxMul) {
#pragma unroll
        for (int csub = 0; csub < 2; ++csub) {
          const int nc = n0 + (cp * 2 + csub) * 32;
          auxv[csub] = row_ok && (nc + 32 <= p.N) && (p.ldaux % 8 == 0);
          if (auxv[csub]) load_bf16x32(p.aux + z * p.bs_aux + static_cast<long long>(row) * p.ldaux + nc, auxp[csub]);
        }
      }
#pragma unroll
      for (int csub = 0; csub < 2; ++csub) {
        const int c = cp * 2 + csub;
        const int nc = n0 + c * 32;
        if (nc >= p.N) continue;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        const bool full = (nc + 32 <= p.N);
        // row-indexed epilogue operands are requested before the accumulator wait so that both latencies overlap
        uint32_t resw[16];
        const uint32_t* auxw = auxp[csub];
        // (the two-output GELU forms take no residual: the launcher refuses it, and its 16 registers stay free)
        const bool res_vec = !kOutF32 && !kTwoOut && p.residual && row_ok && full && (p.ldr % 8 == 0);
        const bool aux_vec = auxv[csub];
        if (res_vec) load_bf16x32(p.residual + z * p.bs_res + static_cast<long long>(row) * p.ldr + nc, resw);
        tmem_ld_wait();
        if ((!row_ok && !p.tma_out) || empty_split) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (bias && split == 0) {
          if (full) {
            const uint4* bp = reinterpret_cast<const uint4*>(bias + nc);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 b = __ldg(bp + q);
              const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[q * 8 + e * 2] += bf16_lo(bw[e]);
                v[q * 8 + e * 2 + 1] += bf16_hi(bw[e]);
              }
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) v[j] += __bfloat162float(bias[nc + j]);
          }
        }
        if (kOutF32) {
          float* o = reinterpret_cast<float*>(p.out) + z * p.bs_out + static_cast<long long>(row) * p.ldo + nc;
          if (p.accumulate || p.splits > 1) {
            if (full && (p.ldo % 4 == 0)) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + q * 4), "f"(v[q * 4]),
                             "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                             : "memory");
            } else {
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) atomicAdd(o + j, v[j]);
            }
          } else {
            if (full && (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(o) & 31) == 0)) {
#pragma unroll
              for (int q = 0; q < 4; ++q) st_global_32B(o + q * 8, reinterpret_cast<const uint32_t*>(v) + q * 8);
            } else if (full && (p.ldo % 4 == 0)) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                reinterpret_cast<float4*>(o)[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) o[j] = v[j];
            }
          }
          continue;
        }
        // ---- bf16 outputs ----
        const bool vec = full && (p.ldo % 8 == 0);
        if (!kTwoOut && p.residual && row_ok) {
          if (res_vec) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              v[e * 2] += bf16_lo(resw[e]);
              v[e * 2 + 1] += bf16_hi(resw[e]);
            }
          } else {
            const __nv_bfloat16* rp = p.residual + z * p.bs_res + static_cast<long long>(row) * p.ldr + nc;
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) v[j] += __bfloat162float(rp[j]);
          }
        }
        if (kAuxMul && row_ok) {
          if (aux_vec) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              v[e * 2] *= kEpi == EPI_MUL ? bf16_lo(auxw[e]) : dgelu_erf(bf16_lo(auxw[e]));
              v[e * 2 + 1] *= kEpi == EPI_MUL ? bf16_hi(auxw[e]) : dgelu_erf(bf16_hi(auxw[e]));
            }
          } else {
            const __nv_bfloat16* ap = p.aux + z * p.bs_aux + static_cast<long long>(row) * p.ldaux + nc;
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) v[j] *= kEpi == EPI_MUL ? __bfloat162float(ap[j]) : dgelu_erf(__bfloat162float(ap[j]));
          }
        }
        if (p.tma_out) {
          // (reached by every lane of the warp: rows >= M compute on zeros and are clipped by the store)
          const int sub = csub;
          const bool last_of_group = sub == 1 || nc + 32 >= p.N;
          uint32_t wds[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) wds[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
          if (kTwoOut) {
            // two outputs, one staging tile: the first leaves with direct 32-byte row stores, gelu(z) through
            // the staging tile (waiting for a bulk store to release the tile twice per group would stall the warp)
            uint32_t act[16];
            if (kEpi == EPI_GELU_GRAD) {
              // first output = gelu'(z), second = gelu(z), both of the bf16-rounded pre-activation, from one cdf/pdf pair
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float z0 = bf16_lo(wds[i]), z1 = bf16_hi(wds[i]);
                float c0, d0, c1, d1;
                normal_cdf_pdf(z0, c0, d0);
                normal_cdf_pdf(z1, c1, d1);
                act[i] = pack_bf16(z0 * c0, z1 * c1);
                wds[i] = pack_bf16(fmaf(z0, d0, c0), fmaf(z1, d1, c1));
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) act[i] = pack_bf16(gelu_erf(bf16_lo(wds[i])), gelu_erf(bf16_hi(wds[i])));
            }
            if (row_ok && full) {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + z * p.bs_out + static_cast<long long>(row) * p.ldo + nc;
              store_words16(o, wds);
            } else if (row_ok) {  // ragged last chunk: element by element, from the packed words (v is dead by now)
              unsigned short* o = reinterpret_cast<unsigned short*>(p.out) + z * p.bs_out + static_cast<long long>(row) * p.ldo + nc;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) o[j] = static_cast<unsigned short>((j & 1) ? (wds[j >> 1] >> 16) : (wds[j >> 1] & 0xffffu));
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) wds[i] = act[i];
          }
          if (sub == 0) stage_acquire();
          stage_words(wds, sub);
          if (last_of_group) stage_flush(kTwoOut ? &tmap_out2 : &tmap_out, nc - sub * 32, m0 + quad * 32, z);
          continue;
        }
        __nv_bfloat16* o =
            reinterpret_cast<__nv_bfloat16*>(p.out) + z * p.bs_out + static_cast<long long>(row) * p.ldo + nc;
        float act2[kTwoOut ? 32 : 1];
        if (kTwoOut) {  // gelu (and for EPI_GELU_GRAD the derivative, which replaces the first output) of the rounded value
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float zr = __bfloat162float(__float2bfloat16(v[j]));
            float c, d;
            normal_cdf_pdf(zr, c, d);
            act2[j] = zr * c;
            if (kEpi == EPI_GELU_GRAD) v[j] = fmaf(zr, d, c);
          }
        }
        if (vec) {
          store_bf16x32(o, v);
        } else {
          for (int j = 0; j < 32; ++j)
            if (nc + j < p.N) o[j] = __float2bfloat16(v[j]);
        }
        if (kTwoOut) {
          __nv_bfloat16* o2 = p.out2 + z * p.bs_out2 + static_cast<long long>(row) * p.ldo2 + nc;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = act2[j];
          if (full && (p.ldo2 % 8 == 0)) {
            store_bf16x32(o2, v);
          } else {
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) o2[j] = __float2bfloat16(v[j]);
          }
        }
      }
      }
      if constexpr (kRowSum) {
        if (want_sum && n0 == 0 && half == 0 && z == 0) {  // warp-uniform
          uint32_t sum_bits;
          asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];"
                       : "=r"(sum_bits)
                       : "r"(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kSumCol + acc * 16));
          tmem_ld_wait();
          if (row_ok && !empty_split) atomicAdd(p.a_sum + row, __uint_as_float(sum_bits));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }
      }  // regular (non-CE) epilogue
    }
    if (lane == 0) tma_store_wait_all();  // shared memory must outlive the bulk stores that read it
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

constexpr int kMaxDevices = 16;
int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}
int g_num_sms[kMaxDevices] = {};
int num_sms() {  // per device: a process may drive more than one GPU
  const int dev = current_device();
  if (g_num_sms[dev] == 0) {
    cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms[dev] <= 0) g_num_sms[dev] = 148;
  }
  return g_num_sms[dev];
}

template <int BN, bool A_MN, bool B_MN, int MODE>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& to2, const DevParams& p,
           int grid, cudaStream_t stream) {
  using L = SmemLayout<BN, MODE>;
  constexpr int kThreads = gemm_threads<BN, MODE>();
  static bool configured[kMaxDevices] = {};  // the shared-memory opt-in is a per-device attribute of the function
  auto kern = gemm_kernel<BN, A_MN, B_MN, MODE>;
  const int dev = current_device();
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return -3;
    configured[dev] = true;
  }
  return launch_pdl(kern, dim3(grid), dim3(kThreads), L::kTotal, stream, ta, tb, to, to2, p) == cudaSuccess ? 0 : -4;
}

}  // namespace

// Build a 3-D bf16 tensor map {inner, rows, batch} with a {64, box_rows, 1} box and 128B swizzle.
//
// Encoding a map costs a driver call of a microsecond or two, and a training step asks for several thousand maps over
// the same few hundred (pointer, shape, stride) combinations: parameters sit in the engine's flat buffers and the
// caching allocator hands activations the same addresses step after step. A map is a pure function of its
// description, so descriptions are looked up in a small direct-mapped, per-thread table first.
namespace {
struct TmapKey {
  const void* ptr;
  long long inner, rows, batch, row_stride, batch_stride;
  int box_rows;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && inner == o.inner && rows == o.rows && batch == o.batch && row_stride == o.row_stride &&
           batch_stride == o.batch_stride && box_rows == o.box_rows;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapSlots = 4096;
inline size_t tmap_hash(const TmapKey& k) {
  unsigned long long h = reinterpret_cast<unsigned long long>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<unsigned long long>(k.inner) * 0xC2B2AE3D27D4EB4Full + static_cast<unsigned long long>(k.rows) * 0x165667B19E3779F9ull;
  h ^= static_cast<unsigned long long>(k.row_stride) * 0x85EBCA77C2B2AE63ull + static_cast<unsigned long long>(k.batch) * 0x27D4EB2F165667C5ull;
  h ^= static_cast<unsigned long long>(k.batch_stride) * 0xD6E8FEB86659FD93ull + static_cast<unsigned long long>(k.box_rows);
  return static_cast<size_t>((h ^ (h >> 29)) % kTmapSlots);
}
}  // namespace

int db200_make_tmap_bf16(CUtensorMap* out, const void* ptr, long long inner, long long rows, long long batch,
                         long long row_stride_elems, long long batch_stride_elems, int box_rows) {
  static thread_local TmapSlot* table = nullptr;
  if (!table) table = new TmapSlot[kTmapSlots]();
  const TmapKey key{ptr, inner, rows, batch, row_stride_elems, batch_stride_elems, box_rows};
  TmapSlot& slot = table[tmap_hash(key)];
  if (slot.used && slot.key == key) {
    *out = slot.map;
    return 0;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride_elems) * 2,
                           static_cast<cuuint64_t>(batch > 1 ? batch_stride_elems : row_stride_elems * rows) * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -2;
  slot.key = key;
  slot.map = *out;
  slot.used = true;
  return 0;
}

// Width of the column range one partial result of EPI_CE_FWD covers: the share of a tile that one set of four
// epilogue warps reduces (a quarter of the 256-column tile, half of the 128-column one).
extern "C" int db200_gemm_tile_n(int N) { (void)N; return 64; }

// Combine the per-vocabulary-tile partials of EPI_CE_FWD: per row log-sum-exp (natural log),
// cross-entropy against the label logit, and the candidate id with the largest sampling key (the sample).
// block (32 rows, 16 tile slices): every thread folds the tiles t = slice, slice + 16, ... of its row, the slices are
// then combined through shared memory (online log-sum-exp, arg-max of the sampling keys).
__global__ void __launch_bounds__(512)
ce_combine_kernel(const float* __restrict__ part, const float* __restrict__ label_logit, int tiles_n, int M,
                  float* __restrict__ lse_out, float* __restrict__ loss_rows, long long* __restrict__ sampled) {
  constexpr int kSlices = 16;
  __shared__ float s_m[kSlices][33], s_s[kSlices][33], s_b[kSlices][33];
  __shared__ int s_i[kSlices][33];
  const int rl = threadIdx.x, slice = threadIdx.y;
  const int row = blockIdx.x * 32 + rl;
  const long long plane = static_cast<long long>(tiles_n) * M;
  float m = -INFINITY, sum = 0.f, best = -INFINITY;
  int idx = 0;
  if (row < M) {
    for (int t = slice; t < tiles_n; t += kSlices) {
      const long long o = static_cast<long long>(t) * M + row;
      const float tm = part[o], ts = part[plane + o], tb = part[2 * plane + o];
      const float nm = fmaxf(m, tm);
      if (nm > -INFINITY) sum = sum * __expf(m - nm) + ts * __expf(tm - nm);
      m = nm;
      if (tb > best) { best = tb; idx = __float_as_int(part[3 * plane + o]); }
    }
  }
  s_m[slice][rl] = m; s_s[slice][rl] = sum; s_b[slice][rl] = best; s_i[slice][rl] = idx;
  __syncthreads();
  if (slice == 0 && row < M) {
    // slices are folded in a fixed order; ties of the largest key go to the lowest tile index seen first
    for (int k = 1; k < kSlices; ++k) {
      const float tm = s_m[k][rl], ts = s_s[k][rl];
      const float nm = fmaxf(m, tm);
      if (nm > -INFINITY) sum = sum * __expf(m - nm) + ts * __expf(tm - nm);
      m = nm;
      if (s_b[k][rl] > best) { best = s_b[k][rl]; idx = s_i[k][rl]; }
    }
    const float lse = m + logf(sum);
    lse_out[row] = lse;
    loss_rows[row] = lse - label_logit[row];
    sampled[row] = idx;
  }
}

// Load the code of the cross-entropy forward path (both tile widths and the combine kernel) on the current device
// without launching anything: under CUDA's lazy module loading a kernel's code reaches the device on first use, and
// that is a device-memory request made by the driver. Callers that must not cause one later call this at start-up.
extern "C" int db200_gemm_preload_ce(void) {
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, gemm_kernel<256, false, false, 4>) != cudaSuccess) return -3;
  if (cudaFuncGetAttributes(&attr, gemm_kernel<128, false, false, 4>) != cudaSuccess) return -3;
  if (cudaFuncGetAttributes(&attr, ce_combine_kernel) != cudaSuccess) return -3;
  (void)num_sms();
  return get_encode_fn() ? 0 : -1;
}

extern "C" int db200_ce_combine(const float* part, const float* label_logit, int tiles_n, int M, float* lse,
                                float* loss_rows, long long* sampled, void* stream) {
  if (M <= 0) return 0;
  ce_combine_kernel<<<(M + 31) / 32, dim3(32, 16), 0, reinterpret_cast<cudaStream_t>(stream)>>>(part, label_logit, tiles_n, M,
                                                                                            lse, loss_rows, sampled);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int db200_gemm_bf16(const GemmArgs* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0) return 0;
  // TMA needs 16-byte aligned bases and strides.
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) || (a->lda % 8) ||
      (a->ldb % 8) || (a->bs_a % 8) || (a->bs_b % 8))
    return -10;
  const int BN = (a->N > 128) ? 256 : 128;
  DevParams p{};
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.tiles_m = (a->M + BM - 1) / BM;
  p.tiles_n = (a->N + BN - 1) / BN;
  p.batch = a->batch;
  p.kb_total = (a->K + BK - 1) / BK;
  p.alpha = a->alpha;
  p.epi = a->epi;
  p.out_f32 = a->out_f32;
  p.accumulate = a->accumulate;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.aux = reinterpret_cast<const __nv_bfloat16*>(a->aux);
  p.out = a->out;
  p.out2 = reinterpret_cast<__nv_bfloat16*>(a->out2);
  p.ldo = a->ldo; p.ldr = a->ldr; p.ldaux = a->ldaux; p.ldo2 = a->ldo2;
  p.bs_out = a->bs_out; p.bs_res = a->bs_res; p.bs_aux = a->bs_aux; p.bs_out2 = a->bs_out2; p.bs_bias = a->bs_bias;
  p.status = db200_status_ptr();
  p.labels = reinterpret_cast<const long long*>(a->labels);
  p.forbidden = reinterpret_cast<const unsigned char*>(a->forbidden);
  p.inv_temp = a->inv_temp;
  p.seed = a->seed;
  p.ce_part = a->ce_part;
  p.label_logit = a->label_logit;
  p.row_lse = a->row_lse;
  p.gscale = a->gscale;
  p.gscale_ptr = a->gscale_ptr;
  p.a_sum = a->a_sum;
  if (p.a_sum && (!a->out_f32 || !a->a_mn || a->batch != 1)) return -11;
  if ((p.epi == EPI_CE_FWD) && (!p.labels || !p.ce_part || !p.label_logit || a->batch != 1)) return -11;
  if ((p.epi == EPI_CE_BWD) && (!p.labels || !p.row_lse || p.out_f32 || a->batch != 1)) return -11;
  const bool two_out = p.epi == EPI_GELU || p.epi == EPI_GELU_GRAD;
  if (two_out && (p.out_f32 || !p.out2 || a->residual)) return -11;
  if ((p.epi == EPI_DGELU || p.epi == EPI_MUL) && (p.out_f32 || !p.aux)) return -11;
  if (p.epi == EPI_SWIGLU && (p.out_f32 || !p.out2 || a->batch != 1 || (a->N % 2) || a->a_mn || a->b_mn || a->N <= 128 ||
                              a->residual))
    return -11;
  if (p.epi == EPI_SWIGLU_BWD && (p.out_f32 || !p.aux || a->batch != 1 || a->a_mn || !a->b_mn || a->residual)) return -11;
  p.half_n = p.epi == EPI_SWIGLU ? a->N / 2 : (p.epi == EPI_SWIGLU_BWD ? a->N : 0);
  if (p.epi == EPI_SWIGLU) p.tiles_n = (p.half_n + 127) / 128;  // a tile = 128 gate columns + their 128 up columns

  const int tiles = p.tiles_m * p.tiles_n * p.batch;
  int splits = 1;
  if (a->out_f32 && a->allow_split_k && a->residual == nullptr) {
    // Fill the machine when the output grid is small (weight gradients: K = tokens). Cost of a split count s in
    // k-block units: waves of work items x (k-blocks per item + a fixed epilogue share, an fp32 tile of reductions).
    const int sms = num_sms();
    constexpr int kEpilogueCost = 6;
    long long best_cost = -1;
    for (int s = 1; s <= 16; s *= 2) {
      if (s > 1 && p.kb_total / s < 4) break;
      const long long waves = (static_cast<long long>(tiles) * s + sms - 1) / sms;
      const long long cost = waves * ((p.kb_total + s - 1) / s + kEpilogueCost);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; splits = s; }
    }
  }
  p.splits = splits;
  if (splits > 1 && !p.accumulate) {
    // partial sums are combined with red.add, so the destination has to start at zero
    for (int z = 0; z < a->batch; ++z) {
      if (cudaMemset2DAsync(reinterpret_cast<float*>(a->out) + z * a->bs_out, a->ldo * sizeof(float), 0,
                            static_cast<size_t>(a->N) * sizeof(float), a->M, stream) != cudaSuccess)
        return -5;
    }
  }

  CUtensorMap ta, tb;
  int rc;
  if (!a->a_mn) rc = db200_make_tmap_bf16(&ta, a->A, a->K, a->M, a->batch, a->lda, a->bs_a, BM);
  else          rc = db200_make_tmap_bf16(&ta, a->A, a->M, a->K, a->batch, a->lda, a->bs_a, BK);
  if (rc) return rc;
  if (!a->b_mn) rc = db200_make_tmap_bf16(&tb, a->B, a->K, a->N, a->batch, a->ldb, a->bs_b, 128);
  else          rc = db200_make_tmap_bf16(&tb, a->B, a->N, a->K, a->batch, a->ldb, a->bs_b, BK);
  if (rc) return rc;

  // bf16 outputs go through shared memory + TMA stores when their layout allows a tensor map
  CUtensorMap to = ta, to2 = ta;  // placeholders when unused (never dereferenced by the kernel)
  auto tma_ok = [&](const void* ptr, long long ld, long long bs) {
    return ptr && !(reinterpret_cast<uintptr_t>(ptr) & 15) && (ld % 8 == 0) && (a->batch == 1 || bs % 8 == 0);
  };
  p.tma_out = 0;
  if (!p.out_f32 && splits == 1 && p.epi != EPI_CE_FWD && p.epi != EPI_CE_BWD && p.epi != EPI_SWIGLU &&
      p.epi != EPI_SWIGLU_BWD && tma_ok(a->out, a->ldo, a->bs_out) &&
      (!two_out || tma_ok(a->out2, a->ldo2, a->bs_out2))) {
    if (db200_make_tmap_bf16(&to, a->out, a->N, a->M, a->batch, a->ldo, a->bs_out, 32) == 0 &&
        (!two_out || db200_make_tmap_bf16(&to2, a->out2, a->N, a->M, a->batch, a->ldo2, a->bs_out2, 32) == 0))
      p.tma_out = 1;
  }

  const int grid = min(tiles * splits, num_sms());
  const int mode = p.out_f32 ? 3 : p.epi == EPI_GELU ? 1 : p.epi == EPI_DGELU ? 2 : p.epi == EPI_CE_FWD ? 4
                   : p.epi == EPI_CE_BWD ? 5 : p.epi == EPI_GELU_GRAD ? 6 : p.epi == EPI_MUL ? 7 : 0;
  if (p.epi == EPI_SWIGLU) return launch<256, false, false, 8>(ta, tb, to, to2, p, grid, stream);
  if (p.epi == EPI_SWIGLU_BWD)
    return BN == 256 ? launch<256, false, true, 9>(ta, tb, to, to2, p, grid, stream)
                     : launch<128, false, true, 9>(ta, tb, to, to2, p, grid, stream);
#define DISPATCH_MODE(BN_, AM_, BM_)                                                         \
  switch (mode) {                                                                            \
    case 0: return launch<BN_, AM_, BM_, 0>(ta, tb, to, to2, p, grid, stream);               \
    case 1: return launch<BN_, AM_, BM_, 1>(ta, tb, to, to2, p, grid, stream);               \
    case 2: return launch<BN_, AM_, BM_, 2>(ta, tb, to, to2, p, grid, stream);               \
    case 3: return launch<BN_, AM_, BM_, 3>(ta, tb, to, to2, p, grid, stream);               \
    case 4: return launch<BN_, AM_, BM_, 4>(ta, tb, to, to2, p, grid, stream);               \
    case 5: return launch<BN_, AM_, BM_, 5>(ta, tb, to, to2, p, grid, stream);               \
    case 6: return launch<BN_, AM_, BM_, 6>(ta, tb, to, to2, p, grid, stream);               \
    default: return launch<BN_, AM_, BM_, 7>(ta, tb, to, to2, p, grid, stream);              \
  }
#define DISPATCH(BN_, AM_, BM_) DISPATCH_MODE(BN_, AM_, BM_)
  if (BN == 256) {
    if (!a->a_mn && !a->b_mn) { DISPATCH(256, false, false); }
    if (!a->a_mn && a->b_mn) { DISPATCH(256, false, true); }
    if (a->a_mn && !a->b_mn) { DISPATCH(256, true, false); }
    DISPATCH(256, true, true);
  } else {
    if (!a->a_mn && !a->b_mn) { DISPATCH(128, false, false); }
    if (!a->a_mn && a->b_mn) { DISPATCH(128, false, true); }
    if (a->a_mn && !a->b_mn) { DISPATCH(128, true, false); }
    DISPATCH(128, true, true);
  }
#undef DISPATCH
#undef DISPATCH_MODE
}
