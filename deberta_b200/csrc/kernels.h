// C ABI of the sm_100a kernel library. Every launcher takes raw device pointers and a
// CUDA stream handle and returns 0 on success or a negative code when the arguments
// are rejected before any launch. The Python bindings mirror these structs with ctypes.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ----- status word written by kernels whose bounded waits ran out -------------------
int* db200_status_ptr(void);          // device address of the status word (lazily allocated)
int db200_status_read_and_clear(void);  // synchronises the device; 0 = no error recorded
int db200_status_snapshot(int* dst, void* stream);
// Programmatic dependent launch (overlap of a kernel's set-up with its predecessor's tail) for the kernels that support it.
int db200_pdl_enabled(void);
int db200_set_pdl(int on);  // returns the previous setting  // stream-ordered copy of the word into device / pinned memory

// ----- GEMM ---------------------------------------------------------------------------
enum { EPI_NONE = 0, EPI_GELU = 1, EPI_DGELU = 2, EPI_CE_FWD = 3, EPI_CE_BWD = 4,
       EPI_GELU_GRAD = 5,  // out = gelu'(z), out2 = gelu(z): the backward pass then needs no transcendental
       EPI_MUL = 6,        // out = acc * aux (aux = the gelu'(z) written by EPI_GELU_GRAD)
       // SwiGLU inside the GEMMs around it. B = W12 [2F, K] (gate rows, then up rows), N = 2F:
       // out [M, 2F] = [gate | up] (kept for the backward pass), out2 [M, F] = silu(gate) * up.
       EPI_SWIGLU = 7,
       // its backward: A·B = dh [M, F] (N = F), aux = [gate | up] [M, 2F]; out [M, 2F] = [dh*up*silu'(gate) | dh*silu(gate)]
       EPI_SWIGLU_BWD = 8 };

typedef struct GemmArgs {
  const void* A;     // bf16
  const void* B;     // bf16
  void* out;         // bf16 or fp32 (out_f32)
  void* out2;        // bf16, EPI_GELU / EPI_GELU_GRAD: gelu of the pre-activation
  const void* bias;  // bf16 [N] or null
  const void* residual;  // bf16 [M, N] or null (added before the activation derivative)
  const void* aux;       // bf16 [M, N]: pre-activation for EPI_DGELU, factor for EPI_MUL
  int M, N, K, batch;
  int a_mn, b_mn;    // operand majors, see gemm.cu
  int epi, out_f32, accumulate, allow_split_k;
  float alpha;
  long long lda, ldb, ldo, ldo2, ldr, ldaux;                       // leading dims (elements)
  long long bs_a, bs_b, bs_out, bs_out2, bs_res, bs_aux, bs_bias;  // batch strides (elements)
  // vocabulary cross-entropy epilogues: A = hidden rows [M,K], B = embedding table [N,K], bias [N]
  const void* labels;        // int64 [M]
  const void* forbidden;     // uint8 [N] or null
  float inv_temp;
  unsigned long long seed;
  float* ce_part;            // fp32 [4, ceil(N / db200_gemm_tile_n(N)), M] scratch (EPI_CE_FWD)
  float* label_logit;        // fp32 [M]                       (EPI_CE_FWD)
  const float* row_lse;      // fp32 [M]                       (EPI_CE_BWD)
  float gscale;              // scale of the logit gradient     (EPI_CE_BWD)
  const float* gscale_ptr;   // optional device scalar multiplied into gscale
  float* a_sum;              // fp32 [M] or null: a_sum[m] += sum_k A[m,k] (needs out_f32, a_mn, batch 1); alpha is not applied
} GemmArgs;

int db200_gemm_bf16(const GemmArgs* args, void* stream);
int db200_gemm_preload_ce(void);  // loads the EPI_CE_FWD kernels and db200_ce_combine's kernel on the current device, launches nothing
int db200_gemm_tile_n(int N);  // width of the vocabulary range one EPI_CE_FWD partial covers
int db200_ce_combine(const float* part, const float* label_logit, int tiles_n, int M, float* lse, float* loss_rows,
                     long long* sampled, void* stream);

// ----- LayerNorm / RMSNorm (bf16 in/out, fp32 stats; row_keep: optional uint8 per-row multiplier) -----
int db200_norm_fwd(const void* x, const void* gamma, const void* beta, const void* row_keep, void* y, float* mean,
                   float* rstd, int rows, int H, float eps, int rms, void* stream);
int db200_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                   const void* row_keep, void* dx, float* dgamma, float* dbeta, int rows, int H, int rms,
                   void* stream);

// ----- reductions ----------------------------------------------------------------------------
// out_accum[n] += sum_m x[m, n]   (x bf16 [M, N] with leading dim ld, out fp32 [N])
int db200_colsum_bf16(const void* x, long long ld, int M, int N, float* out_accum, void* stream);

// ----- optimizer (flat fp32 ranges) ---------------------------------------------------------
int db200_sumsq(const float* g, long long n, float* out_accum, void* stream);
// gate (may be null): device float; the update is skipped when it is not > 0 (decided without a host round trip).
int db200_adamw(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr, float wd,
                float b1, float b2, float eps, float inv_bc1, float inv_sqrt_bc2, const float* norm_sq,
                float max_norm, float grad_scale, const float* gate, void* stream);

// ----- elementwise kernels of the RoPE backbone (see elementwise.cu) ---------------------------
// Interleaved-pair rotary embedding of the first rotary_dim features of every head: y = rot(x) (inverse != 0: the
// transposed rotation, i.e. the backward pass). x, y: bf16 [tokens, ld*] with heads*head_dim features; cos/sin: fp32
// [S, rotary_dim] with each frequency stored twice; token t sits at position t % S. x == y is allowed.
int db200_rotary_bf16(const void* x, void* y, long long ldx, long long ldy, const float* cos_t, const float* sin_t,
                      long long tokens, int S, int heads, int head_dim, int rotary_dim, int inverse, void* stream);
// out[r, c] = silu(gate_up[r, c]) * gate_up[r, F + c]  and its backward (d_gate_up has the layout of gate_up).
// y[r, 0:cols] = bf16(x[r, 0:cols]); x dense fp32 [rows, cols], y bf16 with row stride ld_y (cols, ld_y multiples of 8).
int db200_cast_f32_bf16(const float* x, void* y, long long ld_y, long long rows, int cols, void* stream);
int db200_swiglu_fwd(const void* gate_up, long long ld_in, void* out, long long ld_out, long long rows, int F, void* stream);
int db200_swiglu_bwd(const void* gate_up, long long ld_in, const void* dout, long long ld_do, void* d_gate_up,
                     long long ld_dg, long long rows, int F, void* stream);

// Embedding lookup out[t] = table[ids[t]] (+ delta[ids[t]]) over bf16 tables [vocab, H], and the fp32 gradient
// scatter grad[ids[t]] += dout[t] (tokens with ids[t] == padding_idx skipped; pass -1 for none).
int db200_embed_fwd(const long long* ids, const void* table, const void* delta, void* out, long long tokens, int H,
                    long long vocab, void* stream);
int db200_embed_bwd(const long long* ids, const void* dout, long long ld_do, float* grad, long long tokens, int H,
                    long long vocab, long long padding_idx, void* stream);

// Masked-row gather out[n] = x[idx[n]] over bf16 rows of `cols` features (idx: distinct int64 rows of x); `inv`
// (int32 [m_rows], may be null) receives the inverse map (-1 = row not selected). Its gradient writes every row of dx:
// dx[m] = dout[inv[m]] or 0, so dx needs no clearing.
int db200_rows_gather(const void* x, long long ld_x, const long long* idx, void* out, int* inv, long long m_rows,
                      long long n_rows, int cols, void* stream);
int db200_rows_scatter(const void* dout, long long ld_do, const int* inv, void* dx, long long m_rows, int cols, void* stream);

// Tail of the replaced-token-detection head. Forward: logit[t] = a[t,:].w + bias (rounded to bf16), and
// stats[0..3] += {BCE-with-logits summed over active tokens, correct predictions, active tokens, positive labels}.
// Backward: d_pre[t,:] = dz[t] * w * gelu'(pre[t,:]) (pre null: no activation derivative), dw += sum dz * a[t,:],
// db += sum dz, with dz = (sigmoid(logit) - label) * active * grad[0] / max(stats[2], 1). H <= 1024, H % 8 == 0.
int db200_rtd_tail_fwd(const void* a, long long lda, const void* w, const void* bias, const long long* labels,
                       const unsigned char* active, float* logits, float* stats, long long tokens, int H, void* stream);
int db200_rtd_tail_bwd(const void* a, long long lda, const void* pre, long long ldp, const void* w, const float* logits,
                       const long long* labels, const unsigned char* active, const float* grad, const float* stats,
                       void* d_pre, long long ldd, float* dw, float* db, long long tokens, int H, void* stream);

// ----- fused gradient collectives over NVLink peer memory (see comm.cu) -----------------------
#define DB200_COMM_MAX_WORLD 8
#define DB200_COMM_VEC_MAX 128      // longest vector db200_comm_vector_sum takes
#define DB200_COMM_PAD_WORDS 2048   // 32-bit words of the symmetric flag pad every rank allocates (zeroed once)
typedef struct Db200CommCtx {
  int world, rank;
  void* grads[DB200_COMM_MAX_WORLD];   // every rank's fp32 gradient buffer as mapped into this process
  void* params[DB200_COMM_MAX_WORLD];  // every rank's bf16 parameter buffer (only db200_comm_adamw needs it)
  void* pads[DB200_COMM_MAX_WORLD];    // every rank's flag pad
  void* mc_grads;                      // multicast address covering all gradient buffers, or null: plain peer loads/stores
  void* mc_params;                     // the same for the parameter buffers
  unsigned long long timeout_ns;       // longest wait for a peer flag; 0 = 20 s
} Db200CommCtx;
typedef struct Db200AdamSegment {
  long long begin, end;  // element range inside the slab (multiples of 8)
  float lr, weight_decay;
} Db200AdamSegment;
// Sum `count` gradients at `offset` (this rank's slab) over all ranks, times `scale`. to_all = 0: result in this
// rank's buffer only, squared-norm share published to the peers (db200_comm_adamw picks it up). to_all = 1: result
// in every rank's buffer, *norm_sq_out = squared norm over all slabs once all ranks are through. *extra_share (may
// be null) is added to this rank's share of the squared norm (an infinity there makes every rank skip the update).
int db200_comm_reduce(const Db200CommCtx* ctx, long long offset, long long count, float scale, int to_all,
                      unsigned epoch, const float* extra_share, float* norm_sq_out, void* stream);
// AdamW on this rank's slab after db200_comm_reduce(to_all = 0) with the same epoch; bf16 parameters go to all ranks.
int db200_comm_adamw(const Db200CommCtx* ctx, long long offset, long long count, float* master, float* exp_avg,
                     float* exp_avg_sq, const Db200AdamSegment* segs, int nseg, float b1, float b2, float eps,
                     float inv_bc1, float inv_sqrt_bc2, float max_norm, unsigned epoch, float* norm_sq_out,
                     const float* gate, void* local_params, void* stream);
// local_params (may be null): bf16 buffer of `count` elements that receives the updated slab INSTEAD of the push into
// every rank's parameter buffer (parameters stay sharded; peers fetch what they need with db200_comm_copy_pieces).
// Copy `count` (<= 16) byte ranges, each possibly read from a peer GPU's memory, into local memory; sizes and
// addresses are multiples of 16 bytes.
int db200_comm_copy_pieces(const void* const* src, void* const* dst, const long long* bytes, int count, void* stream);
// out[i] = sum over ranks of in[i], i < n <= DB200_COMM_VEC_MAX (in/out: this rank's own device memory).
int db200_comm_vector_sum(const Db200CommCtx* ctx, const float* in, float* out, int n, unsigned epoch, void* stream);

// ----- attention (head dim 64; token-major bf16 operands; see attention.cu) -------------------------
typedef struct AttnArgs {
  const void *q, *k, *v;          // bf16 [B*S, ld*]
  long long ldq, ldk, ldv;
  void* out;                      // bf16 [B*S, ldo]           (forward)
  long long ldo;
  float* lse;                     // fp32 [B, heads, S], log2 domain
  int B, S, heads, span2;         // span2 = rows of the position score tables, 0 = none
  float scale;                    // scores are divided by this
  const void *c2p, *p2c;          // bf16 [B*S, heads, span2] or null
  const void *lut_c2p, *lut_p2c;  // uint16 [2S-1]
  const void* key_keep;           // uint8 [B*S] or null
  const void* doc_ids;            // int32 [B*S] or null
  const void* dout;               // bf16 [B*S, ld_do]         (backward)
  long long ld_do;
  const float* delta;             // fp32 [B, heads, S]
  float* dq_acc;                  // fp32 [B*S, heads*64], zeroed by the caller
  void *dk, *dv;                  // bf16 [B*S, ld_dk / ld_dv]
  long long ld_dk, ld_dv;
  float *d_c2p, *d_p2c;           // fp32 [B*S, heads, span2], zeroed by the caller, or null
  const void* bias;               // bf16 [B, heads, S, ldb] pre-gathered position bias (then span2 = 0), or null
  void* dbias;                    // bf16 [B, heads, S, ldb] its gradient (backward)
  long long ldb;                  // multiple of 128
  const void* doc_tiles;          // int32 [B, ceil(S/128), 2] from db200_attn_doc_tiles, or null: with it the kernels
                                  // skip the tiles no document of theirs reaches (bias gradient must then be zeroed)
} AttnArgs;

// key-indexed position bias: build from / scatter back to the bucket-indexed score tables (posbias.cu)
int db200_posbias_build(const void* c2p, const void* p2c, const void* lut_c2p, const void* lut_p2c, void* bias, int B,
                        int S, int ldb, int heads, int span2, void* stream);
int db200_posbias_scatter(const void* dbias, const void* lut, void* dtab, int rows_are_keys, int B, int S, int ldb,
                          int heads, int span2, void* stream);
// The same reduction for bucket maps that are monotone in q-k, by differences of prefix sums instead of atomics.
// ranges: int[span2 + 2] = {sign, E_0 .. E_span2}: with sign = +1 bucket j collects E_j <= q-k < E_{j+1}, with
// sign = -1 it collects E_{j+1} <= q-k < E_j; unused buckets have E_j = E_{j+1}. span2 must be a multiple of 8.
int db200_posbias_scatter_ranges(const void* dbias, const void* ranges, void* dtab, int rows_are_keys, int B, int S,
                                 int ldb, int heads, int span2, void* stream);

// Position terms on the tensor cores (posbias_tc.cu): the [q, k] bias and the gradients it induces, computed from
// Q, K and the projected position tables directly; the bucket-indexed score tables never exist in global memory.
typedef struct PosBiasArgs {
  const void *q, *k;                        // bf16 [B*S, ld*], a head is a 64-column slice
  long long ldq, ldk;
  const void *pos_k, *pos_q;                // bf16 [span2, ld_pos] projected position tables (either may be null)
  long long ld_pos;
  const void *lut_c2p, *lut_p2c;            // device uint16 [2S-1]: table row of offset q-k (index q-k+S-1)
  const void *lut_c2p_host, *lut_p2c_host;  // the same tables in host memory (window planning)
  int B, S, heads, span2;
  void* bias;                               // bf16 [B, heads, S, ldb]: written by the forward
  long long ldb;                            // multiple of 128, >= S rounded up to 128
  const void* dbias;                        // bf16 [B, heads, S, ldb]: gradient of the bias (backward input)
  float* dq_acc;                            // fp32 [B*S, heads*64]: the c2p part of dQ is added here
  void* dk;                                 // bf16 [B*S, ld_dk]: the p2c part of dK is added here (read-modify-write)
  long long ld_dk;
  float *d_pos_k, *d_pos_q;                 // fp32 [span2, heads*64]: gradients of the tables are added here
} PosBiasArgs;
// -13: some tile needs more than 256 consecutive table rows (or, backward, span2 > 512): use the table path instead.
int db200_posbias_tc_fwd(const PosBiasArgs* args, void* stream);
int db200_posbias_tc_bwd(const PosBiasArgs* args, void* stream);

int db200_attn_fwd(const AttnArgs* args, void* stream);
int db200_attn_bwd(const AttnArgs* args, void* stream);
// delta[b,h,s] = sum over the head dim of dO * O (fp32 [B, heads, S]); input of db200_attn_bwd. `zero_f32` (may be
// null): a dense fp32 [B*S, heads*64] buffer that the same launch clears (the dQ accumulator of db200_attn_bwd).
int db200_attn_delta(const void* dout, long long ld_do, const void* out, long long ldo, float* delta, float* zero_f32,
                     int B, int S, int heads, void* stream);
// tiles[b, t] = (smallest, largest) non-zero document id of tokens [128 t, 128 t + 128) of row b (int32 [B, tiles, 2]).
int db200_attn_doc_tiles(const void* doc_ids, void* tiles, int B, int S, void* stream);

#ifdef __cplusplus
}
// internal: 3-D bf16 tensor map {inner, rows, batch}, box {64, box_rows, 1}, 128B swizzle
#include <cuda.h>
int db200_make_tmap_bf16(CUtensorMap* out, const void* ptr, long long inner, long long rows, long long batch,
                         long long row_stride_elems, long long batch_stride_elems, int box_rows);
#endif
