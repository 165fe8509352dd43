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

// ----- GEMM ---------------------------------------------------------------------------
enum { EPI_NONE = 0, EPI_GELU = 1, EPI_DGELU = 2 };

typedef struct GemmArgs {
  const void* A;     // bf16
  const void* B;     // bf16
  void* out;         // bf16 or fp32 (out_f32)
  void* out2;        // bf16, EPI_GELU: gelu(out)
  const void* bias;  // bf16 [N] or null
  const void* residual;  // bf16 [M, N] or null (added before the activation derivative)
  const void* aux;       // bf16 [M, N] pre-activation for EPI_DGELU
  int M, N, K, batch;
  int a_mn, b_mn;    // operand majors, see gemm.cu
  int epi, out_f32, accumulate, allow_split_k;
  float alpha;
  long long lda, ldb, ldo, ldo2, ldr, ldaux;                       // leading dims (elements)
  long long bs_a, bs_b, bs_out, bs_out2, bs_res, bs_aux, bs_bias;  // batch strides (elements)
} GemmArgs;

int db200_gemm_bf16(const GemmArgs* args, void* stream);

// ----- LayerNorm / RMSNorm (bf16 in/out, fp32 stats; row_keep: optional uint8 per-row multiplier) -----
int db200_norm_fwd(const void* x, const void* gamma, const void* beta, const void* row_keep, void* y, float* mean,
                   float* rstd, int rows, int H, float eps, int rms, void* stream);
int db200_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                   const void* row_keep, void* dx, float* dgamma, float* dbeta, int rows, int H, int rms,
                   void* stream);

// ----- optimizer (flat fp32 ranges) ---------------------------------------------------------
int db200_sumsq(const float* g, long long n, float* out_accum, void* stream);
int db200_adamw(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr, float wd,
                float b1, float b2, float eps, float inv_bc1, float inv_sqrt_bc2, const float* norm_sq,
                float max_norm, float grad_scale, void* stream);

#ifdef __cplusplus
}
#endif
