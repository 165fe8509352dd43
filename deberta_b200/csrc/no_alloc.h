// Allocation-free entry point of the fused vocabulary cross-entropy / sampling forward.
// This entry point has no counterpart in the reference implementation.
//
// Who it is for: code that calls this library from a place where device memory cannot be
// requested: a real-time serving loop that runs on a memory plan fixed at start-up, an embedding
// application whose allocator this library must not touch, a latency-critical section that cannot
// afford the device-wide synchronisation a cudaMalloc or cudaFree may imply. The regular entry point
// (db200_gemm_bf16 with EPI_CE_FWD followed by db200_ce_combine) needs a caller-provided scratch
// buffer of 4 * ceil(vocab / tile) * rows + rows floats; callers like the ones above often have
// nowhere to get one from. Here the scratch lives inside the library instead.
//
// What it costs: the scratch is a fixed device array of DB200_NOALLOC_SCRATCH_BYTES that every
// GPU which loads the library keeps until the process exits. Problems whose partial-result table
// does not fit (ceil(vocab / tile) * rows > DB200_NOALLOC_MAX_PARTIALS or rows >
// DB200_NOALLOC_MAX_ROWS) are rejected with DB200_NOALLOC_TOO_LARGE before anything is launched.
//
// Sharing: every call, on every stream, uses the same array, and the array keeps what the last
// call left in it. The entry point clears the part that must start at zero itself, but two calls
// whose kernels overlap on the GPU (different streams without ordering, or two host threads)
// race on the scratch and produce garbage: order them.
//
// Set-up, once per device, from a place where device memory may still be requested: db200_noalloc_prepare().
// It looks up the device address of the array (the host-side name of a __device__ array is not a device pointer),
// caches it, and loads the kernels of this path. Both are moments at which the CUDA driver itself takes device
// memory: with lazy module loading (the default since CUDA 12) a library's device image, the scratch array in it and
// each kernel's code reach the GPU on first use, not when the library is opened; measured on a B200, free device
// memory drops by 34 MiB (the array, rounded up by the driver) at the first use. An entry-point call on a device that
// was not prepared does the same set-up itself, so that first call is NOT allocation-free. Make the set-up from one
// host thread (the caches are plain variables; later calls only read them).
// After the set-up no call allocates or frees device memory, neither through the CUDA runtime nor through any
// library, and the driver has nothing left to load for it. (Host side: a thread's first GEMM launch creates that
// thread's table of encoded tensor maps, about 600 KB of heap; db200_noalloc_prepare() on the same thread does not
// cover it, a first call does.)
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define DB200_NOALLOC_MAX_PARTIALS (1 << 21)  // vocabulary tiles x rows
#define DB200_NOALLOC_MAX_ROWS 8192
#define DB200_NOALLOC_SCRATCH_BYTES ((4ll * DB200_NOALLOC_MAX_PARTIALS + DB200_NOALLOC_MAX_ROWS) * 4)  // 32 MiB + 32 KiB

#define DB200_NOALLOC_OK 0
#define DB200_NOALLOC_TOO_LARGE (-20)   // rows / vocabulary exceed the built-in scratch
#define DB200_NOALLOC_BAD_ARGS (-21)    // null pointer, misaligned operand, hidden size not a multiple of 8
#define DB200_NOALLOC_NO_DEVICE (-22)   // the scratch address could not be resolved on the current device

// x [rows, hidden] bf16, weight [vocab, hidden] bf16 (row-major, 16-byte aligned), bias [vocab] bf16 or null,
// labels [rows] int64, forbidden [vocab] uint8 or null. Outputs (caller-owned device memory):
// lse [rows] fp32 natural-log log-sum-exp, loss_rows [rows] fp32 per-row cross-entropy,
// sampled [rows] int64 Gumbel-max sample of softmax(logits / temperature) with forbidden ids excluded.
int db200_vocab_ce_forward_noalloc(const void* x, const void* weight, const void* bias, const long long* labels,
                                   const unsigned char* forbidden, int rows, int vocab, int hidden, float temperature,
                                   unsigned long long seed, float* lse, float* loss_rows, long long* sampled,
                                   void* stream);

// One-time set-up on the current device (see above). Idempotent; returns DB200_NOALLOC_OK or DB200_NOALLOC_NO_DEVICE.
int db200_noalloc_prepare(void);

// Human-readable text for the codes above (and for the launcher codes passed through unchanged).
const char* db200_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
