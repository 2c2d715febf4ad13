// C declarations of entry points of libcubic_b200.so that are meant to be called
// directly from C / C++ / ctypes without the Python wrappers.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// ---------------------------------------------------------------------------
// Split-K weight-quantized GEMM that allocates nothing.
//
// This entry point has no counterpart in the reference project; it exists for
// callers of this library that are not able to allocate device memory:
//   * a serving process that handed every free byte of the GPU to its KV page
//     pool at start-up, so a later cudaMalloc for GEMM scratch would simply fail;
//   * a latency-critical loop that must not risk the device-wide synchronisation
//     a cudaMalloc / cudaFree can cause;
//   * a plain C host (a plugin, a test harness) that has raw device pointers for
//     inputs and outputs but no caching allocator to ask for temporaries.
//
// It computes  y[M, N] = alpha * x[M, K] * W[N, K]^T (+ residual)  with the same
// kernel as cb_wq_gemm in its workspace form (the K splits of an output tile meet
// through fp32 partial sums in global memory; the last split to arrive adds them
// in split order) and the same argument meaning (fmt: 0 cubic4, 1 affine4,
// 2 nvfp4, 3 bf16 weights; x and y are bf16 row-major; codes / meta are the packed
// weight produced by ops/wq_pack.py).  The split-K partial sums and the per-tile
// arrival counters live in a scratch array that is part of the library image
// (CB_NOALLOC_SCRATCH_BYTES per GPU that loads the library, held until the
// process exits) instead of a buffer supplied by the caller.
//
// Limits and rules:
//   * the partial sums need  ceil(N/128) * splits * round_up(M, 16) * 128 * 4
//     bytes (M <= 256); a call that needs more than CB_NOALLOC_PARTIAL_BYTES,
//     or more than CB_NOALLOC_MAX_TILES output tiles, is rejected with
//     CB_NOALLOC_ERR_TOO_LARGE and nothing is launched;
//   * the first call on each device looks up the device address of the scratch
//     array (with that device current) and configures the kernel; make that
//     first call before starting any stream capture on the device;
//   * every call uses the same array: the counters are cleared on the caller's
//     stream before each launch, the partial sums are fully rewritten by each
//     launch, and two calls that can overlap on the GPU (different streams
//     without an ordering between them) race on it -- serialise them;
//   * no cudaMalloc, cudaFree or allocating library routine is called.
//
// Returns 0 on success, a negative CB_NOALLOC_ERR_* / argument code, or a positive
// cudaError_t from the launch.
// ---------------------------------------------------------------------------
#define CB_NOALLOC_PARTIAL_BYTES (8u << 20)
#define CB_NOALLOC_MAX_TILES 4096u
#define CB_NOALLOC_SCRATCH_BYTES (CB_NOALLOC_PARTIAL_BYTES + CB_NOALLOC_MAX_TILES * 4u + 256u)
#define CB_NOALLOC_ERR_TOO_LARGE (-40)
#define CB_NOALLOC_ERR_SYMBOL (-41)
#define CB_NOALLOC_ERR_DEVICE (-42)

int cb_wq_gemm_splitk_noalloc(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                              const void* residual, float alpha, int M, int N, int K, int group_k, int splits,
                              void* stream);

// Device status word of the last no-alloc calls on the current device (0 = no
// device-side wait ran out); reading it synchronises the device.
int cb_wq_gemm_splitk_noalloc_status(unsigned* status_out);

#ifdef __cplusplus
}
#endif
