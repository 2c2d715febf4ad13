// Split-K GEMM entry point whose scratch memory is a static device array
// (see cubic_b200.h for who needs it and for the rules).
#include "cubic_b200.h"

#include <cuda_runtime.h>
#include <stdint.h>

// Scratch shared by every call on a device: [partial sums | tile counters | status word].
// In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CB_NOALLOC_SCRATCH_BYTES];

// the regular split-K entry point in its workspace form (wq_gemm.cu): the K splits meet through the partial sums and
// counters handed in as plain device pointers, never through a cluster's shared memory
extern "C" int cb_wq_gemm_workspace_splitk(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y,
                                           int ldy, const void* residual, float alpha, int M, int N, int K, int group_k,
                                           int splits, void* workspace, void* counters, void* status, void* stream);

namespace {

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device, filled on first use

// Device address of the scratch array on the CURRENT device (set-up on first use).
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return CB_NOALLOC_ERR_DEVICE;
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return CB_NOALLOC_ERR_SYMBOL;
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int cb_wq_gemm_splitk_noalloc(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y,
                                         int ldy, const void* residual, float alpha, int M, int N, int K, int group_k,
                                         int splits, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || splits < 1) return -10;
  if (M > 256) return CB_NOALLOC_ERR_TOO_LARGE;   // one batch tile: keeps the bound on the partial sums simple
  const unsigned long long mb = static_cast<unsigned long long>((M + 15) / 16) * 16;
  const unsigned long long n_tiles = static_cast<unsigned long long>((N + 127) / 128);
  const unsigned long long need = splits > 1 ? n_tiles * static_cast<unsigned long long>(splits) * mb * 128ull * 4ull : 0ull;
  if (need > CB_NOALLOC_PARTIAL_BYTES || n_tiles > CB_NOALLOC_MAX_TILES) return CB_NOALLOC_ERR_TOO_LARGE;

  unsigned char* base = nullptr;
  const int rc = scratch_for_current_device(&base);
  if (rc != 0) return rc;
  unsigned char* counters = base + CB_NOALLOC_PARTIAL_BYTES;
  unsigned char* status = counters + CB_NOALLOC_MAX_TILES * 4u;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the arrival counters must be zero when the kernel starts; an earlier launch that was
  // cut short may have left some raised
  const cudaError_t e = cudaMemsetAsync(counters, 0, n_tiles * 4u, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  return cb_wq_gemm_workspace_splitk(fmt, x, ldx, codes, meta, y, ldy, residual, alpha, M, N, K, group_k, splits, base,
                                     counters, status, stream);
}

extern "C" int cb_wq_gemm_splitk_noalloc_status(unsigned* status_out) {
  unsigned char* base = nullptr;
  const int rc = scratch_for_current_device(&base);
  if (rc != 0) return rc;
  const cudaError_t e = cudaMemcpy(status_out, base + CB_NOALLOC_PARTIAL_BYTES + CB_NOALLOC_MAX_TILES * 4u,
                                   sizeof(unsigned), cudaMemcpyDeviceToHost);
  return static_cast<int>(e);
}
