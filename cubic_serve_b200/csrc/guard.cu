// Canary regions: guard bands around device buffers, filled with a pattern and checked after the kernels under
// audit ran.  A kernel that writes outside the tensor it was given (a tile epilogue that ignores a ragged edge, a
// row count rounded up to the tile) lands in a band and is reported with the band's index and the first damaged
// byte offset, instead of silently corrupting a neighbouring allocation.
//
// Counterpart of the reference's debug-only snapshot / owner-copy kernels (guardrail layer, native unit N32); the
// poisoned-padding audit of whole decode graphs is guardrail/graph_audit.py.
#include "ptx.cuh"

namespace cb {

__global__ void __launch_bounds__(256)
canary_fill_kernel(uint32_t* __restrict__ p, long long words, uint32_t pattern) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < words;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    p[i] = pattern ^ static_cast<uint32_t>(i);
}

// report[0] += damaged words, report[1] = smallest damaged word index seen (atomicMin), report[2] = band index of it
__global__ void __launch_bounds__(256)
canary_check_kernel(const uint32_t* __restrict__ p, long long words, uint32_t pattern, int band,
                    unsigned long long* __restrict__ report) {
  unsigned int bad = 0;
  long long first = -1;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < words;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (p[i] != (pattern ^ static_cast<uint32_t>(i))) {
      ++bad;
      if (first < 0) first = i;
    }
  }
  if (bad) {
    atomicAdd(&report[0], static_cast<unsigned long long>(bad));
    const unsigned long long key = (static_cast<unsigned long long>(band) << 40) | static_cast<unsigned long long>(first);
    atomicMin(&report[1], key);
  }
}

}  // namespace cb

extern "C" {

int cb_canary_fill(void* p, long long bytes, unsigned pattern, void* stream) {
  if (bytes <= 0) return 0;
  if (bytes % 4 != 0 || (reinterpret_cast<uintptr_t>(p) & 3u)) return -10;
  const long long words = bytes / 4;
  const unsigned grid = static_cast<unsigned>(words / 256 + 1 > 1024 ? 1024 : words / 256 + 1);
  cb::canary_fill_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t*>(p), words, pattern);
  return static_cast<int>(cudaGetLastError());
}

// report: three 64-bit words, {damaged words so far, (band << 40 | first damaged word) minimum, unused}; the caller
// sets report[1] to all ones before the first check of an audit.
int cb_canary_check(const void* p, long long bytes, unsigned pattern, int band, void* report, void* stream) {
  if (bytes <= 0) return 0;
  if (bytes % 4 != 0 || (reinterpret_cast<uintptr_t>(p) & 3u) || !report) return -10;
  const long long words = bytes / 4;
  const unsigned grid = static_cast<unsigned>(words / 256 + 1 > 1024 ? 1024 : words / 256 + 1);
  cb::canary_check_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(p), words, pattern, band, static_cast<unsigned long long*>(report));
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
