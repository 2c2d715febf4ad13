// Row kernels: RMSNorm (+residual), SwiGLU, embedding gather.
//
// Counterparts in the reference: normalization/row_norm_native.cu:40 (RMSNorm
// with plain / zero-centred epilogues), the Triton residual+norm kernel
// normalization/rms_norm.py:47, pointwise/qwen_decode.py:300 (packed SwiGLU),
// embedding/immutable.cu:3.  All are bandwidth-bound: 128-bit accesses, one
// pass over the row held in registers.
#include "ptx.cuh"
#include "launch.cuh"
#include <atomic>

namespace cb {

static constexpr int kNormThreads = 256;
static constexpr int kNormMaxVec = 4;  // up to 256 * 4 * 8 = 8192 columns

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// out = rmsnorm(x [+ residual]) * (w or 1+w);  when residual != null the sum is
// written back to residual_out (may alias residual) rounded to bf16 first, as
// the reference's fused kernel does.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* residual, __nv_bfloat16* residual_out,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, int H, float eps,
               int zero_centered, const long long* __restrict__ x_rows) {
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const int nvec = H >> 3;  // 8 bf16 per 16 bytes
  pdl_wait();
  pdl_launch_dependents();
  // x_rows: output row i is the norm of input row x_rows[i] (the rows whose logits are wanted, gathered in passing)
  if (x_rows) x += (static_cast<size_t>(x_rows[row]) - row) * H;
  float vals[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kNormMaxVec; ++it) {
    const int v = threadIdx.x + it * kNormThreads;
    if (v < nvec) {
      uint4 xv = reinterpret_cast<const uint4*>(x + row * H)[v];
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      if (residual) {
        uint4 rv = reinterpret_cast<const uint4*>(residual + row * H)[v];
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
        uint4 ov;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 a = __bfloat1622float2(xp[j]), b = __bfloat1622float2(rp[j]);
          op[j] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
          float2 s = __bfloat1622float2(op[j]);
          vals[it][2 * j] = s.x;
          vals[it][2 * j + 1] = s.y;
        }
        reinterpret_cast<uint4*>(residual_out + row * H)[v] = ov;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 a = __bfloat1622float2(xp[j]);
          vals[it][2 * j] = a.x;
          vals[it][2 * j + 1] = a.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[it][j] * vals[it][j];
    }
  }
  const float total = block_sum(ss, red);
  const float inv = rsqrtf(total / static_cast<float>(H) + eps);
#pragma unroll
  for (int it = 0; it < kNormMaxVec; ++it) {
    const int v = threadIdx.x + it * kNormThreads;
    if (v < nvec) {
      uint4 wv = reinterpret_cast<const uint4*>(w)[v];
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 ov;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 ww = __bfloat1622float2(wp[j]);
        if (zero_centered) { ww.x += 1.f; ww.y += 1.f; }
        op[j] = __floats2bfloat162_rn(vals[it][2 * j] * inv * ww.x, vals[it][2 * j + 1] * inv * ww.y);
      }
      reinterpret_cast<uint4*>(out + row * H)[v] = ov;
    }
  }
}

// out[m, i] = silu(gu[m, i]) * gu[m, I + i]   (gate and up halves concatenated)
__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I) {
  // grid = (vector blocks of a row, rows): no per-thread 64-bit division
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  if (v >= (I >> 3)) return;
  const size_t row = blockIdx.y;
  const uint4 g = reinterpret_cast<const uint4*>(gu + row * 2 * I)[v];
  const uint4 u = reinterpret_cast<const uint4*>(gu + row * 2 * I + I)[v];
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 a = __bfloat1622float2(gp[j]), b = __bfloat1622float2(up[j]);
    op[j] = __floats2bfloat162_rn(cb::silu_fast(a.x) * b.x, cb::silu_fast(a.y) * b.y);
  }
  reinterpret_cast<uint4*>(out + row * I)[v] = o;
}

// out[t, :] = table[ids[t] - vocab_start, :] for owned ids, +0 otherwise
// (vocab-sharded tables: the non-owners contribute zeros to the rank sum).
__global__ void __launch_bounds__(128)
embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out,
                 int H, int vocab_start, int vocab_count) {
  const size_t t = blockIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  const int id = ids[t] - vocab_start;
  const bool owned = id >= 0 && id < vocab_count;
  const int nvec = H >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 val = make_uint4(0, 0, 0, 0);
    if (owned) val = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H)[v];
    reinterpret_cast<uint4*>(out + t * H)[v] = val;
  }
}

}  // namespace cb

static std::atomic<int> g_pdl{1};

extern "C" {

// Programmatic dependent launch of the library's kernels (see launch.cuh): 1 (default) on, 0 off.
void cb_set_pdl(int on) { g_pdl.store(on ? 1 : 0); }
int cb_pdl_enabled() { return g_pdl.load(std::memory_order_relaxed); }

int cb_rmsnorm(const void* x, const void* residual, void* residual_out, const void* w, void* out, int rows, int H,
               float eps, int zero_centered, void* stream) {
  using namespace cb;
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H > kNormThreads * kNormMaxVec * 8) return -10;
  return static_cast<int>(launch(rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(residual_out), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(out), H, eps, zero_centered, static_cast<const long long*>(nullptr)));
}

// out[i] = rmsnorm(x[x_rows[i]]): the final norm of a step over the rows that feed the output projection.
int cb_rmsnorm_rows(const void* x, const void* x_rows, const void* w, void* out, int rows, int H, float eps,
                    int zero_centered, void* stream) {
  using namespace cb;
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H > kNormThreads * kNormMaxVec * 8 || !x_rows) return -10;
  return static_cast<int>(launch(rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(nullptr),
      static_cast<__nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(out), H, eps, zero_centered, static_cast<const long long*>(x_rows)));
}

int cb_swiglu(const void* gate_up, void* out, int rows, int I, void* stream) {
  using namespace cb;
  if (rows <= 0) return 0;
  if (I % 8 != 0) return -10;
  if (rows > 65535) {
    // the row index rides in gridDim.y: split very long batches
    for (int r0 = 0; r0 < rows; r0 += 65535) {
      const int n = rows - r0 < 65535 ? rows - r0 : 65535;
      const int rc = cb_swiglu(static_cast<const __nv_bfloat16*>(gate_up) + static_cast<size_t>(r0) * 2 * I,
                               static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(r0) * I, n, I, stream);
      if (rc) return rc;
    }
    return 0;
  }
  const dim3 grid(static_cast<unsigned>(((I >> 3) + 255) / 256), static_cast<unsigned>(rows));
  return static_cast<int>(launch(swiglu_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), I));
}

int cb_embedding(const void* ids, const void* table, void* out, int tokens, int H, int vocab_start, int vocab_count,
                 void* stream) {
  using namespace cb;
  if (tokens <= 0) return 0;
  if (H % 8 != 0) return -10;
  return static_cast<int>(launch(embedding_kernel, dim3(tokens), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const int*>(ids), static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), H,
      vocab_start, vocab_count));
}

}  // extern "C"
