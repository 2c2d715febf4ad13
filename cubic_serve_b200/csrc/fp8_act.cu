// Dynamic per-token FP8 (e4m3) quantization of activations, alone and fused behind RMSNorm / SwiGLU.
//
// The fp8 weight GEMM (wq_gemm.cu, kFmtFp8) multiplies e4m3 weights with e4m3 activations on the tensor cores; its
// activation operand is made here.  Semantics of the reference's dynamic-token quantizer
// (quantization/extensions/fp8/reference.py:47-59, kernels.py:78-104 there):
//   scale[m] = max(amax_k |x[m, k]| / 448, 1 / (448 * 512)),   q[m, k] = e4m3_rn(clamp(x[m, k] / scale[m], +-448))
// with a correctly rounded division.  The fused forms quantize the value the unfused chain would have stored (the
// bf16-rounded norm output / activation), so fusing changes no bit.
#include "ptx.cuh"
#include "launch.cuh"
#include <cuda_fp8.h>

namespace cb {

static constexpr int kQThreads = 256;
static constexpr int kQMaxVec = 6;          // up to 256 * 6 * 8 = 12288 columns held in registers
static constexpr float kFp8Max = 448.f;
static constexpr float kFp8MinScale = 1.f / (448.f * 512.f);

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  __syncthreads();
  return t;
}

__device__ __forceinline__ float block_sum_q(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// eight fp32 values -> eight e4m3 bytes (value j in byte j)
__device__ __forceinline__ uint2 pack_e4m3x8(const float (&v)[8], float scale) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t acc = 0;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float2 f;
      f.x = fminf(fmaxf(__fdiv_rn(v[4 * h + 2 * j], scale), -kFp8Max), kFp8Max);
      f.y = fminf(fmaxf(__fdiv_rn(v[4 * h + 2 * j + 1], scale), -kFp8Max), kFp8Max);
      const uint32_t pair = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);   // x -> low byte, y -> high byte
      acc |= pair << (16 * j);
    }
    w[h] = acc;
  }
  return make_uint2(w[0], w[1]);
}

// MODE 0: q = quant(x)                                   (x bf16 [rows, K], row stride ldx)
// MODE 1: q = quant(bf16(rmsnorm(x [+ residual]) * w))   (the residual sum is written back like rmsnorm_kernel)
// MODE 2: q = quant(bf16(silu(x[:, :K]) * x[:, K:]))     (x = [gate | up], 2 K columns)
// `phase` (MODE 0 only) splits the work for operands whose K dimension is sharded over tensor-parallel ranks: 1 = write
// the row's scale only (the ranks then take the maximum of their scales), 2 = quantize with the scale found in `scales`.
template <int MODE>
__global__ void __launch_bounds__(kQThreads)
fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* residual, __nv_bfloat16* residual_out,
                const __nv_bfloat16* __restrict__ w, float eps, int zero_centered, uint8_t* __restrict__ q, int ldq,
                float* __restrict__ scales, int K, int phase) {
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const int nvec = K >> 3;
  pdl_wait();
  pdl_launch_dependents();
  float vals[kQMaxVec][8];
  float ss = 0.f, amax = 0.f;
  const __nv_bfloat16* xr = x + row * ldx;
#pragma unroll
  for (int it = 0; it < kQMaxVec; ++it) {
    const int v = threadIdx.x + it * kQThreads;
    if (v < nvec) {
      const uint4 xv = reinterpret_cast<const uint4*>(xr)[v];
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      if (MODE == 2) {
        const uint4 uv = reinterpret_cast<const uint4*>(xr + K)[v];
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(xp[j]), b = __bfloat1622float2(up[j]);
          const float2 o = __bfloat1622float2(__floats2bfloat162_rn(silu_fast(a.x) * b.x, silu_fast(a.y) * b.y));
          vals[it][2 * j] = o.x;
          vals[it][2 * j + 1] = o.y;
        }
      } else if (MODE == 1 && residual) {
        const uint4 rv = reinterpret_cast<const uint4*>(residual + row * K)[v];
        const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
        uint4 ov;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(xp[j]), b = __bfloat1622float2(rp[j]);
          op[j] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
          const float2 s = __bfloat1622float2(op[j]);
          vals[it][2 * j] = s.x;
          vals[it][2 * j + 1] = s.y;
        }
        reinterpret_cast<uint4*>(residual_out + row * K)[v] = ov;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(xp[j]);
          vals[it][2 * j] = a.x;
          vals[it][2 * j + 1] = a.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (MODE == 1) ss += vals[it][j] * vals[it][j];
        else amax = fmaxf(amax, fabsf(vals[it][j]));
      }
    }
  }
  if (MODE == 1) {
    const float total = block_sum_q(ss, red);
    const float inv = rsqrtf(total / static_cast<float>(K) + eps);
#pragma unroll
    for (int it = 0; it < kQMaxVec; ++it) {
      const int v = threadIdx.x + it * kQThreads;
      if (v < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(w)[v];
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 ww = __bfloat1622float2(wp[j]);
          if (zero_centered) { ww.x += 1.f; ww.y += 1.f; }
          const float2 o = __bfloat1622float2(
              __floats2bfloat162_rn(vals[it][2 * j] * inv * ww.x, vals[it][2 * j + 1] * inv * ww.y));
          vals[it][2 * j] = o.x;
          vals[it][2 * j + 1] = o.y;
          amax = fmaxf(amax, fmaxf(fabsf(o.x), fabsf(o.y)));
        }
      }
    }
  }
  float scale;
  if (phase == 2) {
    scale = scales[row];
  } else {
    amax = block_max(amax, red);
    scale = fmaxf(__fdiv_rn(amax, kFp8Max), kFp8MinScale);
    if (threadIdx.x == 0) scales[row] = scale;
    if (phase == 1) return;
  }
  uint8_t* qr = q + row * ldq;
#pragma unroll
  for (int it = 0; it < kQMaxVec; ++it) {
    const int v = threadIdx.x + it * kQThreads;
    if (v < nvec) reinterpret_cast<uint2*>(qr)[v] = pack_e4m3x8(vals[it], scale);
  }
}

}  // namespace cb

extern "C" {

static int fp8_check(int rows, int K, int ldq) {
  if (rows <= 0) return 1;
  if (K % 8 != 0 || K > cb::kQThreads * cb::kQMaxVec * 8 || ldq % 16 != 0 || ldq < K) return -10;
  return 0;
}

// q[m, :K] (e4m3, ldq bytes per row), scales[m] = dynamic per-token quantization of x [rows, K] bf16.
int cb_fp8_quantize_rows(const void* x, int ldx, void* q, int ldq, void* scales, int rows, int K, void* stream) {
  using namespace cb;
  const int c = fp8_check(rows, K, ldq);
  if (c) return c < 0 ? c : 0;
  if (ldx % 8 != 0) return -10;
  return static_cast<int>(launch(fp8_rows_kernel<0>, dim3(rows), dim3(kQThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(nullptr),
      static_cast<__nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(nullptr), 0.f, 0,
      static_cast<uint8_t*>(q), ldq, static_cast<float*>(scales), K, 0));
}

// The same in two launches for an operand whose K dimension is sharded over tensor-parallel ranks: phase 1 writes
// every row's local scale, the caller reduces `scales` with MAX over the ranks, phase 2 quantizes with the result --
// every rank then uses the scale the unsharded row would have had (reference: the `_ScaleCollective` all_reduce(MAX)
// of its FP8 linears, quantization/extensions/fp8/linear.py there).
int cb_fp8_quantize_rows_phase(const void* x, int ldx, void* q, int ldq, void* scales, int rows, int K, int phase,
                               void* stream) {
  using namespace cb;
  const int c = fp8_check(rows, K, ldq);
  if (c) return c < 0 ? c : 0;
  if (ldx % 8 != 0 || (phase != 1 && phase != 2)) return -10;
  return static_cast<int>(launch(fp8_rows_kernel<0>, dim3(rows), dim3(kQThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(nullptr),
      static_cast<__nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(nullptr), 0.f, 0,
      static_cast<uint8_t*>(q), ldq, static_cast<float*>(scales), K, phase));
}

// RMSNorm (optionally of x + residual, the sum written to residual_out) whose output leaves as e4m3 + scales.
int cb_rmsnorm_fp8(const void* x, const void* residual, void* residual_out, const void* w, void* q, int ldq, void* scales,
                   int rows, int H, float eps, int zero_centered, void* stream) {
  using namespace cb;
  const int c = fp8_check(rows, H, ldq);
  if (c) return c < 0 ? c : 0;
  return static_cast<int>(launch(fp8_rows_kernel<1>, dim3(rows), dim3(kQThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), H, static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(residual_out), static_cast<const __nv_bfloat16*>(w), eps, zero_centered,
      static_cast<uint8_t*>(q), ldq, static_cast<float*>(scales), H, 0));
}

// SwiGLU of gate_up [rows, 2 I] whose output leaves as e4m3 [rows, I] + scales.
int cb_swiglu_fp8(const void* gate_up, void* q, int ldq, void* scales, int rows, int I, void* stream) {
  using namespace cb;
  const int c = fp8_check(rows, I, ldq);
  if (c) return c < 0 ? c : 0;
  return static_cast<int>(launch(fp8_rows_kernel<2>, dim3(rows), dim3(kQThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(gate_up), 2 * I, static_cast<const __nv_bfloat16*>(nullptr),
      static_cast<__nv_bfloat16*>(nullptr), static_cast<const __nv_bfloat16*>(nullptr), 0.f, 0,
      static_cast<uint8_t*>(q), ldq, static_cast<float*>(scales), I, 0));
}

}  // extern "C"
