// Gated DeltaNet (linear attention) layer kernels of the hybrid decoder family.
//
// A step's tokens arrive as SEGMENTS: the contiguous rows [row0, row0 + count) of one request, whose first row has
// absolute position pos0; `slot` is the request's row of the persistent state tensors.  A request that starts at
// position 0 starts from zero state (slots are reused without clearing).
//
//   gdn_conv_kernel    depthwise causal conv1d (kernel 4) + SiLU over the mixed q/k/v channels, history in registers,
//                      per-request conv state (the last three inputs of every channel)
//   gdn_delta_kernel   per (segment, value head): L2-normalised q / k, beta = sigmoid(b),
//                      decay = exp(-exp(A_log) * softplus(a + dt_bias)), the gated delta rule
//                          S <- S * decay;  delta = (v - S k) * beta;  S <- S + delta k^T;  o = S q
//                      with the 128 x 128 fp32 state of the head held in registers for the whole segment, then the
//                      gated RMSNorm of the head (o * rsqrt(mean o^2 + eps) * w * silu(z))
//
// Speculative review passes run both kernels with commit = 0: outputs are produced for every row, the persistent
// state is left as it was.  Once the accepted prefix is known (on the device), the SAME kernels run again over the
// recorded inputs of the review rows with segments whose count is the accepted length and commit = 1: that fold
// brings conv and delta state to the accepted position without a host round trip (the reference's separate fold
// kernel: ops/cuda/linear_attention/gated_delta_fold.cu:22).
//
// Reference counterparts: ops/cuda/linear_attention/causal_conv_native.cu:13, gated_delta_native.cu:36,
// gated_delta_coefficients_native.cu:17 and the oracle ops/eager/hybrid.py:255-548 (fp32 recurrence branch).
#include "ptx.cuh"

namespace cb {

static constexpr int kGdnDim = 128;            // key and value head width (d_k = d_v = 128)

struct GdnSegments {
  const int* row0;      // [S] first row of the segment in the step's token order
  const int* count;     // [S] rows of the segment (0 = padding)
  const int* slot;      // [S] state slot of the request
  const int* pos0;      // [S] absolute position of the first row (0 = fresh state)
};

// grid (ceil(C / 128), segments); one thread per channel walks the segment's rows in order.
__global__ void __launch_bounds__(128)
gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* __restrict__ y, int ldy,
                const float* __restrict__ w,            // [C, 4], tap 3 multiplies the current input
                const float* __restrict__ bias,         // [C] or null
                __nv_bfloat16* __restrict__ state,      // [slots, 3, C]
                GdnSegments seg, int C, int commit) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int s = blockIdx.y;
  const int n = seg.count[s];
  if (c >= C || n <= 0) return;
  const int row0 = seg.row0[s];
  __nv_bfloat16* st = state + static_cast<size_t>(seg.slot[s]) * 3 * C + c;
  float h0 = 0.f, h1 = 0.f, h2 = 0.f;                   // inputs at t-3, t-2, t-1
  if (seg.pos0[s] > 0) {
    h0 = __bfloat162float(st[0]);
    h1 = __bfloat162float(st[static_cast<size_t>(C)]);
    h2 = __bfloat162float(st[static_cast<size_t>(2) * C]);
  }
  const float4 wv = *reinterpret_cast<const float4*>(w + static_cast<size_t>(c) * 4);
  const float b = bias ? bias[c] : 0.f;
  const __nv_bfloat16* xp = x + static_cast<size_t>(row0) * ldx + c;
  __nv_bfloat16* yp = y + static_cast<size_t>(row0) * ldy + c;
  // four rows per trip: the loads do not depend on the arithmetic, so they are issued together
  int t = 0;
  for (; t + 4 <= n; t += 4) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(xp[static_cast<size_t>(t + j) * ldx]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = b + wv.x * h0 + wv.y * h1 + wv.z * h2 + wv.w * v[j];
      yp[static_cast<size_t>(t + j) * ldy] = __float2bfloat16(silu_fast(a));
      h0 = h1; h1 = h2; h2 = v[j];
    }
  }
  for (; t < n; ++t) {
    const float v = __bfloat162float(xp[static_cast<size_t>(t) * ldx]);
    const float a = b + wv.x * h0 + wv.y * h1 + wv.z * h2 + wv.w * v;
    yp[static_cast<size_t>(t) * ldy] = __float2bfloat16(silu_fast(a));
    h0 = h1; h1 = h2; h2 = v;
  }
  if (!commit) return;
  st[0] = __float2bfloat16(h0);
  st[static_cast<size_t>(C)] = __float2bfloat16(h1);
  st[static_cast<size_t>(2) * C] = __float2bfloat16(h2);
}

struct GdnDeltaParams {
  const __nv_bfloat16* qkv;   // [T, ldqkv] after the convolution: q [Hk * 128] | k [Hk * 128] | v [Hv * 128]
  int ldqkv;
  const __nv_bfloat16* z;     // [T, ldz] gate of the output norm, [Hv * 128]
  int ldz;
  const __nv_bfloat16* ba;    // [T, ldba]: b [Hv] | a [Hv]
  int ldba;
  const float* a_log;         // [Hv]
  const float* dt_bias;       // [Hv]
  const float* norm_w;        // [128]
  float* state;               // [slots, Hv, 128 (v), 128 (k)] fp32
  __nv_bfloat16* out;         // [T, ldo]: [Hv * 128]
  int ldo;
  int Hk, Hv;
  float eps_norm;             // RMSNorm epsilon
  float eps_l2;               // L2-normalisation epsilon
  int commit;                 // 0: the state is read but not written back (speculative review pass)
  GdnSegments seg;
};

// grid (Hv, segments), 256 threads.  Eight lanes share a state row: lane l8 = lane & 7 owns the float4 chunks
// l8, l8 + 8, l8 + 16, l8 + 24 of the row's 128 key columns, so one load instruction of a warp covers four whole
// 512-byte rows (fully coalesced; the state is the only large operand: 64 KiB per CTA read and written once per
// step).  A thread holds four rows: warp * 16 + (lane >> 3) + 4 i.  Row sums (S k and S q) are reduced over the
// eight lanes by shuffles.  Two CTAs per SM (128 registers per thread): one CTA's state load / store overlaps the
// other's arithmetic.
//
// A segment is walked in blocks of 16 tokens, three phases per block:
//   A (parallel, four warp tasks per token)  L2-normalised q / k, v, z, beta and decay of the block's tokens into shared memory
//   B (the recurrence, no CTA barrier inside)  per token: decay, S k, delta, rank-one update, S q; outputs to shared memory
//   C (parallel, a warp per token)  gated RMSNorm of the block's outputs, coalesced stores
// so the token-serial part is only the arithmetic that really depends on the state.
static constexpr int kGdnBlock = 16;

__global__ void __launch_bounds__(256, 2)
gdn_delta_kernel(const GdnDeltaParams p) {
  const int head = blockIdx.x;
  const int s = blockIdx.y;
  const int n = p.seg.count[s];
  if (n <= 0) return;
  const int row0 = p.seg.row0[s];
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int l8 = lane & 7;
  const int vrow = warp * 16 + (lane >> 3);              // + 4 i
  const int khead = head / (p.Hv / p.Hk);
  __shared__ __align__(16) float qs[kGdnBlock][kGdnDim];
  __shared__ __align__(16) float ks[kGdnBlock][kGdnDim];
  __shared__ float vs[kGdnBlock][kGdnDim];
  __shared__ float os[kGdnBlock][kGdnDim];
  __shared__ float zs[kGdnBlock][kGdnDim];
  __shared__ float2 coef[kGdnBlock];                      // {beta, decay}

  float* sp = p.state + ((static_cast<size_t>(p.seg.slot[s]) * p.Hv + head) * kGdnDim + vrow) * kGdnDim + l8 * 4;
  float4 S[4][4];                                        // [row i][chunk c]: columns 4 (l8 + 8 c) .. + 3
  if (p.seg.pos0[s] > 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) S[i][c] = *reinterpret_cast<const float4*>(sp + (4 * i) * kGdnDim + 32 * c);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) S[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float neg_exp_a = -__expf(p.a_log[head]);
  const float dtb = p.dt_bias[head];
  const int q_off = khead * kGdnDim, k_off = (p.Hk + khead) * kGdnDim, v_off = (2 * p.Hk + head) * kGdnDim;
  float nw[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) nw[a] = p.norm_w[lane + 32 * a];

  for (int t0 = 0; t0 < n; t0 += kGdnBlock) {
    const int nb = min(kGdnBlock, n - t0);
    // ---- A: operands of the block's tokens.  Four independent tasks per token (q, k, v + z, coefficients) dealt
    // to the eight warps, so that a one-token decode step still uses four warps at once
    for (int task = warp; task < nb * 4; task += 8) {
      const int j = task >> 2, part = task & 3;
      const size_t r = static_cast<size_t>(row0 + t0 + j);
      const __nv_bfloat16* row = p.qkv + r * p.ldqkv;
      if (part < 2) {
        // stored boundary of the oracle: normalised q / k are rounded to bf16; q carries the 1 / sqrt(d_k) scale
        const __nv_bfloat16* src = row + (part == 0 ? q_off : k_off);
        float x[4];
        float ss = 0.f;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          x[a] = __bfloat162float(src[lane + 32 * a]);
          ss = fmaf(x[a], x[a], ss);
        }
        const float inv = rsqrtf(warp_sum(ss) + p.eps_l2);
        float* dst = part == 0 ? qs[j] : ks[j];
        const float scale = part == 0 ? 0.08838834764831845f : 1.f;
#pragma unroll
        for (int a = 0; a < 4; ++a) dst[lane + 32 * a] = __bfloat162float(__float2bfloat16(x[a] * inv)) * scale;
      } else if (part == 2) {
        const __nv_bfloat16* zrow = p.z + r * p.ldz + head * kGdnDim;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          vs[j][lane + 32 * a] = __bfloat162float(row[v_off + lane + 32 * a]);
          zs[j][lane + 32 * a] = __bfloat162float(zrow[lane + 32 * a]);
        }
      } else if (lane == 0) {
        const float bb = __bfloat162float(p.ba[r * p.ldba + head]);
        const float x = __bfloat162float(p.ba[r * p.ldba + p.Hv + head]) + dtb;
        const float softplus = x > 20.f ? x : log1pf(__expf(x));
        coef[j] = make_float2(1.f / (1.f + __expf(-bb)), __expf(neg_exp_a * softplus));
      }
    }
    __syncthreads();
    // ---- B: the recurrence
    for (int j = 0; j < nb; ++j) {
      const float beta = coef[j].x, decay = coef[j].y;
      float4 kv[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) kv[c] = *reinterpret_cast<const float4*>(&ks[j][4 * (l8 + 8 * c)]);
      float mem[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float m = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float4& e = S[i][c];
          e.x *= decay; e.y *= decay; e.z *= decay; e.w *= decay;
          m = fmaf(e.x, kv[c].x, m); m = fmaf(e.y, kv[c].y, m); m = fmaf(e.z, kv[c].z, m); m = fmaf(e.w, kv[c].w, m);
        }
        mem[i] = m;
      }
#pragma unroll
      for (int sh = 1; sh < 8; sh <<= 1)
#pragma unroll
        for (int i = 0; i < 4; ++i) mem[i] += __shfl_xor_sync(0xffffffffu, mem[i], sh);
      float4 qv[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) qv[c] = *reinterpret_cast<const float4*>(&qs[j][4 * (l8 + 8 * c)]);
      float o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float delta = (vs[j][vrow + 4 * i] - mem[i]) * beta;
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float4& e = S[i][c];
          e.x = fmaf(delta, kv[c].x, e.x); e.y = fmaf(delta, kv[c].y, e.y);
          e.z = fmaf(delta, kv[c].z, e.z); e.w = fmaf(delta, kv[c].w, e.w);
          acc = fmaf(e.x, qv[c].x, acc); acc = fmaf(e.y, qv[c].y, acc); acc = fmaf(e.z, qv[c].z, acc); acc = fmaf(e.w, qv[c].w, acc);
        }
        o[i] = acc;
      }
#pragma unroll
      for (int sh = 1; sh < 8; sh <<= 1)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] += __shfl_xor_sync(0xffffffffu, o[i], sh);
      if (l8 == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) os[j][vrow + 4 * i] = __bfloat162float(__float2bfloat16(o[i]));   // stored in bf16
      }
    }
    __syncthreads();
    // ---- C: gated RMSNorm over each token's 128 outputs
    for (int j = warp; j < nb; j += 8) {
      const size_t r = static_cast<size_t>(row0 + t0 + j);
      float ob[4];
      float ss = 0.f;
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        ob[a] = os[j][lane + 32 * a];
        ss = fmaf(ob[a], ob[a], ss);
      }
      const float inv = rsqrtf(warp_sum(ss) * (1.f / kGdnDim) + p.eps_norm);
      __nv_bfloat16* orow = p.out + r * p.ldo + head * kGdnDim;
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float normed = __bfloat162float(__float2bfloat16(ob[a] * inv));
        orow[lane + 32 * a] = __float2bfloat16(normed * nw[a] * silu_fast(zs[j][lane + 32 * a]));
      }
    }
    // (the next block's phase A writes q / k / v / z: z of this block is still being read here, hence the barrier)
    if (t0 + kGdnBlock < n) __syncthreads();
  }
  if (!p.commit) return;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) *reinterpret_cast<float4*>(sp + (4 * i) * kGdnDim + 32 * c) = S[i][c];
}

// out = x * sigmoid(gate): the output gate of the hybrid family's full-attention layers (bf16, in place allowed)
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ gate, int ldg,
                    __nv_bfloat16* __restrict__ out, int ldo, int cols) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= (cols >> 1)) return;
  const size_t r = blockIdx.y;
  const float2 a = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + r * ldx)[v]);
  const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(gate + r * ldg)[v]);
  reinterpret_cast<__nv_bfloat162*>(out + r * ldo)[v] =
      __floats2bfloat162_rn(a.x / (1.f + __expf(-g.x)), a.y / (1.f + __expf(-g.y)));
}

}  // namespace cb

extern "C" {

struct CbGdnSegments {
  const void* row0;
  const void* count;
  const void* slot;
  const void* pos0;
  int num;
};

int cb_gdn_conv(const void* x, int ldx, void* y, int ldy, const void* w, const void* bias, void* state,
                const CbGdnSegments* seg, int C, int commit, void* stream) {
  if (!seg || seg->num <= 0 || C <= 0 || seg->num > 65535) return -60;
  cb::GdnSegments s{static_cast<const int*>(seg->row0), static_cast<const int*>(seg->count),
                    static_cast<const int*>(seg->slot), static_cast<const int*>(seg->pos0)};
  dim3 grid((C + 127) / 128, seg->num);
  cb::gdn_conv_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_bfloat16*>(y), ldy, static_cast<const float*>(w),
      static_cast<const float*>(bias), static_cast<__nv_bfloat16*>(state), s, C, commit);
  return static_cast<int>(cudaGetLastError());
}

struct CbGdnDelta {
  const void* qkv; int ldqkv;
  const void* z; int ldz;
  const void* ba; int ldba;
  const void* a_log;
  const void* dt_bias;
  const void* norm_w;
  void* state;
  void* out; int ldo;
  int Hk, Hv;
  float eps_norm, eps_l2;
  int commit;
};

int cb_gdn_delta(const CbGdnDelta* a, const CbGdnSegments* seg, void* stream) {
  if (!a || !seg || seg->num <= 0 || seg->num > 65535 || a->Hk <= 0 || a->Hv <= 0 || (a->Hv % a->Hk) != 0) return -61;
  cb::GdnDeltaParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(a->qkv); p.ldqkv = a->ldqkv;
  p.z = static_cast<const __nv_bfloat16*>(a->z); p.ldz = a->ldz;
  p.ba = static_cast<const __nv_bfloat16*>(a->ba); p.ldba = a->ldba;
  p.a_log = static_cast<const float*>(a->a_log);
  p.dt_bias = static_cast<const float*>(a->dt_bias);
  p.norm_w = static_cast<const float*>(a->norm_w);
  p.state = static_cast<float*>(a->state);
  p.out = static_cast<__nv_bfloat16*>(a->out); p.ldo = a->ldo;
  p.Hk = a->Hk; p.Hv = a->Hv;
  p.eps_norm = a->eps_norm; p.eps_l2 = a->eps_l2;
  p.commit = a->commit;
  p.seg = cb::GdnSegments{static_cast<const int*>(seg->row0), static_cast<const int*>(seg->count),
                          static_cast<const int*>(seg->slot), static_cast<const int*>(seg->pos0)};
  dim3 grid(a->Hv, seg->num);
  cb::gdn_delta_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int cb_sigmoid_gate(const void* x, int ldx, const void* gate, int ldg, void* out, int ldo, int rows, int cols,
                    void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 1) || (ldx & 1) || (ldg & 1) || (ldo & 1)) return -62;
  for (int r0 = 0; r0 < rows; r0 += 65535) {
    const int nr = rows - r0 < 65535 ? rows - r0 : 65535;
    dim3 grid((cols / 2 + 255) / 256, nr);
    cb::sigmoid_gate_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x) + static_cast<size_t>(r0) * ldx, ldx,
        static_cast<const __nv_bfloat16*>(gate) + static_cast<size_t>(r0) * ldg, ldg,
        static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(r0) * ldo, ldo, cols);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
