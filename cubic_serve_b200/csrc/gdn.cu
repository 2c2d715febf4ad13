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
                GdnSegments seg, int C) {
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
  GdnSegments seg;
};

// grid (Hv, segments), 256 threads.  Eight lanes share a state row: lane l8 = lane & 7 owns the float4 chunks
// l8, l8 + 8, l8 + 16, l8 + 24 of the row's 128 key columns, so one load instruction of a warp covers four whole
// 512-byte rows (fully coalesced; the state is the only large operand: 64 KiB per CTA read and written once per
// step).  A thread holds four rows: warp * 16 + (lane >> 3) + 4 i.  Row sums (S k and S q) are reduced over the
// eight lanes by shuffles.  Two CTAs per SM (128 registers per thread): one CTA's state load / store overlaps the
// other's arithmetic.
__global__ void __launch_bounds__(256, 2)
gdn_delta_kernel(const GdnDeltaParams p) {
  const int head = blockIdx.x;
  const int s = blockIdx.y;
  const int n = p.seg.count[s];
  if (n <= 0) return;
  const int row0 = p.seg.row0[s];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int l8 = lane & 7;
  const int vrow = (tid >> 5) * 16 + (lane >> 3);        // + 4 i
  const int khead = head / (p.Hv / p.Hk);
  __shared__ __align__(16) float qs[kGdnDim];
  __shared__ __align__(16) float ks[kGdnDim];
  __shared__ float red[3][8];

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
  for (int i = 0; i < 4; ++i) nw[i] = p.norm_w[vrow + 4 * i];

  // operands of a row: thread tid carries q[tid] (tid < 128) or k[tid - 128] into the norm, every thread the v and
  // z of its four state rows; each iteration loads the next row's before it computes
  float qk_next, v_next[4], z_next[4], b_next, a_next;
  auto load_row = [&](size_t r) {
    const __nv_bfloat16* row = p.qkv + r * p.ldqkv;
    qk_next = __bfloat162float(tid < 128 ? row[q_off + tid] : row[k_off + tid - 128]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v_next[i] = __bfloat162float(row[v_off + vrow + 4 * i]);
      z_next[i] = __bfloat162float(p.z[r * p.ldz + head * kGdnDim + vrow + 4 * i]);
    }
    b_next = __bfloat162float(p.ba[r * p.ldba + head]);
    a_next = __bfloat162float(p.ba[r * p.ldba + p.Hv + head]);
  };
  load_row(static_cast<size_t>(row0));

  for (int t = 0; t < n; ++t) {
    const float qk = qk_next, bb = b_next, aa = a_next;
    float v[4], zz[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[i] = v_next[i]; zz[i] = z_next[i]; }
    if (t + 1 < n) load_row(static_cast<size_t>(row0 + t + 1));
    // L2 norms of q (warps 0-3) and k (warps 4-7)
    const float sq = warp_sum(qk * qk);
    if (lane == 0) red[0][tid >> 5] = sq;
    __syncthreads();
    {
      const int base = tid < 128 ? 0 : 4;
      const float tot = red[0][base] + red[0][base + 1] + red[0][base + 2] + red[0][base + 3];
      const float inv = rsqrtf(tot + p.eps_l2);
      // stored boundary of the oracle: normalised q / k are rounded to bf16; q carries the 1 / sqrt(d_k) scale
      const float nv = __bfloat162float(__float2bfloat16(qk * inv));
      if (tid < 128) qs[tid] = nv * 0.08838834764831845f;
      else ks[tid - 128] = nv;
    }
    __syncthreads();
    const float beta = 1.f / (1.f + __expf(-bb));
    const float x = aa + dtb;
    const float softplus = x > 20.f ? x : log1pf(__expf(x));
    const float decay = __expf(neg_exp_a * softplus);

    float4 kv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) kv[c] = *reinterpret_cast<const float4*>(ks + 4 * (l8 + 8 * c));
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
      m += __shfl_xor_sync(0xffffffffu, m, 1);
      m += __shfl_xor_sync(0xffffffffu, m, 2);
      m += __shfl_xor_sync(0xffffffffu, m, 4);
      mem[i] = m;
    }
    float4 qv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) qv[c] = *reinterpret_cast<const float4*>(qs + 4 * (l8 + 8 * c));
    float ob[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float delta = (v[i] - mem[i]) * beta;
      float o = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float4& e = S[i][c];
        e.x = fmaf(delta, kv[c].x, e.x); e.y = fmaf(delta, kv[c].y, e.y);
        e.z = fmaf(delta, kv[c].z, e.z); e.w = fmaf(delta, kv[c].w, e.w);
        o = fmaf(e.x, qv[c].x, o); o = fmaf(e.y, qv[c].y, o); o = fmaf(e.z, qv[c].z, o); o = fmaf(e.w, qv[c].w, o);
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      ob[i] = __bfloat162float(__float2bfloat16(o));       // the recurrence output is stored in bf16
      if (l8 == 0) ss = fmaf(ob[i], ob[i], ss);            // every row counted once
    }
    // gated RMSNorm over the head's 128 outputs
    ss = warp_sum(ss);
    if (lane == 0) red[1 + (t & 1)][tid >> 5] = ss;
    __syncthreads();
    if (l8 == 0) {
      const float* rr = red[1 + (t & 1)];
      const float tot = rr[0] + rr[1] + rr[2] + rr[3] + rr[4] + rr[5] + rr[6] + rr[7];
      const float inv = rsqrtf(tot * (1.f / kGdnDim) + p.eps_norm);
      __nv_bfloat16* orow = p.out + static_cast<size_t>(row0 + t) * p.ldo + head * kGdnDim + vrow;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float normed = __bfloat162float(__float2bfloat16(ob[i] * inv));
        orow[4 * i] = __float2bfloat16(normed * nw[i] * silu_fast(zz[i]));
      }
    }
  }
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
                const CbGdnSegments* seg, int C, void* stream) {
  if (!seg || seg->num <= 0 || C <= 0 || seg->num > 65535) return -60;
  cb::GdnSegments s{static_cast<const int*>(seg->row0), static_cast<const int*>(seg->count),
                    static_cast<const int*>(seg->slot), static_cast<const int*>(seg->pos0)};
  dim3 grid((C + 127) / 128, seg->num);
  cb::gdn_conv_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_bfloat16*>(y), ldy, static_cast<const float*>(w),
      static_cast<const float*>(bias), static_cast<__nv_bfloat16*>(state), s, C);
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
