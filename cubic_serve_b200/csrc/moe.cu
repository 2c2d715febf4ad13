// Mixture-of-experts routing: stable top-k, per-expert counts, permutation, gather, weighted combine.
//
// Counterparts in the reference: ops/cuda/moe/fused.py (_stable_topk_logits :44,
// _sort_and_normalize_topk :71, _count/_prefix/_scatter_local_routes :159-222,
// _route_combine :444).  Semantics kept: top-k over router logits with the
// lowest expert id winning ties, softmax over the SELECTED logits only
// (= softmax over all experts renormalised to the top-k), routes of one expert
// contiguous for the grouped GEMM (wq_gemm.cu, grouped mode), combine in fixed
// route order per token so the result does not depend on the permutation.
//
// Expert parallelism: `expert_lo / expert_count` select the experts THIS rank
// owns; routes to other experts get position -1 and contribute +0 (the
// reference's replicated-token EP, runtime/README.md:140-160 there), so the same
// kernels serve EP = 1 and the EP shards whose partial outputs are then reduced
// like any row-parallel partial sum.
#include "ptx.cuh"

namespace cb {

static constexpr int kMaxTopK = 8;

// One warp per token: E <= 256 experts, lane l holds experts l, l+32, ...
__global__ void __launch_bounds__(128)
moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int T, int E, int k, int normalize,
                 int expert_lo, int expert_count, int* __restrict__ topk_ids, float* __restrict__ topk_w,
                 int* __restrict__ counts) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? __bfloat162float(logits[static_cast<size_t>(t) * ld + e]) : -INFINITY;
    if (!(v[j] == v[j])) v[j] = -INFINITY;
  }
  float sel_v[kMaxTopK];
  int sel_e[kMaxTopK];
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      if (v[j] > bv || (v[j] == bv && e < be)) { bv = v[j]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    sel_v[r] = bv;
    sel_e[r] = be;
    if ((be & 31) == lane) v[be >> 5] = -INFINITY;   // remove the winner
  }
  if (lane == 0) {
    float w[kMaxTopK], sum = 0.f;
    for (int r = 0; r < k; ++r) { w[r] = __expf(sel_v[r] - sel_v[0]); sum += w[r]; }
    // normalize = 1: softmax over the selected logits.  normalize = 0: softmax over ALL experts, not
    // renormalised: needs the full denominator
    float denom = sum;
    if (!normalize) {
      denom = 0.f;
      for (int e = 0; e < E; ++e) denom += __expf(__bfloat162float(logits[static_cast<size_t>(t) * ld + e]) - sel_v[0]);
    }
    for (int r = 0; r < k; ++r) {
      topk_ids[t * k + r] = sel_e[r];
      topk_w[t * k + r] = w[r] / denom;
      const int local = sel_e[r] - expert_lo;
      if (local >= 0 && local < expert_count) atomicAdd(&counts[local], 1);
    }
  }
}

// Single CTA: exclusive scan of the counts -> offsets (cursors start there), and the work list of the grouped
// GEMM: one item per (expert, block of `mb` rows) = {expert, first row, rows}; at most ceil(routes / mb) + E items.
__global__ void __launch_bounds__(256)
moe_scan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursors, int E, int mb,
                int* __restrict__ total, int* __restrict__ tiles /* [0] = count, then {expert,row0,rows} triples */) {
  __shared__ int sm[256];
  __shared__ int st[256];
  const int e = threadIdx.x;
  const int cnt = e < E ? counts[e] : 0;
  const int nt = (cnt + mb - 1) / mb;
  sm[e] = cnt;
  st[e] = nt;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {
    const int a = e >= o ? sm[e - o] : 0;
    const int b = e >= o ? st[e - o] : 0;
    __syncthreads();
    sm[e] += a;
    st[e] += b;
    __syncthreads();
  }
  if (e < E) {
    const int off = sm[e] - cnt;
    offsets[e] = off;
    cursors[e] = off;
    const int t0 = st[e] - nt;
    for (int i = 0; i < nt; ++i) {
      tiles[1 + 3 * (t0 + i)] = e;
      tiles[2 + 3 * (t0 + i)] = off + i * mb;
      tiles[3 + 3 * (t0 + i)] = min(mb, cnt - i * mb);
    }
  }
  if (e == 255) {
    *total = sm[255];
    tiles[0] = st[255];
  }
}

// One warp per route: claim a slot in the expert's range and copy the token's row there.
__global__ void __launch_bounds__(128)
moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_ids, int T, int k, int H,
                   int expert_lo, int expert_count, int* __restrict__ cursors, int* __restrict__ route_pos,
                   __nv_bfloat16* __restrict__ xs) {
  const int route = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (route >= T * k) return;
  const int local = topk_ids[route] - expert_lo;
  int pos = -1;
  if (local >= 0 && local < expert_count) {
    if (lane == 0) pos = atomicAdd(&cursors[local], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    const int t = route / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
    uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(pos) * H);
    for (int i = lane; i < (H >> 3); i += 32) dst[i] = src[i];
  }
  if (lane == 0) route_pos[route] = pos;
}

// out[t] (+)= sum_r w[t, r] * y[route_pos[t, r]]   (fixed r order; absent routes contribute +0)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_pos,
                   const float* __restrict__ topk_w, int k, int H, const __nv_bfloat16* residual,
                   __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < k; ++r) {
      const int pos = route_pos[t * k + r];
      if (pos < 0) continue;
      const float w = topk_w[t * k + r];
      const uint4 yv = reinterpret_cast<const uint4*>(y + static_cast<size_t>(pos) * H)[v];
      const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(yp[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    if (residual) {
      const uint4 rv = reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H)[v];
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(rp[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 ov;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[v] = ov;
  }
}

}  // namespace cb

extern "C" {

// Routing + permutation in one call: zeroes the counts, selects the top-k, scans, scatters the rows.
// Buffers: topk_ids [T,k] i32, topk_w [T,k] f32, counts/offsets/cursors [expert_count] i32, total [1] i32,
// tiles [1 + 3 * (ceil(T*k / mb) + expert_count)] i32 (work list of the grouped GEMM with `mb` rows per item),
// route_pos [T,k] i32, xs [T*k, H] bf16 (rows of owned routes, expert-major).
int cb_moe_route(const void* logits, int ld, const void* x, int T, int E, int k, int H, int normalize, int expert_lo,
                 int expert_count, int mb, void* topk_ids, void* topk_w, void* counts, void* offsets, void* cursors,
                 void* total, void* tiles, void* route_pos, void* xs, void* stream) {
  using namespace cb;
  if (T <= 0) return 0;
  if (E > 256 || k > kMaxTopK || k < 1 || H % 8 != 0 || expert_count > 256) return -10;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * expert_count, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  moe_route_kernel<<<(T + 3) / 4, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, T, E, k, normalize,
                                                 expert_lo, expert_count, static_cast<int*>(topk_ids),
                                                 static_cast<float*>(topk_w), static_cast<int*>(counts));
  moe_scan_kernel<<<1, 256, 0, st>>>(static_cast<const int*>(counts), static_cast<int*>(offsets),
                                     static_cast<int*>(cursors), expert_count, mb, static_cast<int*>(total),
                                     static_cast<int*>(tiles));
  moe_scatter_kernel<<<(T * k + 3) / 4, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                       static_cast<const int*>(topk_ids), T, k, H, expert_lo,
                                                       expert_count, static_cast<int*>(cursors),
                                                       static_cast<int*>(route_pos), static_cast<__nv_bfloat16*>(xs));
  return static_cast<int>(cudaGetLastError());
}

// Scan + permutation only, for callers that have already filled topk_ids ([T,k], -1 = no route) and counts
// (expert-parallel receive side: the "tokens" are the records received from the other ranks).
int cb_moe_permute(const void* x, const void* topk_ids, int T, int k, int H, int expert_lo, int expert_count, int mb,
                   const void* counts, void* offsets, void* cursors, void* total, void* tiles, void* route_pos,
                   void* xs, void* stream) {
  using namespace cb;
  if (T <= 0) return 0;
  if (k > kMaxTopK || k < 1 || H % 8 != 0 || expert_count > 256) return -10;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  moe_scan_kernel<<<1, 256, 0, st>>>(static_cast<const int*>(counts), static_cast<int*>(offsets),
                                     static_cast<int*>(cursors), expert_count, mb, static_cast<int*>(total),
                                     static_cast<int*>(tiles));
  moe_scatter_kernel<<<(T * k + 3) / 4, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                       static_cast<const int*>(topk_ids), T, k, H, expert_lo,
                                                       expert_count, static_cast<int*>(cursors),
                                                       static_cast<int*>(route_pos), static_cast<__nv_bfloat16*>(xs));
  return static_cast<int>(cudaGetLastError());
}

int cb_moe_combine(const void* y, const void* route_pos, const void* topk_w, int T, int k, int H, const void* residual,
                   void* out, void* stream) {
  using namespace cb;
  if (T <= 0) return 0;
  if (H % 8 != 0) return -10;
  moe_combine_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), static_cast<const int*>(route_pos), static_cast<const float*>(topk_w), k, H,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
