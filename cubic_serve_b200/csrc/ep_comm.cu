// Expert-parallel dispatch / combine over NVLink peer memory, fused with the router's top-k and the permutation.
//
// Reference behaviour being replaced: the eager EP reference dispatches rows to expert owners and combines them
// with NCCL all-to-all (models/qwen3_5_moe/distributed.py:191, executor/parallel/nccl.py ep_dispatch/combine);
// the serving path there keeps tokens replicated and all-reduces partial outputs.  Here the residual stream is
// ROW-SHARDED across the ranks (as in the fused tensor-parallel path, tp_comm.cu), and a MoE block is:
//
//   ep_dispatch     (home rank of a token)  top-k over the router logits; for every rank that owns at least one
//                   selected expert: claim a slot in that rank's receive region for this source, store the
//                   normalised activation row and its {expert ids, weights} there with P2P stores; after the
//                   last row, publish the per-destination counts and raise the destinations' arrival counters
//   ep_unpack       (expert owner)  wait (bounded) for every source's counter; turn the received records into
//                   the {token, top-k ids, weights} arrays of cb_moe_permute and count routes per local expert
//   cb_moe_permute + grouped tcgen05 GEMMs (moe.cu, wq_gemm.cu)  unchanged
//   ep_combine_push (expert owner)  per received token: sum_r w_r * y[route r] over ITS local routes in route
//                   order, one bf16 row back into the home rank's return region (slot = the slot it came in)
//   ep_finish       (home rank)  wait for every rank's return counter; h[row] += sum over ranks IN ASCENDING
//                   RANK ORDER of the returned rows (deterministic), rounded like the tensor-parallel sum
//
// A token row crosses NVLink once per destination rank (not once per route), and only to ranks that own one of
// its experts; nothing is all-gathered or all-reduced.  Plain P2P loads/stores only (no multimem, no TMA from
// peer memory).  Counters only increase; consumers keep the number of arrivals already consumed (tp_comm.cu).
#include "ptx.cuh"

namespace cb {

static constexpr int kEpMaxRanks = 8;
static constexpr int kEpMaxTopK = 8;

__device__ __forceinline__ uint32_t ep_ld_acq(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ep_red_rel(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool ep_wait_ge(const uint32_t* p, uint32_t target) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ep_ld_acq(p) - target) < 0) {
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
  return true;
}

struct EpDispatchParams {
  const __nv_bfloat16* logits;   // [cnt, ld] router logits of this rank's rows
  const __nv_bfloat16* x;        // [cnt, H] normalised rows
  int ld, cnt, E, k, H, normalize, experts_per_rank;
  int rank, size, cap;           // cap = rows a source may send (= rows_per_rank capacity of the regions)
  __nv_bfloat16* xin_peer[kEpMaxRanks];   // every rank's receive rows    [size][cap][H]
  int* ids_peer[kEpMaxRanks];             // every rank's received ids    [size][cap][k]
  float* w_peer[kEpMaxRanks];             // every rank's received weights [size][cap][k]
  int* cnt_peer[kEpMaxRanks];             // every rank's per-source counts [size]
  uint32_t* flag_peer[kEpMaxRanks];       // every rank's dispatch arrival counters [size]
  int* local_cnt;                // [size] slots claimed per destination; zero on entry, zero on exit
  int* sent;                     // [cap][size] slot of the row at each destination, -1 = not sent there
  uint32_t* done;                // CTA counter; zero on entry, zero on exit
};

// One warp per token (E <= 256, lane l holds experts l, l + 32, ...), as moe_route_kernel.
__global__ void __launch_bounds__(128)
ep_dispatch_kernel(const EpDispatchParams p) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t < p.cnt) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < p.E ? __bfloat162float(p.logits[static_cast<size_t>(t) * p.ld + e]) : -INFINITY;
      if (!(v[j] == v[j])) v[j] = -INFINITY;
    }
    float sel_v[kEpMaxTopK];
    int sel_e[kEpMaxTopK];
#pragma unroll
    for (int r = 0; r < kEpMaxTopK; ++r) { sel_v[r] = -INFINITY; sel_e[r] = -1; }
#pragma unroll
    for (int r = 0; r < kEpMaxTopK; ++r) {
      if (r >= p.k) break;
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
    // weights: softmax over the selected logits, or over all experts (then the full denominator is needed)
    float w[kEpMaxTopK], sum = 0.f;
#pragma unroll
    for (int r = 0; r < kEpMaxTopK; ++r) { w[r] = r < p.k ? __expf(sel_v[r] - sel_v[0]) : 0.f; sum += w[r]; }
    float denom = sum;
    if (!p.normalize) {
      float part = 0.f;
      for (int e = lane; e < p.E; e += 32) part += __expf(__bfloat162float(p.logits[static_cast<size_t>(t) * p.ld + e]) - sel_v[0]);
      denom = warp_sum(part);
    }
    // lane d claims the slot at destination d
    int slot = -1;
    if (lane < p.size) {
      bool has = false;
#pragma unroll
      for (int r = 0; r < kEpMaxTopK; ++r) has = has || (r < p.k && sel_e[r] / p.experts_per_rank == lane);
      if (has) slot = atomicAdd(&p.local_cnt[lane], 1);
      p.sent[t * p.size + lane] = slot;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t) * p.H);
    for (int d = 0; d < p.size; ++d) {
      const int s = __shfl_sync(0xffffffffu, slot, d);
      if (s < 0) continue;
      const size_t rec = static_cast<size_t>(p.rank) * p.cap + s;
      uint4* dst = reinterpret_cast<uint4*>(p.xin_peer[d] + rec * p.H);
      for (int i = lane; i < (p.H >> 3); i += 32) dst[i] = src[i];
#pragma unroll
      for (int r = 0; r < kEpMaxTopK; ++r) {
        if (r < p.k && lane == r) {
          p.ids_peer[d][rec * p.k + r] = sel_e[r];
          p.w_peer[d][rec * p.k + r] = w[r] / denom;
        }
      }
    }
  }
  // every row of this CTA is on its way: CTA barrier, count the CTA in (acquire-release); the last CTA
  // publishes the per-destination counts and raises the arrival counters with a release at system scope
  __syncthreads();
  __shared__ uint32_t is_last;
  if (threadIdx.x == 0) is_last = atom_add_acq_rel_gpu(p.done, 1u) == gridDim.x - 1u ? 1u : 0u;
  __syncthreads();
  if (is_last && threadIdx.x < p.size) {
    // the release below is cumulative: it covers the rows of every CTA (release sequence on `done`, CTA barriers)
    const int c = atomicExch(&p.local_cnt[threadIdx.x], 0);
    p.cnt_peer[threadIdx.x][p.rank] = c;
    ep_red_rel(p.flag_peer[threadIdx.x] + p.rank, 1u);
    if (threadIdx.x == 0) *p.done = 0;
  }
}

struct EpUnpackParams {
  const int* ids_in;       // local [size][cap][k]
  const float* w_in;       // local [size][cap][k]
  const int* cnt_in;       // local [size]
  const uint32_t* flag;    // local dispatch arrival counters [size]
  uint32_t* state;         // local {arrivals consumed so far, done CTAs}
  int size, cap, k, expert_lo, expert_count;
  int* topk_ids;           // out [size * cap][k]   (-1 for records that do not exist)
  float* topk_w;           // out [size * cap][k]
  int* counts;             // out [expert_count], zero on entry
  uint32_t* status;
};

__global__ void __launch_bounds__(256)
ep_unpack_kernel(const EpUnpackParams p) {
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < p.size) {
    if (!ep_wait_ge(p.flag + threadIdx.x, p.state[0] + 1u)) ok_flag = 0;
  }
  __syncthreads();
  const bool ok = ok_flag != 0;
  const int te = blockIdx.x * blockDim.x + threadIdx.x;
  if (te < p.size * p.cap) {
    const int src = te / p.cap;
    const int slot = te - src * p.cap;
    const bool valid = ok && slot < __ldcg(p.cnt_in + src);
    for (int r = 0; r < p.k; ++r) {
      const int id = valid ? __ldcg(p.ids_in + static_cast<size_t>(te) * p.k + r) : -1;
      p.topk_ids[static_cast<size_t>(te) * p.k + r] = id;
      p.topk_w[static_cast<size_t>(te) * p.k + r] = valid ? __ldcg(p.w_in + static_cast<size_t>(te) * p.k + r) : 0.f;
      const int local = id - p.expert_lo;
      if (id >= 0 && local >= 0 && local < p.expert_count) atomicAdd(&p.counts[local], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) atomicExch(p.status, static_cast<uint32_t>(kErrFlagTimeout));
    if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1u) {
      p.state[1] = 0;
      __threadfence();
      atomicAdd(&p.state[0], 1u);      // every CTA of this launch has read the old value by now
    }
  }
}

struct EpCombineParams {
  const __nv_bfloat16* y;        // [routes][H] expert outputs, expert-major (moe_permute order)
  const int* route_pos;          // [size * cap][k]
  const float* topk_w;           // [size * cap][k]
  const int* cnt_in;             // [size]
  int size, cap, k, H, rank;
  __nv_bfloat16* yin_peer[kEpMaxRanks];   // every rank's return rows [size][cap][H]
  uint32_t* flag_peer[kEpMaxRanks];       // every rank's return arrival counters [size]
  uint32_t* done;
};

// One CTA per received record: weighted sum over its local routes (fixed route order), one row back home.
__global__ void __launch_bounds__(256)
ep_combine_push_kernel(const EpCombineParams p) {
  const int te = blockIdx.x;
  const int src = te / p.cap;
  const int slot = te - src * p.cap;
  if (slot < p.cnt_in[src]) {
    __nv_bfloat16* dst = p.yin_peer[src] + (static_cast<size_t>(p.rank) * p.cap + slot) * p.H;
    for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < p.k; ++r) {
        const int pos = p.route_pos[static_cast<size_t>(te) * p.k + r];
        if (pos < 0) continue;
        const float w = p.topk_w[static_cast<size_t>(te) * p.k + r];
        const uint4 yv = reinterpret_cast<const uint4*>(p.y + static_cast<size_t>(pos) * p.H)[v];
        const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(yp[j]);
          acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
          acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
        }
      }
      uint4 ov;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      reinterpret_cast<uint4*>(dst)[v] = ov;
    }
  }
  __syncthreads();
  __shared__ uint32_t is_last;
  if (threadIdx.x == 0) is_last = atom_add_acq_rel_gpu(p.done, 1u) == gridDim.x - 1u ? 1u : 0u;
  __syncthreads();
  if (is_last && threadIdx.x < p.size) {
    ep_red_rel(p.flag_peer[threadIdx.x] + p.rank, 1u);
    if (threadIdx.x == 0) *p.done = 0;
  }
}

struct EpFinishParams {
  const __nv_bfloat16* yin;      // local [size][cap][H]
  const int* sent;               // [cap][size]
  const uint32_t* flag;          // local return arrival counters [size]
  uint32_t* state;               // {consumed, done CTAs}
  __nv_bfloat16* h;              // local residual rows [cnt][H], read-modify-write
  int size, cap, H, cnt;
  uint32_t* status;
};

__global__ void __launch_bounds__(256)
ep_finish_kernel(const EpFinishParams p) {
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < p.size) {
    if (!ep_wait_ge(p.flag + threadIdx.x, p.state[0] + 1u)) ok_flag = 0;
  }
  __syncthreads();
  const bool ok = ok_flag != 0;
  const int row = blockIdx.x;
  if (ok && row < p.cnt) {
    for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int d = 0; d < p.size; ++d) {            // ascending rank order, fp32
        const int slot = p.sent[row * p.size + d];
        if (slot < 0) continue;
        const uint4 yv = __ldcg(reinterpret_cast<const uint4*>(p.yin + (static_cast<size_t>(d) * p.cap + slot) * p.H) + v);
        const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(yp[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 hv = reinterpret_cast<const uint4*>(p.h + static_cast<size_t>(row) * p.H)[v];
      const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&hv);
      uint4 ov;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // bf16(residual + bf16(sum)): the rounding points of the tensor-parallel sum
        const float2 s = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
        const float2 hh = __bfloat1622float2(hp[j]);
        op[j] = __floats2bfloat162_rn(hh.x + s.x, hh.y + s.y);
      }
      reinterpret_cast<uint4*>(p.h + static_cast<size_t>(row) * p.H)[v] = ov;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) atomicExch(p.status, static_cast<uint32_t>(kErrFlagTimeout));
    if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1u) {
      p.state[1] = 0;
      __threadfence();
      atomicAdd(&p.state[0], 1u);
    }
  }
}

}  // namespace cb

extern "C" {

struct CbEpDispatch {
  const void* logits; const void* x; int ld, cnt, E, k, H, normalize, experts_per_rank, rank, size, cap;
  void* xin_peer[8]; void* ids_peer[8]; void* w_peer[8]; void* cnt_peer[8]; void* flag_peer[8];
  void* local_cnt; void* sent; void* done;
};

int cb_ep_dispatch(const CbEpDispatch* a, void* stream) {
  using namespace cb;
  if (a->size < 1 || a->size > kEpMaxRanks || a->k < 1 || a->k > kEpMaxTopK || a->E > 256 || a->H % 8 != 0 ||
      a->cnt > a->cap || a->experts_per_rank * a->size != a->E)
    return -10;
  EpDispatchParams p;
  p.logits = static_cast<const __nv_bfloat16*>(a->logits);
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.ld = a->ld; p.cnt = a->cnt; p.E = a->E; p.k = a->k; p.H = a->H; p.normalize = a->normalize;
  p.experts_per_rank = a->experts_per_rank; p.rank = a->rank; p.size = a->size; p.cap = a->cap;
  for (int r = 0; r < a->size; ++r) {
    p.xin_peer[r] = static_cast<__nv_bfloat16*>(a->xin_peer[r]);
    p.ids_peer[r] = static_cast<int*>(a->ids_peer[r]);
    p.w_peer[r] = static_cast<float*>(a->w_peer[r]);
    p.cnt_peer[r] = static_cast<int*>(a->cnt_peer[r]);
    p.flag_peer[r] = static_cast<uint32_t*>(a->flag_peer[r]);
  }
  p.local_cnt = static_cast<int*>(a->local_cnt);
  p.sent = static_cast<int*>(a->sent);
  p.done = static_cast<uint32_t*>(a->done);
  const int ctas = a->cnt > 0 ? (a->cnt + 3) / 4 : 1;      // a rank without rows still reports zero counts
  ep_dispatch_kernel<<<ctas, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// Zeroes `counts`, waits for the dispatch of every source and fills topk_ids / topk_w / counts for
// cb_moe_permute over size * cap virtual tokens.
int cb_ep_unpack(const void* ids_in, const void* w_in, const void* cnt_in, const void* flag, void* state, int size,
                 int cap, int k, int expert_lo, int expert_count, void* topk_ids, void* topk_w, void* counts,
                 void* status, void* stream) {
  using namespace cb;
  if (size < 1 || size > kEpMaxRanks || cap < 1 || k < 1 || k > kEpMaxTopK) return -10;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * expert_count, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  EpUnpackParams p;
  p.ids_in = static_cast<const int*>(ids_in);
  p.w_in = static_cast<const float*>(w_in);
  p.cnt_in = static_cast<const int*>(cnt_in);
  p.flag = static_cast<const uint32_t*>(flag);
  p.state = static_cast<uint32_t*>(state);
  p.size = size; p.cap = cap; p.k = k; p.expert_lo = expert_lo; p.expert_count = expert_count;
  p.topk_ids = static_cast<int*>(topk_ids);
  p.topk_w = static_cast<float*>(topk_w);
  p.counts = static_cast<int*>(counts);
  p.status = static_cast<uint32_t*>(status);
  ep_unpack_kernel<<<(size * cap + 255) / 256, 256, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

struct CbEpCombine {
  const void* y; const void* route_pos; const void* topk_w; const void* cnt_in; int size, cap, k, H, rank;
  void* yin_peer[8]; void* flag_peer[8]; void* done;
};

int cb_ep_combine_push(const CbEpCombine* a, void* stream) {
  using namespace cb;
  if (a->size < 1 || a->size > kEpMaxRanks || a->H % 8 != 0) return -10;
  EpCombineParams p;
  p.y = static_cast<const __nv_bfloat16*>(a->y);
  p.route_pos = static_cast<const int*>(a->route_pos);
  p.topk_w = static_cast<const float*>(a->topk_w);
  p.cnt_in = static_cast<const int*>(a->cnt_in);
  p.size = a->size; p.cap = a->cap; p.k = a->k; p.H = a->H; p.rank = a->rank;
  for (int r = 0; r < a->size; ++r) {
    p.yin_peer[r] = static_cast<__nv_bfloat16*>(a->yin_peer[r]);
    p.flag_peer[r] = static_cast<uint32_t*>(a->flag_peer[r]);
  }
  p.done = static_cast<uint32_t*>(a->done);
  ep_combine_push_kernel<<<a->size * a->cap, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int cb_ep_finish(const void* yin, const void* sent, const void* flag, void* state, void* h, int size, int cap, int H,
                 int cnt, void* status, void* stream) {
  using namespace cb;
  if (size < 1 || size > kEpMaxRanks || H % 8 != 0 || cnt > cap) return -10;
  EpFinishParams p;
  p.yin = static_cast<const __nv_bfloat16*>(yin);
  p.sent = static_cast<const int*>(sent);
  p.flag = static_cast<const uint32_t*>(flag);
  p.state = static_cast<uint32_t*>(state);
  p.h = static_cast<__nv_bfloat16*>(h);
  p.size = size; p.cap = cap; p.H = H; p.cnt = cnt;
  p.status = static_cast<uint32_t*>(status);
  ep_finish_kernel<<<cnt > 0 ? cnt : 1, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
