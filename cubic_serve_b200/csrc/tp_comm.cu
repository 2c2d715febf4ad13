// Tensor-parallel glue kernels over NVLink peer memory (plain P2P loads/stores,
// release/acquire flags at system scope, every wait bounded).
//
// Together with the scatter-push / gather-wait modes of wq_gemm.cu they replace
// the reference's "all_gather_single + ordered rank-sum (+ residual + RMSNorm)"
// sequence (ops/cuda/collective/fixed_rank_sum.py:350-373,596-722) with a
// reduce-scatter -> norm -> all-gather pipeline that moves the minimum number of
// bytes over the links and has no NCCL call:
//
//   row-parallel GEMM  --(epilogue pushes partial rows to their owner)-->
//   tp_reduce_norm     : owner waits for all partials, sums them in ASCENDING
//                        RANK ORDER in fp32 (the reference's determinism
//                        contract), adds the residual it keeps for its rows,
//                        applies RMSNorm and pushes the normalised rows to every
//                        rank's gathered activation buffer
//   column-parallel GEMM waits for all rows (inside its producer warp).
//
// Counters only ever increase; a consumer keeps the cumulative number of arrivals
// it has already consumed in its own state word and waits for (consumed +
// expected of this launch), so nothing is reset while a peer may still write and
// the expected count may differ from launch to launch (prefill vs decode shapes).
#include "ptx.cuh"
#include "launch.cuh"

namespace cb {

static constexpr int kMaxRanksTp = 8;

__device__ __forceinline__ uint32_t ld_acq_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_rel_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool wait_ge(const uint32_t* p, uint32_t target) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ld_acq_sys(p) - target) < 0) {
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
  return true;
}

// NVLS: one instruction addressed to a multicast mapping of a symmetric buffer acts on every rank's copy, inside the
// NVSwitch.  The sum of `multimem.ld_reduce` is accumulated in fp32 and rounded once to bf16, like the ordered sum it
// replaces, but in an order the switch chooses: results may differ in the last bit from run to run.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

struct ReduceNormParams {
  const __nv_bfloat16* recv;     // local [size][rows_per_rank][H] partial rows, slot = source rank
  const uint32_t* rs_flag;       // local arrival counters [size]
  uint32_t* rs_state;            // local {arrivals consumed so far, done CTAs}
  uint32_t rs_expected;          // arrivals per source per epoch; 0 = nothing to reduce (input is h itself)
  __nv_bfloat16* h;              // local residual rows [rows_per_rank][H] (read-modify-write)
  const __nv_bfloat16* norm_w;   // [H]
  __nv_bfloat16* x_peer[kMaxRanksTp];   // every rank's gathered activations [M_pad][H]
  uint32_t* ag_flag_peer[kMaxRanksTp];  // every rank's gather arrival counters [size]
  uint32_t* status;
  int rank, size, rows_per_rank, H, M;
  float eps;
  int zero_centered;
  int local_only;                // 1: keep the normalised rows on this rank (no all-gather, no counters); the
                                 // consumer is a later kernel of the same stream (expert-parallel dispatch)
  // NVLS forms (null = plain peer loads / stores):
  const __nv_bfloat16* recv_mc;  // multicast mapping of the partial-sum buffers, every rank's laid out [M_pad][H] by
                                 // GLOBAL row (the GEMMs wrote their partial rows locally): one ld_reduce per 16 bytes
                                 // sums all ranks' partials in the switch
  __nv_bfloat16* x_mc;           // multicast mapping of the gathered activation buffers: one store reaches every rank
};

static constexpr int kRnThreads = 256;
static constexpr int kRnMaxVec = 4;  // H <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(kRnThreads)
tp_reduce_norm_kernel(const ReduceNormParams p) {
  __shared__ float red[8];
  __shared__ uint32_t ok_flag;
  const int row = blockIdx.x;
  const int m = p.rank * p.rows_per_rank + row;
  if (threadIdx.x == 0) ok_flag = 1;
  pdl_launch_dependents();
  pdl_wait();                     // the residual rows and the counters' base are written by earlier kernels of this GPU
  __syncthreads();
  if (p.rs_expected) {
    if (threadIdx.x < p.size) {
      const uint32_t target = p.rs_state[0] + p.rs_expected;
      if (!wait_ge(p.rs_flag + threadIdx.x, target)) ok_flag = 0;
    }
    __syncthreads();
  }
  const bool ok = ok_flag != 0;
  const int nvec = p.H >> 3;
  if (ok && m < p.M) {
    float vals[kRnMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kRnMaxVec; ++it) {
      const int v = threadIdx.x + it * kRnThreads;
      if (v < nvec) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        uint4 hv = reinterpret_cast<const uint4*>(p.h + static_cast<size_t>(row) * p.H)[v];
        if (p.rs_expected && p.recv_mc) {
          const uint4 pv = multimem_ld_reduce_bf16x8(p.recv_mc + static_cast<size_t>(m) * p.H + static_cast<size_t>(v) * 8);
          const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&pv);
          const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&hv);
          uint4 ov;
          __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 sm = __bfloat1622float2(pp[j]);            // bf16(sum), rounded by the switch
            const float2 hh = __bfloat1622float2(hp[j]);
            op[j] = __floats2bfloat162_rn(hh.x + sm.x, hh.y + sm.y);
          }
          reinterpret_cast<uint4*>(p.h + static_cast<size_t>(row) * p.H)[v] = ov;
          hv = ov;
        } else if (p.rs_expected) {
          // all ranks' partial vectors are requested before the first is used (the loads are independent; a loop
          // with a run-time bound would issue them one round trip at a time), then summed in ascending rank order
          uint4 pv[kMaxRanksTp];
#pragma unroll
          for (int r = 0; r < kMaxRanksTp; ++r)
            if (r < p.size)
              pv[r] = __ldcg(reinterpret_cast<const uint4*>(p.recv + (static_cast<size_t>(r) * p.rows_per_rank + row) * p.H) + v);
#pragma unroll
          for (int r = 0; r < kMaxRanksTp; ++r) {
            if (r < p.size) {
              const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&pv[r]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(pp[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
              }
            }
          }
          // bf16(residual + bf16(sum)), the reference's rounding points
          const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&hv);
          uint4 ov;
          __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 s = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
            const float2 hh = __bfloat1622float2(hp[j]);
            op[j] = __floats2bfloat162_rn(hh.x + s.x, hh.y + s.y);
          }
          reinterpret_cast<uint4*>(p.h + static_cast<size_t>(row) * p.H)[v] = ov;
          hv = ov;
        }
        const __nv_bfloat162* hp2 = reinterpret_cast<const __nv_bfloat162*>(&hv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(hp2[j]);
          vals[it][2 * j] = f.x;
          vals[it][2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    // block reduction of the sum of squares
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = (threadIdx.x & 31) < (kRnThreads >> 5) ? red[threadIdx.x & 31] : 0.f;
    tot = warp_sum(tot);
    const float inv = rsqrtf(tot / static_cast<float>(p.H) + p.eps);
#pragma unroll
    for (int it = 0; it < kRnMaxVec; ++it) {
      const int v = threadIdx.x + it * kRnThreads;
      if (v < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(p.norm_w)[v];
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
        uint4 ov;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 ww = __bfloat1622float2(wp[j]);
          if (p.zero_centered) { ww.x += 1.f; ww.y += 1.f; }
          op[j] = __floats2bfloat162_rn(vals[it][2 * j] * inv * ww.x, vals[it][2 * j + 1] * inv * ww.y);
        }
        // all-gather by push: the same 16 bytes to every rank's buffer (self included)
        if (p.local_only) {
          reinterpret_cast<uint4*>(p.x_peer[p.rank] + static_cast<size_t>(m) * p.H)[v] = ov;
        } else if (p.x_mc) {
          multimem_st_16(p.x_mc + static_cast<size_t>(m) * p.H + static_cast<size_t>(v) * 8, ov);
        } else {
          for (int r = 0; r < p.size; ++r)
            reinterpret_cast<uint4*>(p.x_peer[r] + static_cast<size_t>(m) * p.H)[v] = ov;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < p.size && !p.local_only) {
    // release at system scope, cumulative: covers the row pushed by the whole CTA (ordered by the barrier above)
    red_rel_sys_add(p.ag_flag_peer[threadIdx.x] + p.rank, 1u);
  }
  if (threadIdx.x == 0) {
    if (!ok) atomicExch(p.status, static_cast<uint32_t>(kErrFlagTimeout));
    if (p.rs_expected) {
      if (atomicAdd(&p.rs_state[1], 1u) == gridDim.x - 1u) {
        p.rs_state[1] = 0;
        __threadfence();
        atomicAdd(&p.rs_state[0], p.rs_expected);   // every CTA of this launch has read the old value by now
      }
    }
  }
}

// Stand-alone wait for a gathered buffer (for consumers that are not the GEMM).
__global__ void tp_wait_kernel(const uint32_t* ag_flag, uint32_t* ag_state, uint32_t expected, int size,
                               uint32_t* status) {
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  pdl_launch_dependents();
  pdl_wait();
  __syncthreads();
  if (threadIdx.x < size) {
    if (!wait_ge(ag_flag + threadIdx.x, ag_state[0] + expected)) ok_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok_flag) atomicExch(status, static_cast<uint32_t>(kErrFlagTimeout));
    atomicAdd(&ag_state[0], expected);
  }
}

// Vocab-sharded greedy merge: every rank publishes its local (best logit, global id) per row
// to all ranks, then each rank takes the best over ranks (ties: lowest id), so all ranks agree.
struct ArgmaxMergeParams {
  const float* local_val;    // [rows]
  const int* local_id;       // [rows] already global ids
  float* slot_val[kMaxRanksTp];   // every rank's exchange area [size][rows_max]
  int* slot_id[kMaxRanksTp];
  uint32_t* flag_peer[kMaxRanksTp];  // every rank's counters [size]
  const float* my_val;       // local exchange area
  const int* my_id;
  const uint32_t* my_flag;
  uint32_t* my_state;        // {epoch}
  int* out_id;               // [rows]
  uint32_t* status;
  int rank, size, rows, rows_max;
};

__global__ void __launch_bounds__(256)
tp_argmax_merge_kernel(const ArgmaxMergeParams p) {
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < p.rows; i += blockDim.x) {
    const float v = p.local_val[i];
    const int id = p.local_id[i];
    for (int r = 0; r < p.size; ++r) {
      p.slot_val[r][p.rank * p.rows_max + i] = v;
      p.slot_id[r][p.rank * p.rows_max + i] = id;
    }
  }
  __syncthreads();
  if (threadIdx.x < p.size) {
    red_rel_sys_add(p.flag_peer[threadIdx.x] + p.rank, 1u);
    if (!wait_ge(p.my_flag + threadIdx.x, p.my_state[0] + 1u)) ok_flag = 0;
  }
  __syncthreads();
  if (ok_flag) {
    for (int i = threadIdx.x; i < p.rows; i += blockDim.x) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int r = 0; r < p.size; ++r) {
        const float v = __ldcg(p.my_val + r * p.rows_max + i);
        const int id = __ldcg(p.my_id + r * p.rows_max + i);
        if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
      }
      p.out_id[i] = bi;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok_flag) atomicExch(p.status, static_cast<uint32_t>(kErrFlagTimeout));
    atomicAdd(&p.my_state[0], 1u);
  }
}

// Small all-gather by push: every rank stores `segments` runs of `seg_words` 32-bit words (run g starts at
// local + g * seg_stride) into slot `rank` of every rank's exchange area (same inner layout), raises the peers'
// counters and waits for all of theirs, so that when the kernel ends the local area holds every rank's data.
// Used for the candidates of vocab-sharded sampling; like the greedy merge it is also a step barrier.
struct ExchangeParams {
  const uint32_t* local;
  uint32_t* area_peer[kMaxRanksTp];   // every rank's area [size][area_words]
  uint32_t* flag_peer[kMaxRanksTp];   // every rank's counters [size]
  const uint32_t* my_flag;
  uint32_t* my_state;                 // {epoch}
  uint32_t* status;
  int rank, size, segments, seg_words, seg_stride, area_words;
};

__global__ void __launch_bounds__(256)
tp_exchange_kernel(const ExchangeParams p) {
  __shared__ uint32_t ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  pdl_launch_dependents();
  pdl_wait();
  for (int g = 0; g < p.segments; ++g) {
    for (int i = threadIdx.x; i < p.seg_words; i += blockDim.x) {
      const uint32_t v = p.local[g * p.seg_stride + i];
      for (int r = 0; r < p.size; ++r)
        p.area_peer[r][static_cast<size_t>(p.rank) * p.area_words + g * p.seg_stride + i] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < p.size) {
    red_rel_sys_add(p.flag_peer[threadIdx.x] + p.rank, 1u);      // release at system scope, cumulative over the CTA
    if (!wait_ge(p.my_flag + threadIdx.x, p.my_state[0] + 1u)) ok_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok_flag) atomicExch(p.status, static_cast<uint32_t>(kErrFlagTimeout));
    atomicAdd(&p.my_state[0], 1u);
  }
}

}  // namespace cb

extern "C" {

struct CbExchange {
  const void* local; void* area_peer[8]; void* flag_peer[8]; const void* my_flag; void* my_state; void* status;
  int rank, size, segments, seg_words, seg_stride, area_words;
};

int cb_tp_exchange(const CbExchange* a, void* stream) {
  using namespace cb;
  if (a->size < 1 || a->size > kMaxRanksTp || a->segments < 1 || a->seg_words < 0 ||
      (a->segments - 1) * a->seg_stride + a->seg_words > a->area_words)
    return -10;
  ExchangeParams p;
  p.local = static_cast<const uint32_t*>(a->local);
  for (int r = 0; r < a->size; ++r) {
    p.area_peer[r] = static_cast<uint32_t*>(a->area_peer[r]);
    p.flag_peer[r] = static_cast<uint32_t*>(a->flag_peer[r]);
  }
  p.my_flag = static_cast<const uint32_t*>(a->my_flag);
  p.my_state = static_cast<uint32_t*>(a->my_state);
  p.status = static_cast<uint32_t*>(a->status);
  p.rank = a->rank; p.size = a->size; p.segments = a->segments; p.seg_words = a->seg_words;
  p.seg_stride = a->seg_stride; p.area_words = a->area_words;
  return static_cast<int>(launch(tp_exchange_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), p));
}

struct CbReduceNorm {
  const void* recv; const void* rs_flag; void* rs_state; unsigned rs_expected;
  void* h; const void* norm_w; void* x_peer[8]; void* ag_flag_peer[8]; void* status;
  int rank, size, rows_per_rank, H, M; float eps; int zero_centered; int local_only;
  const void* recv_mc; void* x_mc;
};

int cb_tp_reduce_norm(const CbReduceNorm* a, void* stream) {
  using namespace cb;
  if (a->size < 1 || a->size > kMaxRanksTp || a->H % 8 != 0 || a->H > kRnThreads * kRnMaxVec * 8) return -10;
  ReduceNormParams p;
  p.recv = static_cast<const __nv_bfloat16*>(a->recv);
  p.rs_flag = static_cast<const uint32_t*>(a->rs_flag);
  p.rs_state = static_cast<uint32_t*>(a->rs_state);
  p.rs_expected = a->rs_expected;
  p.h = static_cast<__nv_bfloat16*>(a->h);
  p.norm_w = static_cast<const __nv_bfloat16*>(a->norm_w);
  for (int r = 0; r < a->size; ++r) {
    p.x_peer[r] = static_cast<__nv_bfloat16*>(a->x_peer[r]);
    p.ag_flag_peer[r] = static_cast<uint32_t*>(a->ag_flag_peer[r]);
  }
  p.status = static_cast<uint32_t*>(a->status);
  p.rank = a->rank; p.size = a->size; p.rows_per_rank = a->rows_per_rank; p.H = a->H; p.M = a->M;
  p.eps = a->eps; p.zero_centered = a->zero_centered; p.local_only = a->local_only;
  p.recv_mc = static_cast<const __nv_bfloat16*>(a->recv_mc);
  p.x_mc = static_cast<__nv_bfloat16*>(a->x_mc);
  return static_cast<int>(launch(tp_reduce_norm_kernel, dim3(a->rows_per_rank), dim3(kRnThreads), 0,
                                 static_cast<cudaStream_t>(stream), p));
}

int cb_tp_wait(const void* ag_flag, void* ag_state, unsigned expected, int size, void* status, void* stream) {
  return static_cast<int>(cb::launch(cb::tp_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
      static_cast<const uint32_t*>(ag_flag), static_cast<uint32_t*>(ag_state), expected, size,
      static_cast<uint32_t*>(status)));
}

struct CbArgmaxMerge {
  const void* local_val; const void* local_id; void* slot_val[8]; void* slot_id[8]; void* flag_peer[8];
  const void* my_val; const void* my_id; const void* my_flag; void* my_state; void* out_id; void* status;
  int rank, size, rows, rows_max;
};

int cb_tp_argmax_merge(const CbArgmaxMerge* a, void* stream) {
  using namespace cb;
  if (a->size < 1 || a->size > kMaxRanksTp || a->rows > a->rows_max) return -10;
  ArgmaxMergeParams p;
  p.local_val = static_cast<const float*>(a->local_val);
  p.local_id = static_cast<const int*>(a->local_id);
  for (int r = 0; r < a->size; ++r) {
    p.slot_val[r] = static_cast<float*>(a->slot_val[r]);
    p.slot_id[r] = static_cast<int*>(a->slot_id[r]);
    p.flag_peer[r] = static_cast<uint32_t*>(a->flag_peer[r]);
  }
  p.my_val = static_cast<const float*>(a->my_val);
  p.my_id = static_cast<const int*>(a->my_id);
  p.my_flag = static_cast<const uint32_t*>(a->my_flag);
  p.my_state = static_cast<uint32_t*>(a->my_state);
  p.out_id = static_cast<int*>(a->out_id);
  p.status = static_cast<uint32_t*>(a->status);
  p.rank = a->rank; p.size = a->size; p.rows = a->rows; p.rows_max = a->rows_max;
  return static_cast<int>(launch(tp_argmax_merge_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), p));
}

}  // extern "C"
