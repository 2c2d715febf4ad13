// Token sampling over full-vocabulary bf16 logits: greedy (first-max, lowest id
// wins ties), temperature / top-k (<= 20) / top-p with a counter-based Philox
// stream, optional grammar bitmask, and the speculative accept/resample step.
//
// Counterparts in the reference: sampling/greedy.cu:14-117 (vocab-sharded exact
// argmax with min-id ties and grammar mask), sampling/topk_topp.py:23 (root
// top-k/top-p/temperature + Philox), sampling/speculative.py (K=1 verify).
#include "ptx.cuh"
#include "launch.cuh"

namespace cb {

static constexpr int kSampleThreads = 512;
static constexpr int kMaxTopK = 20;

struct Cand {
  float v;
  int i;
};
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__device__ __forceinline__ Cand block_best(Cand c, Cand* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, c.v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, c.i, o);
    if (better(ov, oi, c.v, c.i)) { c.v = ov; c.i = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = c;
  __syncthreads();
  Cand r = (l < (blockDim.x >> 5)) ? red[l] : Cand{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, r.v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, r.i, o);
    if (better(ov, oi, r.v, r.i)) { r.v = ov; r.i = oi; }
  }
  __syncthreads();
  return r;
}

// Philox4x32-10, one 128-bit draw per (seed, row counter)
__device__ __forceinline__ float philox_uniform(unsigned long long seed, unsigned long long ctr) {
  uint32_t c0 = static_cast<uint32_t>(ctr), c1 = static_cast<uint32_t>(ctr >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return (static_cast<float>(c0 >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct SampleParams {
  const __nv_bfloat16* logits;  // [rows, ld]
  const uint32_t* mask;         // [rows, mask_words] allowed-token bits or null
  const float* temperature;     // [rows] 0 = greedy
  const float* top_p;           // [rows]
  const int* top_k;             // [rows] 0 = up to kMaxTopK
  const unsigned long long* seeds;     // [rows]
  const unsigned long long* counters;  // [rows] per-request draw index
  int* out_ids;                 // [rows]
  float* out_logprob;           // [rows] log-prob of the chosen token within the candidate set (or null)
  float* out_value;             // [rows] raw logit of the chosen token (or null); used by the vocab-sharded merge
  int vocab, ld, mask_words;
  int id_offset;                // added to every emitted id (first vocabulary id of this shard)
  // vocab-sharded sampling: instead of sampling, emit the row's K best (value, global id) pairs, padded to
  // kMaxTopK with (-inf, INT_MAX); cb_sample_merge draws from the union over the ranks
  float* cand_val;              // [rows, kMaxTopK] or null
  int* cand_id;                 // [rows, kMaxTopK]
};

// The draw itself, shared by the one-GPU sampler and the merge of rank-local candidates: `top` holds K
// candidates in (value desc, id asc) order.
struct Draw {
  int id;
  float logprob, value;
};
__device__ __forceinline__ Draw draw_from_top(const Cand* top, int K, float temp, float tp, unsigned long long seed,
                                              unsigned long long ctr) {
  if (K == 0) return Draw{0, 0.f, -INFINITY};
  if (temp <= 0.f || K == 1) return Draw{top[0].i, 0.f, top[0].v};
  float probs[kMaxTopK];
  const float inv_t = 1.f / temp;
  float sum = 0.f;
  for (int k = 0; k < K; ++k) { probs[k] = __expf((top[k].v - top[0].v) * inv_t); sum += probs[k]; }
  int keep = K;
  if (tp < 1.f) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k) { acc += probs[k] / sum; if (acc >= tp) { keep = k + 1; break; } }
  }
  float ksum = 0.f;
  for (int k = 0; k < keep; ++k) ksum += probs[k];
  const float u = philox_uniform(seed, ctr) * ksum;
  float acc = 0.f;
  int pick = keep - 1;
  for (int k = 0; k < keep; ++k) { acc += probs[k]; if (u < acc) { pick = k; break; } }
  return Draw{top[pick].i, __logf(probs[pick] / ksum), top[pick].v};
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const SampleParams p) {
  __shared__ Cand red[kSampleThreads / 32];
  __shared__ Cand top[kMaxTopK];
  const int row = blockIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  const __nv_bfloat16* lg = p.logits + static_cast<size_t>(row) * p.ld;
  const uint32_t* mk = p.mask ? p.mask + static_cast<size_t>(row) * p.mask_words : nullptr;
  const float temp = p.temperature ? p.temperature[row] : 0.f;
  int K = 1;
  if (temp > 0.f) {
    K = p.top_k ? p.top_k[row] : 0;
    if (K <= 0 || K > kMaxTopK) K = kMaxTopK;
  }
  float pv = INFINITY;
  int pi = -1;
  for (int k = 0; k < K; ++k) {
    Cand best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < p.vocab; i += kSampleThreads) {
      if (mk && !((mk[i >> 5] >> (i & 31)) & 1u)) continue;
      float v = __bfloat162float(lg[i]);
      if (!(v == v)) v = -INFINITY;  // NaN never wins
      // strictly after the previous pick in (value desc, id asc) order
      if (v < pv || (v == pv && i > pi)) {
        if (better(v, i, best.v, best.i)) { best.v = v; best.i = i; }
      }
    }
    best = block_best(best, red);
    if (threadIdx.x == 0) top[k] = best;
    pv = best.v;
    pi = best.i;
    if (best.i == 0x7fffffff) { K = k; break; }  // fewer allowed tokens than K (uniform across the block)
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (p.cand_val) {
    for (int k = 0; k < kMaxTopK; ++k) {
      p.cand_val[row * kMaxTopK + k] = k < K ? top[k].v : -INFINITY;
      p.cand_id[row * kMaxTopK + k] = k < K ? top[k].i + p.id_offset : 0x7fffffff;
    }
    return;
  }
  const Draw d = draw_from_top(top, K, temp, p.top_p ? p.top_p[row] : 1.f, p.seeds ? p.seeds[row] : 0ull,
                               p.counters ? p.counters[row] : 0ull);
  p.out_ids[row] = d.id + p.id_offset;
  if (p.out_logprob) p.out_logprob[row] = d.logprob;
  if (p.out_value) p.out_value[row] = d.value;
}

// Merge of the ranks' candidates (vocab-sharded sampling; reference: generation/tp_sampling.py:681
// sample_sharded_broadcast_tp): the global top-K of a row is contained in the union of the local top-Ks, so the
// draw over the merged set equals the draw over the full vocabulary.  Every rank runs this on the same gathered
// data with the same Philox stream and gets the same token: no broadcast.  One warp per row.
__global__ void __launch_bounds__(128)
sample_merge_kernel(const float* cand_val, const int* cand_id, int sources, long long source_stride, int rows,
                    const float* temperature, const float* top_p, const int* top_k, const unsigned long long* seeds,
                    const unsigned long long* counters, int* out_ids, float* out_logprob) {
  __shared__ Cand tops[4][kMaxTopK];
  const int wrp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + wrp;
  pdl_wait();
  pdl_launch_dependents();
  if (row >= rows) return;
  const float temp = temperature ? temperature[row] : 0.f;
  int K = 1;
  if (temp > 0.f) {
    K = top_k ? top_k[row] : 0;
    if (K <= 0 || K > kMaxTopK) K = kMaxTopK;
  }
  // lane l holds candidates l, l + 32, ... of the sources x kMaxTopK pool (<= 8 x 20 = 160 -> 5 per lane)
  Cand mine[5];
  const int pool = sources * kMaxTopK;
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int c = lane + 32 * j;
    mine[j] = Cand{-INFINITY, 0x7fffffff};
    if (c < pool) {
      const int src = c / kMaxTopK, k = c - src * kMaxTopK;
      const long long off = static_cast<long long>(src) * source_stride + static_cast<long long>(row) * kMaxTopK + k;
      mine[j] = Cand{__ldcg(cand_val + off), __ldcg(cand_id + off)};
    }
  }
  int found = 0;
  for (int r = 0; r < K; ++r) {
    Cand best{-INFINITY, 0x7fffffff};
    int bj = -1;
#pragma unroll
    for (int j = 0; j < 5; ++j)
      if (mine[j].i != 0x7fffffff && better(mine[j].v, mine[j].i, best.v, best.i)) { best = mine[j]; bj = j; }
    Cand w = best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, w.v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, w.i, o);
      if (better(ov, oi, w.v, w.i)) { w.v = ov; w.i = oi; }
    }
    if (w.i == 0x7fffffff) break;                        // pool exhausted (uniform over the warp)
    if (bj >= 0 && best.i == w.i) {                      // ids are unique across shards: exactly one lane owns it
#pragma unroll
      for (int j = 0; j < 5; ++j)
        if (j == bj) mine[j].i = 0x7fffffff;
    }
    if (lane == 0) tops[wrp][r] = w;
    ++found;
  }
  __syncwarp();
  if (lane != 0) return;
  const Draw d = draw_from_top(tops[wrp], found, temp, top_p ? top_p[row] : 1.f, seeds ? seeds[row] : 0ull,
                               counters ? counters[row] : 0ull);
  out_ids[row] = d.id;
  if (out_logprob) out_logprob[row] = d.logprob;
}

// Greedy speculative verification: per request, row r holds the target's choice
// after consuming draft token r (row 0 = after the root).  accepted = length of
// the longest prefix with draft[r] == target[r]; the bonus token is
// target[accepted].  (reference: generation/tp_sampling.py:154, greedy branch)
__global__ void verify_greedy_kernel(const int* target_ids, const int* draft_ids, const int* depth, int max_depth,
                                     const int* forced_reject_at, int* accepted, int* bonus, int requests) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  if (r >= requests) return;
  const int d = depth[r];
  int a = 0;
  const int cap = forced_reject_at ? forced_reject_at[r] : d;  // acceptance-forcing hook (benchmarks)
  while (a < d && a < cap && draft_ids[r * max_depth + a] == target_ids[r * (max_depth + 1) + a]) ++a;
  accepted[r] = a;
  bonus[r] = target_ids[r * (max_depth + 1) + a];
}

// Speculative verification for SAMPLED requests: p / q rejection sampling over sparse candidate distributions
// (reference: generation/tp_sampling.py:154-217 verify_speculative_chain, ops/cuda/sampling/speculative.py:54).
// Row (r, i) of `q_*` holds the draft head's top candidates when it proposed draft token i, row (r, i) of `p_*` the
// target's candidates after consuming the root and drafts 0 .. i - 1 ([.., kMaxTopK] (value desc, id asc), padded
// with (-inf, INT_MAX)).  Both are shaped by the request's temperature / top-k / top-p exactly like a plain draw.
//   accept draft i  iff  q(d_i) > 0 and u_i < min(1, p(d_i) / q(d_i));
//   at the first rejection the next token is drawn from normalise(max(0, p - q)) (from p if that is empty);
//   with every draft accepted the bonus token is drawn from the last target row.
// A greedy request (temperature 0) has one-hot p and q: the rule reduces to the longest-matching-prefix check.
// Uniforms come from the request's Philox stream at counter draws | (sub-draw + 1) << 40: sub-draw 2 i decides draft
// i, sub-draw 2 i + 1 draws its replacement, sub-draw 2 depth draws the bonus token, so a replay of the round draws
// the same numbers.  emitted[r] = accepted drafts followed by the next token ([.., max_depth + 1]).
struct VerifySampledParams {
  const float* q_val; const int* q_id;      // [requests, max_depth, kMaxTopK]
  const float* p_val; const int* p_id;      // [requests, max_depth + 1, kMaxTopK]
  const int* draft_ids;                     // [requests, max_depth]
  const int* depth;                         // [requests]
  const float* temperature; const float* top_p; const int* top_k;
  const unsigned long long* seeds; const unsigned long long* counters;
  int* accepted; int* bonus; int* emitted;
  int max_depth, requests;
};

// Shaped probabilities of one candidate row; returns the number of real candidates kept (the rest get 0).
__device__ __forceinline__ int shaped_probs(const float* val, const int* id, float temp, float tp, int top_k, float* probs) {
  int K = 0;
  const int cap = temp <= 0.f ? 1 : ((top_k <= 0 || top_k > kMaxTopK) ? kMaxTopK : top_k);
  while (K < cap && id[K] != 0x7fffffff && val[K] > -INFINITY) ++K;
  for (int k = 0; k < kMaxTopK; ++k) probs[k] = 0.f;
  if (K == 0) return 0;
  if (temp <= 0.f) { probs[0] = 1.f; return 1; }
  const float inv_t = 1.f / temp;
  float sum = 0.f;
  for (int k = 0; k < K; ++k) { probs[k] = __expf((val[k] - val[0]) * inv_t); sum += probs[k]; }
  int keep = K;
  if (tp < 1.f) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k) { acc += probs[k] / sum; if (acc >= tp) { keep = k + 1; break; } }
  }
  float ksum = 0.f;
  for (int k = 0; k < keep; ++k) ksum += probs[k];
  for (int k = 0; k < kMaxTopK; ++k) probs[k] = k < keep ? probs[k] / ksum : 0.f;
  return keep;
}

__device__ __forceinline__ int draw_index(const float* probs, int n, float u) {
  float total = 0.f;
  for (int k = 0; k < n; ++k) total += probs[k];
  float acc = 0.f;
  int pick = -1;
  for (int k = 0; k < n; ++k) {
    if (probs[k] <= 0.f) continue;
    pick = k;                                  // the last candidate with mass catches rounding at the top end
    acc += probs[k];
    if (u * total < acc) break;
  }
  return pick;
}

__global__ void __launch_bounds__(64)
verify_sampled_kernel(const VerifySampledParams p) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  if (r >= p.requests) return;
  const int D = p.max_depth, d = min(p.depth[r], D);
  const float temp = p.temperature ? p.temperature[r] : 0.f;
  const float tp = p.top_p ? p.top_p[r] : 1.f;
  const int tk = p.top_k ? p.top_k[r] : 0;
  const unsigned long long seed = p.seeds ? p.seeds[r] : 0ull;
  const unsigned long long base = p.counters ? p.counters[r] : 0ull;
  auto uniform = [&](int sub) { return philox_uniform(seed, base | (static_cast<unsigned long long>(sub + 1) << 40)); };
  float pp[kMaxTopK], qq[kMaxTopK];
  int* out = p.emitted + static_cast<size_t>(r) * (D + 1);
  int a = 0, next = 0;
  bool done = false;
  for (; a < d; ++a) {
    const float* pv = p.p_val + (static_cast<size_t>(r) * (D + 1) + a) * kMaxTopK;
    const int* pi = p.p_id + (static_cast<size_t>(r) * (D + 1) + a) * kMaxTopK;
    const float* qv = p.q_val + (static_cast<size_t>(r) * D + a) * kMaxTopK;
    const int* qi = p.q_id + (static_cast<size_t>(r) * D + a) * kMaxTopK;
    const int np_ = shaped_probs(pv, pi, temp, tp, tk, pp);
    const int nq = shaped_probs(qv, qi, temp, tp, tk, qq);
    const int tok = p.draft_ids[r * D + a];
    float pd = 0.f, qd = 0.f;
    for (int k = 0; k < np_; ++k) if (pi[k] == tok) pd = pp[k];
    for (int k = 0; k < nq; ++k) if (qi[k] == tok) qd = qq[k];
    if (qd > 0.f && uniform(2 * a) < fminf(1.f, pd / qd)) { out[a] = tok; continue; }
    // rejected: residual max(0, p - q) over the target's candidates
    float res[kMaxTopK];
    float mass = 0.f;
    for (int k = 0; k < kMaxTopK; ++k) {
      float q_here = 0.f;
      if (k < np_) for (int j = 0; j < nq; ++j) if (qi[j] == pi[k]) q_here = qq[j];
      res[k] = k < np_ ? fmaxf(0.f, pp[k] - q_here) : 0.f;
      mass += res[k];
    }
    const int pick = mass > 0.f ? draw_index(res, np_, uniform(2 * a + 1)) : draw_index(pp, np_, uniform(2 * a + 1));
    next = pick >= 0 ? pi[pick] : (np_ > 0 ? pi[0] : 0);
    done = true;
    break;
  }
  if (!done) {
    const float* pv = p.p_val + (static_cast<size_t>(r) * (D + 1) + d) * kMaxTopK;
    const int* pi = p.p_id + (static_cast<size_t>(r) * (D + 1) + d) * kMaxTopK;
    const int np_ = shaped_probs(pv, pi, temp, tp, tk, pp);
    const int pick = draw_index(pp, np_, uniform(2 * d));
    next = pick >= 0 ? pi[pick] : 0;
    a = d;
  }
  out[a] = next;
  p.accepted[r] = a;
  p.bonus[r] = next;
}

// Thinking-token budgets, enforced on the device so that decode graphs (and steps launched ahead of the host) need no
// host decision: an integer state machine per request slot, run on every sampled id right after the sampler.
//   left[slot]  >= 0: the request is in its reasoning phase and may still emit that many thinking tokens; < 0: inactive
//   fpos[slot]  > 0 : the forced end sequence is being emitted, next index
// A row's `init` value re-arms its slot first: -2 = keep, -1 = no budget, >= 0 = reasoning starts (or resumes after a
// re-prefill) with that many tokens left.  When the budget is used up the sampled id is replaced by the tokens of the
// end sequence, one per step; sampling the closing token on its own ends the phase.
// Reference: ops/cuda/sampling/reasoning_budget.cu:94 (sampling rows; its review / proposal prefixes belong to the
// speculative path, which does not enforce budgets here).
__global__ void __launch_bounds__(128)
reasoning_budget_kernel(int* __restrict__ ids, const int* __restrict__ row_slot, const int* __restrict__ init,
                        int* __restrict__ left, int* __restrict__ fpos, int rows, int end_id, int4 seq, int seq_len) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_launch_dependents();
  if (row >= rows) return;
  const int slot = row_slot[row];
  if (slot < 0) return;
  const int in = init[row];
  int L = left[slot], f = fpos[slot];
  if (in >= -1) { L = in; f = 0; }
  if (L >= 0) {
    int tok = ids[row];
    if (f > 0 || L == 0) {
      tok = f == 0 ? seq.x : (f == 1 ? seq.y : (f == 2 ? seq.z : seq.w));
      if (++f >= seq_len) { L = -1; f = 0; }
    } else if (tok == end_id) {
      L = -1;
    } else {
      --L;
    }
    ids[row] = tok;
  }
  left[slot] = L;
  fpos[slot] = f;
}

}  // namespace cb

extern "C" {

int cb_sample(const void* logits, int ld, const void* mask, int mask_words, const void* temperature,
              const void* top_p, const void* top_k, const void* seeds, const void* counters, void* out_ids,
              void* out_logprob, void* out_value, int id_offset, int rows, int vocab, void* stream) {
  using namespace cb;
  if (rows <= 0) return 0;
  SampleParams p;
  p.logits = static_cast<const __nv_bfloat16*>(logits);
  p.mask = static_cast<const uint32_t*>(mask);
  p.temperature = static_cast<const float*>(temperature);
  p.top_p = static_cast<const float*>(top_p);
  p.top_k = static_cast<const int*>(top_k);
  p.seeds = static_cast<const unsigned long long*>(seeds);
  p.counters = static_cast<const unsigned long long*>(counters);
  p.out_ids = static_cast<int*>(out_ids);
  p.out_logprob = static_cast<float*>(out_logprob);
  p.out_value = static_cast<float*>(out_value);
  p.id_offset = id_offset;
  p.vocab = vocab; p.ld = ld; p.mask_words = mask_words;
  p.cand_val = nullptr;
  p.cand_id = nullptr;
  return static_cast<int>(launch(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), p));
}

// Rank-local half of vocab-sharded sampling: the row's best candidates (20 slots per row, see SampleParams).
int cb_sample_candidates(const void* logits, int ld, const void* mask, int mask_words, const void* temperature,
                         const void* top_k, void* cand_val, void* cand_id, int id_offset, int rows, int vocab,
                         void* stream) {
  using namespace cb;
  if (rows <= 0) return 0;
  SampleParams p{};
  p.logits = static_cast<const __nv_bfloat16*>(logits);
  p.mask = static_cast<const uint32_t*>(mask);
  p.temperature = static_cast<const float*>(temperature);
  p.top_k = static_cast<const int*>(top_k);
  p.id_offset = id_offset;
  p.vocab = vocab; p.ld = ld; p.mask_words = mask_words;
  p.cand_val = static_cast<float*>(cand_val);
  p.cand_id = static_cast<int*>(cand_id);
  return static_cast<int>(launch(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), p));
}

// Merge `sources` candidate sets (source s at cand + s * source_stride elements, [rows, 20] each) and draw.
int cb_sample_merge(const void* cand_val, const void* cand_id, int sources, long long source_stride, int rows,
                    const void* temperature, const void* top_p, const void* top_k, const void* seeds,
                    const void* counters, void* out_ids, void* out_logprob, void* stream) {
  using namespace cb;
  if (rows <= 0) return 0;
  if (sources < 1 || sources > 8) return -10;
  return static_cast<int>(launch(sample_merge_kernel, dim3((rows + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const float*>(cand_val), static_cast<const int*>(cand_id), sources, source_stride, rows,
      static_cast<const float*>(temperature), static_cast<const float*>(top_p), static_cast<const int*>(top_k),
      static_cast<const unsigned long long*>(seeds), static_cast<const unsigned long long*>(counters),
      static_cast<int*>(out_ids), static_cast<float*>(out_logprob)));
}

int cb_verify_greedy(const void* target_ids, const void* draft_ids, const void* depth, int max_depth,
                     const void* forced_reject_at, void* accepted, void* bonus, int requests, void* stream) {
  if (requests <= 0) return 0;
  return static_cast<int>(cb::launch(cb::verify_greedy_kernel, dim3((requests + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const int*>(target_ids), static_cast<const int*>(draft_ids), static_cast<const int*>(depth),
      max_depth, static_cast<const int*>(forced_reject_at), static_cast<int*>(accepted), static_cast<int*>(bonus),
      requests));
}

// p / q rejection sampling of a speculative round (see verify_sampled_kernel); candidate arrays as written by
// cb_sample_candidates, `emitted` [requests, max_depth + 1] receives the accepted drafts and the next token.
int cb_verify_sampled(const void* q_val, const void* q_id, const void* p_val, const void* p_id, const void* draft_ids,
                      const void* depth, int max_depth, const void* temperature, const void* top_p, const void* top_k,
                      const void* seeds, const void* counters, void* accepted, void* bonus, void* emitted, int requests,
                      void* stream) {
  if (requests <= 0) return 0;
  if (max_depth <= 0) return -10;
  cb::VerifySampledParams p;
  p.q_val = static_cast<const float*>(q_val); p.q_id = static_cast<const int*>(q_id);
  p.p_val = static_cast<const float*>(p_val); p.p_id = static_cast<const int*>(p_id);
  p.draft_ids = static_cast<const int*>(draft_ids); p.depth = static_cast<const int*>(depth);
  p.temperature = static_cast<const float*>(temperature); p.top_p = static_cast<const float*>(top_p);
  p.top_k = static_cast<const int*>(top_k);
  p.seeds = static_cast<const unsigned long long*>(seeds); p.counters = static_cast<const unsigned long long*>(counters);
  p.accepted = static_cast<int*>(accepted); p.bonus = static_cast<int*>(bonus); p.emitted = static_cast<int*>(emitted);
  p.max_depth = max_depth; p.requests = requests;
  return static_cast<int>(cb::launch(cb::verify_sampled_kernel, dim3((requests + 63) / 64), dim3(64), 0,
                                     static_cast<cudaStream_t>(stream), p));
}

// ids[rows] (in place), row_slot / init [rows], left / fpos [slots]; `seq` = 1..4 tokens of the forced end sequence
// (it contains `end_id`).
int cb_reasoning_budget(void* ids, const void* row_slot, const void* init, void* left, void* fpos, int rows, int end_id,
                        const int* seq, int seq_len, void* stream) {
  if (rows <= 0) return 0;
  if (!seq || seq_len < 1 || seq_len > 4) return -20;
  int4 q = make_int4(seq[0], seq_len > 1 ? seq[1] : 0, seq_len > 2 ? seq[2] : 0, seq_len > 3 ? seq[3] : 0);
  return static_cast<int>(cb::launch(cb::reasoning_budget_kernel, dim3((rows + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<int*>(ids), static_cast<const int*>(row_slot), static_cast<const int*>(init), static_cast<int*>(left),
      static_cast<int*>(fpos), rows, end_id, q, seq_len));
}

}  // extern "C"
