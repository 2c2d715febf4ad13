// Persistent stream-K form of the weight-quantized GEMM (see wq_gemm.cu for the operand roles, the packed
// weight layout and the decode arithmetic, which are shared through wq_gemm_common.cuh).
//
// Why a second kernel.  Profiles of the one-CTA-per-tile kernel at decode batch 256 showed three losses that
// no tuning inside that structure removes:
//   * wave quantisation: 192 weight tiles on 148 SMs run as two waves (35 % of the machine idle on average);
//   * prologue (barrier set-up, first copies, first decode) and epilogue (TMEM -> global) are 14 % of a tile
//     and overlap with nothing, because shared memory allows one CTA per SM;
//   * the four-stage ring that carried {activation tile, decoded tile, packed codes} together was latency
//     bound: a stage went release -> copy issue -> copy latency -> decode -> MMA before it could be reused.
// This kernel launches at most one CTA per SM and deals K-BLOCKS, not tiles, to the CTAs:
//   * tiles [0, sk_tiles) are "streamed": their sk_tiles * k_blocks units are split evenly over sk_ctas CTAs,
//     so a tile may be produced by several CTAs, each writing an fp32 partial; the last to arrive sums the
//     partials in part order (deterministic) and writes the result;
//   * the remaining tiles are whole tiles, tile = sk_tiles + w * grid + cta for w = 0, 1, ...
//   Every CTA therefore gets the same number of k-blocks (+-1) whatever the tile count.
// Inside a CTA the rings are decoupled and the accumulator is double buffered:
//   warp 0      activation tiles (and bf16 weight tiles) by TMA into the AX ring          -> full
//   warp 2      packed codes + metadata by bulk copy into the deeper C ring               -> c_full
//   warps 7-22  decode, four groups of 4 warps, group g takes every fourth k-block: wait c_full, decode 64
//               weights per thread in registers (two 16-byte code loads, eight 16-byte tile stores),
//               wait for the AX slot to be free, store the swizzled bf16 tile             -> full, c_empty
//               (per-k-block costs -- waits, fence, arrive, metadata -- are paid by 4 warps, not 16)
//   warp 1      MMA: wait full, 4 x tcgen05.mma into accumulator (segment & 1),
//               commit -> ax_empty; after a segment's last k-block commit -> acc_full
//   warps 3-6   epilogue: wait acc_full, tcgen05.ld, write bf16 output (or the fp32 partial),
//               release the accumulator -> acc_empty; fix-up reduction for streamed tiles;
//               tensor-parallel push + arrival counters when the launch carries a TpLink.
// The epilogue of segment i overlaps the main loop of segment i + 1.
// Every wait is bounded (ptx.cuh); on a timeout the CTA-wide abort flag makes every role fall through to the
// common exit, which frees tensor memory and records a status word.
#include "wq_gemm_common.cuh"
#include "launch.cuh"

namespace cb {

static constexpr int kSkDecodeWarps = 16;
static constexpr int kSkDecodeGroups = 4;       // group g decodes the k-blocks with (index & 3) == g
static constexpr int kSkGroupWarps = kSkDecodeWarps / kSkDecodeGroups;
static constexpr int kSkEpiScratchBytes = 4 * 16 * 32 * 4;   // per epilogue warp: 16 rows x 32 features fp32
static constexpr int kSkEpiWarps = 4;
static constexpr int kSkFirstEpiWarp = 3;      // any four consecutive warps cover the four TMEM lane quadrants
static constexpr int kSkFirstDecodeWarp = 7;
static constexpr int kSkThreads = (kSkFirstDecodeWarp + kSkDecodeWarps) * 32;   // 736
static constexpr int kSkMaxAx = 6;
static constexpr int kSkMaxC = 8;
__host__ __device__ constexpr int sk_cstage_bytes(int fmt) { return kCodeBytes + meta_bytes(fmt); }

// One contiguous run of k-blocks of one tile, as dealt to a CTA.
struct SkSegment {
  int tile, kb_lo, kb_hi;
  int part, parts;               // this run is part `part` of `parts` runs that make up the tile
};

struct __align__(8) SkCtl {
  uint64_t full[kSkMaxAx];       // activation (and bf16 weight) tile landed (transaction bytes + the producer's
                                 // arrival) AND decoded weight tile stored by the 4 warps of a group (4 arrivals)
  uint64_t ax_empty[kSkMaxAx];   // the MMAs that read the slot have retired            (tcgen05.commit)
  uint64_t c_full[kSkMaxC];      // packed codes + metadata landed                      (transaction bytes)
  uint64_t c_empty[kSkMaxC];     // the group's warps hold the codes in registers       (4 arrivals)
  uint64_t acc_full[2];          // accumulator of a segment complete                   (tcgen05.commit)
  uint64_t acc_empty[2];         // epilogue warps have read the accumulator            (4 arrivals)
  uint64_t tail_full;            // accumulator of the CTA's LAST segment complete; completes once, so waiters
                                 // that arrive many segments early cannot mistake an older phase for it
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t is_last;
  // streamed tiles whose LAST partial arrived from this CTA while it still had segments to run: their fix-up
  // waits for the end of the CTA, where all 20 epilogue + decode warps do it (at most two: the CTA's first run
  // and the run before its whole tiles)
  uint32_t deferred_count;
  uint32_t deferred_next;        // fix-ups [0, deferred_next) are done (sliced form: by the epilogue warps, in the background)
  SkSegment deferred[2];
};

// The deal.  Identical arithmetic on every thread of every role, so all roles of a CTA walk the same list.
struct SkIter {
  // 32-bit arithmetic throughout: the streamed region has at most one tile per SM, so units * CTAs < 2^31
  // (checked on the host); 64-bit divisions cost several hundred cycles each at kernel start
  uint32_t u, u_end, total;      // streamed units of this CTA, and of the whole launch
  int next_whole;
  int tiles;                     // whole-tile bound: p.tiles, or (work items) x n_tiles in grouped mode
  __device__ __forceinline__ void init(const WqGemmParams& p, int cta) {
    tiles = p.group_tiles ? p.group_tiles[0] * p.n_tiles : p.tiles;
    total = static_cast<uint32_t>(p.sk_tiles) * static_cast<uint32_t>(p.k_blocks);
    if (cta < p.sk_ctas) {
      u = total * static_cast<uint32_t>(cta) / static_cast<uint32_t>(p.sk_ctas);
      u_end = total * static_cast<uint32_t>(cta + 1) / static_cast<uint32_t>(p.sk_ctas);
    } else {
      u = u_end = 0;
    }
    next_whole = p.sk_tiles + cta;
  }
  __device__ __forceinline__ bool has_more(const WqGemmParams&) const { return u < u_end || next_whole < tiles; }
  __device__ __forceinline__ bool next(const WqGemmParams& p, int cta, int grid, SkSegment& s) {
    if (u < u_end) {
      const uint32_t kbs = static_cast<uint32_t>(p.k_blocks);
      const uint32_t ctas = static_cast<uint32_t>(p.sk_ctas);
      const uint32_t tile = u / kbs;
      const uint32_t first = tile * kbs;
      const uint32_t end = (u_end < first + kbs) ? u_end : first + kbs;
      s.tile = static_cast<int>(tile);
      s.kb_lo = static_cast<int>(u - first);
      s.kb_hi = static_cast<int>(end - first);
      // CTA that owns unit v: the largest g with floor(total * g / ctas) <= v
      const int g_first = static_cast<int>(((first + 1u) * ctas - 1u) / total);
      const int g_last = static_cast<int>(((first + kbs) * ctas - 1u) / total);
      s.parts = g_last - g_first + 1;
      s.part = cta - g_first;
      u = end;
      return true;
    }
    if (next_whole < tiles) {
      s.tile = next_whole;
      s.kb_lo = 0;
      s.kb_hi = p.k_blocks;
      s.part = 0;
      s.parts = 1;
      next_whole += grid;
      return true;
    }
    return false;
  }
};

// Where a tile lives: first batch row, number of valid rows, weight tile index, and (grouped expert GEMMs) the
// expert whose weights it uses.  Dense: tile = m_tile * n_tiles + n_tile.  Grouped: tile = item * n_tiles +
// n_tile with item = {expert, first row, rows} from the device work list written by the MoE routing kernels.
struct SkCoords {
  int m0, rows, n_tile, expert;
  int tile_id;                   // index of the (row tile, weight tile) this CTA produces: arrival counter of the tile
};
// `rank`: rank of the CTA in its pair (0 without pairs).  With pairs the schedule's tile is a pair of adjacent
// weight tiles and rank r owns weight tile 2 * pair_tile + r.
__device__ __forceinline__ SkCoords sk_coords(const WqGemmParams& p, int tile, int rank) {
  SkCoords c;
  const int nts = p.n_tiles >> p.pair;
  const int outer = tile / nts;
  c.n_tile = ((tile - outer * nts) << p.pair) + rank;
  c.tile_id = outer * p.n_tiles + c.n_tile;
  if (p.group_tiles) {
    c.expert = p.group_tiles[1 + 3 * outer];
    c.m0 = p.group_tiles[2 + 3 * outer];
    c.rows = p.group_tiles[3 + 3 * outer];
  } else {
    c.expert = 0;
    c.m0 = outer * p.mb;
    c.rows = min(p.mb, p.M - c.m0);
  }
  return c;
}

// Ring position: slot index and how many times the ring has wrapped.
struct SkRing {
  int s = 0;
  uint32_t wraps = 0;
  __device__ __forceinline__ void advance(int depth) {
    if (++s == depth) { s = 0; ++wraps; }
  }
  __device__ __forceinline__ void advance_by(int n, int depth) {   // n <= 4, depth >= 2
    s += n;
    if (s >= depth) { s -= depth; ++wraps; }
    if (s >= depth) { s -= depth; ++wraps; }
  }
};

// fp32 partial slot of (cta, part): a CTA has at most one run that starts inside a tile (its first, part > 0)
// and at most one that ends inside a tile (its last, part == 0)
// (`unit` = the CTA's index in the launch: the pair index * 2 + rank with CTA pairs)
__device__ __forceinline__ float* sk_slot(const WqGemmParams& p, int unit, int part) {
  return p.workspace + (static_cast<size_t>(unit) * 2 + (part == 0 ? 1 : 0)) * (static_cast<size_t>(p.mb) * kTileN);
}

__device__ __forceinline__ void epi_bar() {
  asm volatile("bar.sync 1, %0;" ::"r"(kSkEpiWarps * 32));
}

__device__ __forceinline__ void tail_bar() {
  asm volatile("bar.sync 2, %0;" ::"r"((kSkEpiWarps + kSkDecodeWarps) * 32));
}

// Four consecutive output features n0..n0+3 of row m from unscaled fp32 accumulators: scale, add the residual,
// round once to bf16, store locally or (scatter-push) into the receive buffer of the rank that owns row m.
__device__ __forceinline__ void sk_store4(const WqGemmParams& p, int m, int n0, const float4 v) {
  if (n0 >= p.N) return;
  float o4[4] = {v.x * p.alpha, v.y * p.alpha, v.z * p.alpha, v.w * p.alpha};
  __nv_bfloat16* dst;
  const __nv_bfloat16* res = nullptr;
  bool vec;
  if (p.tp.mode & kTpScatterPush) {
    const int o = m / p.tp.rows_per_rank;
    const int lr = m - o * p.tp.rows_per_rank;
    dst = p.tp.recv[o] + (static_cast<size_t>(p.tp.rank) * p.tp.rows_per_rank + lr) * p.N + n0;
    vec = (p.N & 3) == 0;
  } else {
    const size_t off = static_cast<size_t>(m) * p.ldy + n0;
    dst = p.y + off;
    if (p.residual) res = p.residual + off;
    vec = (p.ldy & 3) == 0;
  }
  if (vec && n0 + 3 < p.N) {
    if (res) {
      const uint2 rv = *reinterpret_cast<const uint2*>(res);
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
      const float2 a0 = __bfloat1622float2(rp[0]), a1 = __bfloat1622float2(rp[1]);
      o4[0] += a0.x; o4[1] += a0.y; o4[2] += a1.x; o4[3] += a1.y;
    }
    uint2 ov;
    ov.x = pack_bf16x2(o4[0], o4[1]);
    ov.y = pack_bf16x2(o4[2], o4[3]);
    *reinterpret_cast<uint2*>(dst) = ov;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (n0 + j < p.N) {
        float w = o4[j];
        if (res) w += __bfloat162float(res[j]);
        dst[j] = __float2bfloat16(w);
      }
    }
  }
}

// The same fix-up with the fused SwiGLU epilogue: 16 items of four activation features per row, each from the gate
// and the up float4 of every part.  Out of line: it runs once per streamed tile and its registers stay out of the
// kernel's allocation.
__device__ __noinline__ void sk_reduce_write_act(const WqGemmParams& p, const float* slots, int parts, int own_part,
                                                 const float* own, int tid, int nthreads, int m0, int row_lo, int row_hi,
                                                 int n_tile) {
  const size_t part_elems = static_cast<size_t>(p.mb) * kTileN;
  const size_t stride = static_cast<size_t>(2) << p.pair;      // slots between consecutive parts of a tile
  constexpr int kB = 1;                                        // items per thread and round: 2 loads of 16 bytes per part,
                                                               // four parts in flight (the sum stays in part order)
  const int items = (row_hi - row_lo) * 16;
  for (int base = tid; base < items; base += nthreads * kB) {
    float4 g[kB], u[kB];
    int e[kB];
#pragma unroll
    for (int b = 0; b < kB; ++b) {
      const int idx = base + b * nthreads;
      const int safe = idx < items ? idx : tid;            // out-of-range slots re-read a valid item, never stored
      e[b] = (row_lo + (safe >> 4)) * kTileN + act_gate_col((safe & 15) * 4);
      g[b] = make_float4(0.f, 0.f, 0.f, 0.f);
      u[b] = g[b];
    }
#pragma unroll 4
    for (int sp = 0; sp < parts; ++sp) {
      float4 a[kB], c[kB];
      if (sp == own_part) {
#pragma unroll
        for (int b = 0; b < kB; ++b) {
          a[b] = *reinterpret_cast<const float4*>(own + e[b]);
          c[b] = *reinterpret_cast<const float4*>(own + e[b] + 16);
        }
      } else {
        const float* src = slots + (static_cast<size_t>(sp) * stride + (sp == 0 ? 1 : 0)) * part_elems;
#pragma unroll
        for (int b = 0; b < kB; ++b) {
          a[b] = __ldcg(reinterpret_cast<const float4*>(src + e[b]));
          c[b] = __ldcg(reinterpret_cast<const float4*>(src + e[b] + 16));
        }
      }
#pragma unroll
      for (int b = 0; b < kB; ++b) {
        g[b].x += a[b].x; g[b].y += a[b].y; g[b].z += a[b].z; g[b].w += a[b].w;
        u[b].x += c[b].x; u[b].y += c[b].y; u[b].z += c[b].z; u[b].w += c[b].w;
      }
    }
#pragma unroll
    for (int b = 0; b < kB; ++b) {
      const int idx = base + b * nthreads;
      if (idx < items) {
        g[b].x *= p.alpha; g[b].y *= p.alpha; g[b].z *= p.alpha; g[b].w *= p.alpha;
        u[b].x *= p.alpha; u[b].y *= p.alpha; u[b].z *= p.alpha; u[b].w *= p.alpha;
        store_act4(p, m0 + row_lo + (idx >> 4), n_tile, (idx & 15) * 4, g[b], u[b]);
      }
    }
  }
}

// Fix-up of rows [row_lo, row_hi) of a streamed tile: sum the fp32 partials of all parts IN PART ORDER (bit-identical
// whoever does it) and write those rows.  `own` (optional) is this CTA's own part
// still in shared memory, read instead of its copy in L2.  kBatch items per thread are in flight at once: the
// partials come from L2 at ~1 k cycles per round trip, so the loop is latency bound without batching.
template <int kBatch, int kPartUnroll>
__device__ __forceinline__ void sk_reduce_write(const WqGemmParams& p, const SkSegment& seg, int unit, int tid,
                                                int nthreads, int m0, int row_lo, int row_hi, int n_base, const float* own) {
  const size_t part_elems = static_cast<size_t>(p.mb) * kTileN;
  const size_t stride = static_cast<size_t>(2) << p.pair;      // slots between consecutive parts (CTAs, or pairs of CTAs)
  const int g_first = unit - (seg.part << p.pair);             // the CTA (of this rank) that holds part 0
  const int parts = seg.parts;
  const int own_part = own ? seg.part : -1;
  const float* slots = p.workspace + static_cast<size_t>(g_first) * 2 * part_elems;   // part q > 0 at + q * stride * part_elems
  if (p.swiglu) {
    sk_reduce_write_act(p, slots, parts, own_part, own, tid, nthreads, m0, row_lo, row_hi, n_base / kTileN);
    return;
  }
  const int items = (row_hi - row_lo) * (kTileN / 4);
  for (int base = tid; base < items; base += nthreads * kBatch) {
    float4 acc[kBatch];
    int e[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int idx = base + b * nthreads;
      const int safe = idx < items ? idx : tid;            // out-of-range slots re-read a valid item, never stored
      e[b] = (row_lo + (safe >> 5)) * kTileN + (safe & 31) * 4;
      acc[b] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // the test on the part is uniform over the CTA and sits OUTSIDE the batch loop, so the kBatch loads of a
    // part are issued back to back; unrolling over the parts lets the loads of several parts be in flight at once
    // (the sum stays in part order)
#pragma unroll kPartUnroll
    for (int sp = 0; sp < parts; ++sp) {
      float4 v[kBatch];
      if (sp == own_part) {
#pragma unroll
        for (int b = 0; b < kBatch; ++b) v[b] = *reinterpret_cast<const float4*>(own + e[b]);
      } else {
        const float* src = slots + (static_cast<size_t>(sp) * stride + (sp == 0 ? 1 : 0)) * part_elems;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) v[b] = __ldcg(reinterpret_cast<const float4*>(src + e[b]));
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) { acc[b].x += v[b].x; acc[b].y += v[b].y; acc[b].z += v[b].z; acc[b].w += v[b].w; }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const int idx = base + b * nthreads;
      if (idx < items) sk_store4(p, m0 + row_lo + (idx >> 5), n_base + (idx & 31) * 4, acc[b]);
    }
  }
}

// PAIR: the launch is made of clusters of two CTAs that issue MMAs of M = 256 together (cta_group::2).  Rank r of a
// pair owns weight tile 2 * pair_tile + r and HALF of the activation tile (batch rows r * mb / 2 ...), so every SM
// fetches half the activation bytes per k-block; that traffic is what bounds the one-CTA form at 256 batch rows.
// Rank 0 issues the MMAs for both.  Barriers rank 0 waits on (full, acc_empty) also count the arrivals
// of rank 1; the completions of the MMAs (ax_empty, acc_full, tail_full) are multicast to both CTAs.
template <int FMT, bool PAIR>
__global__ void __launch_bounds__(kSkThreads, 1)
wq_gemm_sk_kernel(const __grid_constant__ CUtensorMap tmap_x,
                  const __grid_constant__ CUtensorMap tmap_w,  // only for the direct formats (bf16, fp8)
                  const __grid_constant__ WqGemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t x_bytes = static_cast<uint32_t>(PAIR ? p.mb >> 1 : p.mb) * 128u;   // this CTA's rows of the activation tile
  const uint32_t ax_bytes = x_bytes + kATileBytes;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* c_ring = smem + static_cast<size_t>(p.ax_stages) * ax_bytes;
  constexpr uint32_t kMeta = static_cast<uint32_t>(meta_bytes(FMT));
  constexpr uint32_t kCStage = kCodeBytes + kMeta;
  float* epi_scratch = reinterpret_cast<float*>(c_ring + (fmt_is_direct(FMT) ? 0 : static_cast<size_t>(p.c_stages) * kCStage));
  SkCtl* ctl = reinterpret_cast<SkCtl*>(reinterpret_cast<uint8_t*>(epi_scratch) + kSkEpiScratchBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int cta = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);   // index in the deal
  const int grid = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int unit = blockIdx.x;                   // owner index of the fp32 partial slots
  constexpr uint32_t kPeers = PAIR ? 2u : 1u;
  const int S = p.ax_stages;
  const int NC = p.c_stages;
  // timeline of CTA 0 (debug hook): row i = i-th k-block this CTA processes; slots as in wq_gemm.cu
  // (with CTA pairs rank 1 of the first pair records too, in rows 64..127, on its own SM's clock)
  CB_TRACE_ONLY(unsigned long long* trace = (p.trace && blockIdx.x <= (PAIR ? 1u : 0u)) ? p.trace + blockIdx.x * 64 * 8 : nullptr;)
  CB_STAMP(threadIdx.x == 0, 6);
  // every CTA: wall-clock entry / exit in slots 0 / 1 of row `cta` (the buffer has >= gridDim.x rows)
  CB_WALL_STAMP(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSkMaxAx; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1 + (fmt_is_direct(FMT) ? 0 : kSkGroupWarps * kPeers));
      mbar_init(smem_u32(&ctl->ax_empty[s]), 1);
    }
    for (int s = 0; s < kSkMaxC; ++s) {
      mbar_init(smem_u32(&ctl->c_full[s]), 1);
      mbar_init(smem_u32(&ctl->c_empty[s]), kSkGroupWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[b]), kSkEpiWarps * kPeers);
    }
    mbar_init(smem_u32(&ctl->tail_full), 1);
    ctl->abort_flag = 0;
    ctl->is_last = 0;
    ctl->deferred_count = 0;
    ctl->deferred_next = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(&ctl->tmem_base), p.tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&ctl->tmem_base), p.tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();        // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  // Programmatic dependent launch: the set-up above and the first copies of the packed weights (which no kernel
  // writes) may run while the previous kernel of the stream is still finishing; every role that reads activations,
  // residuals, counters or a device work list, or writes results, waits for it first.
  pdl_launch_dependents();
  if (p.group_tiles) pdl_wait();            // the deal itself reads the work list written by the routing kernels
  SkIter it;
  it.init(p, cta);
  SkSegment seg;

  if (warp == 0) {
    // ------------------------------------------------ activation (and bf16 weight) tiles
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      if (fmt_is_direct(FMT)) tma_prefetch_desc(&tmap_w);
      pdl_wait();
      bool ok = true;
      if (p.tp.mode & kTpGatherWait) {
        // the packed weights stream meanwhile (warp 2 does not wait): all-gather overlapped with weight traffic
        const uint32_t target = p.tp.ag_state[0] + p.tp.ag_expected;
        for (int r = 0; r < p.tp.size && ok; ++r) ok = wait_counter(p.tp.ag_flag + r, target, abort_flag);
      }
      const uint32_t tx = x_bytes + (fmt_is_direct(FMT) ? static_cast<uint32_t>(kATileBytes) : 0u);
      constexpr int kBK = fmt_block_k(FMT);        // K columns per stage: 64 bf16 or 128 e4m3 (128 bytes either way)
      SkRing r;
      CB_TRACE_ONLY(int ti = 0;)
      while (ok && it.next(p, cta, grid, seg)) {
        const SkCoords c = sk_coords(p, seg.tile, rank);
        const int w_row = c.expert * p.N + c.n_tile * kTileN;   // bf16 weights: experts stacked as [E * N, K]
        for (int kb = seg.kb_lo; kb < seg.kb_hi; ++kb) {
          if (r.wraps && !mbar_wait_park(smem_u32(&ctl->ax_empty[r.s]), (r.wraps - 1u) & 1u, abort_flag)) { ok = false; break; }
          CB_STAMP(ti < 64, ti * 8 + 0);
          CB_TRACE_ONLY(++ti;)
          uint8_t* st = smem + static_cast<size_t>(r.s) * ax_bytes;
          const uint32_t bar = smem_u32(&ctl->full[r.s]);
          if (PAIR) {
            // both CTAs' copies complete on rank 0's barrier, which expects the bytes of both; a completion that
            // lands before the expectation is posted only drives the count negative inside the same phase
            const uint32_t bar0 = cluster_map(bar, 0);
            if (rank == 0) mbar_expect_tx(bar, 2u * tx);
            tma_load_2d_pair(smem_u32(st), &tmap_x, kb * kBK, c.m0 + rank * (p.mb >> 1), bar0);
            if (fmt_is_direct(FMT)) tma_load_2d_pair(smem_u32(st + x_bytes), &tmap_w, kb * kBK, w_row, bar0);
          } else {
            mbar_expect_tx(bar, tx);
            tma_load_2d(smem_u32(st), &tmap_x, kb * kBK, c.m0, bar);
            if (fmt_is_direct(FMT)) tma_load_2d(smem_u32(st + x_bytes), &tmap_w, kb * kBK, w_row, bar);
          }
          r.advance(S);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------ packed codes + metadata
    if (!fmt_is_direct(FMT) && lane == 0) {
      bool ok = true;
      SkRing r;
      while (ok && it.next(p, cta, grid, seg)) {
        const SkCoords c = sk_coords(p, seg.tile, rank);
        const uint8_t* cbase = p.codes + static_cast<size_t>(c.expert) * p.group_code_stride +
                               static_cast<size_t>(c.n_tile) * p.k_blocks * kCodeBytes;
        const uint8_t* mbase = p.meta + static_cast<size_t>(c.expert) * p.group_meta_stride +
                               static_cast<size_t>(c.n_tile) * p.meta_blocks * kMeta;
        for (int kb = seg.kb_lo; kb < seg.kb_hi; ++kb) {
          if (r.wraps && !mbar_wait_park(smem_u32(&ctl->c_empty[r.s]), (r.wraps - 1u) & 1u, abort_flag)) { ok = false; break; }
          const uint32_t dst = smem_u32(c_ring + static_cast<size_t>(r.s) * kCStage);
          const uint32_t bar = smem_u32(&ctl->c_full[r.s]);
          mbar_expect_tx(bar, kCStage);
          bulk_g2s(dst, cbase + static_cast<size_t>(kb) * kCodeBytes, kCodeBytes, bar);
          bulk_g2s(dst + kCodeBytes, mbase + static_cast<size_t>(kb >> p.meta_shift) * kMeta, kMeta, bar);
          r.advance(NC);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (warp-uniform loop, one elected lane issues).
    // The chain of dependent instructions per k-block (barrier test, vote, fence, four MMAs, commit) is the pace of
    // the kernel when the operands are ready ahead of time, so the activation tile and the decoded weight tile
    // complete ONE barrier (`full`), tested once.  (A loop run by a single thread of the warp was measured slower:
    // 550-700 cycles from the barrier to the commit instead of 150-300.)
    const bool leader = elect_one();
    // operand formats: bf16 x bf16 (kind::f16) or e4m3 x e4m3 (kind::f8f6f4)
    const uint32_t idesc = umma_idesc(PAIR ? 2 * kTileN : kTileN, static_cast<uint32_t>(p.mb), FMT == kFmtFp8 ? 0u : 1u,
                                      FMT == kFmtFp8 ? 0u : 1u);
    const uint32_t smem_base = smem_u32(smem);
    const uint64_t desc_hi = umma_desc_sw128(0);
    SkRing r;
    int seg_idx = 0;
    int i_global = 0;
    bool ok = !(PAIR && rank != 0);        // rank 1 of a pair issues nothing: rank 0's MMAs use both CTAs' operands
    while (ok && it.next(p, cta, grid, seg)) {
      const int buf = seg_idx & 1;
      const uint32_t use = static_cast<uint32_t>(seg_idx >> 1);
      const bool tail = !it.has_more(p);
      if (use) {
        ok = mbar_wait_park(smem_u32(&ctl->acc_empty[buf]), (use - 1u) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf) * p.acc_cols;
      uint32_t accumulate = 0;
      for (int kb = seg.kb_lo; kb < seg.kb_hi; ++kb, ++i_global) {
        ok = mbar_wait_park(smem_u32(&ctl->full[r.s]), r.wraps & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        CB_STAMP(leader && i_global < 64, i_global * 8 + 4);
        tc_fence_after();
        const uint32_t st = smem_base + static_cast<uint32_t>(r.s) * ax_bytes;
        const uint64_t bdesc = desc_hi | static_cast<uint64_t>((st & 0x3FFFFu) >> 4);
        const uint64_t adesc = desc_hi | static_cast<uint64_t>(((st + x_bytes) & 0x3FFFFu) >> 4);
        if (leader) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            // +32 bytes along K inside the swizzle atom = +2 in the (addr >> 4) field
            if constexpr (FMT == kFmtFp8) {
              if (PAIR) umma_f8f6f4_pair(tmem_d, adesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : accumulate);
              else umma_f8f6f4(tmem_d, adesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : accumulate);
            } else {
              if (PAIR) umma_f16_pair(tmem_d, adesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : accumulate);
              else umma_f16(tmem_d, adesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : accumulate);
            }
          }
          if (PAIR) {
            tc_commit_pair(smem_u32(&ctl->ax_empty[r.s]), 3u);
            if (kb == seg.kb_hi - 1) {
              tc_commit_pair(smem_u32(&ctl->acc_full[buf]), 3u);
              if (tail) tc_commit_pair(smem_u32(&ctl->tail_full), 3u);
            }
          } else {
            tc_commit(smem_u32(&ctl->ax_empty[r.s]));
            if (kb == seg.kb_hi - 1) {
              tc_commit(smem_u32(&ctl->acc_full[buf]));
              if (tail) tc_commit(smem_u32(&ctl->tail_full));
            }
          }
        }
        accumulate = 1;
        CB_STAMP(leader && i_global < 64, i_global * 8 + 5);
        r.advance(S);
      }
      ++seg_idx;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ decode (warps 7..22) and epilogue (warps 3..6)
    // Geometry of the current segment (set by seg_geometry) and the shared LAST-segment epilogue.
    int m0 = 0, rows_here = 0, n_base = 0, tile_id = 0, w_base = 0;
    auto seg_geometry = [&]() {
      const SkCoords c = sk_coords(p, seg.tile, rank);
      tile_id = c.tile_id;
      m0 = c.m0;
      rows_here = c.rows;
      n_base = c.n_tile * kTileN;
      w_base = c.expert * p.N;              // first weight row of the tile's expert in the stacked matrix
    };
    // fp8: the feature's weight scale times the token's activation scale, applied as the sums leave tensor memory
    // (partial sums of a streamed tile are linear in both, so every later path sees finished values); `quad` is the
    // warp's lane quadrant, c0 the first batch row of the 16-column chunk
    auto scale_acc = [&](uint32_t (&acc)[16], int quad, int c0) {
      if constexpr (FMT == kFmtFp8) {
        const int nn = n_base + quad * 32 + lane;
        const float ws = nn < p.N ? p.row_scale[w_base + nn] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int r = c0 + j;
          const float xs = r < rows_here ? __ldg(p.col_scale + m0 + r) : 0.f;
          acc[j] = __float_as_uint(__uint_as_float(acc[j]) * (ws * xs));
        }
      }
    };
    // Last segment of the CTA: nothing is left to overlap with, so all 20 of these warps (640 threads) do the
    // epilogue together.  The rings are idle once the accumulator is complete, so the whole fp32 tile is staged
    // in their memory ([row][128 features]); then every warp writes full 256-byte rows (or 512-byte fp32 rows
    // of the partial), and a last arriver reduces with 640 threads, reading its own part from shared memory.
    // All 640 threads execute every tail_bar() whatever happened before: work is switched off by `ok`, never
    // the control flow.
    // Streamed tiles are finished by ALL their contributors, each summing its share of the rows at the end of its CTA,
    // instead of by the last contributor alone (15 us of serial tail on a third of the CTAs at 256 batch rows).
    // Rows pushed to other ranks keep the single finisher: their arrival counters are raised once per tile.
    const bool sliced = !(p.tp.mode & kTpScatterPush);
    auto tail_epilogue = [&](int seg_idx, bool ok) {
      pdl_wait();                                             // long since satisfied; orders this thread's global accesses
      const int tt = threadIdx.x - kSkFirstEpiWarp * 32;      // 0..639
      const int nthr = (kSkEpiWarps + kSkDecodeWarps) * 32;
      const int buf = seg_idx & 1;
      ok = ok && mbar_wait_park(smem_u32(&ctl->tail_full), 0u, abort_flag);
      ok = __all_sync(0xffffffffu, ok) && !*abort_flag;
      tc_fence_after();
      CB_STAMP(tt == 0 && seg_idx < 4, (8 + seg_idx) * 8 + 6);
      seg_geometry();
      const bool whole = seg.parts == 1;
      float* stg = reinterpret_cast<float*>(smem);
      if (ok) {
        const int quad = warp & 3;                              // TMEM lane quadrant this warp may read
        const int slice = (warp - kSkFirstEpiWarp) >> 2;        // five warps share a quadrant
        const uint32_t taddr = tmem_base + static_cast<uint32_t>(buf) * p.acc_cols + (static_cast<uint32_t>(quad * 32) << 16);
        for (int ci = slice; ci < (p.mb >> 4); ci += (kSkEpiWarps + kSkDecodeWarps) / 4) {
          uint32_t acc[16];
          tmem_ld_32x16(taddr + ci * 16, acc);
          tmem_ld_wait();
          scale_acc(acc, quad, ci * 16);
#pragma unroll
          for (int j = 0; j < 16; ++j) stg[(ci * 16 + j) * kTileN + quad * 32 + lane] = __uint_as_float(acc[j]);
        }
      }
      tc_fence_before();
      tail_bar();
      bool finalized = whole;
      if (whole) {
        if (ok && p.swiglu) {
          for (int idx = tt; idx < rows_here * 16; idx += nthr) {
            const int mm = idx >> 4, j0 = (idx & 15) * 4;
            const float* gp = stg + mm * kTileN + act_gate_col(j0);
            float4 g = *reinterpret_cast<const float4*>(gp), u = *reinterpret_cast<const float4*>(gp + 16);
            g.x *= p.alpha; g.y *= p.alpha; g.z *= p.alpha; g.w *= p.alpha;
            u.x *= p.alpha; u.y *= p.alpha; u.z *= p.alpha; u.w *= p.alpha;
            store_act4(p, m0 + mm, n_base / kTileN, j0, g, u);
          }
        } else if (ok)
          for (int idx = tt; idx < rows_here * (kTileN / 4); idx += nthr)
            sk_store4(p, m0 + (idx >> 5), n_base + (idx & 31) * 4, *reinterpret_cast<const float4*>(stg + static_cast<size_t>(idx) * 4));
      } else {
        if (ok) {
          float* slot = sk_slot(p, unit, seg.part);
          for (int idx = tt; idx < p.mb * (kTileN / 4); idx += nthr)
            *reinterpret_cast<float4*>(slot + static_cast<size_t>(idx) * 4) = *reinterpret_cast<const float4*>(stg + static_cast<size_t>(idx) * 4);
        }
        __threadfence();
        tail_bar();
        if (tt == 0) {
          uint32_t last = 0;
          if (ok) {
            const uint32_t prev = atomicAdd(&p.counters[tile_id], 1u);
            if (sliced) {
              // every contributor sums its own share of the rows further down (SkCtl::deferred)
              ctl->deferred[ctl->deferred_count] = seg;
              ctl->deferred_count = ctl->deferred_count + 1;
            } else {
              last = (prev == static_cast<uint32_t>(seg.parts) - 1u) ? 1u : 0u;
              if (last) p.counters[tile_id] = 0;
            }
          }
          ctl->is_last = last;
        }
        tail_bar();
        if (ctl->is_last && !*abort_flag) {
          __threadfence();
          finalized = true;
          sk_reduce_write<4, 2>(p, seg, unit, tt, nthr, m0, 0, rows_here, n_base, stg);
        }
      }
      if (p.tp.mode & kTpScatterPush) {
        // every row of the finished tile is on its way: barrier (all stores ordered before thread 0), then the
        // owners' arrival counters after ONE release fence at system scope (cumulative)
        tail_bar();
        if (finalized && tt == 0 && !*abort_flag) {
          const int m_last = min(p.M, m0 + p.mb) - 1;
          fence_acq_rel_sys();
          for (int o = m0 / p.tp.rows_per_rank; o <= m_last / p.tp.rows_per_rank; ++o)
            red_relaxed_sys_add(p.tp.rs_flag[o] + p.tp.rank, 1u);
        }
      }
      // fix-ups deferred by the segments of this CTA (see SkCtl::deferred), now with 640 threads.  Sliced form:
      // this CTA sums ITS share of the rows of every streamed tile it contributed to, once all parts of the tile
      // have landed (they were written long ago as a rule: streamed runs come first in every CTA's deal); the
      // arrival counter counts the parts, then the finished shares, and the last share puts it back to zero.
      tail_bar();
      const uint32_t n_def = ctl->deferred_count;
      for (uint32_t di = ctl->deferred_next; di < n_def; ++di) {
        const SkSegment ds = ctl->deferred[di];
        const SkCoords c = sk_coords(p, ds.tile, rank);
        int row_lo = 0, row_hi = c.rows;
        if (sliced) {
          row_lo = c.rows * ds.part / ds.parts;
          row_hi = c.rows * (ds.part + 1) / ds.parts;
          if (tt == 0 && !wait_counter_gpu(&p.counters[c.tile_id], static_cast<uint32_t>(ds.parts), abort_flag)) *abort_flag = 2;
          tail_bar();
        }
        if (!*abort_flag) {
          // sliced: thread 0 has acquired the counter and the barrier orders the CTA behind it; the partials are
          // read from L2 (ld.cg), where the writers' fences put them
          if (!sliced) __threadfence();
          if (sliced) sk_reduce_write<2, 4>(p, ds, unit, tt, nthr, c.m0, row_lo, row_hi, c.n_tile * kTileN, nullptr);
          else sk_reduce_write<4, 2>(p, ds, unit, tt, nthr, c.m0, row_lo, row_hi, c.n_tile * kTileN, nullptr);
        }
        if (sliced) {
          tail_bar();
          if (tt == 0 && !*abort_flag) {
            const uint32_t prev = atomicAdd(&p.counters[c.tile_id], 1u);
            if (prev == 2u * static_cast<uint32_t>(ds.parts) - 1u) p.counters[c.tile_id] = 0;
          }
        }
        if (p.tp.mode & kTpScatterPush) {
          tail_bar();
          if (tt == 0 && !*abort_flag) {
            const int m_last = min(p.M, c.m0 + p.mb) - 1;
            fence_acq_rel_sys();
            for (int o = c.m0 / p.tp.rows_per_rank; o <= m_last / p.tp.rows_per_rank; ++o)
              red_relaxed_sys_add(p.tp.rs_flag[o] + p.tp.rank, 1u);
          }
        }
      }
      CB_STAMP(tt == 0 && seg_idx < 4, (8 + seg_idx) * 8 + 7);
    };

    if (warp >= kSkFirstDecodeWarp) {
      // ---------------------------------------------- decode
      const int g = (warp - kSkFirstDecodeWarp) / kSkGroupWarps;                   // this warp's group
      const int r = threadIdx.x - kSkFirstDecodeWarp * 32 - g * kSkGroupWarps * 32;    // row of the weight tile, 0..127
      // A thread decodes one whole 128-byte row of the k-block (64 weights: two 16-byte code chunks, the halves
      // h = 0, 1), so that what is paid per k-block and thread (barrier waits and arrivals, ring arithmetic, the
      // proxy fence) is paid once per 64 weights; a profile of the two-group form (32 weights per thread) showed
      // ~270 instructions per thread and k-block against ~110 of decode arithmetic.
      const uint32_t code_off = static_cast<uint32_t>(r * 16);
      const uint32_t a_off = x_bytes + static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128);
      const uint32_t sw = static_cast<uint32_t>(r & 7);
      SkRing rc, ra;
      int i_global = 0;
      int seg_idx = 0;
      bool ok = true;
      // never leaves the loop early: the last segment ends at barriers shared with the epilogue warps
      while (it.next(p, cta, grid, seg)) {
        const bool tail = !it.has_more(p);
        if (!fmt_is_direct(FMT) && ok) {
          // this group's k-blocks are every fourth one; the rings are stepped over the other groups' k-blocks
          // arithmetically instead of by empty loop iterations
          const int len = seg.kb_hi - seg.kb_lo;
          const int skip = (g - i_global) & (kSkDecodeGroups - 1);
          rc.advance_by(skip < len ? skip : len, NC);
          ra.advance_by(skip < len ? skip : len, S);
          for (int jj = skip; jj < len; jj += kSkDecodeGroups) {
            const int ig = i_global + jj;
            if (!mbar_wait_park(smem_u32(&ctl->c_full[rc.s]), rc.wraps & 1u, abort_flag)) { ok = false; break; }
            CB_STAMP(r == 0 && ig < 64, ig * 8 + 2);
            const uint8_t* pk = c_ring + static_cast<size_t>(rc.s) * kCStage;
            const uint4 w0 = *reinterpret_cast<const uint4*>(pk + code_off);
            const uint4 w1 = *reinterpret_cast<const uint4*>(pk + code_off + 128 * 16);
            // metadata: Cubic = the row's level table (16 bytes; one scale group covers the whole k-block); the other
            // formats = bf16 pairs {scale, offset} (or the two 16-column block scales) of each 32-column half
            uint4 t = make_uint4(0u, 0u, 0u, 0u);
            if constexpr (FMT == kFmtCubic4) {
              t = *reinterpret_cast<const uint4*>(pk + kCodeBytes + code_off);
            } else {
              const uint32_t* meta = reinterpret_cast<const uint32_t*>(pk + kCodeBytes);
              t.x = meta[r];
              t.y = meta[128 + r];
            }
            // the codes and metadata are in registers: hand the slot back to the copy warp right away
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->c_empty[rc.s]));
            uint8_t* arow = nullptr;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint4 words = h ? w1 : w0;
              uint32_t o[4][4];
              if constexpr (FMT == kFmtCubic4) {
                cubic_lut8(words.x, t, o[0]);
                cubic_lut8(words.y, t, o[1]);
                cubic_lut8(words.z, t, o[2]);
                cubic_lut8(words.w, t, o[3]);
              } else {
                const uint32_t so = h ? t.y : t.x;
                const uint32_t c0 = bf2_dup(so), c1 = bf2_dup_hi(so);
                if constexpr (FMT == kFmtNvfp4) {
                  // columns 32h + 8j: the 16-column block scale is the low half for j < 2, the high half after
                  decode8<FMT>(words.x, c0, 0u, 0u, o[0]);
                  decode8<FMT>(words.y, c0, 0u, 0u, o[1]);
                  decode8<FMT>(words.z, c1, 0u, 0u, o[2]);
                  decode8<FMT>(words.w, c1, 0u, 0u, o[3]);
                } else {
                  decode8<FMT>(words.x, c0, c1, 0u, o[0]);
                  decode8<FMT>(words.y, c0, c1, 0u, o[1]);
                  decode8<FMT>(words.z, c0, c1, 0u, o[2]);
                  decode8<FMT>(words.w, c0, c1, 0u, o[3]);
                }
              }
              if (h == 0) {
                // the arithmetic above ran while the slot may still be read by MMAs; only the stores wait for it
                if (ra.wraps && !mbar_wait_park(smem_u32(&ctl->ax_empty[ra.s]), (ra.wraps - 1u) & 1u, abort_flag)) { ok = false; break; }
                arow = smem + static_cast<size_t>(ra.s) * ax_bytes + a_off;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(arow + (((static_cast<uint32_t>(h * 4 + j)) ^ sw) << 4)) =
                    make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
            }
            if (!ok) break;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (PAIR && rank != 0) mbar_arrive_cluster(cluster_map(smem_u32(&ctl->full[ra.s]), 0));
              else mbar_arrive(smem_u32(&ctl->full[ra.s]));
            }
            CB_STAMP(r == 0 && ig < 64, ig * 8 + 3);
            const int step = len - jj < kSkDecodeGroups ? len - jj : kSkDecodeGroups;
            rc.advance_by(step, NC);
            ra.advance_by(step, S);
          }
          i_global += len;
        }
        if (tail) tail_epilogue(seg_idx, ok);
        ++seg_idx;
      }
    } else {
      // ---------------------------------------------- epilogue of every segment but the last (warps 3..6)
      // These four warps meet at a named barrier inside the loop, so none of them may leave the loop early:
      // after a failed wait they keep walking the segment list with the work switched off.
      const int quad = warp & 3;                                 // TMEM lane quadrant this warp may read
      const int et = threadIdx.x - kSkFirstEpiWarp * 32;         // 0..127
      int seg_idx = 0;
      pdl_wait();
      while (it.next(p, cta, grid, seg)) {
        if (!it.has_more(p)) {
          tail_epilogue(seg_idx, true);
          break;
        }
        const int buf = seg_idx & 1;
        const uint32_t use = static_cast<uint32_t>(seg_idx >> 1);
        bool ok = mbar_wait_park(smem_u32(&ctl->acc_full[buf]), use & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok) && !*abort_flag;
        tc_fence_after();
        CB_STAMP(et == 0 && seg_idx < 4, (8 + seg_idx) * 8 + 6);
        seg_geometry();
        const bool whole = seg.parts == 1;
        if (ok) {
          // TMEM gives a thread one output feature (lane) and 16 batch rows (registers); memory wants rows of
          // consecutive features.  Each warp transposes 16 x 32 fp32 through its own 2 KiB of shared memory:
          // lane L then owns rows (L >> 3) + 4 i, features 4 (L & 7) .. + 3 of the chunk: 8-byte bf16 (or
          // 16-byte fp32 partial) stores, eight lanes covering the 64 contiguous bytes of one row.
          float* scr = epi_scratch + (warp - kSkFirstEpiWarp) * (16 * 32);
          const int f4 = (lane & 7) * 4;
          float* slot = whole ? nullptr : sk_slot(p, unit, seg.part) + quad * 32 + f4;
          const uint32_t taddr = tmem_base + static_cast<uint32_t>(buf) * p.acc_cols + (static_cast<uint32_t>(quad * 32) << 16);
          for (int c0 = 0; c0 < p.mb; c0 += 16) {
            uint32_t acc[16];
            tmem_ld_32x16(taddr + c0, acc);
            tmem_ld_wait();
            scale_acc(acc, quad, c0);
#pragma unroll
            for (int j = 0; j < 16; ++j) scr[j * 32 + lane] = __uint_as_float(acc[j]);
            __syncwarp();
            if (whole && p.swiglu) {
              // this warp's 32 tile rows are 16 gate + 16 up rows of the same 16 features: lane L owns rows
              // (L >> 2) + 8 i, features 4 (L & 3) .. + 3 (all 32 lanes busy, 32 contiguous bytes per row)
              const int a4 = (lane & 3) * 4;
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int row = (lane >> 2) + 8 * i;
                if (c0 + row < rows_here) {
                  float4 g = *reinterpret_cast<const float4*>(scr + row * 32 + a4);
                  float4 u = *reinterpret_cast<const float4*>(scr + row * 32 + 16 + a4);
                  g.x *= p.alpha; g.y *= p.alpha; g.z *= p.alpha; g.w *= p.alpha;
                  u.x *= p.alpha; u.y *= p.alpha; u.z *= p.alpha; u.w *= p.alpha;
                  store_act4(p, m0 + c0 + row, n_base / kTileN, quad * 16 + a4, g, u);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int row = (lane >> 3) + 4 * i;
                const float4 v = *reinterpret_cast<const float4*>(scr + row * 32 + f4);
                if (!whole) {
                  *reinterpret_cast<float4*>(slot + static_cast<size_t>(c0 + row) * kTileN) = v;
                } else if (c0 + row < rows_here) {
                  sk_store4(p, m0 + c0 + row, n_base + quad * 32 + f4, v);
                }
              }
            }
            __syncwarp();                                  // the scratch is rewritten by the next chunk
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR && rank != 0) mbar_arrive_cluster(cluster_map(smem_u32(&ctl->acc_empty[buf]), 0));
          else mbar_arrive(smem_u32(&ctl->acc_empty[buf]));
        }
        CB_STAMP(et == 0 && seg_idx < 4, (8 + seg_idx) * 8 + 7);

        bool finalized = whole;
        if (!whole) {
          // streamed tile: publish the partial, count arrivals; the last arriver sums all parts in part order
          __threadfence();
          epi_bar();
          if (et == 0) {
            uint32_t last = 0;
            if (ok) {
              const uint32_t prev = atomicAdd(&p.counters[tile_id], 1u);
              if (sliced) {
                last = 1u;                                  // every contributor finishes its share at the end of the CTA
              } else {
                last = (prev == static_cast<uint32_t>(seg.parts) - 1u) ? 1u : 0u;
                if (last) p.counters[tile_id] = 0;
              }
            }
            ctl->is_last = last;
          }
          epi_bar();
          const bool last = ctl->is_last != 0;
          epi_bar();                                   // is_last has been read by all before it can change again
          if (last && !*abort_flag && et == 0) {
            // summing the partials here would hold these four warps (and with them the accumulator hand-off of
            // the running main loop) for tens of microseconds: note the tile, finish it at the end of the CTA
            ctl->deferred[ctl->deferred_count] = seg;
            ctl->deferred_count = ctl->deferred_count + 1;
          }
        }
        if (p.tp.mode & kTpScatterPush) {
          epi_bar();
          if (finalized && et == 0 && !*abort_flag) {
            const int m_last = min(p.M, m0 + p.mb) - 1;
            fence_acq_rel_sys();
            for (int o = m0 / p.tp.rows_per_rank; o <= m_last / p.tp.rows_per_rank; ++o)
              red_relaxed_sys_add(p.tp.rs_flag[o] + p.tp.rank, 1u);
          }
        }
        ++seg_idx;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  // a CTA of a pair leaves only when its peer is done too: until then the peer may arrive on this CTA's barriers
  // and rank 0's MMAs may read this CTA's shared memory; the tensor memory of the pair is freed after it
  if (PAIR) cluster_sync_all();
  CB_STAMP(threadIdx.x == 0, 7);
  CB_WALL_STAMP(1);
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, p.tmem_cols);
    else tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if ((p.tp.mode & kTpGatherWait) && threadIdx.x == 0) {
    // the last CTA of the grid closes the epoch of the gathered buffer
    if (atomicAdd(&p.tp.ag_state[1], 1u) == gridDim.x - 1u) {
      p.tp.ag_state[1] = 0;
      __threadfence();
      atomicAdd(&p.tp.ag_state[0], p.tp.ag_expected);
    }
  }
  if (threadIdx.x == 0 && ctl->abort_flag)
    atomicExch(p.status, static_cast<uint32_t>(ctl->abort_flag == 2 ? kErrFlagTimeout : kErrBarrierTimeout));
}

template <int FMT>
static int launch_sk_fmt(const CUtensorMap& tx, const CUtensorMap& tw, const WqGemmParams& p, int grid, size_t smem,
                         cudaStream_t stream) {
  static bool configured[64] = {};     // per device, like the attribute itself
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -18;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(wq_gemm_sk_kernel<FMT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  return static_cast<int>(launch(wq_gemm_sk_kernel<FMT, false>, dim3(static_cast<unsigned>(grid)), dim3(kSkThreads), smem,
                                 stream, tx, tw, p));
}

// CTA pairs: `grid` CTAs (even) launched as clusters of two.
template <int FMT>
static int launch_sk_pair_fmt(const CUtensorMap& tx, const CUtensorMap& tw, const WqGemmParams& p, int grid, size_t smem,
                              cudaStream_t stream) {
  static bool configured[64] = {};     // per device, like the attribute itself
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -18;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(wq_gemm_sk_kernel<FMT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  return static_cast<int>(launch(wq_gemm_sk_kernel<FMT, true>, dim3(static_cast<unsigned>(grid)), dim3(kSkThreads), smem,
                                 stream, dim3(2, 1, 1), tx, tw, p));
}

// How many CTA pairs can be resident at once (both CTAs of a cluster sit in one GPC, so a GPC with an odd number of
// usable SMs leaves one out): the persistent schedule must not launch more, or the surplus pairs run as a second wave.
template <int FMT>
static int max_resident_pairs() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    if (cudaFuncSetAttribute(wq_gemm_sk_kernel<FMT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024) != cudaSuccess)
      return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kSkThreads, 1, 1);
    cfg.dynamicSmemBytes = 232448 - 1024;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, wq_gemm_sk_kernel<FMT, true>, &cfg) != cudaSuccess) n = 0;
    cached[dev] = n > 0 ? n : -1;
  }
  return cached[dev] > 0 ? cached[dev] : 0;
}
static int max_resident_pairs_fmt(int fmt) {
  switch (fmt) {
    case kFmtCubic4: return max_resident_pairs<kFmtCubic4>();
    case kFmtAffine4: return max_resident_pairs<kFmtAffine4>();
    case kFmtNvfp4: return max_resident_pairs<kFmtNvfp4>();
    case kFmtFp8: return max_resident_pairs<kFmtFp8>();
    default: return max_resident_pairs<kFmtBf16>();
  }
}

int streamk_resident_pairs(int fmt) { return max_resident_pairs_fmt(fmt); }

// Whether a launch with these sizes runs on CTA pairs: 256 batch rows per tile (that is where the activation tile
// bounds the one-CTA form), an even number of weight tiles, not the grouped (expert) mode.
bool streamk_pair_eligible(const WqGemmParams& p, int N) {
  const int n_tiles = (N + kTileN - 1) / kTileN;
  return p.mb == 256 && (n_tiles & 1) == 0 && p.group_tiles == nullptr;
}

// Schedule and launch.  `min_units` > 0 overrides the smallest run of k-blocks a CTA may be dealt in the
// streamed region (tests use 1..2 to force many-part tiles); 0 picks it from a cost model: a run costs about
// 0.34 us per k-block, every extra part of a tile costs the reducer about mb / 256 us, so the best number of
// parts is sqrt(k_blocks * 0.34 * 256 / mb) and the run length k_blocks over that.
int launch_streamk(int fmt, const CUtensorMap& tx, const CUtensorMap& tw, WqGemmParams p, size_t workspace_bytes,
                   int sm_count, int min_units, cudaStream_t stream, int grouped_max_items) {
  if (sm_count < 1) return -15;
  p.n_tiles = (p.N + kTileN - 1) / kTileN;
  const int m_tiles = (p.M + p.mb - 1) / p.mb;
  p.tiles = p.n_tiles * m_tiles;
  if (p.pair) {
    // the deal is over PAIRS of CTAs and pairs of adjacent weight tiles; below, "CTA" and "SM" read "pair"
    if (!streamk_pair_eligible(p, p.N) || sm_count < 2) return -15;
    p.tiles = (p.n_tiles >> 1) * m_tiles;
    sm_count >>= 1;
    const int resident = max_resident_pairs_fmt(fmt);
    if (resident < 1) return -15;
    if (sm_count > resident) sm_count = resident;
  }
  if (p.group_tiles) {
    // grouped expert GEMMs: whole tiles only (the tile count lives on the device), one persistent CTA per SM at
    // most; what this buys over one CTA per tile is the set-up and epilogue of ~30 waves of small tiles
    p.tiles = 0;
    workspace_bytes = 0;
  }
  if (p.meta_k_blocks < 1 || (p.meta_k_blocks & (p.meta_k_blocks - 1)) != 0) return -16;
  p.meta_shift = 0;
  while ((1 << p.meta_shift) < p.meta_k_blocks) ++p.meta_shift;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(p.mb)) cols <<= 1;
  p.acc_cols = cols;
  p.tmem_cols = 2 * cols;

  if (min_units <= 0) {
    int est = 1;
    while (static_cast<long long>(est) * est * 87 < static_cast<long long>(p.k_blocks) * p.mb) ++est;   // ceil(sqrt(kb * mb / 87))
    min_units = est < 4 ? 4 : est;
  }
  p.sk_tiles = p.tiles <= sm_count ? p.tiles : p.tiles % sm_count;
  p.sk_ctas = 0;
  if (p.group_tiles) p.sk_tiles = 0;
  if (p.sk_tiles > 0) {
    // a CTA of the streamed region owns two fp32 partial slots (see sk_slot)
    const size_t part_bytes = static_cast<size_t>(p.mb) * kTileN * sizeof(float);
    const long long slots_fit =
        (p.workspace && p.counters) ? static_cast<long long>(workspace_bytes / ((p.pair ? 4 : 2) * part_bytes)) : 0;
    long long want = static_cast<long long>(p.sk_tiles) * p.k_blocks / min_units;
    if (want > sm_count) want = sm_count;
    if (want < 1) want = 1;
    if (want > slots_fit) want = slots_fit;
    if (want < 1) {
      p.sk_tiles = 0;            // no scratch: every tile stays whole, one per CTA and wave
    } else {
      p.sk_ctas = static_cast<int>(want);   // may be < sk_tiles: a CTA then covers several tiles, split only at run ends
    }
  }
  if (static_cast<long long>(p.sk_tiles) * p.k_blocks * (sm_count + 1) >= (1LL << 31)) return -19;   // SkIter is 32-bit
  int grid = p.group_tiles ? grouped_max_items * p.n_tiles : p.tiles - p.sk_tiles;
  if (grid > sm_count) grid = sm_count;
  if (grid < p.sk_ctas) grid = p.sk_ctas;
  if (grid < 1) return -17;

  const size_t ax = static_cast<size_t>(p.pair ? p.mb >> 1 : p.mb) * 128 + kATileBytes;
  const size_t budget = 232448 - 1024 - 1024 - sizeof(SkCtl) - kSkEpiScratchBytes;
  const size_t kSkCStageBytes = static_cast<size_t>(sk_cstage_bytes(fmt));
  int S, NC;
  if (fmt_is_direct(fmt)) {
    NC = 0;
    S = static_cast<int>(budget / ax);
  } else {
    S = static_cast<int>((budget - 4 * kSkCStageBytes) / ax);
    if (S > kSkMaxAx) S = kSkMaxAx;
    NC = static_cast<int>((budget - S * ax) / kSkCStageBytes);
    if (NC > kSkMaxC) NC = kSkMaxC;
  }
  if (S > kSkMaxAx) S = kSkMaxAx;
  if (S < 2 || (!fmt_is_direct(fmt) && NC < 2)) return -14;
  if (fmt == kFmtFp8Block) return -14;            // block scales need the per-stage promotion of the per-tile kernel
  p.ax_stages = S;
  p.c_stages = NC;
  size_t smem = S * ax + static_cast<size_t>(NC) * kSkCStageBytes + kSkEpiScratchBytes + sizeof(SkCtl) + 1024;
  if (p.pair) {
    // the last segment's epilogue stages the fp32 tile [mb][128] in the ring memory
    const size_t stage_bytes = static_cast<size_t>(p.mb) * kTileN * sizeof(float);
    const size_t rings = S * ax + static_cast<size_t>(NC) * kSkCStageBytes;
    if (rings < stage_bytes) smem += stage_bytes - rings;
    switch (fmt) {
      case kFmtCubic4: return launch_sk_pair_fmt<kFmtCubic4>(tx, tw, p, 2 * grid, smem, stream);
      case kFmtAffine4: return launch_sk_pair_fmt<kFmtAffine4>(tx, tw, p, 2 * grid, smem, stream);
      case kFmtNvfp4: return launch_sk_pair_fmt<kFmtNvfp4>(tx, tw, p, 2 * grid, smem, stream);
      case kFmtFp8: return launch_sk_pair_fmt<kFmtFp8>(tx, tw, p, 2 * grid, smem, stream);
      default: return launch_sk_pair_fmt<kFmtBf16>(tx, tw, p, 2 * grid, smem, stream);
    }
  }
  switch (fmt) {
    case kFmtCubic4: return launch_sk_fmt<kFmtCubic4>(tx, tw, p, grid, smem, stream);
    case kFmtAffine4: return launch_sk_fmt<kFmtAffine4>(tx, tw, p, grid, smem, stream);
    case kFmtNvfp4: return launch_sk_fmt<kFmtNvfp4>(tx, tw, p, grid, smem, stream);
    case kFmtFp8: return launch_sk_fmt<kFmtFp8>(tx, tw, p, grid, smem, stream);
    default: return launch_sk_fmt<kFmtBf16>(tx, tw, p, grid, smem, stream);
  }
}

}  // namespace cb
