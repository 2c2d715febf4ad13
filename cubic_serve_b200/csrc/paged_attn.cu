// Paged GQA attention over the quantized KV cache, decode and chunked-prefill rows.
//
// Counterpart of the reference's paged_decode_native.cu:282 (one CTA per row /
// kv-head tile / KV split, fused INT8/INT4 dequant, split-KV with in-kernel
// last-arriver merge).  Differences that matter on B200:
//   * whole (page, kv-head) blobs (codes + scales of K and V) arrive with ONE
//     bulk async copy each into a per-warp multi-stage ring, completion on an
//     mbarrier -- the kernel is a pure HBM stream;
//   * the cache is stored pre-permuted (kv_layout.cuh) so MMA fragments are
//     plain 32/64-bit shared loads; int8 -> f16 conversion is one byte-permute
//     plus one packed subtract; group scales are applied to the 4 fp32
//     accumulators of a channel group (K) or folded into P (V), never per code;
//   * a row block is 16 MMA rows = (16 / G) consecutive query positions x G
//     query heads of one kv head, so the same kernel serves decode (one
//     position), speculative review rows and causal prefill chunks.
//
// Waits are bounded; on a timeout the CTA records Status and exits cleanly.
#include "ptx.cuh"
#include "launch.cuh"
#include "kv_layout.cuh"

namespace cb {

static constexpr int kAttnWarps = 4;
#ifdef CB_ATTN_OCC4
static constexpr int kAttnStages = 3;
static constexpr int kAttnMinCtas = 4;
#else
static constexpr int kAttnStages = 4;
static constexpr int kAttnMinCtas = 1;
#endif
static constexpr int kD = 128;

struct AttnParams {
  const __nv_bfloat16* q;   // [T, Hq, D]
  __nv_bfloat16* out;       // [T, Hq, D]
  const uint8_t* cache;     // [pages][Hkv][blob]
  const int* page_table;    // [requests, max_pages]
  const int* rb_req;        // [row_blocks] request (page-table row)
  const int* rb_qstart;     // [row_blocks] index of first query token in q/out
  const int* rb_qcount;     // [row_blocks] query positions in this block (<= 16/G); 0 = padding block
  const int* rb_ctx;        // [row_blocks] tokens visible to the FIRST query position (its own included)
  float* partial;           // [row_blocks][Hkv][splits][16][D + 2] fp32 (splits > 1)
  uint32_t* counters;       // [row_blocks * Hkv] zero on entry, zero on exit
  uint32_t* status;
  int Hq, Hkv, G;
  int max_pages;
  int splits;
  float scale_log2;         // softmax scale * log2(e)
  KvLayout lay;
};

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// two offset-binary bytes (selected by `sel` against the 0x64 magic) -> f16x2 of the signed codes
__device__ __forceinline__ uint32_t u8x2_to_f16x2(uint32_t word, uint32_t sel, uint32_t bias_f16x2) {
  uint32_t v = prmt(word, 0x64646464u, sel);
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(bias_f16x2));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct WarpState {
  float m[2];       // running max (log2 domain) for rows g and g+8
  float l[2];       // running partial sum (this lane's columns only)
  float o[16][4];   // O accumulators: n-tile (cg*4 + sub) x {row g: 2 cols, row g+8: 2 cols}
};

// UPPER = false: MMA rows 8..15 of the block hold no query (decode: one position x G <= 8 heads), so their scores,
// softmax state and output rescaling are skipped; the tensor-core instructions still compute them, at no cost.
template <int KBITS, int VBITS, bool UPPER>
__device__ __forceinline__ void process_page(const uint8_t* blob, const KvLayout& lay, const uint32_t (&qf)[8][4],
                                             WarpState& st, int page_tok0, int limit_lo, int limit_hi, int g,
                                             int t4) {
  // limit_lo / limit_hi: number of visible tokens for row g / row g+8
  const float* ksc = reinterpret_cast<const float*>(blob + lay.k_scale_off);
  const float* vsc = reinterpret_cast<const float*>(blob + lay.v_scale_off);
  const uint8_t* vcodes = blob + lay.v_code_off;
  float s[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;

  // ---- S = Q K^T, one channel group (2 k-steps) at a time, scaled per (token, group)
#pragma unroll
  for (int cg = 0; cg < 4; ++cg) {
    float acc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
    if (KBITS == 8) {
#pragma unroll
      for (int jh = 0; jh < 2; ++jh) {
        const int j = cg * 2 + jh;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(blob + j * 256 + (nt * 8 + g) * 16 + t4 * 4);
          const uint32_t b0 = u8x2_to_f16x2(w, 0x5140u, 0x64806480u);
          const uint32_t b1 = u8x2_to_f16x2(w, 0x5342u, 0x64806480u);
          mma_f16(acc[nt], qf[j], b0, b1);
        }
      }
    } else if (KBITS == 6) {
      // nibble plane as for 4 bits; one 32-bit word of high bits serves both tokens (g and g + 8) of this lane,
      // every 2-bit field already at the byte of its code (kv_layout.cuh)
      const uint32_t hb = *reinterpret_cast<const uint32_t*>(blob + kPageTokens * kD / 2 + cg * 128 + g * 16 + t4 * 4);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(blob + cg * 256 + (nt * 8 + g) * 16 + t4 * 4);
        const uint32_t h1 = nt == 0 ? hb : (hb << 4);
        const uint32_t h2 = nt == 0 ? (hb >> 2) : (hb << 2);
        const uint32_t lo = (w & 0x0F0F0F0Fu) | (h1 & 0x30303030u);
        const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) | (h2 & 0x30303030u);
        mma_f16(acc[nt], qf[cg * 2], u8x2_to_f16x2(lo, 0x5140u, 0x64206420u), u8x2_to_f16x2(lo, 0x5342u, 0x64206420u));
        mma_f16(acc[nt], qf[cg * 2 + 1], u8x2_to_f16x2(hi, 0x5140u, 0x64206420u),
                u8x2_to_f16x2(hi, 0x5342u, 0x64206420u));
      }
    } else {
      // 4-bit: one 32-bit word = this lane's 4 channels of both k-steps of the group
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(blob + cg * 256 + (nt * 8 + g) * 16 + t4 * 4);
        const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
        mma_f16(acc[nt], qf[cg * 2], u8x2_to_f16x2(lo, 0x5140u, 0x64086408u), u8x2_to_f16x2(lo, 0x5342u, 0x64086408u));
        mma_f16(acc[nt], qf[cg * 2 + 1], u8x2_to_f16x2(hi, 0x5140u, 0x64086408u),
                u8x2_to_f16x2(hi, 0x5342u, 0x64086408u));
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float k0 = ksc[(nt * 8 + 2 * t4) * 4 + cg], k1 = ksc[(nt * 8 + 2 * t4 + 1) * 4 + cg];
      s[nt][0] = fmaf(acc[nt][0], k0, s[nt][0]);
      s[nt][1] = fmaf(acc[nt][1], k1, s[nt][1]);
      if (UPPER) {
        s[nt][2] = fmaf(acc[nt][2], k0, s[nt][2]);
        s[nt][3] = fmaf(acc[nt][3], k1, s[nt][3]);
      }
    }
  }
  // ---- causal / length mask and online softmax (log2 domain; Q carries the scale)
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int c = 0; c < (UPPER ? 4 : 2); ++c) {
      const int tok = page_tok0 + nt * 8 + 2 * t4 + (c & 1);
      const int lim = (c < 2) ? limit_lo : limit_hi;
      if (tok >= lim) s[nt][c] = -INFINITY;
      mx[c >> 1] = fmaxf(mx[c >> 1], s[nt][c]);
    }
  float alpha[2] = {1.f, 1.f}, muse[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < (UPPER ? 2 : 1); ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mnew = fmaxf(st.m[r], mx[r]);
    muse[r] = (mnew == -INFINITY) ? 0.f : mnew;
    alpha[r] = fast_exp2(st.m[r] - muse[r]);  // exp2(-inf) = 0 on the first page
    st.m[r] = mnew;
    st.l[r] *= alpha[r];
  }
  float pr[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (UPPER || c < 2) {
        pr[nt][c] = fast_exp2(s[nt][c] - muse[c >> 1]);
        st.l[c >> 1] += pr[nt][c];
      } else {
        pr[nt][c] = 0.f;
      }
    }
  // the running maximum settles after the first pages: skip the 64 multiplies when no row's maximum moved
  if (__any_sync(0xffffffffu, alpha[0] != 1.f || (UPPER && alpha[1] != 1.f))) {
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      st.o[n][0] *= alpha[0];
      st.o[n][1] *= alpha[0];
      if (UPPER) {
        st.o[n][2] *= alpha[1];
        st.o[n][3] *= alpha[1];
      }
    }
  }
  // ---- O += P V, V group scales folded into P per channel group
#pragma unroll
  for (int cg = 0; cg < 4; ++cg) {
    // slots past the longest visible length may hold stale bytes (even NaN bit
    // patterns): their scale is forced to zero so that 0 * scale stays 0
    const int vis = max(limit_lo, limit_hi) - page_tok0;
    const float v00 = (2 * t4 < vis) ? vsc[(2 * t4) * 4 + cg] : 0.f;
    const float v01 = (2 * t4 + 1 < vis) ? vsc[(2 * t4 + 1) * 4 + cg] : 0.f;
    const float v10 = (8 + 2 * t4 < vis) ? vsc[(8 + 2 * t4) * 4 + cg] : 0.f;
    const float v11 = (9 + 2 * t4 < vis) ? vsc[(8 + 2 * t4 + 1) * 4 + cg] : 0.f;
    uint32_t a[4];
    a[0] = pack_f16x2(pr[0][0] * v00, pr[0][1] * v01);
    a[1] = UPPER ? pack_f16x2(pr[0][2] * v00, pr[0][3] * v01) : 0u;
    a[2] = pack_f16x2(pr[1][0] * v10, pr[1][1] * v11);
    a[3] = UPPER ? pack_f16x2(pr[1][2] * v10, pr[1][3] * v11) : 0u;
    const int chunk = (cg * 8 + g) ^ ((t4 & 3) << 2);
    if (VBITS == 8) {
      const uint2 lo = *reinterpret_cast<const uint2*>(vcodes + t4 * 256 + chunk * 8);
      const uint2 hi = *reinterpret_cast<const uint2*>(vcodes + (t4 + 4) * 256 + chunk * 8);
      mma_f16(st.o[cg * 4 + 0], a, u8x2_to_f16x2(lo.x, 0x5140u, 0x64806480u), u8x2_to_f16x2(hi.x, 0x5140u, 0x64806480u));
      mma_f16(st.o[cg * 4 + 1], a, u8x2_to_f16x2(lo.x, 0x5342u, 0x64806480u), u8x2_to_f16x2(hi.x, 0x5342u, 0x64806480u));
      mma_f16(st.o[cg * 4 + 2], a, u8x2_to_f16x2(lo.y, 0x5140u, 0x64806480u), u8x2_to_f16x2(hi.y, 0x5140u, 0x64806480u));
      mma_f16(st.o[cg * 4 + 3], a, u8x2_to_f16x2(lo.y, 0x5342u, 0x64806480u), u8x2_to_f16x2(hi.y, 0x5342u, 0x64806480u));
    } else {
      // byte = channel sub, low nibble = even token, high nibble = odd token
      const uint32_t lo = *reinterpret_cast<const uint32_t*>(vcodes + t4 * 128 + chunk * 4);
      const uint32_t hi = *reinterpret_cast<const uint32_t*>(vcodes + (t4 + 4) * 128 + chunk * 4);
      // spread nibbles: even tokens -> bytes (sub), odd tokens -> bytes (sub) of a second word
      uint32_t le = lo & 0x0F0F0F0Fu, lod = (lo >> 4) & 0x0F0F0F0Fu;
      uint32_t he = hi & 0x0F0F0F0Fu, hod = (hi >> 4) & 0x0F0F0F0Fu;
      if (VBITS == 6) {
        // high bits: one 32-bit word for both token pairs (t4 and t4 + 4) of this lane, fields in place
        const uint32_t hw = *reinterpret_cast<const uint32_t*>(vcodes + kPageTokens * kD / 2 + t4 * 128 + chunk * 4);
        le |= hw & 0x30303030u;
        lod |= (hw >> 2) & 0x30303030u;
        he |= (hw << 4) & 0x30303030u;
        hod |= (hw << 2) & 0x30303030u;
      }
      const uint32_t vbias = VBITS == 6 ? 0x64206420u : 0x64086408u;
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
        // f16x2 (even tok, odd tok) of channel `sub`: byte `sub` of le and of lod
        const uint32_t pl = prmt(le, lod, sub | ((4u + sub) << 4));          // bytes: [e_sub, o_sub, x, x]
        const uint32_t ph = prmt(he, hod, sub | ((4u + sub) << 4));
        const uint32_t b0 = u8x2_to_f16x2(pl, 0x5140u, vbias);
        const uint32_t b1 = u8x2_to_f16x2(ph, 0x5140u, vbias);
        mma_f16(st.o[cg * 4 + sub], a, b0, b1);
      }
    }
  }
}

template <int KBITS, int VBITS>
__global__ void __launch_bounds__(kAttnWarps * 32, kAttnMinCtas)
paged_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int kvh = blockIdx.x, rb = blockIdx.y, split = blockIdx.z;
  pdl_wait();
  pdl_launch_dependents();
  const int qcount = p.rb_qcount[rb];
  if (qcount <= 0) return;  // padding block (uniform across the CTA)
  const int req = p.rb_req[rb], qstart = p.rb_qstart[rb], ctx = p.rb_ctx[rb];
  const int G = p.G;
  const int blob_bytes = p.lay.blob_bytes;
  const int stage_stride = (blob_bytes + 127) & ~127;

  uint8_t* my_stages = smem + static_cast<size_t>(warp) * kAttnStages * stage_stride;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kAttnWarps) * kAttnStages * stage_stride);
  uint64_t* my_bars = bars + warp * kAttnStages;
  __shared__ uint32_t abort_word;
  __shared__ uint32_t is_last;
  if (threadIdx.x == 0) { abort_word = 0; is_last = 0; }
  if (lane == 0) {
    for (int s = 0; s < kAttnStages; ++s) mbar_init(smem_u32(&my_bars[s]), 1);
    mbar_fence_init();
  }
  __syncthreads();
  volatile uint32_t* abort_flag = &abort_word;

  // rows of this lane: row g and row g+8; row r -> (query position r / G, head r % G)
  const int total_tokens = ctx + qcount - 1;
  const int total_pages = (total_tokens + kPageTokens - 1) / kPageTokens;
  const int pps = (total_pages + p.splits - 1) / p.splits;
  const int pg_lo = split * pps;
  const int pg_hi = min(total_pages, pg_lo + pps);

  // The first copies of this warp's page stream are issued before anything else: their DRAM latency then overlaps
  // the query load and conversion below instead of following them (every CTA pays this start-up once).
  const int* ptab = p.page_table + static_cast<size_t>(req) * p.max_pages;
  const int first = pg_lo + warp;
  const int my_pages = first < pg_hi ? (pg_hi - first + kAttnWarps - 1) / kAttnWarps : 0;
  auto issue = [&](int i, int page) {
    const int s = i % kAttnStages;
    const uint8_t* src = p.cache + (static_cast<size_t>(page) * p.Hkv + kvh) * blob_bytes;
    const uint32_t bar = smem_u32(&my_bars[s]);
    mbar_expect_tx(bar, blob_bytes);
    bulk_g2s(smem_u32(my_stages + s * stage_stride), src, blob_bytes, bar);
  };
  if (lane == 0) {
    int pg[kAttnStages];
#pragma unroll
    for (int i = 0; i < kAttnStages; ++i) pg[i] = i < my_pages ? ptab[first + i * kAttnWarps] : 0;   // loads first ...
#pragma unroll
    for (int i = 0; i < kAttnStages; ++i)
      if (i < my_pages) issue(i, pg[i]);                                                               // ... then copies
  }

  const bool upper_rows = qcount * G > 8;     // uniform over the CTA: do MMA rows 8..15 hold a query?
  int limit[2];
  uint32_t qf[8][4];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = g + 8 * rr;
    const int qp = row / G, hh = row - qp * G;
    const bool valid = qp < qcount;
    limit[rr] = valid ? ctx + qp : 0;
    const __nv_bfloat16* qrow = p.q + (static_cast<size_t>(qstart + qp) * p.Hq + kvh * G + hh) * kD;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f[4] = {0.f, 0.f, 0.f, 0.f};
      if (valid) {
        const uint2 raw = *reinterpret_cast<const uint2*>(qrow + j * 16 + t4 * 4);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 x = __bfloat1622float2(bp[0]), y = __bfloat1622float2(bp[1]);
        f[0] = x.x * p.scale_log2; f[1] = x.y * p.scale_log2;
        f[2] = y.x * p.scale_log2; f[3] = y.y * p.scale_log2;
      }
      qf[j][rr] = pack_f16x2(f[0], f[1]);       // a0 / a1 : k = 2*t4 .. (first half of the k-step)
      qf[j][2 + rr] = pack_f16x2(f[2], f[3]);   // a2 / a3 : k = 2*t4 + 8 ..
    }
  }

  WarpState st;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
#pragma unroll
  for (int n = 0; n < 16; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) st.o[n][c] = 0.f;

  // ---- per-warp page stream (set up before the query load, see above): pages pg_lo + warp, + 4, ...
  // The page id of the copy issued at the end of iteration i is loaded at the START of iteration i - 1, so that lane 0
  // never sits on a page-table load between two pages.
  int page_next = (lane == 0 && kAttnStages < my_pages) ? ptab[first + kAttnStages * kAttnWarps] : 0;
  bool ok = true;
  for (int i = 0; i < my_pages && ok; ++i) {
    const int s = i % kAttnStages;
    ok = mbar_wait_t<20>(smem_u32(&my_bars[s]), static_cast<uint32_t>(i / kAttnStages) & 1u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const int page_after = (lane == 0 && i + 1 + kAttnStages < my_pages) ? ptab[first + (i + 1 + kAttnStages) * kAttnWarps] : 0;
    if (upper_rows)
      process_page<KBITS, VBITS, true>(my_stages + s * stage_stride, p.lay, qf, st,
                                       (first + i * kAttnWarps) * kPageTokens, limit[0], limit[1], g, t4);
    else
      process_page<KBITS, VBITS, false>(my_stages + s * stage_stride, p.lay, qf, st,
                                        (first + i * kAttnWarps) * kPageTokens, limit[0], limit[1], g, t4);
    __syncwarp();
    if (lane == 0 && i + kAttnStages < my_pages) issue(i + kAttnStages, page_next);
    page_next = page_after;
  }
  // if a wait gave up, copies may still be in flight: give them a bounded time to land
  if (!ok && lane == 0) {
    for (int s = 0; s < kAttnStages; ++s) {
      const long long t0 = clock64();
      while (!mbar_try_wait(smem_u32(&my_bars[s]), 0) && !mbar_try_wait(smem_u32(&my_bars[s]), 1) &&
             clock64() - t0 < kWaitBudgetCycles / 8) {
      }
    }
  }
  // finish row sums across the 4 lanes sharing a row
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
  }
  __syncthreads();  // all warps are done with their stage memory

  // ---- merge the 4 warps through shared memory: [warp][16 rows][D + 2]
  float* mg = reinterpret_cast<float*>(smem);
  constexpr int RS = kD + 2;
  {
    float* mine = mg + warp * 16 * RS;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const int cgi = n >> 2, sub = n & 3;
      const int c0 = cgi * 32 + (2 * t4) * 4 + sub, c1 = cgi * 32 + (2 * t4 + 1) * 4 + sub;
      mine[g * RS + c0] = st.o[n][0];
      mine[g * RS + c1] = st.o[n][1];
      mine[(g + 8) * RS + c0] = st.o[n][2];
      mine[(g + 8) * RS + c1] = st.o[n][3];
    }
    if (t4 == 0) {
      mine[g * RS + kD] = st.m[0];
      mine[g * RS + kD + 1] = st.l[0];
      mine[(g + 8) * RS + kD] = st.m[1];
      mine[(g + 8) * RS + kD + 1] = st.l[1];
    }
  }
  __syncthreads();
  // thread -> (row = tid / 8, 16 channels starting at (tid % 8) * 16)
  const int row = threadIdx.x >> 3, cbase = (threadIdx.x & 7) * 16;
  float mstar = -INFINITY;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) mstar = fmaxf(mstar, mg[(w * 16 + row) * RS + kD]);
  float lsum = 0.f, ov[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) ov[c] = 0.f;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) {
    const float mw = mg[(w * 16 + row) * RS + kD];
    const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mstar);
    lsum += f * mg[(w * 16 + row) * RS + kD + 1];
#pragma unroll
    for (int c = 0; c < 16; ++c) ov[c] += f * mg[(w * 16 + row) * RS + cbase + c];
  }
  const int qp = row / G, hh = row - qp * G;
  const bool row_valid = qp < qcount;
  __nv_bfloat16* orow = p.out + (static_cast<size_t>(qstart + qp) * p.Hq + kvh * G + hh) * kD + cbase;

  if (p.splits == 1) {
    if (row_valid) {
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      uint32_t pk[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) pk[c] = pack_bf16x2(ov[2 * c] * inv, ov[2 * c + 1] * inv);
      reinterpret_cast<uint4*>(orow)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      reinterpret_cast<uint4*>(orow)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    }
  } else {
    float* part = p.partial + ((static_cast<size_t>(rb) * p.Hkv + kvh) * p.splits + split) * 16 * RS;
#pragma unroll
    for (int c = 0; c < 16; ++c) part[row * RS + cbase + c] = ov[c];
    if ((threadIdx.x & 7) == 0) {
      part[row * RS + kD] = mstar;
      part[row * RS + kD + 1] = lsum;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t idx = rb * p.Hkv + kvh;
      const uint32_t prev = atomicAdd(&p.counters[idx], 1u);
      const uint32_t last = (prev == static_cast<uint32_t>(p.splits) - 1u) ? 1u : 0u;
      if (last) p.counters[idx] = 0;
      is_last = last;
    }
    __syncthreads();
    if (is_last) {
      __threadfence();
      const float* base = p.partial + (static_cast<size_t>(rb) * p.Hkv + kvh) * p.splits * 16 * RS;
      float ms = -INFINITY;
      for (int sp = 0; sp < p.splits; ++sp) ms = fmaxf(ms, __ldcg(base + (sp * 16 + row) * RS + kD));
      float ls = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) ov[c] = 0.f;
      for (int sp = 0; sp < p.splits; ++sp) {
        const float mw = __ldcg(base + (sp * 16 + row) * RS + kD);
        const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - ms);
        ls += f * __ldcg(base + (sp * 16 + row) * RS + kD + 1);
#pragma unroll
        for (int c = 0; c < 16; ++c) ov[c] += f * __ldcg(base + (sp * 16 + row) * RS + cbase + c);
      }
      if (row_valid) {
        const float inv = ls > 0.f ? 1.f / ls : 0.f;
        uint32_t pk[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) pk[c] = pack_bf16x2(ov[2 * c] * inv, ov[2 * c + 1] * inv);
        reinterpret_cast<uint4*>(orow)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        reinterpret_cast<uint4*>(orow)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
    }
  }
  if (threadIdx.x == 0 && abort_word) atomicExch(p.status, static_cast<uint32_t>(kErrBarrierTimeout));
}

template <int KB, int VB>
static int launch_attn(const AttnParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_attn_kernel<KB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return static_cast<int>(launch(paged_attn_kernel<KB, VB>, grid, dim3(kAttnWarps * 32), smem, st, p));
}

}  // namespace cb

extern "C" {

// fp32 scratch elements needed for `splits` > 1
long long cb_paged_attn_partial_floats(int row_blocks, int Hkv, int splits) {
  return splits > 1 ? static_cast<long long>(row_blocks) * Hkv * splits * 16 * (cb::kD + 2) : 0;
}

int cb_paged_attn(const void* q, void* out, const void* cache, const void* page_table, const void* rb_req,
                  const void* rb_qstart, const void* rb_qcount, const void* rb_ctx, int row_blocks, int Hq, int Hkv,
                  int D, int max_pages, int k_bits, int v_bits, float scale, int splits, void* partial,
                  void* counters, void* status, void* stream) {
  using namespace cb;
  if (row_blocks <= 0) return 0;
  if (D != kD || Hkv <= 0 || Hq % Hkv != 0) return -10;
  const int G = Hq / Hkv;
  if (G > 16 || (16 % G) != 0) return -11;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!partial || !counters)) return -12;
  AttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.cache = static_cast<const uint8_t*>(cache);
  p.page_table = static_cast<const int*>(page_table);
  p.rb_req = static_cast<const int*>(rb_req);
  p.rb_qstart = static_cast<const int*>(rb_qstart);
  p.rb_qcount = static_cast<const int*>(rb_qcount);
  p.rb_ctx = static_cast<const int*>(rb_ctx);
  p.partial = static_cast<float*>(partial);
  p.counters = static_cast<uint32_t*>(counters);
  p.status = static_cast<uint32_t*>(status);
  p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.max_pages = max_pages; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lay = make_kv_layout(D, k_bits, v_bits);
  const int stage_stride = (p.lay.blob_bytes + 127) & ~127;
  size_t smem = static_cast<size_t>(kAttnWarps) * kAttnStages * stage_stride + kAttnWarps * kAttnStages * 8;
  const size_t merge = static_cast<size_t>(kAttnWarps) * 16 * (kD + 2) * 4;
  if (smem < merge) smem = merge;
  dim3 grid(Hkv, row_blocks, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k_bits == 8 && v_bits == 8) return launch_attn<8, 8>(p, grid, smem, st);
  if (k_bits == 4 && v_bits == 8) return launch_attn<4, 8>(p, grid, smem, st);
  if (k_bits == 4 && v_bits == 4) return launch_attn<4, 4>(p, grid, smem, st);
  if (k_bits == 8 && v_bits == 4) return launch_attn<8, 4>(p, grid, smem, st);
  if (k_bits == 6 && v_bits == 6) return launch_attn<6, 6>(p, grid, smem, st);
  if (k_bits == 6 && v_bits == 8) return launch_attn<6, 8>(p, grid, smem, st);
  if (k_bits == 8 && v_bits == 6) return launch_attn<8, 6>(p, grid, smem, st);
  if (k_bits == 4 && v_bits == 6) return launch_attn<4, 6>(p, grid, smem, st);
  if (k_bits == 6 && v_bits == 4) return launch_attn<6, 4>(p, grid, smem, st);
  return -13;
}

}  // extern "C"
