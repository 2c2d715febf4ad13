// Weight-quantized GEMM for sm_100a:  y[M,N] = x[M,K] * W[N,K]^T  (+ residual)
//
// Replaces the reference's Marlin / Triton weight-only GEMM family
// (quantization/common/marlin/native/template/kernel.cuh:50,
//  quantization/common/kernels.py:68) with one tcgen05 kernel.
//
// Operand roles are swapped relative to the maths: the *weight* tile is the
// UMMA "A" operand (128 output features -> 128 TMEM lanes) and the activation
// tile is the "B" operand (batch rows -> UMMA N, any multiple of 16 up to 256).
// A decode batch of 16..256 rows therefore always fills the 128-row MMA, and
// one CTA dequantizes each weight exactly once per 256 batch rows.
//
// Pipeline per k-block (64 columns of K), S stages:
//   warp 0   : bulk copy of the packed weight tile (4 KiB) + its group metadata
//              (1 KiB) and a TMA tile load of x (128-byte swizzle)  -> full[s]
//   warps 2-17: wait full[s]; decode 4-bit codes -> bf16, write the swizzled
//              K-major A tile in shared memory                      -> ready[s]
//   warp 1   : wait ready[s]; 4 x tcgen05.mma (K=16) into TMEM; commit -> empty[s]
//   warps 2-17: epilogue, tcgen05.ld -> registers -> bf16 (or fp32 split-K
//              partials whose last-arriving CTA sums them in split order).
//
// Packed weight storage is produced at load time by ops/wq_pack.py:
//   codes  [n_tile][k_block][half h(2)][row r(128)][16 bytes]   (4096 B per stage)
//          word j (0..3) of those 16 bytes covers columns 32h + 8j .. + 7; its
//          nibble i (i < 4) is column 2i, nibble i + 4 is column 2i + 1; codes are
//          stored offset-binary (code + 8; the reserved most-negative code -> 8).
//   meta   [n_tile][meta_block][2][128] 32-bit words            (1024 B per block)
//          CUBIC4 : word0 = bf16x2(A, B), word1 = bf16x2(C, 0) with A = s*a/7,
//                   B = s*b/49, C = s*(1-a-b)/343; one block per K group
//          AFFINE4: word h = bf16x2(scale, offset + 8*scale) of 32-column sub-block h
//                   of the k-block; w = (code - 8) * scale + that; one block per k-block
//          NVFP4  : word h = bf16x2(block scale of columns 32h..32h+15, ..+16..31)
#include "wq_gemm_common.cuh"
#include "launch.cuh"
#include <atomic>

namespace cb {

struct __align__(8) SmemCtl {
  uint64_t full[8];
  uint64_t ready[8];
  uint64_t empty[8];
  uint64_t acc_full;
  uint64_t acc_ready[2];   // kFmtFp8Block: a stage's product is complete in tensor-memory buffer b
  uint64_t acc_free[2];    //               buffer b has been promoted into registers by all epilogue warps
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t is_last;
};

template <int FMT>
__global__ void __launch_bounds__(kThreads, 1)
wq_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x,
               const __grid_constant__ CUtensorMap tmap_w,  // only for the direct formats (bf16, fp8)
               const WqGemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: [stage: x tile | A tile | packed codes+meta] * S, then control block
  const uint32_t x_bytes = static_cast<uint32_t>(p.mb) * 128u;
  constexpr uint32_t kMeta = static_cast<uint32_t>(meta_bytes(FMT));
  constexpr bool kDirect = fmt_is_direct(FMT);
  constexpr int kBK = fmt_block_k(FMT);
  const uint32_t stage_bytes = x_bytes + kATileBytes + (kDirect ? 0 : kCodeBytes + kMeta);
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem + static_cast<size_t>(p.stages) * stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x;
  const bool grouped = p.group_tiles != nullptr;
  const int split = grouped ? 0 : blockIdx.y;
  const int m_tile = blockIdx.z;
  int m0 = m_tile * p.mb;
  int m_end = p.M;                       // first row this CTA must NOT write
  const uint8_t* codes_base = p.codes;
  const uint8_t* meta_base = p.meta;
  int w_row0 = 0;                        // bf16 weights: first row of this expert in the stacked [E * N, K] matrix
  pdl_launch_dependents();
  if (grouped) {
    pdl_wait();                             // the work list is written by the routing kernels
    const int item = blockIdx.y;
    if (item >= p.group_tiles[0]) return;   // uniform for the CTA, before any barrier or TMEM allocation
    const int e = p.group_tiles[1 + 3 * item];
    m0 = p.group_tiles[2 + 3 * item];
    m_end = m0 + p.group_tiles[3 + 3 * item];
    w_row0 = e * p.N;
    codes_base += static_cast<size_t>(e) * p.group_code_stride;
    meta_base += static_cast<size_t>(e) * p.group_meta_stride;
  }
  const int S = p.stages;

  // k-block range of this split (balanced contiguous ranges)
  const int kb_lo = static_cast<int>((static_cast<long long>(p.k_blocks) * split) / p.splits);
  const int kb_hi = static_cast<int>((static_cast<long long>(p.k_blocks) * (split + 1)) / p.splits);
  const int iters = kb_hi - kb_lo;

  // timeline rows 0..2, slots 6/7 hold kernel-level stamps: entry, set-up done, accumulator complete,
  // epilogue stores issued, split-K reduction done
  CB_TRACE_ONLY(unsigned long long* trace = (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.trace : nullptr;)
  CB_STAMP(threadIdx.x == 64, 6);
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->ready[s]), kNumDequantWarps / 4);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->acc_full), 1);
    for (int b2 = 0; b2 < 2; ++b2) {
      mbar_init(smem_u32(&ctl->acc_ready[b2]), 1);
      mbar_init(smem_u32(&ctl->acc_free[b2]), kNumDequantWarps);
    }
    ctl->abort_flag = 0;
    ctl->is_last = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  CB_STAMP(threadIdx.x == 64, 7);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      const uint32_t tx = x_bytes + (kDirect ? kATileBytes : kCodeBytes + kMeta);
      // stage index and phase are carried as counters: `i % S` and `i / S` with a run-time S cost two
      // integer divisions (~300 cycles on one thread), which was most of the per-k-block time of this loop
      auto load_weights = [&](int i, int s) {
        const int kb = kb_lo + i;
        uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
        const uint32_t bar = smem_u32(&ctl->full[s]);
        mbar_expect_tx(bar, tx);
        if (kDirect) {
          tma_load_2d(smem_u32(st + x_bytes), &tmap_w, kb * kBK, w_row0 + n_tile * kTileN, bar);
        } else {
          const uint8_t* csrc = codes_base + (static_cast<size_t>(n_tile) * p.k_blocks + kb) * kCodeBytes;
          const uint8_t* msrc = meta_base + (static_cast<size_t>(n_tile) * p.meta_blocks + kb / p.meta_k_blocks) * kMeta;
          bulk_g2s(smem_u32(st + x_bytes + kATileBytes), csrc, kCodeBytes, bar);
          bulk_g2s(smem_u32(st + x_bytes + kATileBytes + kCodeBytes), msrc, kMeta, bar);
        }
      };
      auto load_x = [&](int i, int s) {
        uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
        tma_load_2d(smem_u32(st), &tmap_x, (kb_lo + i) * kBK, m0, smem_u32(&ctl->full[s]));
      };
      // weights of the first S stages go out before anything else, so that an
      // all-gather still in flight overlaps with weight streaming
      const int pre = iters < S ? iters : S;
      for (int i = 0; i < pre; ++i) load_weights(i, i);
      // everything up to here (set-up, the first weight copies) may overlap the tail of the previous kernel
      pdl_wait();
      bool ok = true;
      if (p.tp.mode & kTpGatherWait) {
        const uint32_t target = p.tp.ag_state[0] + p.tp.ag_expected;   // arrivals consumed so far + this launch's
        for (int r = 0; r < p.tp.size && ok; ++r) ok = wait_counter(p.tp.ag_flag + r, target, abort_flag);
      }
      if (ok) {
        for (int i = 0; i < pre; ++i) load_x(i, i);
        int s = 0;
        uint32_t ph = 1;                      // second pass over the ring: wait for the first release
        for (int i = pre; i < iters; ++i) {
          if (!mbar_wait_park(smem_u32(&ctl->empty[s]), ph ^ 1u, abort_flag)) break;
          CB_STAMP(true, i * 8 + 0);
          load_weights(i, s);
          load_x(i, s);
          CB_STAMP(true, i * 8 + 1);
          if (++s == S) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // The whole warp runs the loop with warp-uniform values and one elected lane issues the tcgen05
    // instructions: descriptors and addresses then live in uniform registers instead of being moved
    // there from a divergent lane's registers before every MMA.
    {
      const bool leader = elect_one();
      // operand formats: bf16 x bf16 (kind::f16) or e4m3 x e4m3 (kind::f8f6f4), fp32 accumulators either way
      const uint32_t idesc = fmt_is_fp8(FMT) ? umma_idesc(kTileN, static_cast<uint32_t>(p.mb), 0u, 0u)
                                             : umma_idesc(kTileN, static_cast<uint32_t>(p.mb), 1u, 1u);
      // block-scaled fp8: stage i accumulates from zero into buffer i & 1 (p.tmem_cols / 2 columns each)
      const uint32_t buf_cols = p.tmem_cols >> 1;
      int buf = 0;
      uint32_t buf_ph = 1;                   // a fresh barrier passes a wait on the previous phase: both buffers start free
      const uint32_t tmem_d = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t desc_hi = umma_desc_sw128(0);      // every field except the start address
      bool ok = true;
      int s = 0;
      uint32_t ph = 0;
      uint32_t accumulate = 0;
      for (int i = 0; i < iters && ok; ++i) {
        // decoded formats: `ready` implies `full` (the decode warps waited for the copies themselves)
        ok = kDirect ? mbar_wait_park(smem_u32(&ctl->full[s]), ph, abort_flag)
                               : mbar_wait_park(smem_u32(&ctl->ready[s]), ph, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        CB_STAMP(leader, i * 8 + 4);
        tc_fence_after();
        const uint32_t st = smem_base + static_cast<uint32_t>(s) * stage_bytes;
        const uint64_t bdesc = desc_hi | static_cast<uint64_t>((st & 0x3FFFFu) >> 4);
        const uint64_t adesc = desc_hi | static_cast<uint64_t>(((st + x_bytes) & 0x3FFFFu) >> 4);
        if constexpr (FMT == kFmtFp8Block) {
          ok = __all_sync(0xffffffffu, mbar_wait_park(smem_u32(&ctl->acc_free[buf]), buf_ph, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (leader) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
              umma_f8f6f4(tmem_d + static_cast<uint32_t>(buf) * buf_cols, adesc + 2u * k4, bdesc + 2u * k4, idesc,
                          k4 > 0 ? 1u : 0u);
            tc_commit(smem_u32(&ctl->empty[s]));
            tc_commit(smem_u32(&ctl->acc_ready[buf]));
          }
          if (++buf == 2) { buf = 0; buf_ph ^= 1u; }
        } else if (leader) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            // +32 bytes along K inside the swizzle atom = +2 in the (addr >> 4) field: 16 bf16 or 32 e4m3 columns,
            // one instruction's K either way
            if constexpr (FMT == kFmtFp8)
              umma_f8f6f4(tmem_d, adesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : accumulate);
            else
              umma_f16(tmem_d, adesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : accumulate);
          }
          tc_commit(smem_u32(&ctl->empty[s]));
        }
        accumulate = 1;
        CB_STAMP(leader, i * 8 + 5);
        if (++s == S) { s = 0; ph ^= 1u; }
      }
      if (leader) tc_commit(smem_u32(&ctl->acc_full));
      __syncwarp();
    }
  } else {
    // ------------------------------------------------- dequant + epilogue
    const int dq = threadIdx.x - 64;  // 0..511
    if (!kDirect) {
      // Four groups of four warps, group g takes every fourth k-block; a thread decodes one whole 128-byte row of
      // the k-block (64 weights: two 16-byte code loads, eight 16-byte tile stores), so the per-k-block costs --
      // barrier wait, metadata, fence, arrive, ring arithmetic -- are paid once per 64 weights by 4 warps (the
      // decode is instruction-issue bound: see the stream-K profile).
      const int grp = dq >> 7;          // decode group
      const int r = dq & 127;           // row of the weight tile
      const uint32_t code_off = static_cast<uint32_t>(r * 16);
      const uint32_t a_off = x_bytes + static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128);
      const uint32_t sw = static_cast<uint32_t>(r & 7);
      int s = grp % S;                  // k-block i lives in stage i % S, phase (i / S) & 1
      uint32_t ph = static_cast<uint32_t>(grp / S) & 1u;
      for (int i = grp; i < iters; i += 4) {
        if (!mbar_wait_park(smem_u32(&ctl->full[s]), ph, abort_flag)) break;
        CB_STAMP(dq == 0, i * 8 + 2);
        uint8_t* st = smem + static_cast<size_t>(s) * stage_bytes;
        const uint8_t* pk = st + x_bytes + kATileBytes;
        const uint4 w0 = *reinterpret_cast<const uint4*>(pk + code_off);
        const uint4 w1 = *reinterpret_cast<const uint4*>(pk + code_off + 128 * 16);
        uint8_t* arow = st + a_off;
        if constexpr (FMT == kFmtCubic4) {
          // the row's level table (16 bytes, see cubic_lut8): one scale group covers the whole k-block
          const uint4 t = *reinterpret_cast<const uint4*>(pk + kCodeBytes + code_off);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 words = h ? w1 : w0;
            uint32_t o[4][4];
            cubic_lut8(words.x, t, o[0]);
            cubic_lut8(words.y, t, o[1]);
            cubic_lut8(words.z, t, o[2]);
            cubic_lut8(words.w, t, o[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(arow + ((static_cast<uint32_t>(h * 4 + j) ^ sw) << 4)) =
                  make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
          }
        } else {
          // metadata words are bf16 pairs prepared on the host (see ops/wq_pack.py): {scale, offset} (or two block
          // scales) of each 32-column half
          const uint32_t* meta = reinterpret_cast<const uint32_t*>(pk + kCodeBytes);
          const uint32_t m0 = meta[r], m1 = meta[128 + r];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 words = h ? w1 : w0;
            const uint32_t so = h ? m1 : m0;
            const uint32_t c0 = bf2_dup(so), c1 = bf2_dup_hi(so);
            uint32_t o[4][4];
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
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(arow + ((static_cast<uint32_t>(h * 4 + j) ^ sw) << 4)) =
                  make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->ready[s]));
        CB_STAMP(dq == 0, i * 8 + 3);
        s += 4;
        while (s >= S) { s -= S; ph ^= 1u; }
      }
    }
    // block-scaled fp8: promote every stage's product into registers with the stage's block scale while the MMA
    // warp fills the other tensor-memory buffer.  A warp owns the same (lane quadrant, 16-column chunks) as in the
    // epilogue below: chunk ci = pair + 4 * it lives in racc[it].
    float racc[FMT == kFmtFp8Block ? 4 : 1][16];
    if constexpr (FMT == kFmtFp8Block) {
      const int pquad = warp & 3, ppair = (warp - 2) >> 2, pchunks = p.mb >> 4;
#pragma unroll
      for (int it = 0; it < 4; ++it)
#pragma unroll
        for (int j = 0; j < 16; ++j) racc[it][j] = 0.f;
      const float* bs = p.row_scale + (static_cast<size_t>(w_row0 / kTileN) + n_tile) * p.k_blocks + kb_lo;
      const uint32_t buf_cols = p.tmem_cols >> 1;
      int buf = 0;
      uint32_t ph = 0;
      for (int i = 0; i < iters; ++i) {
        if (!__all_sync(0xffffffffu, mbar_wait_park(smem_u32(&ctl->acc_ready[buf]), ph, abort_flag))) break;
        tc_fence_after();
        const float sc = __ldg(bs + i);
        // one chunk at a time: 16 values in flight beside the 64 accumulators is what the register budget of 18 warps
        // holds without spilling (two or four loads in flight spilled and ran 1.7 x slower)
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int ci = ppair + 4 * it;
          if (ci < pchunks) {
            uint32_t part[16];
            tmem_ld_32x16(tmem_base + static_cast<uint32_t>(buf) * buf_cols + (static_cast<uint32_t>(pquad * 32) << 16) + ci * 16, part);
            tmem_ld_wait();
            // packed fp32 pairs: the promotion's 64 multiply-adds per thread and stage are what the issue slots of
            // the 16 warps are spent on (58 % issue-active, tensor pipe 31 % before the pairing)
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const float2 r2 = __ffma2_rn(make_float2(sc, sc),
                                           make_float2(__uint_as_float(part[j]), __uint_as_float(part[j + 1])),
                                           make_float2(racc[it][j], racc[it][j + 1]));
              racc[it][j] = r2.x;
              racc[it][j + 1] = r2.y;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_free[buf]));
        if (++buf == 2) { buf = 0; ph ^= 1u; }
      }
    }
    // epilogue: TMEM lane = output feature, column = batch row
    pdl_wait();                             // before this thread's first global access (residual, output, partials)
    const bool acc_ok = __all_sync(0xffffffffu, mbar_wait_park(smem_u32(&ctl->acc_full), 0, abort_flag));
    tc_fence_after();
    CB_STAMP(dq == 0, 8 + 6);
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int pair = (warp - 2) >> 2;        // four warps share a quadrant; they interleave 16-column chunks
    const int chunks = p.mb >> 4;
    // where element (m, n) of the result goes: the local output, or (scatter-push)
    // the receive buffer of the rank that owns row m
    auto store_out = [&](int m, int nn, float v) {
      if (p.tp.mode & kTpScatterPush) {
        const int o = m / p.tp.rows_per_rank;
        const int lr = m - o * p.tp.rows_per_rank;
        p.tp.recv[o][(static_cast<size_t>(p.tp.rank) * p.tp.rows_per_rank + lr) * p.N + nn] = __float2bfloat16(v);
      } else {
        const size_t off = static_cast<size_t>(m) * p.ldy + nn;
        if (p.residual) v += __bfloat162float(p.residual[off]);
        p.y[off] = __float2bfloat16(v);
      }
    };
    // fp8: the feature's weight scale times the token's activation scale, applied as the sums leave tensor memory
    // (partial sums of K splits are linear in both, so every later path sees finished values)
    float w_scale = 1.f;
    if constexpr (FMT == kFmtFp8) {
      const int nn = n_tile * kTileN + quad * 32 + lane;
      w_scale = nn < p.N ? p.row_scale[w_row0 + nn] : 0.f;
    }
    // the accumulators of chunk ci (= pair + 4 * it): from tensor memory, or (block-scaled fp8) the promoted registers
    auto load_acc = [&](uint32_t (&acc)[16], int ci, int it) {
      if constexpr (FMT == kFmtFp8Block) {
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = __float_as_uint(racc[it][j]);
      } else {
        tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ci * 16, acc);
        tmem_ld_wait();
      }
    };
    auto scale_acc = [&](uint32_t (&acc)[16], int ci) {
      if constexpr (fmt_is_fp8(FMT)) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + ci * 16 + j;
          const float xs = m < m_end ? __ldg(p.col_scale + m) : 0.f;
          acc[j] = __float_as_uint(__uint_as_float(acc[j]) * (w_scale * xs));
        }
      }
    };
    if (acc_ok && iters > 0) {
      if (p.splits == 1) {
        // TMEM -> registers -> fp32 tile [row][128 features] in the (now idle) stage memory, then all 512 threads
        // write 16-byte row segments: coalesced for the local output and for the peers' receive buffers alike
        float* stg = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int ci = pair + 4 * it;
          if (ci >= chunks) continue;
          uint32_t acc[16];
          load_acc(acc, ci, it);
          scale_acc(acc, ci);
#pragma unroll
          for (int j = 0; j < 16; ++j) stg[(ci * 16 + j) * kTileN + quad * 32 + lane] = __uint_as_float(acc[j]) * p.alpha;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kNumDequantWarps * 32));
        const int rows_here = min(p.mb, m_end - m0);
        const int n_base = n_tile * kTileN;
        const bool vec_ok = (p.ldy & 7) == 0 && (p.N & 7) == 0;
        if (p.swiglu) {
          // 64 activation features per tile row: 16 items of four
          for (int idx = dq; idx < rows_here * 16; idx += kNumDequantWarps * 32) {
            const int mm = idx >> 4, j0 = (idx & 15) * 4;
            const float* gp = stg + mm * kTileN + act_gate_col(j0);
            store_act4(p, m0 + mm, n_tile, j0, *reinterpret_cast<const float4*>(gp), *reinterpret_cast<const float4*>(gp + 16));
          }
        } else
        for (int idx = dq; idx < rows_here * (kTileN / 8); idx += kNumDequantWarps * 32) {
          const int mm = idx >> 4;                 // kTileN / 8 = 16 segments of 8 features per row
          const int n0 = n_base + (idx & 15) * 8;
          if (n0 >= p.N) continue;
          const int m = m0 + mm;
          const float4 f0 = *reinterpret_cast<const float4*>(stg + mm * kTileN + (idx & 15) * 8);
          const float4 f1 = *reinterpret_cast<const float4*>(stg + mm * kTileN + (idx & 15) * 8 + 4);
          float v[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
          if (vec_ok && n0 + 7 < p.N) {
            __nv_bfloat16* dst;
            if (p.tp.mode & kTpScatterPush) {
              const int o = m / p.tp.rows_per_rank;
              const int lr = m - o * p.tp.rows_per_rank;
              dst = p.tp.recv[o] + (static_cast<size_t>(p.tp.rank) * p.tp.rows_per_rank + lr) * p.N + n0;
            } else {
              const size_t off = static_cast<size_t>(m) * p.ldy + n0;
              dst = p.y + off;
              if (p.residual) {
                const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + off);
                const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 r2 = __bfloat1622float2(rp[j]);
                  v[2 * j] += r2.x;
                  v[2 * j + 1] += r2.y;
                }
              }
            }
            uint4 ov;
            ov.x = pack_bf16x2(v[0], v[1]); ov.y = pack_bf16x2(v[2], v[3]);
            ov.z = pack_bf16x2(v[4], v[5]); ov.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(dst) = ov;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (n0 + j < p.N) store_out(m, n0 + j, v[j]);
          }
        }
      } else if (p.cluster_splitk) {
        // the tile's K splits are one cluster: the raw fp32 partial is staged in this CTA's (now idle) stage memory
        // and summed by the cluster below, after all threads of all its CTAs have met
        float* stg = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int ci = pair + 4 * it;
          if (ci >= chunks) continue;
          uint32_t acc[16];
          load_acc(acc, ci, it);
          scale_acc(acc, ci);
#pragma unroll
          for (int j = 0; j < 16; ++j) stg[(ci * 16 + j) * kTileN + quad * 32 + lane] = __uint_as_float(acc[j]);
        }
      } else {
        float* ws = p.workspace +
                    ((static_cast<size_t>(m_tile) * gridDim.x + n_tile) * p.splits + split) * (static_cast<size_t>(p.mb) * kTileN);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int ci = pair + 4 * it;
          if (ci >= chunks) continue;
          uint32_t acc[16];
          load_acc(acc, ci, it);
          scale_acc(acc, ci);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            ws[static_cast<size_t>(ci * 16 + j) * kTileN + quad * 32 + lane] = __uint_as_float(acc[j]);
        }
      }
    }
    CB_STAMP(dq == 0, 8 + 7);
    if (p.splits > 1 && !p.cluster_splitk) {
      // last-arriving split sums all partials in split order (deterministic)
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"r"(kNumDequantWarps * 32));
      if (dq == 0) {
        const uint32_t idx = m_tile * gridDim.x + n_tile;
        const uint32_t prev = atomicAdd(&p.counters[idx], 1u);
        const uint32_t last = (prev == static_cast<uint32_t>(p.splits) - 1u) ? 1u : 0u;
        if (last) p.counters[idx] = 0;
        ctl->is_last = last;
      }
      asm volatile("bar.sync 1, %0;" ::"r"(kNumDequantWarps * 32));
      if (ctl->is_last && !*abort_flag) {
        __threadfence();
        const float* wsb = p.workspace +
                           (static_cast<size_t>(m_tile) * gridDim.x + n_tile) * p.splits * (static_cast<size_t>(p.mb) * kTileN);
        const size_t part_elems = static_cast<size_t>(p.mb) * kTileN;
        // all 512 threads, four consecutive output features per thread: 16-byte partial loads straight from
        // L2 (.cg), 8-byte bf16 stores
        const int rows_here = min(p.mb, m_end - m0);
        const int n_base = n_tile * kTileN;
        if (p.swiglu) {
          for (int idx = dq; idx < rows_here * 16; idx += kNumDequantWarps * 32) {
            const int mm = idx >> 4, j0 = (idx & 15) * 4;
            const size_t e = static_cast<size_t>(mm) * kTileN + act_gate_col(j0);
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
            for (int sp = 0; sp < p.splits; ++sp) {
              const float4 a = __ldcg(reinterpret_cast<const float4*>(wsb + sp * part_elems + e));
              const float4 b = __ldcg(reinterpret_cast<const float4*>(wsb + sp * part_elems + e + 16));
              g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
              u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
            g.x *= p.alpha; g.y *= p.alpha; g.z *= p.alpha; g.w *= p.alpha;
            u.x *= p.alpha; u.y *= p.alpha; u.z *= p.alpha; u.w *= p.alpha;
            store_act4(p, m0 + mm, n_tile, j0, g, u);
          }
        } else
        for (int idx = dq; idx < rows_here * (kTileN / 4); idx += kNumDequantWarps * 32) {
          const int mm = idx >> 5;             // kTileN / 4 = 32 float4 per row
          const int c4 = (idx & 31) * 4;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int sp = 0; sp < p.splits; ++sp) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(wsb + sp * part_elems + static_cast<size_t>(mm) * kTileN + c4));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          const int m = m0 + mm;
          const float o4[4] = {acc.x, acc.y, acc.z, acc.w};
          if ((p.tp.mode & kTpScatterPush) && n_base + c4 + 3 < p.N && ((p.N & 3) == 0)) {
            const int o = m / p.tp.rows_per_rank;
            const int lr = m - o * p.tp.rows_per_rank;
            uint2 ov;
            ov.x = pack_bf16x2(o4[0] * p.alpha, o4[1] * p.alpha);
            ov.y = pack_bf16x2(o4[2] * p.alpha, o4[3] * p.alpha);
            *reinterpret_cast<uint2*>(p.tp.recv[o] + (static_cast<size_t>(p.tp.rank) * p.tp.rows_per_rank + lr) * p.N +
                                      n_base + c4) = ov;
          } else if (!(p.tp.mode & kTpScatterPush) && n_base + c4 + 3 < p.N && ((p.ldy & 3) == 0)) {
            const size_t off = static_cast<size_t>(m) * p.ldy + n_base + c4;
            float r4[4] = {0.f, 0.f, 0.f, 0.f};
            if (p.residual) {
              const uint2 rv = *reinterpret_cast<const uint2*>(p.residual + off);
              const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
              const float2 a0 = __bfloat1622float2(rp[0]), a1 = __bfloat1622float2(rp[1]);
              r4[0] = a0.x; r4[1] = a0.y; r4[2] = a1.x; r4[3] = a1.y;
            }
            uint2 ov;
            ov.x = pack_bf16x2(o4[0] * p.alpha + r4[0], o4[1] * p.alpha + r4[1]);
            ov.y = pack_bf16x2(o4[2] * p.alpha + r4[2], o4[3] * p.alpha + r4[3]);
            *reinterpret_cast<uint2*>(p.y + off) = ov;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (n_base + c4 + j < p.N) store_out(m, n_base + c4 + j, o4[j] * p.alpha);
          }
        }
      }
    }
  }

  if (p.cluster_splitk) {
    // Split-K through distributed shared memory.  Every thread of every CTA of the cluster meets here (all roles fall
    // through to this point, also after a failed wait); then CTA `rank` sums, in split order, the rows
    // [rank * chunk, (rank + 1) * chunk) of the `splits` partial tiles, read in place from the peers' shared memory,
    // and writes them; nobody leaves before its peers have finished reading.
    cluster_sync_all();
    if (warp >= 2 && !*abort_flag) {
      const int dq = threadIdx.x - 64;
      const int rank = static_cast<int>(cluster_ctarank());
      const int rows_here = min(p.mb, m_end - m0);
      const int chunk = (rows_here + p.splits - 1) / p.splits;
      const int row_lo = rank * chunk, row_hi = min(rows_here, row_lo + chunk);
      const uint32_t stg0 = smem_u32(smem);
      const int n_base = n_tile * kTileN;
      if (p.swiglu) {
        for (int idx = dq; idx < (row_hi - row_lo) * 16; idx += kNumDequantWarps * 32) {
          const int mm = row_lo + (idx >> 4), j0 = (idx & 15) * 4;
          const uint32_t off = static_cast<uint32_t>(mm * kTileN + act_gate_col(j0)) * 4u;
          float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
          for (int sp = 0; sp < p.splits; ++sp) {
            const uint32_t base = cluster_map(stg0, static_cast<uint32_t>(sp)) + off;
            const float4 a = ld_cluster_f4(base), b = ld_cluster_f4(base + 64u);
            g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
            u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
          }
          g.x *= p.alpha; g.y *= p.alpha; g.z *= p.alpha; g.w *= p.alpha;
          u.x *= p.alpha; u.y *= p.alpha; u.z *= p.alpha; u.w *= p.alpha;
          store_act4(p, m0 + mm, n_tile, j0, g, u);
        }
      } else {
        for (int idx = dq; idx < (row_hi - row_lo) * (kTileN / 4); idx += kNumDequantWarps * 32) {
          const int mm = row_lo + (idx >> 5), c4 = (idx & 31) * 4;
          if (n_base + c4 >= p.N) continue;
          const uint32_t off = static_cast<uint32_t>(mm * kTileN + c4) * 4u;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int sp = 0; sp < p.splits; ++sp) {
            const float4 v = ld_cluster_f4(cluster_map(stg0, static_cast<uint32_t>(sp)) + off);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          const float o4[4] = {acc.x * p.alpha, acc.y * p.alpha, acc.z * p.alpha, acc.w * p.alpha};
          if (p.tp.mode & kTpScatterPush) {
            // partial rows go straight to the receive buffer of the rank that owns them (slot = this rank)
            const int m = m0 + mm;
            const int ow = m / p.tp.rows_per_rank;
            const int lr = m - ow * p.tp.rows_per_rank;
            __nv_bfloat16* dst = p.tp.recv[ow] + (static_cast<size_t>(p.tp.rank) * p.tp.rows_per_rank + lr) * p.N + n_base + c4;
            if (n_base + c4 + 3 < p.N && (p.N & 3) == 0) {
              uint2 ov;
              ov.x = pack_bf16x2(o4[0], o4[1]);
              ov.y = pack_bf16x2(o4[2], o4[3]);
              *reinterpret_cast<uint2*>(dst) = ov;
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (n_base + c4 + j < p.N) dst[j] = __float2bfloat16(o4[j]);
            }
            continue;
          }
          const size_t o = static_cast<size_t>(m0 + mm) * p.ldy + n_base + c4;
          if (n_base + c4 + 3 < p.N && (p.ldy & 3) == 0) {
            float r4[4] = {0.f, 0.f, 0.f, 0.f};
            if (p.residual) {
              const uint2 rv = *reinterpret_cast<const uint2*>(p.residual + o);
              const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
              const float2 a0 = __bfloat1622float2(rp[0]), a1 = __bfloat1622float2(rp[1]);
              r4[0] = a0.x; r4[1] = a0.y; r4[2] = a1.x; r4[3] = a1.y;
            }
            uint2 ov;
            ov.x = pack_bf16x2(o4[0] + r4[0], o4[1] + r4[1]);
            ov.y = pack_bf16x2(o4[2] + r4[2], o4[3] + r4[3]);
            *reinterpret_cast<uint2*>(p.y + o) = ov;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (n_base + c4 + j < p.N) {
                float w = o4[j];
                if (p.residual) w += __bfloat162float(p.residual[o + j]);
                p.y[o + j] = __float2bfloat16(w);
              }
            }
          }
        }
      }
    }
    cluster_sync_all();
  }

  if ((p.tp.mode & kTpScatterPush) && warp >= 2) {
    // every partial row of this CTA is on its way: make the stores visible system-wide,
    // then raise the arrival counter of each owner whose rows this tile touched
    // with the K splits in a cluster every CTA pushed its share of the rows before the cluster's second barrier, so
    // CTA 0 of the cluster speaks for all of them: one system-scope fence per tile
    const bool pusher = (p.splits == 1) || (p.cluster_splitk ? cluster_ctarank() == 0 : ctl->is_last != 0);
    // CTA barrier first (every thread's stores then happen before thread 64 continues), then ONE release fence
    // at system scope by that thread (cumulative: it orders all of the tile's stores) and relaxed counter updates
    asm volatile("bar.sync 1, %0;" ::"r"(kNumDequantWarps * 32));
    if (pusher && threadIdx.x == 64 && !ctl->abort_flag) {
      const int m_last = min(p.M, m0 + p.mb) - 1;
      fence_acq_rel_sys();
      for (int o = m0 / p.tp.rows_per_rank; o <= m_last / p.tp.rows_per_rank; ++o)
        red_relaxed_sys_add(p.tp.rs_flag[o] + p.tp.rank, 1u);
    }
  }
  tc_fence_before();
  __syncthreads();
  CB_STAMP(threadIdx.x == 64, 16 + 6);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if ((p.tp.mode & kTpGatherWait) && threadIdx.x == 0) {
    // the last CTA of the grid closes the epoch of the gathered buffer
    const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(&p.tp.ag_state[1], 1u) == total - 1u) {
      p.tp.ag_state[1] = 0;
      __threadfence();
      atomicAdd(&p.tp.ag_state[0], p.tp.ag_expected);
    }
  }
  if (threadIdx.x == 0 && ctl->abort_flag)
    atomicExch(p.status, static_cast<uint32_t>(ctl->abort_flag == 2 ? kErrFlagTimeout : kErrBarrierTimeout));
}

// Clusters of `size` CTAs of the per-tile kernel (one CTA per SM) that can be resident at once; a cluster's CTAs
// share a GPC, so this is less than SMs / size when GPCs do not hold a multiple of `size` usable SMs.
template <int FMT>
static int resident_clusters(int size) {
  // per device: a function attribute set with one device current does not carry over to another device
  static int cached_dev[64][9] = {};
  int dev = 0;
  if (size < 1 || size > 8 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int* cached = cached_dev[dev];
  if (cached[size] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, static_cast<unsigned>(size), 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = 232448 - 1024;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(size);
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaFuncSetAttribute(wq_gemm_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, wq_gemm_kernel<FMT>, &cfg) != cudaSuccess)
      n = 0;
    cached[size] = n > 0 ? n : -1;
  }
  return cached[size] > 0 ? cached[size] : 0;
}

template <int FMT>
static int launch_fmt(const CUtensorMap& tx, const CUtensorMap& tw, WqGemmParams p, dim3 grid, size_t smem,
                      cudaStream_t stream) {
  static bool configured[64] = {};     // per device, like the attribute itself
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -18;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(wq_gemm_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  if (p.cluster_splitk) {
    // the K splits of a tile (grid.y) as one cluster; only if every cluster of the launch can be resident at once
    // (a cluster's CTAs share a GPC), otherwise the launch would run in waves: fall back to the workspace path
    if (resident_clusters<FMT>(static_cast<int>(grid.y)) >= static_cast<int>(grid.x * grid.z))
      return static_cast<int>(launch(wq_gemm_kernel<FMT>, grid, dim3(kThreads), smem, stream, dim3(1, grid.y, 1), tx, tw, p));
    p.cluster_splitk = 0;
    if (!p.workspace || !p.counters) return -13;
  }
  return static_cast<int>(launch(wq_gemm_kernel<FMT>, grid, dim3(kThreads), smem, stream, tx, tw, p));
}

}  // namespace cb

// Per-launch options of the common launcher.  Everything that steers ONE launch travels in this struct (not in
// process-wide variables), so launches made concurrently from several host threads cannot see each other's choices.
struct WqLaunchOpts {
  const float* x_scale = nullptr;      // fp8: one scale per row of x (the weight scales travel as `meta`)
  const int* tiles = nullptr;          // grouped (expert) launch: device work list, see WqGemmParams::group_tiles
  size_t code_stride = 0, meta_stride = 0;
  int max_items = 0, num_experts = 0;
  int mb_hint = 0;                     // grouped launch: batch rows per work item
  int swiglu = 0;                      // fused SwiGLU epilogue (gate / up rows interleaved)
  int cluster_splitk = -1;             // -1: the process default; 0 / 1: workspace / cluster reduction for this launch
  bool stream_k = false;
  int min_units = 0;
  long long workspace_bytes = 0;
};

#ifdef CB_KERNEL_TRACE
static unsigned long long* g_trace_buffer = nullptr;
static int g_stage_override = 0;
#endif

extern "C" {

#ifdef CB_KERNEL_TRACE
// Development builds only: a device buffer of [k-blocks][8] 64-bit words receives the pipeline timeline of CTA (0,0,0)
// of every following launch (null switches it off); a non-zero stage count overrides the automatic choice.
void cb_wq_gemm_debug(void* trace_buffer, int stages) {
  g_trace_buffer = static_cast<unsigned long long*>(trace_buffer);
  g_stage_override = stages;
}
#endif

// Bytes of split-K workspace / counters a launch with these sizes needs.
long long cb_wq_gemm_workspace_bytes(int M, int N, int splits) {
  int mb = M >= 256 ? 256 : ((M + 15) / 16) * 16;
  long long m_tiles = (M + mb - 1) / mb;
  long long n_tiles = (N + 127) / 128;
  return splits > 1 ? m_tiles * n_tiles * splits * mb * 128LL * 4LL : 0;
}

// x: bf16 [M, K] row-major (ldx elements per row); y: bf16 [M, ldy].
// fmt: 0 cubic4, 1 affine4, 2 nvfp4 (W4A16), 3 bf16 weights (codes = W [N,K] bf16).
// Returns 0 or a negative argument error / positive cudaError_t.
// Tensor-parallel link description passed from the host (see TpLink).
struct CbTpLink {
  int mode, rank, size, rows_per_rank;
  void* recv[8];
  void* rs_flag[8];
  const void* ag_flag;
  void* ag_state;
  unsigned ag_expected;
};

int cb_wq_gemm_tp(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                  const void* residual, float alpha, int M, int N, int K, int group_k, int splits, void* workspace,
                  void* counters, void* status, void* stream, const CbTpLink* link);

// Grouped GEMM over experts: x / y rows are sorted by expert; `tiles` is the device work list written by
// cb_moe_route (items of at most `mb` rows); `max_items` sizes the grid (ceil(routes / mb) + experts).
int cb_wq_gemm_grouped(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                       float alpha, int total_rows, int N, int K, int group_k, const void* tiles, int max_items,
                       int mb, int num_experts, long long code_stride, long long meta_stride, void* status,
                       void* stream);

int cb_wq_gemm(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
               const void* residual, float alpha, int M, int N, int K, int group_k, int splits, void* workspace,
               void* counters, void* status, void* stream) {
  return cb_wq_gemm_tp(fmt, x, ldx, codes, meta, y, ldy, residual, alpha, M, N, K, group_k, splits, workspace, counters,
                       status, stream, nullptr);
}

// Persistent stream-K kernel (wq_gemm_sk.cu): the schedule is chosen from the shape; `min_units` > 0 forces
// the smallest run of k-blocks per CTA (0 = automatic).  `workspace_bytes` bounds the fp32 partial slots.
int cb_wq_gemm_sk(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                  const void* residual, float alpha, int M, int N, int K, int group_k, int min_units, void* workspace,
                  long long workspace_bytes, void* counters, void* status, void* stream, const CbTpLink* link);

// 1 (default): the K splits of a tile of the per-tile kernel form a cluster and reduce through distributed shared
// memory; 0: fp32 partial tiles in the workspace, summed by the last split to arrive.
static std::atomic<int> g_cluster_splitk{1};

// Persistent kernel on CTA pairs (cta_group::2): 0 never; 1 (default) eligible launches with more than 256 batch
// rows (measured: 5-20 % faster than one CTA per SM from 512 rows up, 2-8 % slower at exactly 256, where the decode
// warps and not the activation traffic set the pace); 2 every eligible launch.
static std::atomic<int> g_pair_mode{1};

static int wq_gemm_dispatch(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                            const void* residual, float alpha, int M, int N, int K, int group_k, int splits,
                            void* workspace, void* counters, void* status, void* stream, const CbTpLink* link,
                            const WqLaunchOpts& o);

int cb_wq_gemm_tp(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
               const void* residual, float alpha, int M, int N, int K, int group_k, int splits, void* workspace,
               void* counters, void* status, void* stream, const CbTpLink* link) {
  return wq_gemm_dispatch(fmt, x, ldx, codes, meta, y, ldy, residual, alpha, M, N, K, group_k, splits, workspace,
                          counters, status, stream, link, WqLaunchOpts{});
}

// Same as cb_wq_gemm, but the K splits always meet through `workspace` / `counters` (never through a cluster's
// distributed shared memory), whatever the process default says.
int cb_wq_gemm_workspace_splitk(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                                const void* residual, float alpha, int M, int N, int K, int group_k, int splits,
                                void* workspace, void* counters, void* status, void* stream) {
  WqLaunchOpts o;
  o.cluster_splitk = 0;
  return wq_gemm_dispatch(fmt, x, ldx, codes, meta, y, ldy, residual, alpha, M, N, K, group_k, splits, workspace,
                          counters, status, stream, nullptr, o);
}

int cb_wq_gemm_sk(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                  const void* residual, float alpha, int M, int N, int K, int group_k, int min_units, void* workspace,
                  long long workspace_bytes, void* counters, void* status, void* stream, const CbTpLink* link) {
  WqLaunchOpts o;
  o.stream_k = true;
  o.min_units = min_units;
  o.workspace_bytes = workspace_bytes;
  return wq_gemm_dispatch(fmt, x, ldx, codes, meta, y, ldy, residual, alpha, M, N, K, group_k, 1, workspace, counters,
                          status, stream, link, o);
}

static int wq_gemm_dispatch(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                            const void* residual, float alpha, int M, int N, int K, int group_k, int splits,
                            void* workspace, void* counters, void* status, void* stream, const CbTpLink* link,
                            const WqLaunchOpts& o) {
  using namespace cb;
  const bool stream_k = o.stream_k;
  const int min_units = o.min_units;
  const long long workspace_bytes = o.workspace_bytes;
  const int pair_mode = g_pair_mode.load(std::memory_order_relaxed);
  const int cluster_default = o.cluster_splitk >= 0 ? o.cluster_splitk : g_cluster_splitk.load(std::memory_order_relaxed);
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0 || (ldx % (fmt_is_fp8(fmt) ? 16 : 8)) != 0) return -10;
  if (fmt != kFmtBf16 && fmt != kFmtCubic4 && fmt != kFmtAffine4 && fmt != kFmtNvfp4 && !fmt_is_fp8(fmt)) return -11;
  if (fmt_is_fp8(fmt) && (!o.x_scale || !meta || (stream_k && fmt != kFmtFp8))) return -15;
  if (fmt == kFmtFp8Block && o.tiles && (N % kTileN) != 0) return -16;   // stacked experts: whole block rows each
  if (fmt == kFmtCubic4 && (group_k % kBlockK) != 0) return -12;
  WqGemmParams p{};
  p.codes = static_cast<const uint8_t*>(codes);
  p.meta = static_cast<const uint8_t*>(meta);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.workspace = static_cast<float*>(workspace);
  p.counters = static_cast<uint32_t*>(counters);
  p.status = static_cast<uint32_t*>(status);
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.alpha = alpha;
  p.swiglu = o.swiglu;
  if (p.swiglu && (residual || (link && (link->mode & kTpScatterPush)))) return -51;
  p.tp.mode = kTpNone;
  if (link && link->mode != kTpNone) {
    if (link->size < 1 || link->size > kMaxRanks || link->rows_per_rank <= 0 || (link->rows_per_rank % 16) != 0) return -30;
    p.tp.mode = link->mode; p.tp.rank = link->rank; p.tp.size = link->size; p.tp.rows_per_rank = link->rows_per_rank;
    for (int r = 0; r < link->size; ++r) {
      p.tp.recv[r] = static_cast<__nv_bfloat16*>(link->recv[r]);
      p.tp.rs_flag[r] = static_cast<uint32_t*>(link->rs_flag[r]);
    }
    p.tp.ag_flag = static_cast<const uint32_t*>(link->ag_flag);
    p.tp.ag_state = static_cast<uint32_t*>(link->ag_state);
    p.tp.ag_expected = link->ag_expected;
    if ((link->mode & kTpScatterPush) && static_cast<long long>(link->rows_per_rank) * link->size < M) return -31;
  }
  p.mb = M >= 256 ? 256 : ((M + 15) / 16) * 16;
  if (o.tiles && o.mb_hint > 0) p.mb = o.mb_hint;
  p.row_scale = fmt_is_fp8(fmt) ? static_cast<const float*>(meta) : nullptr;
  p.col_scale = o.x_scale;
  // fp8 stages cover 128 columns; a ragged last stage reads zeros from both tensor maps
  p.k_blocks = (K + fmt_block_k(fmt) - 1) / fmt_block_k(fmt);
  if (splits < 1) splits = 1;
  if (splits > p.k_blocks) splits = p.k_blocks;
  // K splits of the per-tile kernel meet in a thread-block cluster (distributed shared memory), also when the tile's
  // rows are pushed to other ranks (CTA 0 of the cluster raises the owners' arrival counters once per tile)
  p.cluster_splitk = (splits > 1 && splits <= 8 && cluster_default && !stream_k && !o.tiles) ? 1 : 0;
  if (splits > 1 && !p.cluster_splitk && (!workspace || !counters)) return -13;
  p.splits = splits;
  p.meta_k_blocks = (fmt == kFmtCubic4) ? group_k / kBlockK : 1;
  p.meta_blocks = (p.k_blocks + p.meta_k_blocks - 1) / p.meta_k_blocks;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(p.mb)) cols <<= 1;
  p.tmem_cols = fmt == kFmtFp8Block ? 2 * cols : cols;     // two alternating stage buffers (at most 2 x 256 columns)
  const size_t stage = static_cast<size_t>(p.mb) * 128 + kATileBytes + (fmt_is_direct(fmt) ? 0 : kCodeBytes + meta_bytes(fmt));
  const size_t budget = 232448 - 1024 - 1024 - sizeof(SmemCtl);
  int stages = static_cast<int>(budget / stage);
  if (stages > 8) stages = 8;
#ifdef CB_KERNEL_TRACE
  if (g_stage_override > 0 && g_stage_override < stages) stages = g_stage_override;
  p.trace = g_trace_buffer;
#endif
  if (stages < 2) return -14;
  p.stages = stages;
  const size_t smem = stages * stage + sizeof(SmemCtl) + 1024;

  if (o.tiles) p.group_tiles = o.tiles;
  p.pair = (stream_k && (pair_mode == 2 || (pair_mode == 1 && M > 256)) && streamk_pair_eligible(p, N)) ? 1 : 0;
  CUtensorMap tx, tw;
  // with CTA pairs each CTA of a pair fetches half of the rows of an activation tile
  if (fmt_is_fp8(fmt)) {
    const uint64_t w_rows = static_cast<uint64_t>(N) * (o.tiles ? o.num_experts : 1);
    if (make_tmap_u8(&tx, x, M, K, ldx, p.pair ? p.mb / 2 : p.mb) != 0) return -20;
    if (make_tmap_u8(&tw, codes, w_rows, K, K, kTileN) != 0) return -21;
  } else if (make_tmap_bf16(&tx, x, M, K, ldx, p.pair ? p.mb / 2 : p.mb) != 0) {
    return -20;
  } else if (fmt == kFmtBf16) {
    const uint64_t w_rows = static_cast<uint64_t>(N) * (o.tiles ? o.num_experts : 1);
    if (make_tmap_bf16(&tw, codes, w_rows, K, K, kTileN) != 0) return -21;
  } else {
    tw = tx;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (stream_k) {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -18;
    if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -18;
    if (o.tiles) {
      p.group_tiles = o.tiles;
      p.group_code_stride = o.code_stride; p.group_meta_stride = o.meta_stride;
    }
    return launch_streamk(fmt, tx, tw, p, static_cast<size_t>(workspace_bytes < 0 ? 0 : workspace_bytes), sms[dev],
                          min_units, st, o.tiles ? o.max_items : 0);
  }
  const int n_tiles = (N + kTileN - 1) / kTileN;
  const int m_tiles = (M + p.mb - 1) / p.mb;
  dim3 grid(n_tiles, splits, m_tiles);
  if (o.tiles) {
    p.group_tiles = o.tiles;
    p.group_code_stride = o.code_stride; p.group_meta_stride = o.meta_stride;
    grid = dim3(n_tiles, o.max_items, 1);
  }
  switch (fmt) {
    case kFmtCubic4: return launch_fmt<kFmtCubic4>(tx, tw, p, grid, smem, st);
    case kFmtAffine4: return launch_fmt<kFmtAffine4>(tx, tw, p, grid, smem, st);
    case kFmtNvfp4: return launch_fmt<kFmtNvfp4>(tx, tw, p, grid, smem, st);
    case kFmtFp8: return launch_fmt<kFmtFp8>(tx, tw, p, grid, smem, st);
    case kFmtFp8Block: return launch_fmt<kFmtFp8Block>(tx, tw, p, grid, smem, st);
    default: return launch_fmt<kFmtBf16>(tx, tw, p, grid, smem, st);
  }
}

static std::atomic<int> g_grouped_persistent{1};

// Gate/up projection with the activation fused: y[M, N / 2] = silu(x Wg^T) * (x Wu^T), W in the interleaved row
// order (16 gate rows, 16 up rows, ...).  `stream_k` picks the persistent kernel; `splits` applies to the per-tile one.
// `link` may make the kernel wait for gathered activation rows; the output is always local.
int cb_wq_gemm_act(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy, float alpha,
                   int M, int N, int K, int group_k, int stream_k, int splits, int min_units, void* workspace,
                   long long workspace_bytes, void* counters, void* status, void* stream, const CbTpLink* link) {
  if ((N % 32) != 0 || ldy < N / 2) return -50;
  WqLaunchOpts o;
  o.swiglu = 1;
  o.stream_k = stream_k != 0;
  o.min_units = min_units;
  o.workspace_bytes = workspace_bytes;
  return wq_gemm_dispatch(fmt, x, ldx, codes, meta, y, ldy, nullptr, alpha, M, N, K, group_k, stream_k ? 1 : splits,
                          workspace, counters, status, stream, link, o);
}

// 1 (default): grouped GEMMs run on the persistent kernel; 0: one CTA per (work item, weight tile).
void cb_wq_gemm_grouped_mode(int persistent) { g_grouped_persistent.store(persistent); }

// 0: one CTA per SM works alone; 1 (default): CTA pairs for eligible launches of more than 256 batch rows; 2: for
// every eligible launch.
void cb_wq_gemm_pair_mode(int pairs) { g_pair_mode.store(pairs); }

// 1 (default): split-K of the per-tile kernel through a cluster's distributed shared memory; 0: through the workspace.
void cb_wq_gemm_cluster_splitk(int on) { g_cluster_splitk.store(on); }

// Clusters of `size` K splits of the per-tile kernel that fit on the current device at once (0: unknown / none).
int cb_wq_gemm_resident_clusters(int fmt, int size) {
  if (!g_cluster_splitk.load()) return 0;
  switch (fmt) {
    case cb::kFmtCubic4: return cb::resident_clusters<cb::kFmtCubic4>(size);
    case cb::kFmtAffine4: return cb::resident_clusters<cb::kFmtAffine4>(size);
    case cb::kFmtNvfp4: return cb::resident_clusters<cb::kFmtNvfp4>(size);
    case cb::kFmtFp8: return cb::resident_clusters<cb::kFmtFp8>(size);
    case cb::kFmtFp8Block: return cb::resident_clusters<cb::kFmtFp8Block>(size);
    default: return cb::resident_clusters<cb::kFmtBf16>(size);
  }
}

// CTA pairs of the persistent kernel that can be resident at once on the current device (0: cannot be launched).
int cb_wq_gemm_resident_pairs(int fmt) { return cb::streamk_resident_pairs(fmt); }

static int wq_gemm_grouped_launch(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                                  float alpha, int total_rows, int N, int K, int group_k, const void* tiles,
                                  int max_items, int mb, int num_experts, long long code_stride, long long meta_stride,
                                  void* status, void* stream, int swiglu) {
  if (!tiles || max_items <= 0 || mb <= 0 || mb > 256 || (mb % 16) != 0 || num_experts <= 0) return -40;
  WqLaunchOpts o;
  o.num_experts = num_experts;
  o.tiles = static_cast<const int*>(tiles);
  o.code_stride = static_cast<size_t>(code_stride);
  o.meta_stride = static_cast<size_t>(meta_stride);
  o.max_items = max_items;
  o.mb_hint = mb;
  o.swiglu = swiglu;
  o.stream_k = g_grouped_persistent.load(std::memory_order_relaxed) != 0;
  // the tensor map spans all rows; every work item starts at its own row offset
  return wq_gemm_dispatch(fmt, x, ldx, codes, meta, y, ldy, nullptr, alpha, total_rows, N, K, group_k, 1, nullptr,
                          nullptr, status, stream, nullptr, o);
}

// Grouped gate/up projection with the fused SwiGLU epilogue (every expert's rows interleaved): y has N / 2 columns.
int cb_wq_gemm_grouped_act(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                           float alpha, int total_rows, int N, int K, int group_k, const void* tiles, int max_items,
                           int mb, int num_experts, long long code_stride, long long meta_stride, void* status,
                           void* stream) {
  if ((N % 32) != 0 || ldy < N / 2) return -50;
  return wq_gemm_grouped_launch(fmt, x, ldx, codes, meta, y, ldy, alpha, total_rows, N, K, group_k, tiles, max_items, mb,
                                num_experts, code_stride, meta_stride, status, stream, 1);
}

int cb_wq_gemm_grouped(int fmt, const void* x, int ldx, const void* codes, const void* meta, void* y, int ldy,
                       float alpha, int total_rows, int N, int K, int group_k, const void* tiles, int max_items,
                       int mb, int num_experts, long long code_stride, long long meta_stride, void* status,
                       void* stream) {
  return wq_gemm_grouped_launch(fmt, x, ldx, codes, meta, y, ldy, alpha, total_rows, N, K, group_k, tiles, max_items, mb,
                                num_experts, code_stride, meta_stride, status, stream, 0);
}

// W8A8 on the fp8 tensor-core path (tcgen05.mma.kind::f8f6f4, e4m3 x e4m3, fp32 accumulate):
//   y[m, n] = x_scale[m] * w_scale[n] * sum_k xq[m, k] * wq[n, k]   (+ residual)
// xq: e4m3 [M, K] (ldx bytes per row, a multiple of 16), x_scale: fp32 [M] (see cb_fp8_quantize_rows);
// wq: e4m3 [N, K] row-major exactly as in the checkpoint, w_scale: fp32 [N].  `swiglu`: wq's rows are in the
// interleaved gate / up order and y has N / 2 columns.  K splits meet in a cluster or in `workspace`.
// Counterpart of the reference's dynamic-token FP8 linear (quantization/extensions/fp8/kernels.py:81-130).
// `block`: w_scale holds one scale per 128 x 128 block, [ceil(N / 128), ceil(K / 128)], instead of one per row.
// `stream_k`: the persistent kernel (row scales only; CTA pairs above 256 rows), `min_units` / `workspace_bytes` as in
// cb_wq_gemm_sk.
int cb_wq_gemm_fp8(const void* xq, int ldx, const void* x_scale, const void* wq, const void* w_scale, int block, void* y,
                   int ldy, const void* residual, int M, int N, int K, int splits, int swiglu, int stream_k,
                   int min_units, void* workspace, long long workspace_bytes, void* counters, void* status, void* stream,
                   const CbTpLink* link) {
  if (swiglu && ((N % 32) != 0 || ldy < N / 2)) return -50;
  WqLaunchOpts o;
  o.x_scale = static_cast<const float*>(x_scale);
  o.swiglu = swiglu;
  o.stream_k = stream_k != 0 && !block;
  o.min_units = min_units;
  o.workspace_bytes = workspace_bytes;
  if (o.stream_k) splits = 1;
  return wq_gemm_dispatch(block ? cb::kFmtFp8Block : cb::kFmtFp8, xq, ldx, wq, w_scale, y, ldy, residual, 1.f, M, N, K, K, splits, workspace,
                          counters, status, stream, link, o);
}

// The grouped (expert) form: wq is the stack [experts * N, K], w_scale [experts * N]; rows of xq / x_scale / y are the
// routed rows in work-list order (see cb_wq_gemm_grouped).
int cb_wq_gemm_fp8_grouped(const void* xq, int ldx, const void* x_scale, const void* wq, const void* w_scale, int block,
                           void* y, int ldy, int total_rows, int N, int K, const void* tiles, int max_items, int mb,
                           int num_experts, int swiglu, void* status, void* stream) {
  if (!tiles || max_items <= 0 || mb <= 0 || mb > 256 || (mb % 16) != 0 || num_experts <= 0) return -40;
  if (swiglu && ((N % 32) != 0 || ldy < N / 2)) return -50;
  WqLaunchOpts o;
  o.x_scale = static_cast<const float*>(x_scale);
  o.num_experts = num_experts;
  o.tiles = static_cast<const int*>(tiles);
  o.max_items = max_items;
  o.mb_hint = mb;
  o.swiglu = swiglu;
  return wq_gemm_dispatch(block ? cb::kFmtFp8Block : cb::kFmtFp8, xq, ldx, wq, w_scale, y, ldy, nullptr, 1.f, total_rows, N, K, K, 1, nullptr,
                          nullptr, status, stream, nullptr, o);
}

}  // extern "C"
