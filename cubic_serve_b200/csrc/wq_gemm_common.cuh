// Shared pieces of the weight-quantized GEMM kernels: formats, tile constants, the tensor-parallel link,
// launch parameters, the packed bf16x2 decoders and the tensor-map helper.  Included by wq_gemm.cu (one CTA
// per tile: grouped expert GEMMs, explicit split-K) and wq_gemm_sk.cu (persistent stream-K kernel).
#pragma once
#include "ptx.cuh"
#include <cuda.h>

namespace cb {

// kFmtFp8: e4m3 weights [N, K] with one fp32 scale per output feature, multiplied on the tensor cores with e4m3
// ACTIVATIONS (one fp32 scale per token) by tcgen05.mma.kind::f8f6f4 -- no software decode at all: both operands go
// from global memory to the swizzled shared-memory tiles by TMA, as for bf16 weights, with 128 K columns per stage.
// kFmtFp8Block: e4m3 weights with one fp32 scale per 128 x 128 block ([ceil(N / 128), ceil(K / 128)], the
// `weight_scale_inv` of block-quantized checkpoints).  A weight tile is one block row and a stage one block column, so
// every stage's product has ONE scale: the MMA warp accumulates each stage into a fresh tensor-memory buffer (two
// buffers alternate) and the epilogue warps, idle in the main loop of a direct format, promote it into fp32
// registers with that scale (acc += s * partial) while the next stage's MMAs run.
enum WqFormat : int { kFmtCubic4 = 0, kFmtAffine4 = 1, kFmtNvfp4 = 2, kFmtBf16 = 3, kFmtFp8 = 4, kFmtFp8Block = 5 };
__host__ __device__ constexpr bool fmt_is_fp8(int fmt) { return fmt == kFmtFp8 || fmt == kFmtFp8Block; }
// formats whose weight tile is fetched by TMA straight into the MMA layout (no decode warps, no code ring)
__host__ __device__ constexpr bool fmt_is_direct(int fmt) { return fmt == kFmtBf16 || fmt_is_fp8(fmt); }
// K columns of one pipeline stage: one 128-byte swizzle row of the operand's element type
__host__ __device__ constexpr int fmt_block_k(int fmt) { return fmt_is_fp8(fmt) ? 128 : 64; }

static constexpr int kTileN = 128;       // output features per CTA (UMMA M)
static constexpr int kBlockK = 64;       // K columns per stage (one 128-byte swizzle row)
static constexpr int kCodeBytes = 4096;  // 128 x 64 x 4 bit
static constexpr int kMetaBytes = 1024;       // affine4 / nvfp4: two 32-bit words per row
static constexpr int kMetaBytesCubic = 2048;  // cubic4: four 32-bit words per row (the row's level table)
__host__ __device__ constexpr int meta_bytes(int fmt) { return fmt == 0 ? kMetaBytesCubic : kMetaBytes; }
static constexpr int kATileBytes = kTileN * kBlockK * 2;  // 16 KiB bf16
static constexpr int kNumDequantWarps = 16;  // 4 per scheduler: the decode chains are latency-bound with fewer
static constexpr int kThreads = (2 + kNumDequantWarps) * 32;

// Tensor-parallel links of a launch (all pointers are device addresses valid on
// THIS GPU: local buffers, or peers' symmetric buffers mapped over NVLink).
//   kTpGatherWait : the activation operand is an all-gathered buffer that peers
//                   fill with plain P2P stores; the producer warp prefetches
//                   weights, then waits (bounded) for every rank's rows before
//                   the first activation TMA load -- all-gather fused into the
//                   column-parallel GEMM.
//   kTpScatterPush: the output is a partial sum; the epilogue stores each bf16
//                   partial tile straight into the row owner's receive buffer
//                   (slot = this rank) and raises that owner's arrival counter
//                   -- reduce-scatter fused into the row-parallel GEMM.
enum TpMode : int { kTpNone = 0, kTpGatherWait = 1, kTpScatterPush = 2 };
static constexpr int kMaxRanks = 8;

struct TpLink {
  int mode;
  int rank, size;
  int rows_per_rank;                  // multiple of 16; row m belongs to rank m / rows_per_rank
  __nv_bfloat16* recv[kMaxRanks];     // push: owner o's receive buffer [size][rows_per_rank][N]
  uint32_t* rs_flag[kMaxRanks];       // push: owner o's arrival counters [size]
  const uint32_t* ag_flag;            // wait: local arrival counters [size]
  uint32_t* ag_state;                 // wait: local {arrivals consumed so far, done CTAs}
  uint32_t ag_expected;               // wait: arrivals per source rank per epoch
};

struct WqGemmParams {
  const uint8_t* codes;
  const uint8_t* meta;
  __nv_bfloat16* y;         // [M, ldy]
  const __nv_bfloat16* residual;  // optional [M, ldy]
  float* workspace;         // split-K partials: [tiles][splits][mb][128] fp32
  uint32_t* counters;       // one per (m_tile, n_tile); zero on entry, zero on exit
  uint32_t* status;         // device status word (Status)
  int M, N, K;
  int ldy;
  int mb;                   // batch rows per CTA (multiple of 16, <= 256)
  int k_blocks;             // K / 64
  int splits;               // split-K factor (k_blocks % splits may be != 0)
  int meta_k_blocks;        // k-blocks covered by one metadata block (1 or group/64)
  int meta_blocks;          // metadata blocks per n-tile
  int stages;
  float alpha;              // epilogue scale (per-tensor global scale), 1.0 when unused
  // kFmtFp8: accumulators are scaled as they leave tensor memory, acc[n][m] *= row_scale[n] * col_scale[m]
  const float* row_scale;   // [N] (grouped: [experts * N]) weight scale per output feature; kFmtFp8Block: the block
                            // scales [n tiles (grouped: experts * n tiles)][k_blocks]
  const float* col_scale;   // [M] activation scale per token (row of x)
  uint32_t tmem_cols;       // power of two >= max(32, mb)
  TpLink tp;
  // grouped (mixture-of-experts) mode: blockIdx.y indexes a device-side work list
  // group_tiles = {count, then {expert, first row, rows} per item}; rows are contiguous in x / y; weights
  // of expert e start at codes + e * group_code_stride (meta likewise).  Split-K is not combined with it.
  const int* group_tiles;
  size_t group_code_stride, group_meta_stride;
  unsigned long long* trace;  // optional pipeline timeline of CTA (0,0,0): [iteration][8] clock64 stamps
  // fused SwiGLU epilogue (gate/up projection): the weight rows were interleaved at load time so that a
  // 128-row tile holds 64 output features as four blocks of {16 gate rows, 16 up rows}; the epilogue writes
  // act[m, 64 * n_tile + 16 * q + i] = silu(tile row 32 q + i) * (tile row 32 q + 16 + i), ldy = row stride of act
  int swiglu;
  // persistent kernel on CTA pairs (cta_group::2): the schedule's tile is a PAIR of adjacent weight tiles, CTA rank r of
  // the pair owns weight tile 2 * pair_tile + r and loads batch rows [m0 + r * mb / 2, + mb / 2) of the activation tile
  int pair;
  // per-tile kernel with K splits: the `splits` CTAs of a tile form a thread-block cluster and sum their fp32 partial
  // tiles through distributed shared memory (no workspace, no fences, no arrival counter)
  int cluster_splitk;
  // persistent stream-K kernel only (wq_gemm_sk.cu)
  int n_tiles, tiles;       // tile = m_tile * n_tiles + n_tile
  int sk_tiles, sk_ctas;    // tiles [0, sk_tiles) are dealt by k-block to CTAs [0, sk_ctas); the rest are whole
  int ax_stages, c_stages;  // ring depths: {activation tile + decoded tile}, {packed codes + metadata}
  int meta_shift;           // log2(meta_k_blocks)
  uint32_t acc_cols;        // TMEM columns per accumulator buffer (two buffers)
};

// Pipeline timeline of the first CTA(s) of a launch, for development builds only (-DCB_KERNEL_TRACE): clock64
// stamps into `p.trace` ([row][8] 64-bit words; rows 256 + CTA hold every CTA's wall-clock entry / exit).  The product build compiles the stamps and the hook out.
#ifdef CB_KERNEL_TRACE
#define CB_TRACE_ONLY(...) __VA_ARGS__
#define CB_STAMP(cond, idx) do { if (trace && (cond)) trace[idx] = clock64(); } while (0)
#define CB_WALL_STAMP(slot) do { if (p.trace && threadIdx.x == 0) { unsigned long long t_; \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.trace[(256 + blockIdx.x) * 8 + (slot)] = t_; } } while (0)
#else
#define CB_TRACE_ONLY(...)
#define CB_STAMP(cond, idx) do { } while (0)
#define CB_WALL_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until a monotonically increasing counter reaches `target` (wrap-safe).
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, volatile uint32_t* abort_flag) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ld_acquire_sys(p) - target) < 0) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitBudgetCycles) {
      *abort_flag = 2;
      return false;
    }
  }
  return true;
}

// The same for a counter that CTAs of THIS kernel raise (device scope), reaching at least `target`.
__device__ __forceinline__ bool wait_counter_gpu(const uint32_t* p, uint32_t target, volatile uint32_t* abort_flag) {
  const long long t0 = clock64();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (v >= target) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitBudgetCycles) return false;
    __nanosleep(200);
  }
}

// SwiGLU on a pair of accumulators, with the rounding points of the unfused path (the projection's output is
// rounded to bf16, the activation is computed in fp32 from those and rounded once)
__device__ __forceinline__ float silu_mul(float g, float u) {
  g = __bfloat162float(__float2bfloat16(g));
  u = __bfloat162float(__float2bfloat16(u));
  return silu_fast(g) * u;
}
// Four consecutive activation features j0..j0+3 (j0 % 4 == 0) of tile `n_tile` for row m from the fp32 gate / up
// values of the tile row (already scaled by alpha)
__device__ __forceinline__ void store_act4(const WqGemmParams& p, int m, int n_tile, int j0, const float4 g, const float4 u) {
  const int n_out = p.N >> 1;
  const int n0 = n_tile * 64 + j0;
  if (n0 >= n_out) return;
  const float a[4] = {silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w)};
  __nv_bfloat16* dst = p.y + static_cast<size_t>(m) * p.ldy + n0;
  if ((p.ldy & 3) == 0 && n0 + 3 < n_out) {
    uint2 ov;
    ov.x = pack_bf16x2(a[0], a[1]);
    ov.y = pack_bf16x2(a[2], a[3]);
    *reinterpret_cast<uint2*>(dst) = ov;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n0 + j < n_out) dst[j] = __float2bfloat16(a[j]);
  }
}
// offset of activation feature j (0..63) of a tile inside a 128-float tile row: gate value there, up value 16 on
__device__ __forceinline__ int act_gate_col(int j) { return ((j >> 4) << 5) + (j & 15); }

// ---- packed bf16x2 decode (affine4, nvfp4) ---------------------------------
// A 32-bit word holds 8 codes; nibble i (i < 4) is column 2i and nibble i + 4 is
// column 2i + 1 of the 8-column chunk, so ONE mask pulls an adjacent column pair
// into the two halves of a register:  ((w >> 4i) & 0x000F000F) | 0x43004300 is
// the bf16 pair (128 + n_lo, 128 + n_hi).  All arithmetic then runs two weights
// per instruction on the FMA pipe and produces bf16 directly -- no float -> bf16
// conversion (those run on the quarter-rate XU pipe and were the bottleneck of
// an fp32 formulation: 87 % XU utilisation in the first profile).
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// low 16 bits of a word duplicated into both halves: one byte permute
__device__ __forceinline__ uint32_t bf2_dup(uint32_t lo16) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %1, 0x1010;" : "=r"(r) : "r"(lo16));
  return r;
}
__device__ __forceinline__ uint32_t bf2_dup_hi(uint32_t w) {      // high 16 bits into both halves
  uint32_t r;
  asm("prmt.b32 %0, %1, %1, 0x3232;" : "=r"(r) : "r"(w));
  return r;
}
__device__ __forceinline__ uint32_t bf2_abs(uint32_t a) {
  uint32_t r;
  asm("abs.bf16x2 %0, %1;" : "=r"(r) : "r"(a));
  return r;
}

template <int FMT>
__device__ __forceinline__ void decode8(uint32_t w, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t (&out)[4]);

template <>
__device__ __forceinline__ void decode8<kFmtBf16>(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t (&)[4]) {}

// CUBIC4 goes through a level table instead of arithmetic.  A Cubic weight is sign(c) * level[|c|] with eight
// levels per (row, K group); the host stores them as bf16, rounded once from the fp32 curve
//   level[m] = s t (a + t (b + t (1 - a - b))),  t = m / 7,
// split into low bytes (words tl0 = levels 0..3, tl1 = levels 4..7) and high bytes (th0, th1).  A code word holds
// eight codes in sign-magnitude form: nibble i carries |c_i| of column i in its low three bits (so that the
// masked word IS a byte-permute selector), the sign of column i (i < 4) sits in bit 8 i + 7 and that of column
// 4 + i in bit 8 i + 3 -- the spare top bits of the nibbles, placed where one mask (after one shift for the second
// four) puts them on the sign bits of the looked-up high bytes.  13 integer instructions per eight weights
// (mask, shift, four look-ups, three for the signs, four interleaves) against 28 for the arithmetic form, and the
// weights are bit-exact roundings of the fp32 curve.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ void cubic_lut8(uint32_t w, const uint4& t, uint32_t (&out)[4]) {
  const uint32_t m = w & 0x77777777u;       // selectors of columns 0..3 (low 16 bits are used by prmt)
  const uint32_t mb = m >> 16;              // ... of columns 4..7
  const uint32_t lo_a = prmt(t.x, t.y, m);
  uint32_t hi_a = prmt(t.z, t.w, m);
  const uint32_t lo_b = prmt(t.x, t.y, mb);
  uint32_t hi_b = prmt(t.z, t.w, mb);
  hi_a ^= w & 0x80808080u;
  hi_b ^= (w << 4) & 0x80808080u;
  out[0] = prmt(lo_a, hi_a, 0x5140u);       // {column 0, column 1} as a bf16 pair
  out[1] = prmt(lo_a, hi_a, 0x7362u);
  out[2] = prmt(lo_b, hi_b, 0x5140u);
  out[3] = prmt(lo_b, hi_b, 0x7362u);
}

// AFFINE4: w = (n - 8) * scale + offset8   (offset8 = offset + 8 * scale, small in magnitude)
template <>
__device__ __forceinline__ void decode8<kFmtAffine4>(uint32_t w, uint32_t scale, uint32_t offset8, uint32_t,
                                                     uint32_t (&out)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
    out[i] = bf2_fma(bf2_sub(x, 0x43084308u), scale, offset8);
  }
}

// NVFP4: the codes arrive as sign-magnitude words like Cubic's (ops/wq_pack.py re-tiles them at load): the low three
// bits of a nibble, exponent and mantissa of the e2m1 value, index ONE constant table whose entry m is the bf16
// pattern m << 6 = magnitude x 2^-126 ({0, .5, 1, 1.5, 2, 3, 4, 6}; the two smallest are bf16 subnormals that the
// multiply below normalises).  One packed multiply per pair by the block scale, stored as scale x 2^118, finishes the
// weights (the remaining 2^8 rides in alpha): 13 integer instructions + 4 multiplies per eight weights against 28
// for the shift-and-mask form.
template <>
__device__ __forceinline__ void decode8<kFmtNvfp4>(uint32_t w, uint32_t scale, uint32_t, uint32_t,
                                                   uint32_t (&out)[4]) {
  const uint4 t = make_uint4(0xC0804000u, 0xC0804000u, 0x00000000u, 0x01010101u);   // low bytes 0..3, 4..7; high bytes
  cubic_lut8(w, t, out);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = bf2_mul(out[i], scale);
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 8-bit row-major [rows, cols] (row stride ld bytes), box = {128 cols, box_rows}, 128-byte swizzle
static inline int make_tmap_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                               uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// bf16 row-major [rows, cols] (row stride ld elements), box = {64 cols, box_rows}, 128-byte swizzle
static inline int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                          uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}


// Persistent stream-K launcher (wq_gemm_sk.cu).  `workspace_bytes` bounds the fp32 partial-tile slots the
// schedule may use; returns 0, a negative argument error or a positive cudaError_t.
bool streamk_pair_eligible(const WqGemmParams& p, int N);
int streamk_resident_pairs(int fmt);
int launch_streamk(int fmt, const CUtensorMap& tx, const CUtensorMap& tw, WqGemmParams p, size_t workspace_bytes,
                   int sm_count, int min_units, cudaStream_t stream, int grouped_max_items = 0);

}  // namespace cb
