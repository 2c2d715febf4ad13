// Fused per-head RMSNorm (optional) + RoPE + KV quantize-on-write.
//
// One launch after the QKV GEMM replaces the reference's separate q/k norm,
// M-RoPE (position/qwen_mrope.py:25) and cache quantization kernels
// (cache_quantization_native.cu:49).  One warp handles one (token, head) at a
// time; lane l holds channels l, l+32, l+64, l+96, so a rotate-half RoPE pair
// (c, c+64) and a 32-channel quantization group (c/32) are both warp-local.
#include "ptx.cuh"
#include "kv_layout.cuh"
#include "launch.cuh"

namespace cb {

struct KvWriteParams {
  const __nv_bfloat16* qkv;    // [T, (Hq + 2*Hkv) * D]
  __nv_bfloat16* q_out;        // [T, Hq * D]
  uint8_t* cache;              // [pages][Hkv][blob]
  const int* positions;        // [T] rotary position (the temporal axis when pos_h / pos_w are given)
  const int* pos_h;            // [T] or null: row-axis positions of the three-axis rotary form
  const int* pos_w;            // [T] or null: column-axis positions
  int mrope_h, mrope_w;        // frequency slots 1, 4, 7, .. (< 3 mrope_h) follow pos_h, slots 2, 5, 8, .. (< 3 mrope_w) pos_w
  const __nv_bfloat16* qkv_bias;  // [(Hq + 2 Hkv) D] or null: bias of the q / k / v projections, added before the norm
  const int* slots;            // [T] page * 16 + offset, < 0: do not write (padding row)
  const __nv_bfloat16* q_norm; // [D] or null
  const __nv_bfloat16* k_norm; // [D] or null
  const float* inv_freq;       // [D/2]
  int T, Hq, Hkv;
  int rotary_dim;              // <= D, multiple of 2; pairs (c, c + rotary_dim/2)
  float eps;
  int rotate;                  // normalised Walsh-Hadamard transform of every q / k / v head vector (after RoPE)
  KvLayout lay;
};

// Normalised Walsh-Hadamard transform of a 128-vector held as v[a] = x[lane + 32 a]: index bits 5-6 are the
// register index, bits 0-4 the lane.  fp32 stages, the caller rounds once (reference:
// ops/cuda/cache_rotation_native.cu:12).  The transform is its own inverse, and q . k is unchanged when both are
// transformed, so attention over a rotated cache needs only the transform of its output (V's rotation undone).
__device__ __forceinline__ void hadamard128(float (&v)[4], int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float o = __shfl_xor_sync(0xffffffffu, v[k], m);
      v[k] = (lane & m) ? o - v[k] : v[k] + o;
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] *= 0.08838834764831845f;     // 1 / sqrt(128)
}

__device__ __forceinline__ void quantize_store(const float (&v)[4], int bits, bool is_v, uint8_t* blob,
                                               const KvLayout& lay, int tok, int lane) {
  const float qmax = bits == 8 ? 127.f : (bits == 6 ? 31.f : 7.f);
  const int bias = bits == 8 ? 128 : (bits == 6 ? 32 : 8);
  uint8_t* codes = blob + (is_v ? lay.v_code_off : 0);
  float* scales = reinterpret_cast<float*>(blob + (is_v ? lay.v_scale_off : lay.k_scale_off));
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float amax = warp_max(fabsf(v[k]));
    const float scale = amax > 0.f ? amax / qmax : 1.f;
    float c = rintf(v[k] / scale);
    c = fminf(fmaxf(c, -qmax), qmax);
    uint32_t code = static_cast<uint32_t>(static_cast<int>(c) + bias);
    const int ch = lane + 32 * k;
    int shift;
    if (bits == 6) {
      // two high bits into the second plane (the fields of one 32-bit word come from several lanes and from
      // several tokens = several warps: atomics), low nibble as a 4-bit code below
      const int pos = is_v ? v_hi_pos(lay.head_dim, tok, ch, &shift) : k_hi_pos(lay.head_dim, tok, ch, &shift);
      uint32_t* word = reinterpret_cast<uint32_t*>(codes + pos);
      atomicAnd(word, ~(0x3u << shift));
      atomicOr(word, (code >> 4) << shift);
      code &= 15u;
    }
    if (bits == 8) {
      const int pos = is_v ? v_code_pos(8, lay.head_dim, tok, ch, &shift) : k_code_pos(8, tok, ch, &shift);
      codes[pos] = static_cast<uint8_t>(code);
    } else if (!is_v) {
      // channels c and c+16 of a 32-block share a byte: lanes l and l+16
      const uint32_t other = __shfl_down_sync(0xffffffffu, code, 16);
      if (lane < 16) {
        const int pos = k_code_pos(4, tok, ch, &shift);
        codes[pos] = static_cast<uint8_t>(code | (other << 4));
      }
    } else {
      // even/odd tokens share a byte and may be written by different warps
      const int pos = v_code_pos(4, lay.head_dim, tok, ch, &shift);
      uint32_t* word = reinterpret_cast<uint32_t*>(codes + (pos & ~3));
      const int bit = (pos & 3) * 8 + shift;
      atomicAnd(word, ~(0xFu << bit));
      atomicOr(word, code << bit);
    }
    if (lane == 0) scales[tok * (lay.head_dim / kKvGroup) + k] = scale;
  }
}

static constexpr int kRopeWarps = 8;

// One CTA per token; its eight warps share the token's heads (warp w takes heads w, w + 8, ...).  The rotary
// angles depend on (position, channel) only, so each lane computes its two sin / cos pairs ONCE and reuses them
// for every head of the token: full-precision sincosf on arguments of thousands of radians is the expensive
// part of this kernel, and one warp per (token, head) paid it 6x as often.
__global__ void __launch_bounds__(kRopeWarps * 32)
rope_kv_write_kernel(const KvWriteParams p) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.Hq + 2 * p.Hkv;
  const int D = p.lay.head_dim;  // == 128
  const int half = p.rotary_dim >> 1;
  const float pos = static_cast<float>(p.positions[t]);
  // three-axis form: frequency slot j turns by the position on its axis (interleaved layout: temporal by default, the
  // row axis on slots 1, 4, 7, .., the column axis on 2, 5, 8, .. as far as their counts reach)
  auto slot_pos = [&](int j) -> float {
    if (p.pos_h == nullptr) return pos;
    const int r = j % 3;
    if (r == 1 && j < 3 * p.mrope_h) return static_cast<float>(p.pos_h[t]);
    if (r == 2 && j < 3 * p.mrope_w) return static_cast<float>(p.pos_w[t]);
    return pos;
  };
  float sn[2] = {0.f, 0.f}, cs[2] = {1.f, 1.f};
  if (half == 64) {
#pragma unroll
    for (int k = 0; k < 2; ++k) sincosf(slot_pos(lane + 32 * k) * p.inv_freq[lane + 32 * k], &sn[k], &cs[k]);
  } else if (half == 32) {
    sincosf(slot_pos(lane) * p.inv_freq[lane], &sn[0], &cs[0]);
  }
  const int slot = p.slots[t];
  for (int h = warp; h < heads; h += kRopeWarps) {
    const __nv_bfloat16* src = p.qkv + (static_cast<size_t>(t) * heads + h) * D;
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __bfloat162float(src[lane + 32 * k]);
    if (p.qkv_bias != nullptr) {
      // the projection's output was rounded to bf16 by the GEMM; the sum is rounded again, as an unfused add would
#pragma unroll
      for (int k = 0; k < 4; ++k)
        v[k] = __bfloat162float(__float2bfloat16(v[k] + __bfloat162float(p.qkv_bias[h * D + lane + 32 * k])));
    }

    const bool is_q = h < p.Hq;
    const bool is_k = !is_q && h < p.Hq + p.Hkv;
    if (is_q || is_k) {
      const __nv_bfloat16* nw = is_q ? p.q_norm : p.k_norm;
      if (nw) {
        float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(D) + p.eps);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // round to bf16 after the norm, as an unfused norm kernel would
          v[k] = __bfloat162float(__float2bfloat16(v[k] * inv * __bfloat162float(nw[lane + 32 * k])));
        }
      }
      // pairs (c, c + half) for c < half; with D = 128 and half = 64: (l, l+64), (l+32, l+96)
      if (half == 64) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float a = v[k], b = v[k + 2];
          v[k] = a * cs[k] - b * sn[k];
          v[k + 2] = b * cs[k] + a * sn[k];
        }
      } else if (half == 32) {
        // partial rotary over the first 64 channels: pairs (l, l+32)
        const float a = v[0], b = v[1];
        v[0] = a * cs[0] - b * sn[0];
        v[1] = b * cs[0] + a * sn[0];
      }
    }
    if (p.rotate) hadamard128(v, lane);
    if (is_q) {
      __nv_bfloat16* dst = p.q_out + (static_cast<size_t>(t) * p.Hq + h) * D;
#pragma unroll
      for (int k = 0; k < 4; ++k) dst[lane + 32 * k] = __float2bfloat16(v[k]);
      continue;
    }
    if (slot < 0) continue;
    const int kvh = is_k ? h - p.Hq : h - p.Hq - p.Hkv;
    const int page = slot >> 4, tok = slot & 15;
    uint8_t* blob = p.cache + (static_cast<size_t>(page) * p.Hkv + kvh) * p.lay.blob_bytes;
    // the cache stores what attention will see: bf16-rounded values
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __bfloat162float(__float2bfloat16(v[k]));
    quantize_store(v, is_k ? p.lay.k_bits : p.lay.v_bits, !is_k, blob, p.lay, tok, lane);
  }
}

// Walsh-Hadamard transform of `vectors` consecutive 128-vectors per row (in place allowed): undoes the rotation of
// V on the attention output.  One warp per vector.
__global__ void __launch_bounds__(256)
hadamard_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* __restrict__ y, int ldy, int vectors,
                int rows) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long w = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (w >= static_cast<long long>(rows) * vectors) return;
  const int r = static_cast<int>(w / vectors), h = static_cast<int>(w - static_cast<long long>(r) * vectors);
  const __nv_bfloat16* src = x + static_cast<size_t>(r) * ldx + h * 128;
  __nv_bfloat16* dst = y + static_cast<size_t>(r) * ldy + h * 128;
  float v[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] = __bfloat162float(src[lane + 32 * k]);
  hadamard128(v, lane);
#pragma unroll
  for (int k = 0; k < 4; ++k) dst[lane + 32 * k] = __float2bfloat16(v[k]);
}

// Copy whole pages (all kv heads) src -> dst: copy-on-write of a shared page.
__global__ void __launch_bounds__(256)
copy_pages_kernel(uint8_t* cache, const int* src_pages, const int* dst_pages, int page_bytes_vec) {
  const int s = src_pages[blockIdx.x], d = dst_pages[blockIdx.x];
  if (s < 0 || d < 0 || s == d) return;
  const uint4* sp = reinterpret_cast<const uint4*>(cache + static_cast<size_t>(s) * page_bytes_vec * 16);
  uint4* dp = reinterpret_cast<uint4*>(cache + static_cast<size_t>(d) * page_bytes_vec * 16);
  // blockIdx.y strides over the page, so that rows of megabytes (recurrent-state rows) use more than one SM
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < page_bytes_vec; i += blockDim.x * gridDim.y) dp[i] = sp[i];
}

}  // namespace cb

extern "C" {

int cb_kv_blob_bytes(int head_dim, int k_bits, int v_bits) {
  return cb::make_kv_layout(head_dim, k_bits, v_bits).blob_bytes;
}

// Three-axis rotary positions: ``positions`` is the temporal axis, ``pos_h`` / ``pos_w`` the row and column axes (both
// null: one axis); ``mrope_h`` / ``mrope_w`` are the frequency-slot counts of those two axes.  ``qkv_bias`` (or null) is
// added to every q / k / v row as it is read.
int cb_rope_kv_write_axes(const void* qkv, void* q_out, void* cache, const void* positions, const void* pos_h,
                          const void* pos_w, int mrope_h, int mrope_w, const void* qkv_bias, const void* slots,
                          const void* q_norm, const void* k_norm, const void* inv_freq, int T, int Hq, int Hkv, int D,
                          int rotary_dim, float eps, int k_bits, int v_bits, int rotate, void* stream);

int cb_rope_kv_write(const void* qkv, void* q_out, void* cache, const void* positions, const void* slots,
                     const void* q_norm, const void* k_norm, const void* inv_freq, int T, int Hq, int Hkv, int D,
                     int rotary_dim, float eps, int k_bits, int v_bits, int rotate, void* stream) {
  return cb_rope_kv_write_axes(qkv, q_out, cache, positions, nullptr, nullptr, 0, 0, nullptr, slots, q_norm, k_norm,
                               inv_freq, T, Hq, Hkv, D, rotary_dim, eps, k_bits, v_bits, rotate, stream);
}

int cb_rope_kv_write_axes(const void* qkv, void* q_out, void* cache, const void* positions, const void* pos_h,
                          const void* pos_w, int mrope_h, int mrope_w, const void* qkv_bias, const void* slots,
                          const void* q_norm, const void* k_norm, const void* inv_freq, int T, int Hq, int Hkv, int D,
                          int rotary_dim, float eps, int k_bits, int v_bits, int rotate, void* stream) {
  using namespace cb;
  if (T <= 0) return 0;
  if (D != 128) return -10;
  if (!(k_bits == 8 || k_bits == 6 || k_bits == 4) || !(v_bits == 8 || v_bits == 6 || v_bits == 4)) return -11;
  if (!(rotary_dim == 128 || rotary_dim == 64 || rotary_dim == 0)) return -12;
  if ((pos_h == nullptr) != (pos_w == nullptr)) return -13;
  if (pos_h != nullptr) {
    const int half = rotary_dim / 2;   // the last slot of either axis has to exist: 3 h - 2 and 3 w - 1 below half
    if (mrope_h <= 0 || mrope_w <= 0 || 3 * mrope_h - 2 >= half || 3 * mrope_w - 1 >= half) return -14;
  }
  KvWriteParams p;
  p.pos_h = static_cast<const int*>(pos_h);
  p.pos_w = static_cast<const int*>(pos_w);
  p.mrope_h = mrope_h;
  p.mrope_w = mrope_w;
  p.qkv_bias = static_cast<const __nv_bfloat16*>(qkv_bias);
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.cache = static_cast<uint8_t*>(cache);
  p.positions = static_cast<const int*>(positions);
  p.slots = static_cast<const int*>(slots);
  p.q_norm = static_cast<const __nv_bfloat16*>(q_norm);
  p.k_norm = static_cast<const __nv_bfloat16*>(k_norm);
  p.inv_freq = static_cast<const float*>(inv_freq);
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.rotary_dim = rotary_dim; p.eps = eps; p.rotate = rotate;
  p.lay = make_kv_layout(D, k_bits, v_bits);
  return static_cast<int>(launch(rope_kv_write_kernel, dim3(static_cast<unsigned>(T)), dim3(kRopeWarps * 32), 0,
                                 static_cast<cudaStream_t>(stream), p));
}

// y[r, 128 h .. 128 h + 127] = normalised Walsh-Hadamard transform of x[r, same], h < vectors (bf16, in place allowed).
int cb_hadamard(const void* x, int ldx, void* y, int ldy, int vectors, int rows, void* stream) {
  if (rows <= 0 || vectors <= 0) return 0;
  const long long warps = static_cast<long long>(rows) * vectors;
  return static_cast<int>(cb::launch(cb::hadamard_kernel, dim3(static_cast<unsigned>((warps + 7) / 8)), dim3(256), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), ldx,
                                     static_cast<__nv_bfloat16*>(y), ldy, vectors, rows));
}

int cb_copy_pages(void* cache, const void* src_pages, const void* dst_pages, int n, long long page_bytes,
                  void* stream) {
  if (n <= 0) return 0;
  if (page_bytes % 16 != 0) return -10;
  const long long vecs = page_bytes / 16;
  const unsigned chunks = static_cast<unsigned>(vecs > 256 * 16 ? (vecs / (256 * 16) > 64 ? 64 : vecs / (256 * 16)) : 1);
  cb::copy_pages_kernel<<<dim3(static_cast<unsigned>(n), chunks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(cache), static_cast<const int*>(src_pages), static_cast<const int*>(dst_pages),
      static_cast<int>(page_bytes / 16));
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
