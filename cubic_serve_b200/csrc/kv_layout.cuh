// Physical layout of one (page, kv-head) blob of the quantized paged KV cache.
//
// A page holds 16 tokens (the reference's page size, runtime/performance.py:212).
// K and V are typed independently (8-, 6- or 4-bit symmetric codes; ranges +-127 /
// +-7; 6-bit: +-31; the most-negative code is never produced) with one fp32 scale per
// (token, head, 32-channel group) -- the reference's row-group form
// (ops/cuda/cache_quantization_native.cu:49, actions 0/2).  Codes are stored
// offset-binary (code + 2^(bits-1)) and pre-permuted so that the attention
// kernel's mma.sync fragments are plain 32/64-bit shared-memory loads:
//
//   blob = [K codes][K scales fp32 [16][D/32]][V codes][V scales fp32 [16][D/32]]
//
//   K codes, 8-bit: [ch/16][tok][16 B]          (a k-step of 16 channels is contiguous per token)
//   K codes, 4-bit: [ch/32][tok][16 B], byte = 4*t + e holds channels
//                   32*blk + 4*t + e (low nibble) and 32*blk + 16 + 4*t + e (high nibble)
//   V codes, 8-bit: [tok/2][chunk'][8 B], chunk = ch/4, chunk' = chunk ^ ((tok/2 & 3) << 2),
//                   byte = (ch%4)*2 + tok%2   (token pairs adjacent = one f16x2 B fragment)
//   V codes, 4-bit: [tok/2][chunk'][4 B], same chunking, byte = ch%4,
//                   low nibble = even token, high nibble = odd token
//
//   6-bit (K or V): the low nibble of the offset-binary code (code + 32) sits in a plane with exactly the
//                   4-bit layout above; the two high bits sit in a second plane right after it (16 * D / 4
//                   bytes) of 32-bit words.  One word serves the TWO nibble words a thread of the attention
//                   kernel loads together (X and Y below), with every 2-bit field already at the byte of its
//                   code, so a code byte is  nibble | ((word >> s) & 0x30)  with one shift per group of four:
//                       field of X, first set : bits 8e + 4, 8e + 5      (word        & 0x30303030)
//                       field of X, second set: bits 8e + 6, 8e + 7      ((word >> 2) & 0x30303030)
//                       field of Y, first set : bits 8e + 0, 8e + 1      ((word << 4) & 0x30303030)
//                       field of Y, second set: bits 8e + 2, 8e + 3      ((word << 2) & 0x30303030)
//                   K: word [ch/32][tok % 8][t]; X = token tok % 8, Y = token tok % 8 + 8; first / second set
//                      = channels 32*blk + 4*t + e / 32*blk + 16 + 4*t + e.
//                   V: word [(tok/2) % 4][chunk']; X = token pair (tok/2) % 4, Y = that pair + 4; first /
//                      second set = even / odd token; e = ch % 4.
//
// Every region is a multiple of 16 bytes so one bulk copy moves a whole blob.
#pragma once
#include <stdint.h>

namespace cb {

static constexpr int kPageTokens = 16;
static constexpr int kKvGroup = 32;

struct KvLayout {
  int head_dim;
  int k_bits, v_bits;
  int k_code_bytes, v_code_bytes, scale_bytes;
  int k_scale_off, v_code_off, v_scale_off, blob_bytes;
};

__host__ __device__ inline KvLayout make_kv_layout(int head_dim, int k_bits, int v_bits) {
  KvLayout l;
  l.head_dim = head_dim;
  l.k_bits = k_bits;
  l.v_bits = v_bits;
  l.k_code_bytes = kPageTokens * head_dim * k_bits / 8;
  l.v_code_bytes = kPageTokens * head_dim * v_bits / 8;
  l.scale_bytes = kPageTokens * (head_dim / kKvGroup) * 4;
  l.k_scale_off = l.k_code_bytes;
  l.v_code_off = l.k_scale_off + l.scale_bytes;
  l.v_scale_off = l.v_code_off + l.v_code_bytes;
  l.blob_bytes = l.v_scale_off + l.scale_bytes;
  return l;
}

// byte offset (and nibble shift for 4-bit) of K element (tok, ch) inside the K code region
__host__ __device__ inline int k_code_pos(int bits, int tok, int ch, int* shift) {
  if (bits == 8) {
    *shift = 0;
    return (ch >> 4) * 256 + tok * 16 + (ch & 15);
  }
  const int blk = ch >> 5, c = ch & 31;
  *shift = (c >= 16) ? 4 : 0;
  return blk * 256 + tok * 16 + (c & 15);
}

// 6-bit: byte offset of the 32-bit word of high bits (relative to the START of the code region, i.e. past the
// nibble plane) and the bit position of the two high bits of element (tok, ch)
__host__ __device__ inline int k_hi_pos(int head_dim, int tok, int ch, int* shift) {
  const int blk = ch >> 5, c = ch & 31;
  *shift = 8 * (c & 3) + ((tok >= 8) ? 0 : 4) + ((c >= 16) ? 2 : 0);
  return kPageTokens * head_dim / 2 + blk * 128 + (tok & 7) * 16 + ((c & 15) >> 2) * 4;
}
__host__ __device__ inline int v_hi_pos(int head_dim, int tok, int ch, int* shift) {
  const int p = tok >> 1;
  const int chunk = (ch >> 2) ^ ((p & 3) << 2);
  *shift = 8 * (ch & 3) + ((p >= 4) ? 0 : 4) + ((tok & 1) ? 2 : 0);
  return kPageTokens * head_dim / 2 + (p & 3) * head_dim + chunk * 4;
}

// byte offset (and nibble shift) of V element (tok, ch) inside the V code region
__host__ __device__ inline int v_code_pos(int bits, int head_dim, int tok, int ch, int* shift) {
  const int p = tok >> 1;
  const int chunk = (ch >> 2) ^ ((p & 3) << 2);
  if (bits == 8) {
    *shift = 0;
    return p * (head_dim * 2) + chunk * 8 + (ch & 3) * 2 + (tok & 1);
  }
  *shift = (tok & 1) ? 4 : 0;
  return p * head_dim + chunk * 4 + (ch & 3);
}

}  // namespace cb
