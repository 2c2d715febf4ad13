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
//                   bytes) whose 16-bit words line up with the 32-bit words of the nibble plane:
//                   K: word [ch/32][tok][t] holds the high bits of channels 32*blk + 4*t + e (bits 2e, 2e+1)
//                      and 32*blk + 16 + 4*t + e (bits 8 + 2e, 9 + 2e);
//                   V: word [tok/2][chunk'] holds those of channels 4*chunk + e for the even token (bits 2e,
//                      2e+1) and the odd token (bits 8 + 2e, 9 + 2e).
//                   One multiply spreads a byte of high bits over four code bytes:
//                   (x * 0x410410) & 0x30303030 puts bits (2e, 2e+1) of x at bits (4, 5) of byte e.
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

// 6-bit: byte offset of the 16-bit word (relative to the START of the code region, i.e. past the nibble
// plane) and the bit position of the two high bits of K element (tok, ch)
__host__ __device__ inline int k_hi_pos(int head_dim, int tok, int ch, int* shift) {
  const int blk = ch >> 5, c = ch & 31;
  *shift = ((c >= 16) ? 8 : 0) + 2 * (c & 3);
  return kPageTokens * head_dim / 2 + blk * 128 + tok * 8 + ((c & 15) >> 2) * 2;
}
__host__ __device__ inline int v_hi_pos(int head_dim, int tok, int ch, int* shift) {
  const int p = tok >> 1;
  const int chunk = (ch >> 2) ^ ((p & 3) << 2);
  *shift = ((tok & 1) ? 8 : 0) + 2 * (ch & 3);
  return kPageTokens * head_dim / 2 + p * (head_dim / 2) + chunk * 2;
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
