// Keys and bins of the radix select, shared by the top-k kernels and by kernels that build a row
// histogram for them (the index-score epilogue).
#pragma once
#include <stdint.h>

namespace ulc {

constexpr int kTopkBins = 2048;

__device__ __forceinline__ uint32_t order_key(float x) {
  uint32_t u = __float_as_uint(x);
  if (x != x) u = 0xff800000u;   // NaN sorts as -inf
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Histogram bin of an order-preserving key: monotone (not strictly) in the key.
__device__ __forceinline__ uint32_t window_bin(uint32_t key) {
  const bool nonneg = (key & 0x80000000u) != 0u;
  const uint32_t mag = (nonneg ? key : ~key) & 0x7fffffffu;        // exponent | mantissa of |x|
  const int t = static_cast<int>(mag >> 18) - (112 << 5);           // exponent 112 = 2^-15
  const uint32_t bp = static_cast<uint32_t>(min(max(t, 0), 1023));
  return nonneg ? 1024u + bp : 1023u - bp;
}

// Smallest key of bin b (0 .. 2047).  Key 0 is reserved for "no element", so bin 0 starts at 1.
__device__ __forceinline__ uint32_t bin_lo_key(uint32_t b) {
  if (b == 0u) return 1u;
  if (b >= 1024u) {
    const uint32_t bp = b - 1024u;
    return 0x80000000u | (bp == 0u ? 0u : ((bp + 3584u) << 18));
  }
  // negative scores: the smallest key of the bin belongs to its LARGEST magnitude
  const uint32_t bp = 1023u - b;
  const uint32_t mhi = bp == 1023u ? 0x7fffffffu : (((bp + 3585u) << 18) - 1u);
  return 0x7fffffffu - mhi;
}

// Workspace of the histogram-first selection (see topk.cu), per row, in 32-bit words.
constexpr int kTopkWsRowBytes = 24832;
constexpr int kTopkWsCtr = 8192 / 4;
constexpr int kTopkWsKey = 8448 / 4;
constexpr int kTopkWsPos = 16640 / 4;


}  // namespace ulc
