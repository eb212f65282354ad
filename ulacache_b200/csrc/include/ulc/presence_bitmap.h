// Hierarchical presence bitmap and the bucketed-recency ring built from it.
//
// PresenceBitmap: a 32-ary tree of bit words over `n` slots.  Level 0 has one
// bit per slot; a bit of level l + 1 says "the word below holds at least one
// set bit".  Setting, clearing and finding the lowest set slot cost one word
// per level (at most 7 levels for 2^31 slots), independent of the pool size.
//
// PresenceRing: 255 recent buckets (one per step epoch, reused modulo 255) and
// one cold bucket, each a PresenceBitmap over the same slots, plus the inverse
// map slot -> bucket.  It makes the same decisions as the stamp-based ring of
// residency.h (victims: cold bucket first, then the oldest recent bucket
// upward, never the current epoch; lowest slot first inside a bucket), but its
// costs follow the number of slots that expire or are taken, not the pool size:
//   touch   : two tree updates
//   advance : drains only the bucket that turned 255 epochs old
//   victim  : one descent of the first non-empty bucket
//
// Reference counterpart: ulacache/csrc/eviction/presence_bitmap.cuh:20-249 and
// presence_recent.cuh:52-229 (the same structure, with warp-cooperative
// variants for concurrent updates).  The functions here are sequential: the
// host oracle uses them as they are; a device caller must give each bitmap word
// one writer at a time (for example one thread per residency group).
#pragma once
#include <stdint.h>
#include "layout.h"

namespace ulc {

constexpr int kPresenceMaxLevels = 7;

// Number of 32-bit words a bitmap over n slots needs (all levels).
ULC_HD int64_t presence_words(int64_t n) {
  int64_t total = 0, w = (n + 31) / 32;
  for (int l = 0; l < kPresenceMaxLevels; ++l) {
    total += w;
    if (w <= 1) break;
    w = (w + 31) / 32;
  }
  return total;
}

struct PresenceBitmap {
  uint32_t* words;                       // all levels, level 0 first
  int64_t level_off[kPresenceMaxLevels]; // first word of each level
  int32_t levels;
  int32_t n;                             // slots
  int32_t count;                         // set bits

  // `storage` must hold presence_words(n) zeroed words.
  ULC_HD void init(uint32_t* storage, int32_t slots) {
    words = storage;
    n = slots;
    count = 0;
    int64_t off = 0, w = (static_cast<int64_t>(slots) + 31) / 32;
    levels = 0;
    for (int l = 0; l < kPresenceMaxLevels; ++l) {
      level_off[l] = off;
      off += w;
      levels = l + 1;
      if (w <= 1) break;
      w = (w + 31) / 32;
    }
  }

  ULC_HD bool test(int32_t slot) const { return (words[level_off[0] + (slot >> 5)] >> (slot & 31)) & 1u; }

  // Returns true when the bit was clear before.
  ULC_HD bool set(int32_t slot) {
    int64_t idx = slot;
    for (int l = 0; l < levels; ++l) {
      uint32_t& w = words[level_off[l] + (idx >> 5)];
      const uint32_t bit = 1u << (idx & 31);
      const bool was_empty = (w == 0);
      if (l == 0 && (w & bit)) return false;
      w |= bit;
      if (!was_empty) break;             // the parents already know about this word
      idx >>= 5;
    }
    ++count;
    return true;
  }

  // Returns true when the bit was set before.
  ULC_HD bool clear(int32_t slot) {
    int64_t idx = slot;
    for (int l = 0; l < levels; ++l) {
      uint32_t& w = words[level_off[l] + (idx >> 5)];
      const uint32_t bit = 1u << (idx & 31);
      if (l == 0 && !(w & bit)) return false;
      w &= ~bit;
      if (w != 0) break;                 // the word is still non-empty: parents unchanged
      idx >>= 5;
    }
    --count;
    return true;
  }

  ULC_HD static int lowest_bit(uint32_t w) {
#if defined(__CUDA_ARCH__)
    return __ffs(static_cast<int>(w)) - 1;
#else
    return __builtin_ctz(w);
#endif
  }

  // Lowest set slot, or -1 when empty: one word per level, top down.
  ULC_HD int32_t find_first() const {
    if (count == 0) return -1;
    int64_t idx = 0;
    for (int l = levels - 1; l >= 0; --l) {
      const uint32_t w = words[level_off[l] + idx];
      idx = (idx << 5) + lowest_bit(w);
    }
    return static_cast<int32_t>(idx);
  }

  // Lowest set slot >= from, or -1.  Climbs until a word has a set bit to the right, then descends.
  ULC_HD int32_t find_next(int32_t from) const {
    if (count == 0 || from >= n) return -1;
    if (from < 0) from = 0;
    int64_t idx = from;
    int l = 0;
    // bits of the current word at or above idx
    while (true) {
      const int64_t word = idx >> 5;
      const int shift = static_cast<int>(idx & 31);
      const int64_t level_words = (l + 1 < levels ? level_off[l + 1] : level_off[l] + 1) - level_off[l];
      uint32_t w = word < level_words ? words[level_off[l] + word] : 0u;
      w = shift ? (w >> shift) << shift : w;
      if (w != 0) {
        idx = (word << 5) + lowest_bit(w);
        break;
      }
      if (l + 1 >= levels) return -1;
      idx = word + 1;                    // continue to the right, one level up
      ++l;
    }
    for (; l > 0; --l) {                 // descend to the lowest set bit below
      const uint32_t w = words[level_off[l - 1] + idx];
      idx = (idx << 5) + lowest_bit(w);
    }
    return static_cast<int32_t>(idx);
  }
};

constexpr int kPresenceRecent = 255;     // recent buckets; bucket kPresenceRecent is the cold one
constexpr int kPresenceBuckets = 256;
constexpr int8_t kPresenceFree = -1;

struct PresenceRing {
  PresenceBitmap bucket[kPresenceBuckets];
  int64_t bucket_epoch[kPresenceRecent]; // epoch a recent bucket stands for, -1 = empty
  int16_t* slot_bucket;                  // [n] bucket of a slot, or kPresenceFree
  int64_t epoch;
  int32_t n;

  // `bits` must hold kPresenceBuckets * presence_words(slots) zeroed words, `inverse` slots entries.
  ULC_HD void init(uint32_t* bits, int16_t* inverse, int32_t slots) {
    n = slots;
    epoch = 0;
    slot_bucket = inverse;
    const int64_t per = presence_words(slots);
    for (int b = 0; b < kPresenceBuckets; ++b) bucket[b].init(bits + per * b, slots);
    for (int b = 0; b < kPresenceRecent; ++b) bucket_epoch[b] = -1;
    bucket_epoch[0] = 0;                 // slots touched before the first advance() belong to epoch 0
    for (int32_t s = 0; s < slots; ++s) inverse[s] = kPresenceFree;
  }

  ULC_HD int current() const { return static_cast<int>(epoch % kPresenceRecent); }

  // New step: the bucket that is reused for `epoch + 1` held slots that are now 255 epochs old;
  // they move to the cold bucket.  Cost: the slots that expire.
  ULC_HD void advance() {
    epoch += 1;
    const int b = current();
    if (bucket_epoch[b] >= 0 && bucket_epoch[b] != epoch) {
      for (int32_t s = bucket[b].find_first(); s >= 0; s = bucket[b].find_first()) {
        bucket[b].clear(s);
        bucket[kPresenceRecent].set(s);
        slot_bucket[s] = kPresenceRecent;
      }
    }
    bucket_epoch[b] = epoch;
  }

  // The slot was used in the current epoch.
  ULC_HD void touch(int32_t slot) {
    const int cur = current();
    const int old = slot_bucket[slot];
    if (old == cur) return;
    if (old != kPresenceFree) bucket[old].clear(slot);
    bucket[cur].set(slot);
    slot_bucket[slot] = static_cast<int16_t>(cur);
  }

  // The slot no longer holds a record.
  ULC_HD void detach(int32_t slot) {
    const int old = slot_bucket[slot];
    if (old == kPresenceFree) return;
    bucket[old].clear(slot);
    slot_bucket[slot] = kPresenceFree;
  }

  // Next victim: lowest slot of the cold bucket, else of the oldest recent bucket; never a slot
  // of the current epoch.  -1 when every attached slot was used in this epoch.
  ULC_HD int32_t victim() const {
    if (bucket[kPresenceRecent].count > 0) return bucket[kPresenceRecent].find_first();
    for (int age = kPresenceRecent - 1; age >= 1; --age) {
      const int64_t e = epoch - age;
      if (e < 0) continue;
      const int b = static_cast<int>(e % kPresenceRecent);
      if (bucket_epoch[b] == e && bucket[b].count > 0) return bucket[b].find_first();
    }
    return -1;
  }

  ULC_HD int32_t attached() const {
    int32_t total = 0;
    for (int b = 0; b < kPresenceBuckets; ++b) total += bucket[b].count;
    return total;
  }
};

}  // namespace ulc
