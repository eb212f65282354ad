// State of one residency group (one directory shared by a set of layers) and
// the bucketed-recency ring used to pick eviction victims.
//
// Policy (same decisions as the reference's presence-bitmap ring,
// ulacache/csrc/eviction/presence_recent.cuh:125-229): recency is tracked in
// epochs (one per forward step).  A slot touched in epoch e belongs to recent
// bucket e % 255 until it is 255 epochs old, then to the cold bucket.  Victims
// come from the cold bucket first, then from the oldest recent bucket upward,
// never from the current epoch.
//
// Representation (different from the reference on purpose): every HBM slot
// carries the epoch of its last touch, and the ring keeps only one COUNT per
// bucket.  Quotas are computed from the 256 counts; victims are enumerated by
// one coalesced scan over the stamps (4 bytes per slot, L2 resident on a 126 MB
// L2) instead of walking eight levels of 32-ary bitmaps.
//
// Everything here is plain integer code usable from host and device; the host
// build is the oracle the GPU kernels are tested against.
#pragma once
#include "layout.h"

namespace ulc {

constexpr int kRecentBuckets = 255;
constexpr int kColdBucket = 255;
constexpr int kRingBuckets = 256;

enum Counter : int32_t {
  kCntEpoch = 0,
  kCntHbmFree = 1,        // entries on the HBM free stack
  kCntHostFree = 2,       // entries on the host free stack
  kCntPromote = 3,        // rows queued for promotion this step
  kCntPlan = 4,           // items in the plan
  kCntVictims = 5,        // victims enumerated so far
  kCntNeedVictims = 6,    // victims wanted by the current plan
  kCntFromFree = 7,       // promotions served from free slots
  kCntHits = 8,           // statistics (monotonic)
  kCntMisses = 9,
  kCntPromotions = 10,
  kCntEvictions = 11,
  kCntRegistered = 12,
  kCntBoundaryBucket = 13,
  kCntBoundaryQuota = 14,
  kCntBoundaryTaken = 15,
  kCntCutoffEpoch = 16,   // victims have stamp < cutoff, or == boundary epoch within quota
  kCntUnserved = 17,      // promotions that could not be served (capacity)
  kCntRingCtl = 24,       // 8 words: control block of the presence-bitmap index (see presence_ring.h)
  kNumCounters = 32,
};

struct ResidencyState {
  int32_t* directory;     // [dir_len] local ID -> slot encoding
  int32_t* hbm_tags;      // [hbm_slots] slot -> local ID, -1 free
  int32_t* host_tags;     // [host_slots]
  int32_t* stamps;        // [hbm_slots] epoch of last touch, -1 free
  int32_t* access_time;   // [dir_len] epoch in which the row was last queued for promotion
  int32_t* hbm_free;      // [hbm_slots] stack
  int32_t* host_free;     // [host_slots] stack
  int32_t* counters;      // [kNumCounters]
  int32_t* ring;          // [kRingBuckets] slots per bucket
  int32_t* promote;       // [plan_capacity] local IDs to promote
  int32_t* plan;          // [kPlanRows, plan_capacity]
  int32_t* victims;       // [plan_capacity] victim slots
  int32_t dir_len, hbm_slots, host_slots, plan_capacity;
  // Optional victim index over the stamps (null = victims are found by scanning the stamps): one bitmap
  // per bucket with a level-1 summary, kept in step with the stamps by every kernel that changes one.
  uint32_t* bits;         // [256][w0]
  uint32_t* summary;      // [256][w1]
  int32_t* vlist;         // [256][3] buckets a plan takes victims from
  int32_t* chunk_count;   // [256][kPrChunks]
  int32_t w0, w1;
};

#if defined(__CUDACC__)
// A slot enters / leaves the bitmap of `bucket` (no-ops without the index).  A clear leaves the summary
// bit set; the victim count drops summary bits of words it finds empty.
__device__ __forceinline__ void bm_set(const ResidencyState& st, int bucket, int32_t slot) {
  if (st.bits == nullptr) return;
  const int w = slot >> 5;
  atomicOr(&st.bits[static_cast<size_t>(bucket) * st.w0 + w], 1u << (slot & 31));
  atomicOr(&st.summary[static_cast<size_t>(bucket) * st.w1 + (w >> 5)], 1u << (w & 31));
}
__device__ __forceinline__ void bm_clear(const ResidencyState& st, int bucket, int32_t slot) {
  if (st.bits == nullptr) return;
  atomicAnd(&st.bits[static_cast<size_t>(bucket) * st.w0 + (slot >> 5)], ~(1u << (slot & 31)));
}
#endif

ULC_HD int32_t bucket_of(int32_t stamp, int32_t epoch) {
  return (epoch - stamp >= kRecentBuckets) ? kColdBucket : (stamp % kRecentBuckets);
}

// Given the ring counts, decide which stamps are victims when `need` slots are
// wanted at epoch `epoch`: every slot with stamp < cutoff, plus `quota` slots
// whose stamp == cutoff (the boundary epoch).  Cold slots (age >= 255) always
// precede.  Returns the number that can actually be served.
ULC_HD int32_t victim_cutoff(const int32_t* ring, int32_t epoch, int32_t need, int32_t* cutoff,
                             int32_t* quota) {
  int32_t got = 0;
  *cutoff = epoch - kRecentBuckets + 1;   // everything colder than the ring
  *quota = 0;
  if (need <= 0) { *cutoff = -0x7fffffff; return 0; }
  const int32_t cold = ring[kColdBucket];
  if (cold >= need) {
    // boundary inside the cold bucket: stamps are unordered there, take any `need`
    *cutoff = -0x7fffffff;   // marker: quota applies to the cold bucket
    *quota = need;
    return need;
  }
  got = cold;
  // oldest recent epoch is epoch-254, newest allowed is epoch-1
  for (int32_t e = epoch - kRecentBuckets + 1; e < epoch; ++e) {
    if (e < 0) continue;
    const int32_t c = ring[e % kRecentBuckets];
    if (got + c >= need) {
      *cutoff = e;
      *quota = need - got;
      return need;
    }
    got += c;
  }
  *cutoff = epoch;   // everything but the current epoch
  *quota = 0;
  return got;
}

}  // namespace ulc
