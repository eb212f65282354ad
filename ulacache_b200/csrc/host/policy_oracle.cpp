// CPU oracle for the replacement policies of the device tier: given a stream of steps (each a
// list of accessed record ids) it replays residency in a pool of `capacity` slots and reports
// hits, misses and the evicted ids.  The GPU policies are checked against it, and the scheduler
// study uses it as the reference arm.
//
// Policies
//   0  bucket ring   255 recent buckets (one per step epoch) + one cold bucket; victims come from
//                    the cold bucket first, then from the oldest recent bucket, lowest slot first
//                    (the policy of the residency kernels)
//   1  exact LRU     victim = smallest (last access epoch, slot)
//   2  linked list   move-to-front list in access order; victim = tail
//   3  clock         circular hand over the slots, skipping slots used in the current step
//   4  per-request   every request owns `per_request` slots with exact LRU inside them
//                    (the hot-buffer scheme of the HiSparse baseline)
//   5  bitmap ring   the decisions of policy 0, taken from hierarchical presence bitmaps
//                    (include/ulc/presence_bitmap.h) instead of a scan over all slots: touch,
//                    epoch advance and victim search cost one word per tree level
//
// Role of the reference's scripts/7_5_scheduler/_runtime/reference.cpp:1-146 (a ctypes-loaded C++
// replay of LRU policies); written independently against the behaviour described there.
#include <algorithm>
#include <cstdint>
#include <list>
#include <unordered_map>
#include <vector>

#include "ulc/presence_bitmap.h"

namespace {

constexpr int kRecentBuckets = 255;

struct Sim {
  int kind = 0;
  int64_t capacity = 0;
  int64_t per_request = 0;
  int64_t epoch = 0;
  std::unordered_map<int64_t, int64_t> slot_of;       // id -> slot
  std::vector<int64_t> id_of;                          // slot -> id or -1
  std::vector<int64_t> stamp;                          // slot -> last access epoch
  std::vector<int64_t> free_slots;                     // stack, lowest slot on top
  // linked list (policy 2): most recent at front
  std::list<int64_t> order;                            // slots
  std::vector<std::list<int64_t>::iterator> where;
  int64_t hand = 0;                                    // policy 3
  // policy 4: request -> its slots
  std::unordered_map<int64_t, std::vector<int64_t>> req_slots;
  std::unordered_map<int64_t, int64_t> req_of_id;
  int64_t next_req_slot = 0;
  // policy 5: presence-bitmap ring over the slots
  ulc::PresenceRing ring;
  std::vector<uint32_t> ring_bits;
  std::vector<int16_t> ring_inverse;

  void init() {
    id_of.assign(capacity, -1);
    stamp.assign(capacity, -1);
    free_slots.clear();
    for (int64_t s = capacity - 1; s >= 0; --s) free_slots.push_back(s);
    where.assign(capacity, order.end());
    if (kind == 5) {
      ring_bits.assign(static_cast<size_t>(ulc::kPresenceBuckets) * ulc::presence_words(capacity), 0u);
      ring_inverse.assign(capacity, ulc::kPresenceFree);
      ring.init(ring_bits.data(), ring_inverse.data(), static_cast<int32_t>(capacity));
    }
  }

  void next_epoch() {
    epoch += 1;
    if (kind == 5) ring.advance();
  }

  void touch(int64_t slot) {
    stamp[slot] = epoch;
    if (kind == 5) ring.touch(static_cast<int32_t>(slot));
    if (kind == 2) {
      if (where[slot] != order.end()) order.erase(where[slot]);
      order.push_front(slot);
      where[slot] = order.begin();
    }
  }

  // slot to evict, or -1 when every slot is in use by the current step
  int64_t victim() {
    if (kind == 5) return ring.victim();
    if (kind == 0) {
      // age >= 255 is the cold bucket; otherwise bucket = stamp % 255.  Cold first (lowest slot),
      // then the oldest epoch (lowest slot).  Equivalent: minimise (min(age,255) descending, ...)
      int64_t best = -1, best_age = -1;
      for (int64_t s = 0; s < capacity; ++s) {
        if (id_of[s] < 0 || stamp[s] == epoch) continue;
        int64_t age = std::min<int64_t>(epoch - stamp[s], kRecentBuckets);
        if (age > best_age) { best_age = age; best = s; }
      }
      return best;
    }
    if (kind == 1 || kind == 4) {
      int64_t best = -1;
      for (int64_t s = 0; s < capacity; ++s) {
        if (id_of[s] < 0 || stamp[s] == epoch) continue;
        if (best < 0 || stamp[s] < stamp[best]) best = s;
      }
      return best;
    }
    if (kind == 2) {
      for (auto it = order.rbegin(); it != order.rend(); ++it)
        if (stamp[*it] != epoch) return *it;
      return -1;
    }
    for (int64_t n = 0; n < capacity; ++n) {           // clock
      const int64_t s = (hand + n) % capacity;
      if (id_of[s] >= 0 && stamp[s] != epoch) { hand = (s + 1) % capacity; return s; }
    }
    return -1;
  }

  void drop(int64_t slot) {
    slot_of.erase(id_of[slot]);
    id_of[slot] = -1;
    if (kind == 5) ring.detach(static_cast<int32_t>(slot));
    if (kind == 2 && where[slot] != order.end()) { order.erase(where[slot]); where[slot] = order.end(); }
  }
};

}  // namespace

extern "C" {

void* ulc_policy_create(int kind, long long capacity, long long per_request) {
  if (kind < 0 || kind > 5 || capacity <= 0 || (kind == 5 && capacity > 0x7fffffffLL)) return nullptr;
  Sim* s = new Sim;
  s->kind = kind;
  s->capacity = capacity;
  s->per_request = per_request;
  s->init();
  return s;
}

void ulc_policy_destroy(void* h) { delete static_cast<Sim*>(h); }

// One step.  ids[n] accessed records (duplicates allowed: later ones hit); requests[n] (policy 4
// only, nullable) the request each access belongs to.  evicted[] (capacity >= n) receives the
// ids that lost their slot, in order.  counts[0..3] = hits, misses, evictions, overflow (misses
// that found no slot).  Returns 0, or -1 on a bad handle.
int ulc_policy_step(void* h, const long long* ids, const long long* requests, long long n, long long* evicted,
                    long long* counts) {
  Sim* s = static_cast<Sim*>(h);
  if (s == nullptr) return -1;
  s->next_epoch();
  long long hits = 0, misses = 0, ev = 0, overflow = 0;
  for (long long i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    auto it = s->slot_of.find(id);
    if (it != s->slot_of.end()) {
      hits += 1;
      s->touch(it->second);
      continue;
    }
    misses += 1;
    int64_t slot = -1;
    if (s->kind == 4 && requests != nullptr && s->per_request > 0) {
      // the request's own slots: claim unused pool slots up to per_request, then LRU inside them
      auto& mine = s->req_slots[requests[i]];
      if (static_cast<int64_t>(mine.size()) < s->per_request && !s->free_slots.empty()) {
        slot = s->free_slots.back();
        s->free_slots.pop_back();
        mine.push_back(slot);
      } else {
        for (int64_t cand : mine)
          if (s->stamp[cand] != s->epoch && (slot < 0 || s->stamp[cand] < s->stamp[slot])) slot = cand;
        if (slot >= 0 && s->id_of[slot] >= 0) { evicted[ev++] = s->id_of[slot]; s->drop(slot); }
      }
    } else if (!s->free_slots.empty()) {
      slot = s->free_slots.back();
      s->free_slots.pop_back();
    } else {
      slot = s->victim();
      if (slot >= 0) { evicted[ev++] = s->id_of[slot]; s->drop(slot); }
    }
    if (slot < 0) { overflow += 1; continue; }
    s->id_of[slot] = id;
    s->slot_of[id] = slot;
    s->touch(slot);
  }
  counts[0] = hits; counts[1] = misses; counts[2] = ev; counts[3] = overflow;
  return 0;
}

// Forget records (request finished): their slots return to the free stack.
int ulc_policy_release(void* h, const long long* ids, long long n) {
  Sim* s = static_cast<Sim*>(h);
  if (s == nullptr) return -1;
  for (long long i = 0; i < n; ++i) {
    auto it = s->slot_of.find(ids[i]);
    if (it == s->slot_of.end()) continue;
    const int64_t slot = it->second;
    s->drop(slot);
    s->stamp[slot] = -1;
    if (s->kind != 4) s->free_slots.push_back(slot);
  }
  return 0;
}

// A bare presence bitmap, for tests of the tree itself: op 0 = set, 1 = clear, 2 = test,
// 3 = lowest set slot at or after `slot` (-1 if none), 4 = number of set bits.
struct BitmapHandle {
  ulc::PresenceBitmap map;
  std::vector<uint32_t> words;
};

void* ulc_presence_create(long long slots) {
  if (slots <= 0 || slots > 0x7fffffffLL) return nullptr;
  BitmapHandle* b = new BitmapHandle;
  b->words.assign(static_cast<size_t>(ulc::presence_words(slots)), 0u);
  b->map.init(b->words.data(), static_cast<int32_t>(slots));
  return b;
}

void ulc_presence_destroy(void* h) { delete static_cast<BitmapHandle*>(h); }

long long ulc_presence_op(void* h, int op, long long slot) {
  BitmapHandle* b = static_cast<BitmapHandle*>(h);
  if (b == nullptr) return -2;
  if (op == 4) return b->map.count;
  if (op == 3) return b->map.find_next(static_cast<int32_t>(slot));
  if (slot < 0 || slot >= b->map.n) return -2;
  if (op == 0) return b->map.set(static_cast<int32_t>(slot)) ? 1 : 0;
  if (op == 1) return b->map.clear(static_cast<int32_t>(slot)) ? 1 : 0;
  if (op == 2) return b->map.test(static_cast<int32_t>(slot)) ? 1 : 0;
  return -2;
}

long long ulc_policy_resident(void* h) {
  Sim* s = static_cast<Sim*>(h);
  return s == nullptr ? -1 : static_cast<long long>(s->slot_of.size());
}

// Scenario check of the sequential presence ring (ulc/presence_bitmap.h) on the host: `early` slots are
// touched BEFORE the first advance (epoch 0), one more slot is touched in every later epoch, and the ring is
// advanced `epochs` times.  The epoch-0 slots must be offered as victims while they are recent (oldest
// first), move to the cold bucket when their bucket is reused (epoch 255), stay attached, and be the first
// victims afterwards.  Returns 0, or the number of the first check that failed.
int ulc_presence_ring_epoch0_check(int slots, int early, int epochs) {
  if (slots <= 0 || early <= 0 || early + epochs > slots) return -1;
  std::vector<uint32_t> bits(static_cast<size_t>(ulc::kPresenceBuckets) * ulc::presence_words(slots), 0u);
  std::vector<int16_t> inverse(slots);
  auto* ring = new ulc::PresenceRing;
  ring->init(bits.data(), inverse.data(), slots);
  int rc = 0;
  for (int s = 0; s < early; ++s) ring->touch(s);                    // epoch 0, before any advance
  if (ring->attached() != early) rc = 1;
  if (!rc && ring->victim() != -1) rc = 2;                           // everything attached is of the current epoch
  for (int e = 1; e <= epochs && !rc; ++e) {
    ring->advance();
    ring->touch(early + e - 1);
    if (ring->attached() != early + e) { rc = 3; break; }
    // the epoch-0 slots are the oldest: the victim is the lowest of them, recent or cold
    if (ring->victim() != 0) { rc = 4; break; }
    const bool cold = e >= ulc::kPresenceRecent;
    if (cold && ring->bucket[ulc::kPresenceRecent].count < early) { rc = 5; break; }
    if (!cold && ring->bucket[ulc::kPresenceRecent].count != 0) { rc = 6; break; }
  }
  if (!rc) {                                                         // evict them all: lowest slot first
    for (int s = 0; s < early; ++s) {
      const int v = ring->victim();
      if (v != s) { rc = 7; break; }
      ring->detach(v);
    }
  }
  if (!rc && epochs >= 2 && ring->victim() != early) rc = 8;         // then the slot of epoch 1 (not current any more)
  delete ring;
  return rc;
}

}  // extern "C"
