// Presence-bitmap recency ring, parallel device form.
//
// State: 255 recent buckets + 1 cold bucket; per bucket a level-0 bitmap over the slots and a
// level-1 summary (one bit per level-0 word), one member count per bucket, the epoch each recent
// bucket stands for, and slot_bucket[slot] (the bucket a slot is in, -1 = detached).
//
//   touch    any number of threads: slot_bucket is exchanged atomically, so exactly one thread moves a
//            slot; the clear of the old bit and the set of the new one are word atomics, lanes of a warp
//            that set bits of the same word are combined into one atomic (match.any);
//   advance  two launches: a scalar step (epoch, counts, labels) and a drain of the bucket being
//            reused into the cold bucket that walks the summary: cost ~ slots/1024 + expiring slots;
//   victims  three launches: a scalar plan (cold first, then the oldest recent buckets, never the
//            current one) listing (bucket, take); a count of set bits per (bucket, chunk); an ordered
//            emit (lowest slots of a bucket first) from a prefix over the chunk counts.
//
// Within a phase a bucket only ever gains bits (the current / cold one) or only ever loses them (the
// others), so summary bits may be left stale-set by a clear: a summary bit means "look at this word".
//
// The host / device header ulc/presence_bitmap.h is the sequential form of the same structure.
//
// Reference roles: ulacache/csrc/eviction/presence_recent.cuh:52-229 (claim / mark / advance /
// enumerate_victims), presence_warp.cuh:11-133 (warp-aggregated updates), victims.cuh:81-194
// (bucket-parallel victim enumeration).
#include <cuda_runtime.h>
#include <stdint.h>

#include "ulc/presence_ring.h"
#include "ulc/status.h"

namespace ulc {

__device__ __forceinline__ uint32_t* pr_bits(const PRing& r, int bucket) { return r.bits + static_cast<size_t>(bucket) * r.w0; }
__device__ __forceinline__ uint32_t* pr_sum(const PRing& r, int bucket) { return r.summary + static_cast<size_t>(bucket) * r.w1; }

// Move `slot` into bucket `cur` (or detach it when cur < 0).  Called by converged or diverged lanes;
// `moving` lanes of a warp that target the same level-0 word share one atomicOr.
__device__ __forceinline__ void pr_move(const PRing& r, int slot, int cur, bool active) {
  int old = cur;
  if (active) old = atomicExch(&r.slot_bucket[slot], cur);
  const bool moved = active && old != cur;
  const int w = slot >> 5;
  const uint32_t m = 1u << (slot & 31);
  if (moved && old >= 0) {
    atomicAnd(&pr_bits(r, old)[w], ~m);
    atomicSub(&r.count[old], 1);
  }
  const bool sets = moved && cur >= 0;
  const unsigned int movers = __ballot_sync(__activemask(), sets);
  if (sets) {
    const unsigned int peers = __match_any_sync(movers, w);
    uint32_t mask = 0;
    for (unsigned int p = peers; p; p &= p - 1) mask |= __shfl_sync(peers, m, __ffs(p) - 1);
    const int lane = threadIdx.x & 31;
    if (lane == __ffs(peers) - 1) {
      atomicOr(&pr_bits(r, cur)[w], mask);
      atomicOr(&pr_sum(r, cur)[w >> 5], 1u << (w & 31));
    }
    if (lane == __ffs(movers) - 1) atomicAdd(&r.count[cur], __popc(movers));
  }
}

__global__ void pring_begin_kernel(PRing r) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int epoch = r.ctl[kPrEpoch] + 1;
  r.ctl[kPrEpoch] = epoch;
  const int b = epoch % kPrRecent;
  int drain = -1;
  if (r.bucket_epoch[b] >= 0 && r.bucket_epoch[b] != epoch) {
    drain = b;
    r.count[kPrCold] += r.count[b];
    r.count[b] = 0;
  }
  r.bucket_epoch[b] = epoch;
  r.ctl[kPrDrain] = drain;
}

// One warp per summary word of the bucket being reused: lane j owns level-0 word 32 i + j.
__global__ void __launch_bounds__(256) pring_drain_kernel(PRing r, int relabel) {
  const int b = r.ctl[kPrDrain];
  if (b < 0) return;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  uint32_t* src = pr_bits(r, b);
  uint32_t* dst = pr_bits(r, kPrCold);
  for (int i = warp; i < r.w1; i += nwarps) {
    const uint32_t sm = pr_sum(r, b)[i];
    if (!sm) continue;
    const int w = i * 32 + lane;
    uint32_t v = 0;
    if (w < r.w0 && ((sm >> lane) & 1u)) v = src[w];
    if (v) {
      atomicOr(&dst[w], v);
      src[w] = 0;
      if (relabel)
        for (uint32_t t = v; t; t &= t - 1) r.slot_bucket[w * 32 + __ffs(t) - 1] = kPrCold;
    }
    const uint32_t live = __ballot_sync(0xffffffffu, v != 0);
    if (lane == 0) {
      if (live) atomicOr(&pr_sum(r, kPrCold)[i], live);
      pr_sum(r, b)[i] = 0;
    }
  }
}

__global__ void __launch_bounds__(256) pring_touch_kernel(PRing r, const int32_t* __restrict__ slots, int n, int detach,
                                                          int32_t* status) {
  const int cur = detach ? -1 : r.ctl[kPrEpoch] % kPrRecent;
  const int base = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  for (int i0 = base; i0 < n; i0 += gridDim.x * blockDim.x) {
    const int i = i0 + (threadIdx.x & 31);
    int s = i < n ? slots[i] : -1;
    if (s >= r.n) { report(status, kErrBounds, s); s = -1; }
    pr_move(r, s < 0 ? 0 : s, cur, s >= 0);
  }
}

// ids -> hit (touch the slot) or miss (flag[i] = 1).  dir: id -> slot or -1.
__global__ void __launch_bounds__(256) pring_lookup_touch_kernel(PRing r, const int32_t* __restrict__ ids, int n,
                                                                 const int32_t* __restrict__ dir, int id_space,
                                                                 int32_t* __restrict__ miss_flag, int32_t* status) {
  const int cur = r.ctl[kPrEpoch] % kPrRecent;
  const int base = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  for (int i0 = base; i0 < n; i0 += gridDim.x * blockDim.x) {
    const int i = i0 + (threadIdx.x & 31);
    int s = -1;
    if (i < n) {
      const int id = ids[i];
      if (id < 0 || id >= id_space) {
        report(status, kErrBounds, id);
        miss_flag[i] = 0;
      } else {
        s = dir[id];
        miss_flag[i] = s < 0;
      }
    }
    pr_move(r, s < 0 ? 0 : s, cur, s >= 0);
  }
}

// (bucket, take, base) list for `need` victims: the cold bucket, then recent buckets from the oldest.
__global__ void pring_victim_plan_kernel(PRing r, int need) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int epoch = r.ctl[kPrEpoch];
  int got = 0, listed = 0;
  auto add = [&](int bucket) {
    const int c = r.count[bucket];
    if (c <= 0 || got >= need) return;
    const int take = min(c, need - got);
    r.vlist[listed * 3] = bucket;
    r.vlist[listed * 3 + 1] = take;
    r.vlist[listed * 3 + 2] = got;
    got += take;
    ++listed;
  };
  if (need > 0) {
    add(kPrCold);
    for (int age = kPrRecent - 1; age >= 1 && got < need; --age) {
      const int e = epoch - age;
      if (e < 0) continue;
      const int b = e % kPrRecent;
      if (r.bucket_epoch[b] == e) add(b);
    }
  }
  r.ctl[kPrServed] = got;
  r.ctl[kPrListed] = listed;
}

// grid (kPrChunks, y): one warp per (listed bucket, chunk of its summary).
__global__ void __launch_bounds__(32) pring_victim_count_kernel(PRing r) {
  const int lane = threadIdx.x, c = blockIdx.x;
  const int listed = r.ctl[kPrListed];
  const int per = (r.w1 + kPrChunks - 1) / kPrChunks;
  for (int j = blockIdx.y; j < listed; j += gridDim.y) {
    const int b = r.vlist[j * 3];
    const uint32_t* bits = pr_bits(r, b);
    const uint32_t* sum = pr_sum(r, b);
    int total = 0;
    for (int i = c * per; i < min(r.w1, (c + 1) * per); ++i) {
      const uint32_t sm = sum[i];
      if (!sm) continue;
      const int w = i * 32 + lane;
      const uint32_t v = (w < r.w0 && ((sm >> lane) & 1u)) ? bits[w] : 0;
      total += __popc(v);
      // a clear leaves the summary bit set: drop the bits of words found empty (nothing sets bits of a
      // listed bucket in this phase, and no other warp reads this summary word)
      const uint32_t live = __ballot_sync(0xffffffffu, v != 0);
      if (lane == 0 && live != sm) pr_sum(r, b)[i] = live;
    }
    total = __reduce_add_sync(0xffffffffu, total);
    if (lane == 0) r.chunk_count[j * kPrChunks + c] = total;
  }
}

// Same grid: emits the chunk's slots in ascending order at their rank within the bucket.
__global__ void __launch_bounds__(32) pring_victim_emit_kernel(PRing r, int32_t* __restrict__ victims, int capacity) {
  const int lane = threadIdx.x, c = blockIdx.x;
  const int listed = r.ctl[kPrListed];
  const int per = (r.w1 + kPrChunks - 1) / kPrChunks;
  for (int j = blockIdx.y; j < listed; j += gridDim.y) {
    const int b = r.vlist[j * 3], take = r.vlist[j * 3 + 1], base = r.vlist[j * 3 + 2];
    int run = 0;                                   // set bits of the chunks before mine
    for (int k = lane; k < c; k += 32) run += r.chunk_count[j * kPrChunks + k];
    run = __reduce_add_sync(0xffffffffu, run);
    if (run >= take) continue;
    const uint32_t* bits = pr_bits(r, b);
    const uint32_t* sum = pr_sum(r, b);
    for (int i = c * per; i < min(r.w1, (c + 1) * per) && run < take; ++i) {
      const uint32_t sm = sum[i];
      if (!sm) continue;
      const int w = i * 32 + lane;
      uint32_t v = (w < r.w0 && ((sm >> lane) & 1u)) ? bits[w] : 0;
      const int cnt = __popc(v);
      int incl = cnt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      int rank = run + incl - cnt;
      for (; v && rank < take; v &= v - 1, ++rank) {
        const int at = base + rank;
        if (at < capacity) victims[at] = w * 32 + __ffs(v) - 1;
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
}

// Place the misses: miss i takes free_stack[nfree - 1 - i] while i < from_free, then victims[i - from_free].
// A victim's old record leaves the directory (its id goes to evicted[i - from_free]).
__global__ void __launch_bounds__(256) pring_place_kernel(PRing r, const int32_t* __restrict__ miss_ids, int n_place,
                                                          int from_free, const int32_t* __restrict__ free_stack, int nfree,
                                                          const int32_t* __restrict__ victims, int32_t* __restrict__ dir,
                                                          int32_t* __restrict__ id_of, int32_t* __restrict__ evicted) {
  const int cur = r.ctl[kPrEpoch] % kPrRecent;
  const int base = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  for (int i0 = base; i0 < n_place; i0 += gridDim.x * blockDim.x) {
    const int i = i0 + (threadIdx.x & 31);
    int s = -1;
    if (i < n_place) {
      if (i < from_free) {
        s = free_stack[nfree - 1 - i];
      } else {
        s = victims[i - from_free];
        const int old = id_of[s];
        evicted[i - from_free] = old;
        if (old >= 0) dir[old] = -1;
      }
      id_of[s] = miss_ids[i];
      dir[miss_ids[i]] = s;
    }
    pr_move(r, s < 0 ? 0 : s, cur, s >= 0);
  }
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// Words of the level-0 bitmap and of the summary of ONE bucket.
int ulc_pring_words(int slots, int* w0, int* w1) {
  if (slots <= 0) return -kErrUnsupported;
  *w0 = (slots + 31) / 32;
  *w1 = (*w0 + 31) / 32;
  return 0;
}

static inline int pring_grid(long long n, int threads, int cap) {
  long long g = (n + threads - 1) / threads;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

// New step: epoch + 1, expired bucket into the cold one.
int ulc_pring_drain(const PRing* r, int relabel, cudaStream_t s) {
  pring_drain_kernel<<<pring_grid(static_cast<long long>(r->w1) * 32, 256, 296), 256, 0, s>>>(*r, relabel);
  return static_cast<int>(cudaGetLastError());
}

int ulc_pring_advance(const PRing* r, cudaStream_t s) {
  pring_begin_kernel<<<1, 32, 0, s>>>(*r);
  return ulc_pring_drain(r, 1, s);
}

int ulc_pring_touch(const PRing* r, const int32_t* slots, int n, int detach, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  pring_touch_kernel<<<pring_grid(n, 256, 592), 256, 0, s>>>(*r, slots, n, detach, status);
  return static_cast<int>(cudaGetLastError());
}

int ulc_pring_lookup_touch(const PRing* r, const int32_t* ids, int n, const int32_t* dir, int id_space, int32_t* miss_flag,
                           int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  pring_lookup_touch_kernel<<<pring_grid(n, 256, 592), 256, 0, s>>>(*r, ids, n, dir, id_space, miss_flag, status);
  return static_cast<int>(cudaGetLastError());
}

// victims[0 .. served) in eviction order; served is left in ctl[kPrServed].
int ulc_pring_victims(const PRing* r, int need, int32_t* victims, int capacity, cudaStream_t s) {
  pring_victim_plan_kernel<<<1, 32, 0, s>>>(*r, need);
  if (need <= 0) return static_cast<int>(cudaGetLastError());
  return ulc_pring_count_emit(r, victims, capacity, s);
}

int ulc_pring_count_emit(const PRing* r, int32_t* victims, int capacity, cudaStream_t s) {
  pring_victim_count_kernel<<<dim3(kPrChunks, 8), 32, 0, s>>>(*r);
  pring_victim_emit_kernel<<<dim3(kPrChunks, 8), 32, 0, s>>>(*r, victims, capacity);
  return static_cast<int>(cudaGetLastError());
}

int ulc_pring_place(const PRing* r, const int32_t* miss_ids, int n_place, int from_free, const int32_t* free_stack,
                    int nfree, const int32_t* victims, int32_t* dir, int32_t* id_of, int32_t* evicted, cudaStream_t s) {
  if (n_place <= 0) return 0;
  if (from_free > nfree || from_free > n_place) return -kErrUnsupported;
  pring_place_kernel<<<pring_grid(n_place, 256, 592), 256, 0, s>>>(*r, miss_ids, n_place, from_free, free_stack, nfree,
                                                                  victims, dir, id_of, evicted);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
