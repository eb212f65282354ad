// Replacement-policy ablations for the scheduler study: exact-timestamp LRU, a linked-list LRU, the
// per-request hot buffer of the HiSparse baseline, and a read-only hit observer.  They run on the
// same directory / slot arrays as the production bucket-ring policy so that a recorded selection
// trace can be replayed through each of them on the GPU and compared with the CPU oracle
// (csrc/host/policy_oracle.cpp).
//
// Reference roles: ulacache/csrc/eviction/naive_lru.cuh:61-139 (timestamps + byte radix select),
// csrc/kvcacheio/linked_list_lru.cuh:75, hisparse_union.cuh:310, trace_hits.cuh.  Independent
// implementations: single-CTA kernels, sized for studies (not for the decode path).
#include <cuda_runtime.h>
#include <stdint.h>

#include "ulc/presence_bitmap.h"
#include "ulc/status.h"

namespace ulc {

// ---------------------------------------------------------------------------------------------
// Exact LRU: the `need` occupied slots with the smallest (stamp, slot), skipping slots stamped
// with the current epoch.  Four 8-bit radix passes over the stamps find the threshold stamp; ties
// are taken lowest slot first.
__global__ void __launch_bounds__(1024)
exact_lru_victims_kernel(const int32_t* __restrict__ stamps, const int32_t* __restrict__ id_of, int n_slots,
                         int cur_epoch, int need, int32_t* __restrict__ out_slots, int32_t* __restrict__ out_count) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned int s_prefix, s_remaining, s_done;
  __shared__ int s_warp_sum[32];
  __shared__ int s_base_less, s_base_eq;
  const int t = threadIdx.x;
  if (t == 0) { s_prefix = 0; s_remaining = need; s_done = 0; s_base_less = 0; s_base_eq = 0; }
  __syncthreads();
  // candidates: occupied, not used this step
  auto cand = [&](int s) { return id_of[s] >= 0 && stamps[s] != cur_epoch && stamps[s] >= 0; };
  unsigned int total = 0;
  for (int s = t; s < n_slots; s += 1024) total += cand(s) ? 1u : 0u;
  // block sum of candidates
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if ((t & 31) == 0) s_warp_sum[t >> 5] = static_cast<int>(total);
  __syncthreads();
  if (t == 0) {
    int all = 0;
    for (int w = 0; w < 32; ++w) all += s_warp_sum[w];
    if (all < need) s_remaining = all;        // fewer candidates than asked: take them all
    out_count[0] = all < need ? all : need;
  }
  __syncthreads();
  const int want = out_count[0];
  if (want <= 0) return;
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = t; i < 256; i += 1024) hist[i] = 0;
    __syncthreads();
    const unsigned int prefix = s_prefix;
    const unsigned int hi_mask = pass == 3 ? 0u : (0xffffffffu << (8 * (pass + 1)));
    for (int s = t; s < n_slots; s += 1024) {
      if (!cand(s)) continue;
      const unsigned int k = static_cast<unsigned int>(stamps[s]);
      if ((k & hi_mask) == (prefix & hi_mask)) atomicAdd(&hist[(k >> (8 * pass)) & 255u], 1u);
    }
    __syncthreads();
    if (t == 0) {
      unsigned int rem = s_remaining, cum = 0;
      int bin = 0;
      for (; bin < 256; ++bin) {
        if (cum + hist[bin] >= rem) break;
        cum += hist[bin];
      }
      if (bin > 255) bin = 255;
      s_remaining = rem - cum;
      s_prefix = prefix | (static_cast<unsigned int>(bin) << (8 * pass));
    }
    __syncthreads();
  }
  const unsigned int thr = s_prefix;
  const int ties = static_cast<int>(s_remaining);       // slots with stamp == thr to take
  const int n_less = want - ties;
  // ordered emission: slots with stamp < thr first (any order inside), then the lowest tie slots
  for (int base = 0; base < n_slots; base += 1024) {
    const int s = base + t;
    const bool c = s < n_slots && cand(s);
    const unsigned int k = c ? static_cast<unsigned int>(stamps[s]) : 0xffffffffu;
    const bool less = c && k < thr, eq = c && k == thr;
    const unsigned int bl = __ballot_sync(0xffffffffu, less), be = __ballot_sync(0xffffffffu, eq);
    const int lane = t & 31, w = t >> 5;
    __syncthreads();
    if (lane == 0) s_warp_sum[w] = (__popc(bl) << 16) | __popc(be);
    __syncthreads();
    int less_before = 0, eq_before = 0;
    for (int i = 0; i < w; ++i) { less_before += s_warp_sum[i] >> 16; eq_before += s_warp_sum[i] & 0xffff; }
    less_before += __popc(bl & ((1u << lane) - 1u));
    eq_before += __popc(be & ((1u << lane) - 1u));
    const int bl_all = s_base_less, be_all = s_base_eq;
    if (less) out_slots[bl_all + less_before] = s;
    if (eq && be_all + eq_before < ties) out_slots[n_less + be_all + eq_before] = s;
    __syncthreads();
    if (t == 0) {
      int tl = 0, te = 0;
      for (int i = 0; i < 32; ++i) { tl += s_warp_sum[i] >> 16; te += s_warp_sum[i] & 0xffff; }
      s_base_less = bl_all + tl;
      s_base_eq = be_all + te;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// Linked-list LRU: one thread replays the accesses in order.  next/prev are slot-indexed, list[0]
// = head (most recent), list[1] = tail, list[2] = free-stack height, list[3] = epoch.
__global__ void linked_lru_step_kernel(int32_t* dir, int32_t* id_of, int32_t* stamp, int32_t* next, int32_t* prev,
                                       int32_t* list, int32_t* free_stack, const int32_t* ids, int n,
                                       int32_t* evicted, int32_t* counts) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int head = list[0], tail = list[1], nfree = list[2];
  const int epoch = list[3] + 1;
  int hits = 0, misses = 0, ev = 0, overflow = 0;
  auto unlink = [&](int s) {
    const int p = prev[s], q = next[s];
    if (p >= 0) next[p] = q; else head = q;
    if (q >= 0) prev[q] = p; else tail = p;
  };
  auto push_front = [&](int s) {
    prev[s] = -1;
    next[s] = head;
    if (head >= 0) prev[head] = s;
    head = s;
    if (tail < 0) tail = s;
  };
  for (int i = 0; i < n; ++i) {
    const int id = ids[i];
    int s = dir[id];
    if (s >= 0) {
      ++hits;
      unlink(s);
      push_front(s);
      stamp[s] = epoch;
      continue;
    }
    ++misses;
    if (nfree > 0) {
      s = free_stack[--nfree];
    } else {
      s = tail;
      while (s >= 0 && stamp[s] == epoch) s = prev[s];     // never a slot used in this step
      if (s >= 0) {
        evicted[ev++] = id_of[s];
        dir[id_of[s]] = -1;
        unlink(s);
      }
    }
    if (s < 0) { ++overflow; continue; }
    id_of[s] = id;
    dir[id] = s;
    stamp[s] = epoch;
    push_front(s);
  }
  list[0] = head; list[1] = tail; list[2] = nfree; list[3] = epoch;
  counts[0] = hits; counts[1] = misses; counts[2] = ev; counts[3] = overflow;
}

// ---------------------------------------------------------------------------------------------
// Per-request hot buffer: request r owns tags[r, 0..width) / stamps[r, 0..width).  One CTA per
// request replays its accesses in order; a miss replaces the entry with the smallest stamp that was
// not used in this step (lowest index on ties).
__global__ void __launch_bounds__(256)
hot_buffer_step_kernel(int32_t* tags, int32_t* stamps, int width, const int32_t* ids, const int32_t* row_offs,
                       int epoch, int32_t* counts /* [R, 2] hits, misses */) {
  __shared__ int s_hit;
  __shared__ unsigned long long s_best;
  const int r = blockIdx.x;
  int32_t* tg = tags + static_cast<size_t>(r) * width;
  int32_t* stp = stamps + static_cast<size_t>(r) * width;
  int hits = 0, misses = 0;
  for (int i = row_offs[r]; i < row_offs[r + 1]; ++i) {
    const int id = ids[i];
    if (threadIdx.x == 0) { s_hit = -1; s_best = ~0ull; }
    __syncthreads();
    for (int j = threadIdx.x; j < width; j += blockDim.x)
      if (tg[j] == id) atomicMax(&s_hit, j);
    __syncthreads();
    if (s_hit >= 0) {
      if (threadIdx.x == 0) stp[s_hit] = epoch;
      ++hits;
      __syncthreads();
      continue;
    }
    ++misses;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
      if (stp[j] == epoch) continue;
      // empty entries (tag -1, stamp -1) sort first: key = (stamp + 1) << 32 | index
      const unsigned long long key = (static_cast<unsigned long long>(static_cast<unsigned int>(stp[j] + 1)) << 32) |
                                     static_cast<unsigned int>(j);
      atomicMin(&s_best, key);
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_best != ~0ull) {
      const int j = static_cast<int>(s_best & 0xffffffffu);
      tg[j] = id;
      stp[j] = epoch;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { counts[2 * r] = hits; counts[2 * r + 1] = misses; }
}

// Read-only observer: how many of the selected ids are resident (directory entry >= 0).
__global__ void trace_hits_kernel(const int32_t* __restrict__ dir, int dir_len, const int32_t* __restrict__ sel,
                                  long long n, unsigned long long* __restrict__ counts /* hits, valid */) {
  unsigned long long hits = 0, valid = 0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int id = sel[i];
    if (id < 0 || id >= dir_len) continue;
    ++valid;
    hits += dir[id] >= 0 ? 1 : 0;
  }
  for (int o = 16; o > 0; o >>= 1) {
    hits += __shfl_xor_sync(0xffffffffu, hits, o);
    valid += __shfl_xor_sync(0xffffffffu, valid, o);
  }
  if ((threadIdx.x & 31) == 0) { atomicAdd(&counts[0], hits); atomicAdd(&counts[1], valid); }
}

// ---------------------------------------------------------------------------------------------
// Presence-bitmap ring: the bucket-ring policy with hierarchical bitmaps (ulc/presence_bitmap.h,
// the code the CPU oracle runs), replayed by one thread.  `ring` lives in global memory; `bits`
// holds kPresenceBuckets bitmaps of presence_words(capacity) words, `inverse` one entry per slot.
// state[0] = free-stack height, state[1] = 1 once the ring is initialised.
__global__ void presence_ring_step_kernel(PresenceRing* ring, uint32_t* bits, int16_t* inverse, int capacity,
                                          int32_t* dir, int id_space, int32_t* id_of, int32_t* free_stack, int32_t* state,
                                          const int32_t* ids, int n, int32_t* evicted, int32_t* counts,
                                          int32_t* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (state[1] == 0) {            // `bits` arrives zeroed
    ring->init(bits, inverse, capacity);
    state[1] = 1;
  }
  ring->advance();
  int nfree = state[0];
  int hits = 0, misses = 0, ev = 0, overflow = 0;
  for (int i = 0; i < n; ++i) {
    const int id = ids[i];
    if (id < 0 || id >= id_space) {      // reported, never dereferenced
      report(status, kErrBounds, id);
      continue;
    }
    int s = dir[id];
    if (s >= 0) {
      ++hits;
      ring->touch(s);
      continue;
    }
    ++misses;
    if (nfree > 0) {
      s = free_stack[--nfree];
    } else {
      s = ring->victim();
      if (s >= 0) {
        evicted[ev++] = id_of[s];
        dir[id_of[s]] = -1;
        ring->detach(s);
      }
    }
    if (s < 0) { ++overflow; continue; }
    id_of[s] = id;
    dir[id] = s;
    ring->touch(s);
  }
  state[0] = nfree;
  counts[0] = hits; counts[1] = misses; counts[2] = ev; counts[3] = overflow;
}

}  // namespace ulc

extern "C" {
using namespace ulc;

int ulc_ablate_exact_lru_victims(const int32_t* stamps, const int32_t* id_of, int n_slots, int cur_epoch, int need,
                                 int32_t* out_slots, int32_t* out_count, cudaStream_t stream) {
  if (n_slots <= 0 || need < 0) return -kErrUnsupported;
  exact_lru_victims_kernel<<<1, 1024, 0, stream>>>(stamps, id_of, n_slots, cur_epoch, need, out_slots, out_count);
  return static_cast<int>(cudaGetLastError());
}

int ulc_ablate_linked_lru_step(int32_t* dir, int32_t* id_of, int32_t* stamp, int32_t* next, int32_t* prev,
                               int32_t* list, int32_t* free_stack, const int32_t* ids, int n, int32_t* evicted,
                               int32_t* counts, cudaStream_t stream) {
  linked_lru_step_kernel<<<1, 32, 0, stream>>>(dir, id_of, stamp, next, prev, list, free_stack, ids, n, evicted, counts);
  return static_cast<int>(cudaGetLastError());
}

int ulc_ablate_hot_buffer_step(int32_t* tags, int32_t* stamps, int requests, int width, const int32_t* ids,
                               const int32_t* row_offs, int epoch, int32_t* counts, cudaStream_t stream) {
  if (requests <= 0) return 0;
  hot_buffer_step_kernel<<<requests, 256, 0, stream>>>(tags, stamps, width, ids, row_offs, epoch, counts);
  return static_cast<int>(cudaGetLastError());
}

// Bytes of the ring object and words of its bitmaps, for the caller's allocations.
long long ulc_presence_ring_bytes() { return static_cast<long long>(sizeof(ulc::PresenceRing)); }
long long ulc_presence_ring_words(int capacity) {
  return static_cast<long long>(ulc::kPresenceBuckets) * ulc::presence_words(capacity);
}

int ulc_ablate_presence_ring_step(void* ring, uint32_t* bits, int16_t* inverse, int capacity, int32_t* dir, int id_space,
                                  int32_t* id_of, int32_t* free_stack, int32_t* state, const int32_t* ids, int n,
                                  int32_t* evicted, int32_t* counts, int32_t* status, cudaStream_t stream) {
  if (capacity <= 0 || id_space <= 0) return -ulc::kErrUnsupported;
  ulc::presence_ring_step_kernel<<<1, 32, 0, stream>>>(static_cast<ulc::PresenceRing*>(ring), bits, inverse, capacity,
                                                        dir, id_space, id_of, free_stack, state, ids, n, evicted, counts,
                                                        status);
  return static_cast<int>(cudaGetLastError());
}

int ulc_trace_hits(const int32_t* dir, int dir_len, const int32_t* sel, long long n, unsigned long long* counts,
                   cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 296) blocks = 296;
  trace_hits_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(dir, dir_len, sel, n, counts);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
