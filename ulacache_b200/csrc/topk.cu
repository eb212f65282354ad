// Radix-select top-k (k <= 2048) over rows of fp32 scores.
//
// Selection works on an order-preserving 32-bit key of the score and proceeds in four steps,
// all of them over keys that stay in shared memory when the row is short enough (every pass is
// then a short rolled loop: between two launches of a decode step the instruction lines of a
// kernel fall out of L2, so the hot path is kept to a few hundred instructions):
//
//  1. FILTER.  Shared-memory atomics are the scarce resource of a histogram (one lane per
//     clock), so most elements must never reach one.  A warp sorts 32 sampled keys, eight of them
//     become candidate cut-offs, every thread counts its keys against the eight (compare + add,
//     no atomics) and the CTA keeps the highest cut-off that still leaves it 1.5 x its share of
//     k elements.  Typically 5 - 15 % of a row passes.
//  2. HISTOGRAM of the survivors over 2048 bins of a WINDOWED key: sign, five exponent bits
//     covering 2^-15 .. 2^16 (everything outside is clamped into the end bins) and five mantissa
//     bits, i.e. 32 bins per octave where scores live.  The CTAs of a cluster add their non-empty
//     bins into every CTA's copy of the row histogram through distributed shared memory; the
//     histogram is exact from the highest filter bin of the cluster upwards, and the scan for the
//     k-th element only looks there.  (If it does not find it - a sample that misjudged the row -
//     the step is redone without a filter.)  A threshold bin with more elements than the
//     candidate store gets a second 2048-bin level inside it.
//  3. EMIT.  Keys above the threshold go straight from registers to the output; every warp claims
//     its range with one atomic, every CTA its range from CTA 0 with one remote atomic.  Keys of
//     the threshold bin are parked in CTA 0's shared memory.
//  4. RESOLVE the threshold bin in CTA 0: with few candidates, a candidate is selected iff fewer
//     than the missing number of candidates beat it (counted by all threads); crowded bins take
//     radix levels over the 64-bit composite of key and position.
//
// Ties at the k-th value go to the lowest position, so the selected SET is deterministic (the
// order inside a row is not).
//
// Launch shape: a cluster of CS (1, 2, 4 or 8) CTAs of 512 threads per row.  Blocks of 512
// consecutive elements are dealt to the CTAs of a cluster in turn; a CTA keeps up to 32 blocks of
// keys in shared memory, so rows up to CS * 512 * 32 elements are read from memory once.
// Distributed shared memory is ordinary ld / st / red / atom on shared::cluster addresses; no
// bulk copy is involved.
//
// Options: per-row lengths, candidate-list input (scores + explicit indices, used for the
// cross-rank merge), an index transform through a table or a page table (position -> logical
// record ID).
//
// Reference counterpart: ulacache/csrc/indexer/topk_v2.cuh:464 (fp16-derived 12 / 10-bit coarse
// histogram of every element, second pass re-reads the row, tie buffer; persistent cluster pool at
// :547).
#include "ulc/launch.h"
#include "ulc/ptx.cuh"
#include "ulc/topk_key.cuh"

namespace ulc {

constexpr int kTopkThreads = 512;
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kTopkCand = 2048;      // shared-memory candidate slots (elements of the threshold bin)
constexpr int kTopkRankMax = 512;    // up to this many candidates are resolved by rank counting
constexpr int kTopkMaxCluster = 8;
constexpr int kTopkFilters = 8;      // candidate cut-offs of the filter step
constexpr uint64_t kNoKey = 1ull << 32;   // "above every key"
// ranks of the sorted sample tried as cut-offs, relative to the expected one
__constant__ float kTopkRankSpread[kTopkFilters] = {0.6f, 0.85f, 1.15f, 1.5f, 2.f, 3.f, 4.5f, 8.f};

struct TopkShared {
  uint32_t hist[kTopkBins];      // this CTA's survivors (level 1, then level 2)
  uint32_t sum[kTopkBins];       // cluster launch: the row, level 1
  uint32_t sum2[kTopkBins];      // cluster launch: the row, level 2 (inside the threshold bin)
  uint32_t cand_key[kTopkCand];  // CTA 0: the threshold bin's elements
  int32_t cand_pos[kTopkCand];
  uint32_t warp_sums[32];
  uint32_t sample[32];
  uint32_t filt_key[kTopkFilters];
  uint32_t filt_count[kTopkFilters];
  uint32_t filt_bin[kTopkMaxCluster];   // filter bin of every CTA of the cluster (written by the peers)
  uint32_t out_count;            // CTA 0: output slots handed out
  uint32_t cand_count;           // CTA 0: candidate slots handed out
  uint32_t local_emit, local_park;
  uint32_t emit_base, park_base;
  uint32_t thr_bin, thr_above, thr_count;
};

// Optional phase timeline of CTA 0 (row 0), compiled in with -DULC_TOPK_TRACE (development only):
// topk_trace[event] = clock64 at that point.
#ifdef ULC_TOPK_TRACE
__device__ long long topk_trace[16];
#define TOPK_T(ev)                                                          \
  do {                                                                      \
    if (blockIdx.x == 0 && threadIdx.x == 0) topk_trace[ev] = clock64();    \
  } while (0)
#else
#define TOPK_T(ev) do {} while (0)
#endif

// ---- distributed shared memory (cluster launch only) ------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dsm_addr(const void* local, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(ptx::smem_u32(local)), "r"(cta));
  return r;
}
__device__ __forceinline__ void dsm_store(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t dsm_atomic_add(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void dsm_add(uint32_t addr, uint32_t v) {
  asm volatile("red.shared::cluster.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// The two halves of the cluster barrier, for work that can go between them.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Hardware barrier over every thread of the cluster; orders shared-memory traffic cluster-wide.
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Find bin d >= floor_bin (scanning from the top bin down) where the running count first reaches
// `need`; thr_above = number of elements in bins above d, thr_count = elements in d.  Bins below
// `floor_bin` are ignored; returns false when the bins from floor_bin up hold fewer than `need`.
template <int NB>
__device__ __forceinline__ bool find_threshold(TopkShared& s, const uint32_t* hist, uint32_t need,
                                               uint32_t floor_bin = 0) {
  constexpr int PER = (NB + kTopkThreads - 1) / kTopkThreads;
  const int t = threadIdx.x;
  uint32_t local[PER];
  uint32_t sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int rev = t * PER + j;   // position counted from the top
    local[j] = (rev < NB && static_cast<uint32_t>(NB - 1 - rev) >= floor_bin) ? hist[NB - 1 - rev] : 0;
    sum += local[j];
  }
  if (t == 0) s.thr_bin = 0xffffffffu;
  // exclusive block scan of `sum`
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if ((t & 31) >= o) incl += v;
  }
  if ((t & 31) == 31) s.warp_sums[t >> 5] = incl;
  __syncthreads();
  if (t < 32) {
    uint32_t w = t < kTopkWarps ? s.warp_sums[t] : 0u;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, w, o);
      if (t >= o) w += v;
    }
    s.warp_sums[t] = w;
  }
  __syncthreads();
  uint32_t before = incl - sum + ((t >> 5) ? s.warp_sums[(t >> 5) - 1] : 0);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int rev = t * PER + j;
    if (rev < NB && before < need && before + local[j] >= need) {
      s.thr_bin = NB - 1 - rev;
      s.thr_above = before;
      s.thr_count = local[j];
    }
    before += local[j];
  }
  __syncthreads();
  return s.thr_bin != 0xffffffffu;
}

// How an emitted position becomes the output value.
struct TopkXform {
  const int32_t* in_idx;      // explicit index per score (candidate-list mode), or null
  const int32_t* table;       // direct table applied to the index, or null
  const int32_t* pages;       // page table of this row's request (paged mode), or null
  int ranks, rank;            // paged mode: id = ((pages[v >> 6] * ranks + rank) << 6) | (v & 63)
  int drop_neg_inf;           // emit -1 for scores equal to -inf
};

__device__ __forceinline__ int32_t xform_value(const TopkXform& x, int32_t pos, float score) {
  if (x.drop_neg_inf && score == -INFINITY) return -1;
  int32_t v = x.in_idx ? x.in_idx[pos] : pos;
  if (v < 0) return -1;
  if (x.table) return x.table[v];
  if (x.pages) {
    const int32_t pg = x.pages[v >> 6];
    return pg < 0 ? -1 : (((pg * x.ranks + x.rank) << 6) | (v & 63));
  }
  return v;
}

// Warp-aggregated slot claim: the lanes with `pred` get consecutive slots from one atomic add on a
// counter in this CTA's shared memory.  Every lane of the warp must call it.
__device__ __forceinline__ uint32_t claim_slots(uint32_t* counter, bool pred) {
  const uint32_t m = __ballot_sync(0xffffffffu, pred);
  if (m == 0) return 0xffffffffu;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t leader = __ffs(m) - 1;
  uint32_t base = 0;
  if (lane == leader) base = atomicAdd(counter, static_cast<uint32_t>(__popc(m)));
  base = __shfl_sync(0xffffffffu, base, leader);
  return pred ? base + __popc(m & ((1u << lane) - 1u)) : 0xffffffffu;
}

__device__ __forceinline__ void write_out(int32_t* out_idx, float* out_val, int k, uint32_t at, int32_t pos,
                                          uint32_t key, const TopkXform& x) {
  if (at < static_cast<uint32_t>(k)) {
    const uint32_t u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
    const float score = __uint_as_float(u);
    out_idx[at] = xform_value(x, pos, score);
    if (out_val) out_val[at] = score;
  }
}

__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v) {
  const uint32_t lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t u = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= static_cast<uint32_t>(o)) v += u;
  }
  return v;
}

// Step 4 of the selection, run by one CTA: `need` of the `in_bin` elements with key_cand <= key <
// key_above are still to be selected.  They sit in s.cand_key / s.cand_pos (`parked`) or are
// re-read from the row `x` of `n` elements.  Output slots are claimed from s.out_count.
__device__ __forceinline__ void resolve_threshold_bin(TopkShared& s, const float* x, int n, bool parked, uint32_t in_bin,
                                                      uint32_t need, uint32_t key_cand, uint64_t key_above,
                                                      int32_t* oi, float* ov, int k, const TopkXform& xf) {
  const int t = threadIdx.x;
  const int cn = parked ? static_cast<int>(in_bin) : n;
  auto in_range = [&](uint32_t key) { return key >= key_cand && static_cast<uint64_t>(key) < key_above; };
  if (in_bin == need) {   // the whole threshold bin is selected
    for (int jb = 0; jb < cn; jb += kTopkThreads) {
      const int j = jb + t;
      uint32_t key = 0; int32_t pos = 0;
      bool take = j < cn;
      if (take) {
        if (parked) { key = s.cand_key[j]; pos = s.cand_pos[j]; }
        else { key = order_key(x[j]); pos = j; take = in_range(key); }
      }
      const uint32_t at = claim_slots(&s.out_count, take);
      if (at != 0xffffffffu) write_out(oi, ov, k, at, pos, key, xf);
    }
  } else if (parked && cn <= kTopkRankMax) {
    // Few candidates: a candidate is selected iff fewer than `need` candidates beat it, where
    // "beats" compares the score and then prefers the lower position.  G threads share a candidate.
    int P = 16;
    while (P < cn) P <<= 1;
    const int G = kTopkThreads / P;              // 1 .. 32 consecutive lanes per candidate
    const int j = t / G, g = t % G;
    uint32_t key = 0; int32_t pos = 0;
    uint32_t rank = 0;
    if (j < cn) {
      key = s.cand_key[j]; pos = s.cand_pos[j];
      for (int i = g; i < cn; i += G) {
        const uint32_t ki = s.cand_key[i];
        const int32_t pi = s.cand_pos[i];
        rank += (ki > key || (ki == key && pi < pos)) ? 1u : 0u;
      }
    }
    for (int o = 1; o < G; o <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
    const bool take = j < cn && g == 0 && rank < need;
    const uint32_t at = claim_slots(&s.out_count, take);
    if (at != 0xffffffffu) write_out(oi, ov, k, at, pos, key, xf);
  } else {
    // Radix levels over the 64-bit composite (key, 0xffffffff - position), 11 bits a level,
    // over the parked candidates or (a threshold range too crowded to park) over the row itself.
    uint64_t prefix = 0, mask = 0;
    bool done = false;
    for (int shift = 53; !done; shift -= 11) {
      const int sh = shift < 0 ? 0 : shift;
      const uint32_t nb_mask = shift < 0 ? 0x1ffu : 0x7ffu;   // the last level has 9 bits
      for (int i = t; i < kTopkBins; i += kTopkThreads) s.hist[i] = 0;
      __syncthreads();
      for (int j = t; j < cn; j += kTopkThreads) {
        uint32_t key; int32_t pos;
        if (parked) { key = s.cand_key[j]; pos = s.cand_pos[j]; }
        else { key = order_key(x[j]); pos = j; if (!in_range(key)) continue; }
        const uint64_t comp = (static_cast<uint64_t>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(pos));
        if ((comp & mask) == prefix) atomicAdd(&s.hist[(comp >> sh) & nb_mask], 1u);
      }
      __syncthreads();
      find_threshold<kTopkBins>(s, s.hist, need);
      const uint32_t d = s.thr_bin;
      const uint32_t above = s.thr_above;
      const uint32_t at_d = s.thr_count;
      const bool last = (at_d == need - above) || shift < 0;
      __syncthreads();
      for (int jb = 0; jb < cn; jb += kTopkThreads) {
        const int j = jb + t;
        uint32_t key = 0; int32_t pos = 0;
        bool take = false;
        if (j < cn) {
          if (parked) { key = s.cand_key[j]; pos = s.cand_pos[j]; take = true; }
          else { key = order_key(x[j]); pos = j; take = in_range(key); }
          const uint64_t comp = (static_cast<uint64_t>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(pos));
          const uint32_t dig = (comp >> sh) & nb_mask;
          take = take && (comp & mask) == prefix && (dig > d || (last && dig == d));
        }
        const uint32_t at = claim_slots(&s.out_count, take);
        if (at != 0xffffffffu) write_out(oi, ov, k, at, pos, key, xf);
      }
      prefix |= static_cast<uint64_t>(d) << sh;
      mask |= static_cast<uint64_t>(nb_mask) << sh;
      need -= above;
      done = last;
      __syncthreads();
    }
  }
}

struct TopkArgs {
  const float* scores; long long row_stride;
  const int32_t* lengths; int max_len, k;
  const int32_t* in_idx; long long in_idx_stride;
  const int32_t* xform; long long xform_stride;
  const int32_t* pages; long long pages_stride;
  int rows_per_request, ranks, rank, drop_neg_inf;
  int32_t* out_idx; float* out_val; int32_t* out_count;
};

// CS CTAs per row (a cluster when CS > 1); `cap` blocks of keys fit the dynamic shared memory.
template <int CS>
__global__ void __launch_bounds__(kTopkThreads, 2)
topk_select_kernel(const TopkArgs a, const int cap) {
  __shared__ TopkShared s;
  extern __shared__ uint32_t topk_keys[];          // [cap][512] keys of this CTA's blocks
  const int row = blockIdx.x / CS;
  const uint32_t crank = CS > 1 ? cluster_cta_rank() : 0u;
  const int t = threadIdx.x;
  const uint32_t lane = t & 31;
  const float* x = a.scores + static_cast<size_t>(row) * a.row_stride;
  TopkXform xf;
  xf.in_idx = a.in_idx ? a.in_idx + static_cast<size_t>(row) * a.in_idx_stride : nullptr;
  xf.table = a.xform ? a.xform + static_cast<size_t>(row) * a.xform_stride : nullptr;
  xf.pages = a.pages ? a.pages + static_cast<size_t>(row / a.rows_per_request) * a.pages_stride : nullptr;
  xf.ranks = a.ranks; xf.rank = a.rank; xf.drop_neg_inf = a.drop_neg_inf;
  const int k = a.k;
  int32_t* oi = a.out_idx + static_cast<size_t>(row) * k;
  float* ov = a.out_val ? a.out_val + static_cast<size_t>(row) * k : nullptr;
  const int n = a.lengths ? min(max(a.lengths[row], 0), a.max_len) : a.max_len;

  if (n <= k) {   // the same decision in every CTA of the cluster, before any cluster barrier
    if (crank == 0) {
      for (int i = t; i < k; i += kTopkThreads) {
        oi[i] = i < n ? xform_value(xf, i, x[i]) : -1;
        if (ov) ov[i] = i < n ? x[i] : -INFINITY;
      }
      if (t == 0 && a.out_count) a.out_count[row] = n;
    }
    return;
  }

  TOPK_T(0);
  // Key 0 marks "no element": no float maps to it (order_key sends every NaN to the key of -inf),
  // and it lies below every cut-off used here.
  const uint32_t un = static_cast<uint32_t>(n);
  const uint32_t nblk = (un + kTopkThreads - 1) / kTopkThreads;
  const uint32_t my_blocks = nblk > crank ? (nblk - crank + CS - 1) / CS : 0;
  const uint32_t E = static_cast<uint32_t>(cap);
  const uint32_t chunks = (my_blocks + E - 1) / E;
  const bool cached = chunks <= 1;
  uint32_t* keys = topk_keys + t;                                // keys[j * 512]: key j of this thread
  constexpr uint32_t KS = kTopkThreads;
  auto element = [&](uint32_t chunk, uint32_t j) -> uint32_t {  // row position of key j of `chunk`
    return (crank + (chunk * E + j) * CS) * kTopkThreads + t;
  };
  auto chunk_len = [&](uint32_t chunk) -> uint32_t { return min(E, my_blocks - chunk * E); };
  auto load_chunk = [&](uint32_t chunk) {
    const uint32_t nj = chunk_len(chunk);
#pragma unroll 4
    for (uint32_t j = 0; j < nj; ++j) {
      const uint32_t i = element(chunk, j);
      keys[j * KS] = i < un ? order_key(__ldg(x + i)) : 0u;
    }
  };
  load_chunk(0);

  for (int i = t; i < kTopkBins; i += kTopkThreads) {
    s.hist[i] = 0;
    if constexpr (CS > 1) { s.sum[i] = 0; s.sum2[i] = 0; }
  }
  if (t < kTopkFilters) s.filt_count[t] = 0;
  if (t == 0) { s.out_count = 0; s.cand_count = 0; s.local_emit = 0; s.local_park = 0; }
  // ---- step 1: filter ---------------------------------------------------------------------
  // 32 keys from 32 threads, spread over this CTA's blocks
  if ((t & 15) == 0) s.sample[t >> 4] = my_blocks ? keys[((t >> 4) % chunk_len(0)) * KS] : 0u;
  __syncthreads();
  // The other CTAs add into `sum` of this one: tell them it is cleared.  The wait for their
  // arrival comes after the local passes.
  if constexpr (CS > 1) cluster_arrive();
  TOPK_T(1);
  const uint32_t target = (3u * static_cast<uint32_t>(k) / 2u + CS - 1) / CS + 32u;   // survivors this CTA wants
  const uint32_t n_local = min(my_blocks * kTopkThreads, un);
  const bool filtering = 2u * target < n_local;
  uint32_t filter_key = 1u, filter_bin = 0u;                     // pass everything
  if (filtering) {
    if (t < 32) {
      uint32_t v = s.sample[lane];
#pragma unroll
      for (int kk = 2; kk <= 32; kk <<= 1)
#pragma unroll
        for (int j = kk >> 1; j > 0; j >>= 1) {                  // bitonic sort, descending
          const uint32_t o = __shfl_xor_sync(0xffffffffu, v, j);
          const bool keep_max = ((lane & j) == 0) == ((lane & kk) == 0);
          v = keep_max ? max(v, o) : min(v, o);
        }
      // eight ranks around the one whose cut-off is expected to leave `target` elements
      const float expect = 33.f * static_cast<float>(target) / static_cast<float>(n_local);
      const int c = lane < kTopkFilters ? lane : 0;
      const int r = min(32, max(1, static_cast<int>(ceilf(expect * kTopkRankSpread[c]))));
      const uint32_t cut = __shfl_sync(0xffffffffu, v, r - 1);
      if (lane < kTopkFilters) s.filt_key[lane] = cut == 0u ? 1u : bin_lo_key(window_bin(cut));   // bin aligned
    }
    __syncthreads();
    uint32_t fk[kTopkFilters], cnt[kTopkFilters];
#pragma unroll
    for (int c = 0; c < kTopkFilters; ++c) { fk[c] = s.filt_key[c]; cnt[c] = 0; }
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
      if (chunk > 0) { __syncthreads(); load_chunk(chunk); }
      const uint32_t nj = chunk_len(chunk);
#pragma unroll 1
      for (uint32_t j = 0; j < nj; ++j) {
        const uint32_t key = keys[j * KS];
#pragma unroll
        for (int c = 0; c < kTopkFilters; ++c) cnt[c] += key >= fk[c] ? 1u : 0u;
      }
    }
#pragma unroll
    for (int c = 0; c < kTopkFilters; ++c) {
      const uint32_t w = __reduce_add_sync(0xffffffffu, cnt[c]);
      if (lane == 0 && w) atomicAdd(&s.filt_count[c], w);
    }
    __syncthreads();
#pragma unroll
    for (int c = kTopkFilters - 1; c >= 0; --c)                   // the highest cut-off that leaves enough
      if (s.filt_count[c] >= target) { filter_key = fk[c]; }
    filter_bin = filter_key == 1u ? 0u : window_bin(filter_key);
  }
  TOPK_T(2);

  // ---- step 2: histogram of the survivors, merged over the cluster ---------------------------
  uint32_t b1 = 0, need = 0, in_bin = 0;
  bool first_try = true;
  while (true) {
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
      if (!cached) load_chunk(chunk);
      const uint32_t nj = chunk_len(chunk);
#pragma unroll 1
      for (uint32_t j = 0; j < nj; ++j) {
        const uint32_t key = keys[j * KS];
        if (key >= filter_key) atomicAdd(&s.hist[window_bin(key)], 1u);
      }
    }
    __syncthreads();
    const uint32_t* row_hist = s.hist;
    uint32_t floor_bin = filter_bin;
    if constexpr (CS > 1) {
      if (first_try) cluster_wait();       // every CTA has cleared its sums
      for (int b = t; b < kTopkBins; b += kTopkThreads) {
        const uint32_t c = s.hist[b];
        if (c == 0) continue;              // most bins are empty
#pragma unroll
        for (int r = 0; r < CS; ++r) dsm_add(dsm_addr(&s.sum[b], r), c);
      }
      if (t < CS) dsm_store(dsm_addr(&s.filt_bin[crank], t), filter_bin);
      cluster_barrier();                   // ... and has received everybody's counts
      row_hist = s.sum;
#pragma unroll
      for (int r = 0; r < CS; ++r) floor_bin = max(floor_bin, s.filt_bin[r]);
    }
    // the row histogram is exact from the cluster's highest filter bin upwards
    const bool found = find_threshold<kTopkBins>(s, row_hist, static_cast<uint32_t>(k), floor_bin);
    if (found) break;
    // The filter cut too deep (a sample that misjudged the row): once more with every element.
    // All CTAs of the cluster read the same histogram, so all of them come here together.
    first_try = false;
    filter_key = 1u;
    filter_bin = 0u;
    if constexpr (CS > 1) cluster_barrier();          // nobody still reads the sums
    for (int i = t; i < kTopkBins; i += kTopkThreads) {
      s.hist[i] = 0;
      if constexpr (CS > 1) s.sum[i] = 0;
    }
    __syncthreads();
    if constexpr (CS > 1) cluster_barrier();          // every sum is cleared before anybody adds
  }
  TOPK_T(3);
  b1 = s.thr_bin;
  need = static_cast<uint32_t>(k) - s.thr_above;      // how many of the threshold bin are selected
  in_bin = s.thr_count;
  uint32_t key_cand = bin_lo_key(b1);                                      // candidates: key_cand <= key < key_above
  uint64_t key_above = b1 < 2047u ? bin_lo_key(b1 + 1u) : kNoKey;          // selected outright
  if (in_bin > static_cast<uint32_t>(kTopkCand) && in_bin != need) {
    // A crowded threshold bin (scores packed into a fraction of an octave): a second level of
    // 2048 equal key ranges inside it.
    const uint32_t lo = key_cand;
    const uint32_t width = static_cast<uint32_t>(key_above - lo);          // modulo 2^32 for the top bin; never 0
    const int sh = width - 1u < 2048u ? 0 : (32 - __clz(width - 1u)) - 11;
    for (int i = t; i < kTopkBins; i += kTopkThreads) s.hist[i] = 0;
    __syncthreads();
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
      if (!cached) load_chunk(chunk);
      const uint32_t nj = chunk_len(chunk);
#pragma unroll 1
      for (uint32_t j = 0; j < nj; ++j) {
        const uint32_t key = keys[j * KS];
        if (key >= lo && static_cast<uint64_t>(key) < key_above) atomicAdd(&s.hist[(key - lo) >> sh], 1u);
      }
    }
    __syncthreads();
    const uint32_t* sub_hist = s.hist;
    if constexpr (CS > 1) {
      for (int b = t; b < kTopkBins; b += kTopkThreads) {
        const uint32_t c = s.hist[b];
        if (c == 0) continue;
#pragma unroll
        for (int r = 0; r < CS; ++r) dsm_add(dsm_addr(&s.sum2[b], r), c);
      }
      cluster_barrier();
      sub_hist = s.sum2;
    }
    find_threshold<kTopkBins>(s, sub_hist, need);     // the bin holds at least `need` elements
    const uint32_t b2 = s.thr_bin;
    need -= s.thr_above;
    in_bin = s.thr_count;
    key_cand = lo + (b2 << sh);
    if (b2 < 2047u) key_above = static_cast<uint64_t>(lo) + (static_cast<uint64_t>(b2 + 1u) << sh);
  }
  const bool parked = in_bin <= static_cast<uint32_t>(kTopkCand);
  TOPK_T(4);

  // ---- step 3: emit ------------------------------------------------------------------------------
  {
    uint32_t na = 0, nc = 0;
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
      if (!cached) load_chunk(chunk);
      const uint32_t nj = chunk_len(chunk);
#pragma unroll 1
      for (uint32_t j = 0; j < nj; ++j) {
        const uint32_t key = keys[j * KS];
        const bool above = static_cast<uint64_t>(key) >= key_above;
        na += above ? 1u : 0u;
        nc += (!above && key >= key_cand) ? 1u : 0u;
      }
    }
    if (!parked) nc = 0;
    const uint32_t ia = warp_inclusive_scan(na), ic = warp_inclusive_scan(nc);
    uint32_t wa = 0, wc = 0;
    if (lane == 31) {
      wa = ia ? atomicAdd(&s.local_emit, ia) : 0u;
      wc = ic ? atomicAdd(&s.local_park, ic) : 0u;
    }
    wa = __shfl_sync(0xffffffffu, wa, 31);
    wc = __shfl_sync(0xffffffffu, wc, 31);
    __syncthreads();
    if (t == 0) {
      const uint32_t above = s.local_emit, park = s.local_park;
      if constexpr (CS > 1) {
        s.emit_base = above ? dsm_atomic_add(dsm_addr(&s.out_count, 0), above) : 0u;
        s.park_base = park ? dsm_atomic_add(dsm_addr(&s.cand_count, 0), park) : 0u;
      } else {
        s.emit_base = 0; s.park_base = 0;
        s.out_count = above; s.cand_count = park;
      }
    }
    __syncthreads();
    TOPK_T(5);
    uint32_t pa = s.emit_base + wa + ia - na, pc = s.park_base + wc + ic - nc;
    const uint32_t m_key = CS > 1 ? dsm_addr(&s.cand_key[0], 0) : 0u;
    const uint32_t m_pos = CS > 1 ? dsm_addr(&s.cand_pos[0], 0) : 0u;
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
      if (!cached) load_chunk(chunk);
      const uint32_t nj = chunk_len(chunk);
#pragma unroll 1
      for (uint32_t j = 0; j < nj; ++j) {
        const uint32_t key = keys[j * KS];
        const uint32_t i = element(chunk, j);
        if (static_cast<uint64_t>(key) >= key_above) {
          write_out(oi, ov, k, pa++, static_cast<int32_t>(i), key, xf);
        } else if (parked && key >= key_cand) {
          if (pc < static_cast<uint32_t>(kTopkCand)) {
            if constexpr (CS > 1) {
              dsm_store(m_key + pc * 4u, key);
              dsm_store(m_pos + pc * 4u, i);
            } else {
              s.cand_key[pc] = key;
              s.cand_pos[pc] = static_cast<int32_t>(i);
            }
          }
          ++pc;
        }
      }
    }
  }
  TOPK_T(6);
  if constexpr (CS > 1) {
    // After this barrier nobody reads or writes another CTA's shared memory: CTA 0 finishes alone.
    cluster_barrier();
    if (crank != 0) return;
  } else {
    __syncthreads();
  }
  TOPK_T(7);

  // ---- step 4: resolve the threshold bin (CTA 0) ---------------------------------------------------
  resolve_threshold_bin(s, x, n, parked, in_bin, need, key_cand, key_above, oi, ov, k, xf);
  __syncthreads();
  TOPK_T(8);
  if (t == 0 && a.out_count) a.out_count[row] = min(static_cast<uint32_t>(k), s.out_count);
}


// ---- selection from a row histogram that already exists in global memory ------------------------
//
// When the histogram of a row is built somewhere else - by `topk_hist_kernel` below, or by the
// index-score kernel in its epilogue, which sees every score anyway - selection needs no
// communication between the CTAs that share a row: each reads the 2048 counts, finds the threshold
// bin itself, and claims output slots per warp from a counter in global memory.  The last CTA of a
// row to finish (a ticket) resolves the threshold bin and puts the workspace back to zero, so the
// next launch can use it as it is.
//
// Workspace (device memory, zero when first used), per row:
//   [0, 8192)        uint32 hist[2048]
//   [8192, 8208)     uint32 emitted, parked, ticket, valid row length (written by the histogram's producer)
//   [8448, 16640)    uint32 cand_key[2048]
//   [16640, 24832)   int32  cand_pos[2048]
struct TopkWsArgs {
  TopkArgs a;
  uint32_t* ws;
  int splits;          // CTAs per row
  int len_from_ws;     // row length = ws counter 3 (set by the producer of the histogram) instead of lengths / max_len
};

__global__ void __launch_bounds__(kTopkThreads)
topk_hist_kernel(const TopkWsArgs w) {
  __shared__ uint32_t hist[kTopkBins];
  const int row = blockIdx.y, t = threadIdx.x;
  const TopkArgs& a = w.a;
  const float* x = a.scores + static_cast<size_t>(row) * a.row_stride;
  const int n = a.lengths ? min(max(a.lengths[row], 0), a.max_len) : a.max_len;
  if (n <= a.k) return;                  // the select kernel copies such a row; it reads no histogram
  for (int i = t; i < kTopkBins; i += kTopkThreads) hist[i] = 0;
  __syncthreads();
  for (uint32_t i = blockIdx.x * kTopkThreads + t; i < static_cast<uint32_t>(n); i += gridDim.x * kTopkThreads)
    atomicAdd(&hist[window_bin(order_key(__ldg(x + i)))], 1u);
  __syncthreads();
  uint32_t* g = w.ws + static_cast<size_t>(row) * (kTopkWsRowBytes / 4);
  for (int b = t; b < kTopkBins; b += kTopkThreads) {
    const uint32_t c = hist[b];
    if (c) atomicAdd(g + b, c);
  }
}

__global__ void __launch_bounds__(kTopkThreads, 2)
topk_select_from_hist_kernel(const TopkWsArgs w) {
  __shared__ TopkShared s;
  __shared__ int s_last;
  const TopkArgs& a = w.a;
  const int row = blockIdx.y, t = threadIdx.x;
  const uint32_t lane = t & 31;
  const uint32_t S = gridDim.x, part = blockIdx.x;
  uint32_t* g = w.ws + static_cast<size_t>(row) * (kTopkWsRowBytes / 4);
  uint32_t* ctr = g + kTopkWsCtr;
  const float* x = a.scores + static_cast<size_t>(row) * a.row_stride;
  TopkXform xf;
  xf.in_idx = a.in_idx ? a.in_idx + static_cast<size_t>(row) * a.in_idx_stride : nullptr;
  xf.table = a.xform ? a.xform + static_cast<size_t>(row) * a.xform_stride : nullptr;
  xf.pages = a.pages ? a.pages + static_cast<size_t>(row / a.rows_per_request) * a.pages_stride : nullptr;
  xf.ranks = a.ranks; xf.rank = a.rank; xf.drop_neg_inf = a.drop_neg_inf;
  const int k = a.k;
  int32_t* oi = a.out_idx + static_cast<size_t>(row) * k;
  float* ov = a.out_val ? a.out_val + static_cast<size_t>(row) * k : nullptr;
  int n = a.max_len;
  if (w.len_from_ws) n = min(static_cast<int>(__ldcg(ctr + 3)), a.max_len);
  else if (a.lengths) n = min(max(a.lengths[row], 0), a.max_len);

  if (n <= k) {
    // short row: everything is selected.  A producer that builds histograms does so for every row,
    // so the row's workspace still goes back to zero.
    if (part == 0) {
      for (int i = t; i < k; i += kTopkThreads) {
        oi[i] = i < n ? xform_value(xf, i, x[i]) : -1;
        if (ov) ov[i] = i < n ? x[i] : -INFINITY;
      }
      if (t == 0 && a.out_count) a.out_count[row] = n;
      if (w.len_from_ws) {
        for (int i = t; i < kTopkBins; i += kTopkThreads) g[i] = 0;
        if (t < 4) ctr[t] = 0;
      }
    }
    return;
  }

  find_threshold<kTopkBins>(s, g, static_cast<uint32_t>(k));
  const uint32_t b1 = s.thr_bin;
  const uint32_t need = static_cast<uint32_t>(k) - s.thr_above;
  const uint32_t in_bin = s.thr_count;
  const uint32_t key_cand = bin_lo_key(b1);
  const uint64_t key_above = b1 < 2047u ? bin_lo_key(b1 + 1u) : kNoKey;
  const bool parked = in_bin <= static_cast<uint32_t>(kTopkCand);

  // this CTA's blocks of the row: part, part + S, ...; eight loads per thread are in flight at once,
  // and a row short enough for one such round (the usual case) is read from memory once
  const uint32_t un = static_cast<uint32_t>(n);
  const uint32_t stride = S * kTopkThreads;
  const uint32_t first = part * kTopkThreads + t;
  const bool single = first + 8u * stride >= un || stride * 8u >= un;
  uint32_t keys[8];
  auto load8 = [&](uint32_t base) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t i = base + j * stride;
      keys[j] = i < un ? order_key(__ldg(x + i)) : 0u;
    }
  };
  uint32_t na = 0, nc = 0;
  for (uint32_t base = first; base < un; base += 8u * stride) {
    load8(base);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool above = static_cast<uint64_t>(keys[j]) >= key_above;
      na += above ? 1u : 0u;
      nc += (!above && keys[j] >= key_cand) ? 1u : 0u;
    }
  }
  if (!parked) nc = 0;
  const uint32_t ia = warp_inclusive_scan(na), ic = warp_inclusive_scan(nc);
  uint32_t wa = 0, wc = 0;
  if (lane == 31) {                                   // one claim per warp, straight from the row's counters
    wa = ia ? atomicAdd(ctr + 0, ia) : 0u;
    wc = ic ? atomicAdd(ctr + 1, ic) : 0u;
  }
  uint32_t pa = __shfl_sync(0xffffffffu, wa, 31) + ia - na;
  uint32_t pc = __shfl_sync(0xffffffffu, wc, 31) + ic - nc;
  for (uint32_t base = first; base < un; base += 8u * stride) {
    if (!single) load8(base);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t key = keys[j];
      const uint32_t i = base + j * stride;
      if (static_cast<uint64_t>(key) >= key_above) {
        write_out(oi, ov, k, pa++, static_cast<int32_t>(i), key, xf);
      } else if (parked && key >= key_cand) {
        if (pc < static_cast<uint32_t>(kTopkCand)) {
          g[kTopkWsKey + pc] = key;
          g[kTopkWsPos + pc] = i;
        }
        ++pc;
      }
    }
  }
  // ticket: the last CTA of the row to get here finishes it
  __threadfence();
  __syncthreads();
  if (t == 0) s_last = atomicAdd(ctr + 2, 1u) == S - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (t == 0) s.out_count = __ldcg(ctr + 0);
  if (parked)
    for (uint32_t i = t; i < in_bin; i += kTopkThreads) {
      s.cand_key[i] = __ldcg(g + kTopkWsKey + i);
      s.cand_pos[i] = static_cast<int32_t>(__ldcg(g + kTopkWsPos + i));
    }
  __syncthreads();
  resolve_threshold_bin(s, x, n, parked, in_bin, need, key_cand, key_above, oi, ov, k, xf);
  __syncthreads();
  if (t == 0 && a.out_count) a.out_count[row] = min(static_cast<uint32_t>(k), s.out_count);
  for (int i = t; i < kTopkBins; i += kTopkThreads) g[i] = 0;      // leave the workspace as it was found
  if (t < 4) ctr[t] = 0;
}

template <int CS>
static int launch_topk(const TopkArgs& a, int rows, int cap, cudaStream_t stream) {
  static PerDeviceOnce once;
  const int key_bytes = cap * kTopkThreads * 4;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(topk_select_kernel<CS>), 32 * kTopkThreads * 4, once);
  if (rc != 0) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows) * CS);
  cfg.blockDim = dim3(kTopkThreads);
  cfg.dynamicSmemBytes = key_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CS > 1 ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, topk_select_kernel<CS>, a, cap);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Throughput form for MANY rows (prefill chunks, large batches): one CTA per row, no cluster, no
// communication between CTAs, CTAs walk the rows in a grid-stride loop.
//
//  1. 2048 evenly spaced samples of the row go into the 2048-bin windowed histogram; the bin that
//     holds the sample of rank 1.75 k / n * 2048 becomes the filter bin.
//  2. The row is streamed once; elements at or above the filter bin (about 1.75 k of them) are
//     compacted into shared memory with a block scan (no atomics).  Rows of up to 8192 elements skip
//     the filter and keep everything.
//  3. The exact k-th element of the survivors is found by radix levels over the 64-bit composite
//     (key, ~position): 11 + 11 + 10 key bits, then, only when equal keys straddle the cut,
//     11 + 11 + 10 position bits.  A level stops the search as soon as its threshold bin holds exactly
//     the number of elements still wanted.  Ties therefore go to the lowest position.
//  4. Survivors at or above the threshold composite are written out through a block scan.
//  If a sample misjudged the row (fewer than k survivors) or equal values flood the candidate store,
//  steps 3 and 4 run over the row in global memory instead (same code, another element source).
//
// Two kernels share this code.  `topk_rows_kernel` (512 threads, two CTAs per SM) streams the row from
// global memory, 16 elements per thread and chunk: every chunk is a dependent round trip to memory.
// `topk_rows_staged_kernel` (1024 threads, one CTA per SM, rows of up to 32768 elements that start on a
// 16-byte boundary) brings the WHOLE row into shared memory with 16-byte cp.async copies - one round
// trip, 128 KB in flight per SM - takes samples and survivors from there, and starts the copy of its
// next row as soon as the survivors are compacted, so that the copy runs under steps 3 and 4.
constexpr int kRowsCand = 8192;
constexpr int kRowsSamples = 2048;
constexpr int kRowsPerThread = 16;
constexpr int kRowsStageMax = 32768;       // elements of a row the staged kernel holds in shared memory

struct RowsShared {
  uint32_t cand_key[kRowsCand];
  int32_t cand_pos[kRowsCand];
  uint32_t hist[kTopkBins];
  uint32_t warp_sums[32];
  uint32_t total;
  uint32_t sel_bin, sel_above, sel_count;
};
constexpr int kRowsSmem = static_cast<int>(sizeof(RowsShared));
constexpr int kRowsStagedSmem = kRowsSmem + 16 + kRowsStageMax * 4;

// exclusive scan of one value per thread over the CTA; s.total receives the sum
template <int TH>
__device__ __forceinline__ uint32_t rows_block_scan(uint32_t v, RowsShared& s) {
  constexpr uint32_t kWarps = TH / 32;
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t incl = warp_inclusive_scan(v);
  __syncthreads();                                   // the previous scan's warp_sums / total are done with
  if (lane == 31) s.warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = lane < kWarps ? s.warp_sums[lane] : 0u;
    const uint32_t wi = warp_inclusive_scan(w);
    if (lane < kWarps) s.warp_sums[lane] = wi - w;
    if (lane == kWarps - 1) s.total = wi;
  }
  __syncthreads();
  return s.warp_sums[warp] + incl - v;
}

// Among the bins [0, nb) of s.hist, counted from the TOP: the bin b with
// (elements in bins above b) < need <= (elements in bins >= b).  Results in s.sel_*; s.sel_count = 0 and
// s.sel_bin = nb when the histogram holds fewer than `need` elements.  Every thread calls it.
template <int TH>
__device__ __forceinline__ void rows_find_bin(RowsShared& s, int nb, uint32_t need) {
  const int per = nb / TH;                           // 1, 2 or 4 bins per thread
  const int t = threadIdx.x;
  uint32_t h[4];
  uint32_t sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    h[j] = j < per ? s.hist[nb - 1 - (t * per + j)] : 0u;     // reversed: j-th bin from the top of my range
    sum += h[j];
  }
  if (t == 0) { s.sel_bin = static_cast<uint32_t>(nb); s.sel_above = 0; s.sel_count = 0; }
  uint32_t run = rows_block_scan<TH>(sum, s);        // (its barriers also order the reset above)
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j < per) {
      if (run < need && need <= run + h[j]) {
        s.sel_bin = static_cast<uint32_t>(nb - 1 - (t * per + j));
        s.sel_above = run;
        s.sel_count = h[j];
      }
      run += h[j];
    }
  }
  __syncthreads();
}

// Histogram add of the lanes with `pred`.  Plain shared-memory atomics: aggregating equal bins of a warp first
// (`match.any` + one atomic per distinct bin) measured SLOWER here (10.8 k against 7.3 k cycles for the three
// levels of a 32K row), the match instruction costing more than the conflicts it removes.
__device__ __forceinline__ void rows_hist_add(uint32_t* hist, uint32_t bin, bool pred) {
  if (pred) atomicAdd(&hist[bin], 1u);
}

struct RowsCandSource {
  const RowsShared* s;
  uint32_t n;
  __device__ __forceinline__ uint64_t at(uint32_t i) const {
    return (static_cast<uint64_t>(s->cand_key[i]) << 32) | static_cast<uint32_t>(~s->cand_pos[i]);
  }
};
struct RowsGlobalSource {
  const float* x;
  uint32_t n;
  __device__ __forceinline__ uint64_t at(uint32_t i) const {
    return (static_cast<uint64_t>(order_key(x[i])) << 32) | static_cast<uint32_t>(~i);
  }
};

// Steps 3 and 4 over `src`; exactly k elements are written (src.n > k).
template <int TH, class Source>
__device__ __forceinline__ void rows_select_emit(RowsShared& s, const Source& src, int k, int32_t* oi, float* ov,
                                                 const TopkXform& xf) {
  const int t = threadIdx.x;
  uint64_t prefix = 0, mask = 0;
  uint32_t need = static_cast<uint32_t>(k);
  for (int level = 0; level < 6; ++level) {
    const int shift = level == 0 ? 53 : level == 1 ? 42 : level == 2 ? 32 : level == 3 ? 21 : level == 4 ? 10 : 0;
    const int nb = (level == 2 || level == 5) ? 1024 : 2048;
    for (int i = t; i < nb; i += TH) s.hist[i] = 0;
    __syncthreads();
    for (uint32_t i0 = 0; i0 < src.n; i0 += TH) {
      const uint32_t i = i0 + static_cast<uint32_t>(t);
      const uint64_t c = i < src.n ? src.at(i) : 0ull;
      rows_hist_add(s.hist, static_cast<uint32_t>(c >> shift) & static_cast<uint32_t>(nb - 1), i < src.n && (c & mask) == prefix);
    }
    __syncthreads();
    rows_find_bin<TH>(s, nb, need);
    const uint32_t bin = s.sel_bin, above = s.sel_above, in_bin = s.sel_count;
    __syncthreads();                                 // everyone has read the result before the next level resets it
    need -= above;
    prefix |= static_cast<uint64_t>(bin) << shift;
    mask |= static_cast<uint64_t>(nb - 1) << shift;
    if (in_bin == need) break;                       // everything that matches the prefix is selected
  }
  TOPK_T(4);
  // selected: masked composite >= prefix.  Per-thread counts, one scan, ordered writes.
  constexpr uint32_t kPer = 8;
  uint32_t base = 0;
  for (uint32_t i0 = 0; i0 < src.n; i0 += TH * kPer) {
    uint32_t cnt = 0;
    uint32_t flags = 0;
#pragma unroll
    for (uint32_t j = 0; j < kPer; ++j) {
      const uint32_t i = i0 + j * TH + static_cast<uint32_t>(t);
      if (i < src.n && (src.at(i) & mask) >= prefix) { flags |= 1u << j; ++cnt; }
    }
    uint32_t at = base + rows_block_scan<TH>(cnt, s);
    base += s.total;
#pragma unroll
    for (uint32_t j = 0; j < kPer; ++j) {
      if (flags & (1u << j)) {
        const uint64_t c = src.at(i0 + j * TH + static_cast<uint32_t>(t));
        write_out(oi, ov, k, at++, static_cast<int32_t>(~static_cast<uint32_t>(c)), static_cast<uint32_t>(c >> 32), xf);
      }
    }
  }
}

// Step 1: the filter of a row of n > kRowsCand elements read through `x` (global or shared memory), as a VALUE:
// the lower edge of the filter bin.  Step 2 then costs one float compare per element instead of a key and a bin
// (the kernels are bound by instruction issue, not by memory: 32K elements x ~25 instructions were 18 k cycles).
// Any value works as long as at least k elements pass; -0.0 / +0.0 and NaN only make the survivors a superset
// or send the row to the exact pass over global memory.
template <int TH>
__device__ __forceinline__ float rows_filter_value(RowsShared& s, const float* x, int n, int k) {
  const int t = threadIdx.x;
  for (int i = t; i < kTopkBins; i += TH) s.hist[i] = 0;
  __syncthreads();
  for (int i = t; i < kRowsSamples; i += TH) {
    const int pos = static_cast<int>((static_cast<long long>(i) * n) / kRowsSamples);
    rows_hist_add(s.hist, window_bin(order_key(x[pos])), true);
  }
  __syncthreads();
  TOPK_T(1);
  long long want = (7ll * k * kRowsSamples + 4ll * n - 1) / (4ll * n);          // ceil(1.75 k / n * samples)
  want = want < 8 ? 8 : (want > kRowsSamples / 2 ? kRowsSamples / 2 : want);
  rows_find_bin<TH>(s, kTopkBins, static_cast<uint32_t>(want));
  const uint32_t bin = s.sel_bin < static_cast<uint32_t>(kTopkBins) ? s.sel_bin : 0u;
  __syncthreads();
  if (bin == 0u) return -INFINITY;
  const uint32_t key = bin_lo_key(bin);
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Step 2 over `x` (global or shared memory; `vec`: x is 16-byte aligned).  Returns the number of survivors
// (more than kRowsCand = the store overflowed and holds only a part).
template <int TH>
__device__ __forceinline__ uint32_t rows_compact(RowsShared& s, const float* x, int n, bool vec, float pivot) {
  const int t = threadIdx.x;
  uint32_t base = 0;
  for (int c0 = 0; c0 < n; c0 += TH * kRowsPerThread) {
    float v[kRowsPerThread];
#pragma unroll
    for (int j = 0; j < kRowsPerThread / 4; ++j) {
      const int i = c0 + (j * TH + t) * 4;
      if (vec && i + 3 < n) {
        const float4 q = *reinterpret_cast<const float4*>(x + i);
        v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[4 * j + e] = i + e < n ? x[i + e] : 0.f;
      }
    }
    uint32_t flags = 0, cnt = 0;
#pragma unroll
    for (int j = 0; j < kRowsPerThread; ++j) {
      const int i = c0 + ((j >> 2) * TH + t) * 4 + (j & 3);
      if (i < n && v[j] >= pivot) { flags |= 1u << j; ++cnt; }
    }
    uint32_t at = base + rows_block_scan<TH>(cnt, s);
    base += s.total;
#pragma unroll
    for (int j = 0; j < kRowsPerThread; ++j) {
      if (flags & (1u << j)) {
        if (at < static_cast<uint32_t>(kRowsCand)) {
          s.cand_key[at] = order_key(v[j]);
          s.cand_pos[at] = c0 + ((j >> 2) * TH + t) * 4 + (j & 3);
        }
        ++at;
      }
    }
    if (base > static_cast<uint32_t>(kRowsCand)) break;      // (uniform: base is the same in every thread)
  }
  __syncthreads();
  return base;
}

struct RowsRow {
  const float* x;
  TopkXform xf;
  int32_t* oi;
  float* ov;
  int n;
};

__device__ __forceinline__ RowsRow rows_row(const TopkArgs& a, int row) {
  RowsRow r;
  r.x = a.scores + static_cast<size_t>(row) * a.row_stride;
  r.xf.in_idx = a.in_idx ? a.in_idx + static_cast<size_t>(row) * a.in_idx_stride : nullptr;
  r.xf.table = a.xform ? a.xform + static_cast<size_t>(row) * a.xform_stride : nullptr;
  r.xf.pages = a.pages ? a.pages + static_cast<size_t>(row / a.rows_per_request) * a.pages_stride : nullptr;
  r.xf.ranks = a.ranks; r.xf.rank = a.rank; r.xf.drop_neg_inf = a.drop_neg_inf;
  r.oi = a.out_idx + static_cast<size_t>(row) * a.k;
  r.ov = a.out_val ? a.out_val + static_cast<size_t>(row) * a.k : nullptr;
  r.n = a.lengths ? min(max(a.lengths[row], 0), a.max_len) : a.max_len;
  return r;
}

template <int TH>
__device__ __forceinline__ void rows_trivial(const RowsRow& r, int k) {
  for (int i = threadIdx.x; i < k; i += TH) {
    r.oi[i] = i < r.n ? xform_value(r.xf, i, r.x[i]) : -1;
    if (r.ov) r.ov[i] = i < r.n ? r.x[i] : -INFINITY;
  }
}

__global__ void __launch_bounds__(512, 2)
topk_rows_kernel(const TopkArgs a, const int rows) {
  constexpr int TH = 512;
  extern __shared__ __align__(16) uint8_t rows_smem_raw[];
  RowsShared& s = *reinterpret_cast<RowsShared*>(rows_smem_raw);
  const int k = a.k;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const RowsRow r = rows_row(a, row);
    TOPK_T(0);
    if (threadIdx.x == 0 && a.out_count) a.out_count[row] = min(r.n, k);
    if (r.n <= k) { rows_trivial<TH>(r, k); continue; }
    const float pivot = r.n > kRowsCand ? rows_filter_value<TH>(s, r.x, r.n, k) : -INFINITY;
    TOPK_T(2);
    const uint32_t got = rows_compact<TH>(s, r.x, r.n, (reinterpret_cast<uintptr_t>(r.x) & 15) == 0, pivot);
    TOPK_T(3);
    if (got <= static_cast<uint32_t>(kRowsCand) && got >= static_cast<uint32_t>(k)) {
      RowsCandSource src{&s, got};
      rows_select_emit<TH>(s, src, k, r.oi, r.ov, r.xf);
    } else {
      RowsGlobalSource src{r.x, static_cast<uint32_t>(r.n)};
      rows_select_emit<TH>(s, src, k, r.oi, r.ov, r.xf);
    }
    __syncthreads();                                 // the candidate store is free for the next row
    TOPK_T(5);
  }
}

// whole row -> shared memory: 16-byte asynchronous copies, the last one shortened to the row's end
template <int TH>
__device__ __forceinline__ void rows_stage(float* buf, const float* x, int n) {
  const int vecs = (n + 3) >> 2;
  for (int i = threadIdx.x; i < vecs; i += TH) {
    const int rem = n - 4 * i;
    ptx::cp_async16_partial(buf + 4 * i, x + 4 * i, rem >= 4 ? 16 : rem * 4);
  }
  ptx::cp_async_commit();
}

__device__ __forceinline__ bool rows_stageable(const RowsRow& r, int k) {
  return r.n > k && r.n <= kRowsStageMax && (reinterpret_cast<uintptr_t>(r.x) & 15) == 0;
}

__global__ void __launch_bounds__(1024, 1)
topk_rows_staged_kernel(const TopkArgs a, const int rows) {
  constexpr int TH = 1024;
  extern __shared__ __align__(16) uint8_t rows_smem_raw[];
  RowsShared& s = *reinterpret_cast<RowsShared*>(rows_smem_raw);
  float* buf = reinterpret_cast<float*>(rows_smem_raw + ((kRowsSmem + 15) & ~15));
  const int k = a.k;
  int row = blockIdx.x;
  if (row >= rows) return;
  RowsRow r = rows_row(a, row);
  bool staged = rows_stageable(r, k);
  if (staged) rows_stage<TH>(buf, r.x, r.n);
  for (;;) {
    const int next = row + static_cast<int>(gridDim.x);
    RowsRow rn = r;
    bool staged_next = false;
    if (next < rows) { rn = rows_row(a, next); staged_next = rows_stageable(rn, k); }
    TOPK_T(0);
    if (threadIdx.x == 0 && a.out_count) a.out_count[row] = min(r.n, k);
    if (r.n <= k) {
      rows_trivial<TH>(r, k);
      if (staged_next) rows_stage<TH>(buf, rn.x, rn.n);          // nothing of this row sits in the buffer
    } else {
      const float* x = r.x;
      bool vec = (reinterpret_cast<uintptr_t>(r.x) & 15) == 0;
      if (staged) {
        ptx::cp_async_wait<0>();
        __syncthreads();
        x = buf;
        vec = true;
      }
      const float pivot = r.n > kRowsCand ? rows_filter_value<TH>(s, x, r.n, k) : -INFINITY;
      TOPK_T(2);
      const uint32_t got = rows_compact<TH>(s, x, r.n, vec, pivot);           // ends with a barrier: the buffer is free
      TOPK_T(3);
      if (staged_next) rows_stage<TH>(buf, rn.x, rn.n);          // runs under the selection below
      if (got <= static_cast<uint32_t>(kRowsCand) && got >= static_cast<uint32_t>(k)) {
        RowsCandSource src{&s, got};
        rows_select_emit<TH>(s, src, k, r.oi, r.ov, r.xf);
      } else {
        RowsGlobalSource src{r.x, static_cast<uint32_t>(r.n)};
        rows_select_emit<TH>(s, src, k, r.oi, r.ov, r.xf);
      }
      __syncthreads();                               // the candidate store is free for the next row
    }
    TOPK_T(5);
    if (next >= rows) break;
    row = next; r = rn; staged = staged_next;
  }
}

static int launch_topk_rows(const TopkArgs& a, int rows, bool staged, cudaStream_t stream) {
  static PerDeviceOnce once, once_staged;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (staged) {
    int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(topk_rows_staged_kernel), kRowsStagedSmem, once_staged);
    if (rc != 0) return rc;
    const int grid = rows < sms ? rows : sms;
    topk_rows_staged_kernel<<<grid, 1024, kRowsStagedSmem, stream>>>(a, rows);
    return static_cast<int>(cudaGetLastError());
  }
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(topk_rows_kernel), kRowsSmem, once);
  if (rc != 0) return rc;
  const int grid = rows < 2 * sms ? rows : 2 * sms;
  topk_rows_kernel<<<grid, 512, kRowsSmem, stream>>>(a, rows);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ulc

static int g_topk_mode = 0;
constexpr int kTopkManyRows = 48;   // rows from which the throughput kernel is taken

extern "C" {

// scores [rows, row_stride] fp32; lengths (nullable) per-row valid length <= max_len.
// in_idx (nullable): explicit index per score (candidate-list mode).
// xform (nullable): table applied to every emitted index (value < 0 stays -1).
// out_idx [rows, k] int32 (padding -1), out_val (nullable) [rows, k] fp32,
// out_count (nullable) [rows].
int ulc_topk(const float* scores, long long row_stride, const int32_t* lengths, int rows, int max_len,
             int k, const int32_t* in_idx, long long in_idx_stride, const int32_t* xform,
             long long xform_stride, int32_t* out_idx, float* out_val, int32_t* out_count,
             cudaStream_t stream);

// Full form.  pages (nullable) [requests, pages_stride]: paged transform, row r belongs to request
// r / rows_per_request and an emitted column v becomes ((pages[v >> 6] * ranks + rank) << 6) | (v & 63).
// drop_neg_inf: entries whose score is -inf are emitted as -1.
int ulc_topk_ex(const float* scores, long long row_stride, const int32_t* lengths, int rows, int max_len,
                int k, const int32_t* in_idx, long long in_idx_stride, const int32_t* xform,
                long long xform_stride, const int32_t* pages, long long pages_stride, int rows_per_request,
                int ranks, int rank, int drop_neg_inf, int32_t* out_idx, float* out_val, int32_t* out_count,
                cudaStream_t stream) {
  using namespace ulc;
  if (rows <= 0) return 0;
  if (k <= 0 || k > 2048 || max_len < 0) return -kErrUnsupported;
  if (rows_per_request < 1) rows_per_request = 1;
  TopkArgs a;
  a.scores = scores; a.row_stride = row_stride; a.lengths = lengths; a.max_len = max_len; a.k = k;
  a.in_idx = in_idx; a.in_idx_stride = in_idx_stride; a.xform = xform; a.xform_stride = xform_stride;
  a.pages = pages; a.pages_stride = pages_stride; a.rows_per_request = rows_per_request;
  a.ranks = ranks; a.rank = rank; a.drop_neg_inf = drop_neg_inf;
  a.out_idx = out_idx; a.out_val = out_val; a.out_count = out_count;
  // CTAs per row: enough that a row's keys stay in shared memory with two CTAs per SM (16 blocks
  // each), then more while the launch still fits the machine in one wave.
  // mode: 0 = choose, 1 = one CTA per row, 2 = a cluster of eight per row.
  const int mode = g_topk_mode;
  // many rows: the one-CTA-per-row throughput kernels
  // (mode 3 / 4 force its streaming / staged form, any other explicit mode keeps it off)
  if (mode == 3 || mode == 4 || (mode == 0 && rows >= kTopkManyRows && max_len > 2 * k)) {
    // staged: one CTA per SM, so it pays while every row has an SM of its own; beyond that two streaming CTAs
    // per SM overlap each other's phases (measured: 20.6 against 22.9 us at 128 rows, 37.8 against 30.9 at 256)
    const bool staged = mode == 4 || (mode == 0 && max_len <= kRowsStageMax && rows <= 148);
    return launch_topk_rows(a, rows, staged, stream);
  }
  int cs = 1;
  while (cs < kTopkMaxCluster && static_cast<long long>(cs) * kTopkThreads * 16 < max_len) cs *= 2;
  while (cs < kTopkMaxCluster && static_cast<long long>(rows) * cs * 2 <= 2 * 148) cs *= 2;
  if (max_len <= 2 * k) cs = 1;       // short candidate lists: one CTA, nothing to share
  if (mode == 1) cs = 1;
  if (mode == 2) cs = kTopkMaxCluster;
  if (mode == 12 || mode == 14) cs = mode - 10;     // (measurements: a forced cluster of two / four)
  // blocks of keys a CTA holds in shared memory: its whole share of the row when that is at most 32
  long long cap = (static_cast<long long>(max_len) + cs * kTopkThreads - 1) / (cs * kTopkThreads);
  cap = cap < 1 ? 1 : (cap > 32 ? 32 : cap);
  switch (cs) {
    case 1: return launch_topk<1>(a, rows, static_cast<int>(cap), stream);
    case 2: return launch_topk<2>(a, rows, static_cast<int>(cap), stream);
    case 4: return launch_topk<4>(a, rows, static_cast<int>(cap), stream);
    default: return launch_topk<8>(a, rows, static_cast<int>(cap), stream);
  }
}


// Bytes of workspace `ulc_topk_ws` needs for `rows` rows.  The memory must be zero the first time it
// is used; every call leaves it zero again.  Calls that share a workspace must not overlap on the GPU.
long long ulc_topk_workspace_bytes(int rows) { return static_cast<long long>(rows) * ulc::kTopkWsRowBytes; }

// As ulc_topk_ex, in two launches without clusters: a histogram kernel, then a selection kernel in
// which the CTAs of a row do not communicate (see topk_select_from_hist_kernel).
//   hist_ready = 1: the row histograms are already in the workspace (built by ulc_index_score with
//   its `topk_ws` argument) together with every row's valid length; `lengths` is then ignored.
int ulc_topk_ws(const float* scores, long long row_stride, const int32_t* lengths, int rows, int max_len,
                int k, const int32_t* in_idx, long long in_idx_stride, const int32_t* xform,
                long long xform_stride, const int32_t* pages, long long pages_stride, int rows_per_request,
                int ranks, int rank, int drop_neg_inf, int32_t* out_idx, float* out_val, int32_t* out_count,
                void* workspace, int hist_ready, cudaStream_t stream) {
  using namespace ulc;
  if (rows <= 0) return 0;
  if (k <= 0 || k > 2048 || max_len < 0 || workspace == nullptr) return -kErrUnsupported;
  if (rows_per_request < 1) rows_per_request = 1;
  TopkWsArgs w;
  TopkArgs& a = w.a;
  a.scores = scores; a.row_stride = row_stride; a.lengths = lengths; a.max_len = max_len; a.k = k;
  a.in_idx = in_idx; a.in_idx_stride = in_idx_stride; a.xform = xform; a.xform_stride = xform_stride;
  a.pages = pages; a.pages_stride = pages_stride; a.rows_per_request = rows_per_request;
  a.ranks = ranks; a.rank = rank; a.drop_neg_inf = drop_neg_inf;
  a.out_idx = out_idx; a.out_val = out_val; a.out_count = out_count;
  w.ws = reinterpret_cast<uint32_t*>(workspace);
  w.len_from_ws = hist_ready ? 1 : 0;
  // eight elements per thread, but no more CTAs than fill the machine a few times over
  long long per_row = (static_cast<long long>(max_len) + kTopkThreads * 8 - 1) / (kTopkThreads * 8);
  while (per_row > 1 && per_row * rows > 8 * 148) per_row = (per_row + 1) / 2;
  w.splits = static_cast<int>(per_row < 1 ? 1 : per_row);
  const dim3 grid(static_cast<unsigned>(w.splits), static_cast<unsigned>(rows));
  if (!hist_ready) topk_hist_kernel<<<grid, kTopkThreads, 0, stream>>>(w);
  topk_select_from_hist_kernel<<<grid, kTopkThreads, 0, stream>>>(w);
  return static_cast<int>(cudaGetLastError());
}

#ifdef ULC_TOPK_TRACE
int ulc_topk_trace_read(long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, ulc::topk_trace, sizeof(long long) * 16));
}
#endif

// Launch shape override for tests and measurements: 0 = choose by size, 1 = one CTA per row, 2 = a cluster of eight per row,
// 3 = the many-rows throughput kernel (streaming form), 4 = its staged form.
void ulc_topk_set_mode(int mode) { g_topk_mode = mode; }

int ulc_topk(const float* scores, long long row_stride, const int32_t* lengths, int rows, int max_len,
             int k, const int32_t* in_idx, long long in_idx_stride, const int32_t* xform,
             long long xform_stride, int32_t* out_idx, float* out_val, int32_t* out_count,
             cudaStream_t stream) {
  return ulc_topk_ex(scores, row_stride, lengths, rows, max_len, k, in_idx, in_idx_stride, xform, xform_stride,
                     nullptr, 0, 1, 1, 0, 0, out_idx, out_val, out_count, stream);
}

}  // extern "C"
