// Indexer scoring over this rank's shard of fp8 index keys (tcgen05, kind::f8f6f4),
// and the peer-store candidate exchange that replaces an all-gather of scores.
//
//   logits[q, t] = key_scale[t] * sum_h w[q, h] * relu( <q8[q, h, :], key8[t, :]> )
//
// Keys are 128 fp8 e4m3 values per token with one fp32 scale, stored in 64-token
// index pages (8192 key bytes then 256 scale bytes).  Index pages are striped
// over the ranks by logical page; a request's context is described by a table of
// allocation pages (one entry per 64 * ranks tokens, the same physical page index
// on every rank), so every rank scores 1/ranks of the context.
//
// One CTA streams a range of pages of one request: a producer thread issues TMA
// loads (non-multicast, local HBM only) of 64 x 128-byte key tiles into a ring;
// one thread issues tcgen05.mma with the 128 tokens of two pages as M and the
// request's query heads (64 per query, up to 4 queries) as N, accumulating in
// TMEM (double buffered); four epilogue warps read the accumulator, apply ReLU,
// the head weights and the token scale, and store fp32 logits.  The queries'
// fp8 scale is folded into `w` by the caller.
//
// Reference: the score step is external there (DeepGEMM fp8_paged_mqa_logits
// injected at patches/sglang.patch:801-804); the score all-gather it feeds is
// FlashAG (ulacache/csrc/flashag/b300/ag_kernels_dynamic.cuh:375) followed by a
// rank-major top-k (ulacache/csrc/indexer/topk_v2.cuh:1467).  Here each rank takes
// its local top-k and peer-stores only (score, token) candidates.
#include "ulc/launch.h"
#include "ulc/layout.h"
#include "ulc/ptx.cuh"
#include "ulc/tmap.h"
#include "ulc/topk_key.cuh"

namespace ulc {

constexpr int kIdxTileTokens = 128;                 // two pages per MMA tile
constexpr int kIdxStageBytes = kIdxTileTokens * 128; // 16 KB of keys
constexpr int kIdxStages = 8;
constexpr int kIdxMaxQueries = 4;
constexpr int kIdxBarrierBytes = 768;                   // IdxBarriers: mbarriers + page-table slice
constexpr int kIdxQBytes = kIdxMaxQueries * 64 * 128;   // 32 KB
constexpr int kIdxSmem = 1024 + kIdxStages * kIdxStageBytes + kIdxQBytes + kIdxMaxQueries * 64 * 4 + kIdxBarrierBytes;

// One query per request (decode): a short ring and small query tile, so that three CTAs share an
// SM (3 x 74 KB of shared memory, 3 x 128 TMEM columns) and one CTA's prologue and ring fill
// overlap the others' streaming.  More queries per request keep the deep ring, one CTA per SM.
// HIST: the epilogue also builds, per score row, the 2048-bin histogram the radix select starts
// from (a shared-memory histogram per CTA, flushed to the select's workspace at the end), so that the
// select kernel needs no pass of its own over the scores to find its threshold bin.
template <int NQ, bool HIST = false>
struct IdxGeom {
  // One query per request: two epilogue warpgroups take alternate tiles (the epilogue, one thread per key
  // reading 64 accumulator columns, is the longest stage), two CTAs per SM, five ring stages each.
  static constexpr int kEpilogueGroups = NQ == 1 ? 2 : 1;
  static constexpr int kThreads = 64 + 128 * kEpilogueGroups;
  static constexpr int kStages = NQ == 1 ? 5 : (HIST && NQ == 4 ? 6 : kIdxStages);
  static constexpr int kQBytes = NQ * 64 * 128;
  static constexpr int kHistBytes = HIST ? NQ * kTopkBins * 4 : 0;
  static constexpr int kSmem = 1024 + kStages * kIdxStageBytes + kQBytes + NQ * 64 * 4 + kIdxBarrierBytes + kHistBytes;
  static constexpr int kCtasPerSm = NQ == 1 ? 2 : 1;
};

struct IndexScoreParams {
  const uint8_t* q8;          // [R, n_q, 64, 128] fp8 e4m3
  const float* w;             // [R, n_q, 64]
  const int32_t* page_table;  // [R, max_pages] physical index page per allocation page, -1 = none
  const int32_t* lengths;     // [R] context length in tokens
  const uint8_t* pool;        // this rank's index page pool (for the scales)
  float* logits;              // [R * n_q, max_pages * 64]
  uint32_t* topk_ws;          // workspace of the histogram-first select (nullable): per row 2048 counts + counters
  int32_t* status;
  int R, n_q, max_pages, ranks, rank, pages_per_rank, pages_per_cta;
};

constexpr int kIdxTablePages = 128;   // page-table entries of a CTA kept in shared memory

struct IdxBarriers {
  uint64_t full[kIdxStages];
  uint64_t empty[kIdxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  // This CTA's slice of the request's page table: the producer would otherwise wait for a global
  // load before every TMA issue, and the epilogue for one before every scale load.
  int32_t pages[kIdxTablePages];
};

static_assert(sizeof(IdxBarriers) <= kIdxBarrierBytes, "barrier block outgrew its shared-memory reservation");

__device__ __forceinline__ int local_valid_tokens(int length, int alloc_page, int ranks, int rank) {
  // tokens of allocation page `alloc_page` that this rank holds and that lie below `length`
  const long long first = (static_cast<long long>(alloc_page) * ranks + rank) * kPageTokens;
  const long long left = length - first;
  return left <= 0 ? 0 : (left >= kPageTokens ? kPageTokens : static_cast<int>(left));
}

template <int NQ, bool HIST>
__global__ void __launch_bounds__(IdxGeom<NQ, HIST>::kThreads, IdxGeom<NQ, HIST>::kCtasPerSm)
index_score_kernel(const __grid_constant__ CUtensorMap tmap_keys, const IndexScoreParams p) {
  constexpr int N = NQ * 64;
  constexpr int kStages = IdxGeom<NQ, HIST>::kStages;
  constexpr int kIdxThreads = IdxGeom<NQ, HIST>::kThreads;          // (shadows the one-group constant)
  constexpr int kGroups = IdxGeom<NQ, HIST>::kEpilogueGroups;
  constexpr uint32_t kCols = N * 2 <= 128 ? 128 : N * 2 <= 256 ? 256 : 512;
  extern __shared__ uint8_t idx_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(idx_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sk = smem;
  uint8_t* sq = smem + kStages * kIdxStageBytes;
  float* sw = reinterpret_cast<float*>(sq + IdxGeom<NQ, HIST>::kQBytes);
  IdxBarriers& bar = *reinterpret_cast<IdxBarriers*>(sw + NQ * 64);
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(&bar) + kIdxBarrierBytes);   // [NQ][2048] when HIST

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.y;
  const int length = p.lengths[r];
  const int req_pages = (length + kPageTokens * p.ranks - 1) / (kPageTokens * p.ranks);
  const int pg0 = blockIdx.x * p.pages_per_cta;
  const int pg1 = min(min(req_pages, p.max_pages), pg0 + p.pages_per_cta);
  const int ntiles = pg1 > pg0 ? (pg1 - pg0 + 1) / 2 : 0;
  const int32_t* table = p.page_table + static_cast<size_t>(r) * p.max_pages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&bar.full[s], 1); ptx::mbar_init(&bar.empty[s], 1); }
    for (int s = 0; s < 2; ++s) { ptx::mbar_init(&bar.acc_full[s], 1); ptx::mbar_init(&bar.acc_empty[s], 4); }
    bar.abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_keys);
  }
  if (warp == 1) { ptx::tmem_alloc<kCols>(&bar.tmem_base); ptx::tmem_relinquish(); }
  if constexpr (HIST) {
    for (int i = threadIdx.x; i < NQ * kTopkBins; i += kIdxThreads) s_hist[i] = 0;
    // the select kernel scans the valid prefix of a row: columns of whole pages this rank holds plus
    // its share of the last, partial stripe of pages
    if (blockIdx.x == 0 && threadIdx.x < NQ) {
      const int stripe = kPageTokens * p.ranks;
      const int full = length / stripe, rem = length - full * stripe;
      const int mine = min(max(rem - p.rank * kPageTokens, 0), kPageTokens);
      const int n_valid = min(full * kPageTokens + mine, p.max_pages * kPageTokens);
      p.topk_ws[static_cast<size_t>(r * NQ + threadIdx.x) * (kTopkWsRowBytes / 4) + kTopkWsCtr + 3] = static_cast<uint32_t>(n_valid);
    }
  }
  for (int i = threadIdx.x; i < kIdxTablePages && pg0 + i < pg1; i += kIdxThreads) bar.pages[i] = table[pg0 + i];
  auto page_of = [&](int a) -> int32_t { return a - pg0 < kIdxTablePages ? bar.pages[a - pg0] : table[a]; };
  // queries of this request -> shared memory, 128-byte swizzled rows (one row per head)
  if (ntiles > 0) {
    const uint4* src = reinterpret_cast<const uint4*>(p.q8 + static_cast<size_t>(r) * NQ * 64 * 128);
    for (int i = threadIdx.x; i < N * 8; i += kIdxThreads)
      *reinterpret_cast<uint4*>(sq + ptx::sw128_offset(i >> 3, i & 7)) = src[i];
    for (int i = threadIdx.x; i < N; i += kIdxThreads) sw[i] = p.w[static_cast<size_t>(r) * N + i];
    ptx::fence_async_smem();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = bar.tmem_base;
  volatile int* abort_flag = &bar.abort_flag;

  if (warp == 0) {
    if (ptx::elect_one()) {
      int issued = 0;
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kStages;
        if (*abort_flag || !ptx::mbar_wait(&bar.empty[s], ((i / kStages) & 1) ^ 1)) {
          if (!*abort_flag) report(p.status, kErrPipeline, 100 + s);
          *abort_flag = 1;
          break;
        }
        const int a0 = pg0 + 2 * i, a1 = a0 + 1;
        const int32_t ph0 = page_of(a0);
        const int32_t ph1 = a1 < pg1 ? page_of(a1) : -1;
        const bool v0 = ph0 >= 0 && ph0 < p.pages_per_rank;
        const bool v1 = ph1 >= 0 && ph1 < p.pages_per_rank;
        // a page that is not loaded leaves stale bytes behind; the epilogue masks its tokens
        // (arrive.expect_tx is this thread's one arrival; with nothing in flight it completes the phase)
        ptx::mbar_expect_tx(&bar.full[s], (v0 ? 8192 : 0) + (v1 ? 8192 : 0));
        uint8_t* dst = sk + s * kIdxStageBytes;
        if (v0) ptx::tma_load_2d(dst, &tmap_keys, &bar.full[s], 0, ph0 * 66);
        if (v1) ptx::tma_load_2d(dst + 8192, &tmap_keys, &bar.full[s], 0, ph1 * 66);
        issued = i + 1;
      }
      if (*abort_flag)
        for (int i = max(0, issued - kStages); i < issued; ++i)
          ptx::mbar_wait(&bar.full[i % kStages], (i / kStages) & 1, 200000000LL);
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc(128, N, 0, 0, 0, 0);   // e4m3 x e4m3 -> f32
      const uint64_t q_desc = ptx::umma_desc_sw128(ptx::smem_u32(sq));
      const uint64_t k_desc0 = ptx::umma_desc_sw128(ptx::smem_u32(sk));
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kStages, ab = i & 1;
        if (*abort_flag || !ptx::mbar_wait(&bar.acc_empty[ab], ((i >> 1) & 1) ^ 1) ||
            !ptx::mbar_wait(&bar.full[s], (i / kStages) & 1)) {
          if (!*abort_flag) report(p.status, kErrPipeline, 200 + s);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after();
        const uint64_t k_desc = ptx::umma_desc_advance(k_desc0, s * kIdxStageBytes);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          ptx::umma_fp8(tmem + ab * N, ptx::umma_desc_advance(k_desc, kk * 32),
                        ptx::umma_desc_advance(q_desc, kk * 32), idesc, kk != 0);
        ptx::umma_commit(&bar.empty[s]);
        ptx::umma_commit(&bar.acc_full[ab]);
      }
    }
  } else {
    const int qd = warp & 3;                  // TMEM lane quarter this warp may read
    const int wg = (warp - 2) >> 2;           // epilogue group: takes tiles wg, wg + kGroups, ...
    const int row = qd * 32 + lane;           // token row in the tile
    const int pg_in_tile = row >> 6, off = row & 63;
    const size_t row_stride = static_cast<size_t>(p.max_pages) * kPageTokens;
    // The key scale of this thread's token is fetched one tile ahead, so that its latency hides
    // behind the wait for the accumulator and the arithmetic of the tile before.
    bool inside_next = false;                 // the token lies below the request's length (whatever its page holds)
    auto fetch_scale = [&](int tile, bool& valid_out) -> float {
      const int a = pg0 + 2 * tile + pg_in_tile;
      int32_t phys = (tile < ntiles && a < pg1) ? page_of(a) : -1;
      if (phys >= p.pages_per_rank) phys = -1;
      inside_next = tile < ntiles && a < pg1 && off < local_valid_tokens(length, a, p.ranks, p.rank);
      valid_out = phys >= 0 && inside_next;
      return valid_out
          ? reinterpret_cast<const float*>(p.pool + static_cast<size_t>(phys) * kIndexPageBytes + kIndexPageKeyBytes)[off]
          : 0.f;
    };
    bool valid_next = false;
    float kscale_next = fetch_scale(wg, valid_next);
    for (int i = wg; i < ntiles; i += kGroups) {
      const int ab = i & 1;
      const bool valid = valid_next;
      const bool inside = inside_next;
      const float kscale = kscale_next;
      kscale_next = fetch_scale(i + kGroups, valid_next);
      if (*abort_flag || !ptx::mbar_wait(&bar.acc_full[ab], (i >> 1) & 1)) {
        if (!*abort_flag && lane == 0) report(p.status, kErrPipeline, 300 + qd);
        *abort_flag = 1;
        break;
      }
      ptx::tc_fence_after();
      const int a = pg0 + 2 * i + pg_in_tile;
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        // both halves of the accumulator row are requested before the first is consumed, and the
        // weighted sum runs as four independent chains (one chain of 64 dependent FMAs would take
        // longer than the tile's share of the key stream)
        uint32_t d0[32], d1[32];
        ptx::tmem_ld32(tmem + (static_cast<uint32_t>(qd * 32) << 16) + ab * N + j * 64, d0);
        ptx::tmem_ld32(tmem + (static_cast<uint32_t>(qd * 32) << 16) + ab * N + j * 64 + 32, d1);
        ptx::tmem_ld_wait();
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 32; ++h) {
          part[h & 3] = fmaf(sw[j * 64 + h], fmaxf(__uint_as_float(d0[h]), 0.f), part[h & 3]);
          part[h & 3] = fmaf(sw[j * 64 + 32 + h], fmaxf(__uint_as_float(d1[h]), 0.f), part[h & 3]);
        }
        const float acc = (part[0] + part[1]) + (part[2] + part[3]);
        const float logit = valid ? acc * kscale : -INFINITY;
        if (a < pg1)
          p.logits[(static_cast<size_t>(r) * NQ + j) * row_stride + static_cast<size_t>(a) * kPageTokens + off] = logit;
        if constexpr (HIST) {
          if (inside) atomicAdd(&s_hist[j * kTopkBins + window_bin(order_key(logit))], 1u);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar.acc_empty[ab]);
    }
    if constexpr (HIST) {
      // the four epilogue warps flush this CTA's non-empty bins into the rows' histograms
      asm volatile("bar.sync 1, %0;" ::"n"(128 * kGroups) : "memory");
      const int et = threadIdx.x - 64;
      for (int i = et; i < NQ * kTopkBins; i += 128 * kGroups) {
        const uint32_t c = s_hist[i];
        if (c) atomicAdd(p.topk_ws + static_cast<size_t>(r * NQ + i / kTopkBins) * (kTopkWsRowBytes / 4) + (i % kTopkBins), c);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc<kCols>(tmem);
}

// Columns that no CTA covers (pages beyond a request's length) must read -inf.
__global__ void index_fill_tail_kernel(IndexScoreParams p) {
  const int r = blockIdx.y;
  const int length = p.lengths[r];
  const int req_pages = min(p.max_pages, (length + kPageTokens * p.ranks - 1) / (kPageTokens * p.ranks));
  const size_t row_stride = static_cast<size_t>(p.max_pages) * kPageTokens;
  const int first = req_pages * kPageTokens;
  for (int j = 0; j < p.n_q; ++j) {
    float* row = p.logits + (static_cast<size_t>(r) * p.n_q + j) * row_stride;
    for (size_t c = first + blockIdx.x * blockDim.x + threadIdx.x; c < row_stride; c += static_cast<size_t>(gridDim.x) * blockDim.x)
      row[c] = -INFINITY;
  }
}

// Local column (alloc_page * 64 + offset) -> logical record ID, for `n` selected columns per row.
__global__ void index_cols_to_ids_kernel(const int32_t* __restrict__ cols, const int32_t* __restrict__ page_table,
                                         int max_pages, int n_q, int k, int ranks, int rank, int rows,
                                         int32_t* __restrict__ ids) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * k) return;
  const int row = i / k;
  const int32_t c = cols[i];
  int32_t out = -1;
  if (c >= 0) {
    const int32_t phys = page_table[static_cast<size_t>(row / n_q) * max_pages + (c >> kPageShift)];
    if (phys >= 0) out = ((phys * ranks + rank) << kPageShift) | (c & (kPageTokens - 1));
  }
  ids[i] = out;
}

// Peer-store this rank's candidates into every rank's merge buffer, laid out
// [row][source rank][k] so that a row's ranks * k candidates are contiguous for the merge.
// vals/ids [rows, k]; dst_vals[r] / dst_ids[r] point at rank r's buffers.  k % 4 == 0.
__global__ void candidate_scatter_kernel(const float* __restrict__ vals, const int32_t* __restrict__ ids,
                                         float* const* dst_vals, int32_t* const* dst_ids, int ranks, int rank,
                                         int rows, int k) {
  const int peer = blockIdx.y;
  float* dv = dst_vals[peer];
  int32_t* di = dst_ids[peer];
  const size_t n4 = static_cast<size_t>(rows) * k / 4;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t e = i * 4;
    const size_t row = e / k, j = e % k;
    const size_t o = (row * ranks + rank) * k + j;
    ptx::st_cg16(dv + o, *reinterpret_cast<const uint4*>(vals + e));
    ptx::st_cg16(di + o, *reinterpret_cast<const uint4*>(ids + e));
  }
  ptx::cta_release_peer_stores();
}

template <int NQ, bool HIST>
static int launch_index_score(const CUtensorMap& tm, const IndexScoreParams& p, dim3 grid, cudaStream_t s) {
  static PerDeviceOnce once;
  const int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(index_score_kernel<NQ, HIST>),
                                     IdxGeom<NQ, HIST>::kSmem, once);
  if (rc != 0) return rc;
  index_score_kernel<NQ, HIST><<<grid, IdxGeom<NQ, HIST>::kThreads, IdxGeom<NQ, HIST>::kSmem, s>>>(tm, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// q8 [R, n_q, 64, 128] fp8; w [R, n_q, 64] fp32; page_table [R, max_pages]; lengths [R];
// pool: this rank's index pages (8448 bytes each); logits [R*n_q, max_pages*64] fp32.
// topk_ws (nullable): workspace of ulc_topk_ws (ulc_topk_workspace_bytes(R * n_q) bytes, zero when first
// used).  When given, the kernel also leaves every row's histogram and valid length there for
// ulc_topk_ws(..., hist_ready = 1), and the columns beyond a request's pages are NOT filled with -inf
// (the select kernel reads only the valid prefix).
int ulc_index_score_hist(const void* q8, const float* w, const int32_t* page_table, const int32_t* lengths,
                         const void* pool, int pages_per_rank, int R, int n_q, int max_pages, int ranks, int rank,
                         int pages_per_cta, float* logits, void* topk_ws, int32_t* status, cudaStream_t stream);

int ulc_index_score(const void* q8, const float* w, const int32_t* page_table, const int32_t* lengths,
                    const void* pool, int pages_per_rank, int R, int n_q, int max_pages, int ranks, int rank,
                    int pages_per_cta, float* logits, int32_t* status, cudaStream_t stream) {
  return ulc_index_score_hist(q8, w, page_table, lengths, pool, pages_per_rank, R, n_q, max_pages, ranks, rank,
                              pages_per_cta, logits, nullptr, status, stream);
}

int ulc_index_score_hist(const void* q8, const float* w, const int32_t* page_table, const int32_t* lengths,
                         const void* pool, int pages_per_rank, int R, int n_q, int max_pages, int ranks, int rank,
                         int pages_per_cta, float* logits, void* topk_ws, int32_t* status, cudaStream_t stream) {
  if (R <= 0 || max_pages <= 0) return 0;
  if (n_q < 1 || n_q > kIdxMaxQueries || n_q == 3) return -kErrUnsupported;
  if (reinterpret_cast<uintptr_t>(pool) & 127) return -kErrAlignment;
  CUtensorMap tm;
  int rc = make_tmap_2d(&tm, pool, 1, static_cast<uint64_t>(pages_per_rank) * 66, 128, 128, 64, 128, true);
  if (rc != 0) return rc;
  IndexScoreParams p;
  p.q8 = reinterpret_cast<const uint8_t*>(q8); p.w = w; p.page_table = page_table; p.lengths = lengths;
  p.pool = reinterpret_cast<const uint8_t*>(pool); p.logits = logits; p.status = status;
  p.topk_ws = reinterpret_cast<uint32_t*>(topk_ws);
  p.R = R; p.n_q = n_q; p.max_pages = max_pages; p.ranks = ranks; p.rank = rank;
  p.pages_per_rank = pages_per_rank;
  if (pages_per_cta <= 0) {
    // one resident wave: 148 SMs x 2 CTAs (one query per request) or two waves of one CTA per SM;
    // at least 8 pages (4 tiles) each
    const long long total = static_cast<long long>(R) * max_pages;
    const long long ctas = 296;
    long long per = (total + ctas - 1) / ctas;
    if (per < 8) per = 8;
    per = (per + 1) / 2 * 2;
    // the grid is R x ceil(max_pages / per): rounding per row must not push it past the resident wave
    // (four CTAs too many cost a whole second wave)
    while (static_cast<long long>(R) * ((max_pages + per - 1) / per) > ctas && per < max_pages) per += 2;
    pages_per_cta = static_cast<int>(per);
  }
  p.pages_per_cta = pages_per_cta + (pages_per_cta & 1);
  dim3 grid((max_pages + p.pages_per_cta - 1) / p.pages_per_cta, R);
  if (topk_ws != nullptr) {
    switch (n_q) {
      case 1: return launch_index_score<1, true>(tm, p, grid, stream);
      case 2: return launch_index_score<2, true>(tm, p, grid, stream);
      default: return launch_index_score<4, true>(tm, p, grid, stream);
    }
  }
  index_fill_tail_kernel<<<dim3(8, R), 256, 0, stream>>>(p);
  switch (n_q) {
    case 1: rc = launch_index_score<1, false>(tm, p, grid, stream); break;
    case 2: rc = launch_index_score<2, false>(tm, p, grid, stream); break;
    default: rc = launch_index_score<4, false>(tm, p, grid, stream); break;
  }
  return rc;
}

int ulc_index_cols_to_ids(const int32_t* cols, const int32_t* page_table, int max_pages, int n_q, int k,
                          int ranks, int rank, int rows, int32_t* ids, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int n = rows * k;
  index_cols_to_ids_kernel<<<(n + 255) / 256, 256, 0, stream>>>(cols, page_table, max_pages, n_q, k, ranks, rank, rows, ids);
  return static_cast<int>(cudaGetLastError());
}

int ulc_candidate_scatter(const float* vals, const int32_t* ids, float* const* dst_vals, int32_t* const* dst_ids,
                          int ranks, int rank, int rows, int k, cudaStream_t stream) {
  if (rows <= 0 || k <= 0) return 0;
  if (k % 4) return -kErrUnsupported;
  const long long n4 = static_cast<long long>(rows) * k / 4;
  int blocks = static_cast<int>((n4 + 255) / 256);
  if (blocks > 64) blocks = 64;
  if (blocks < 1) blocks = 1;
  candidate_scatter_kernel<<<dim3(blocks, ranks), 256, 0, stream>>>(vals, ids, dst_vals, dst_ids, ranks, rank, rows, k);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
