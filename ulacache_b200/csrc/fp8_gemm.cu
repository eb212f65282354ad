// Block-scaled fp8 grouped GEMM for decode (tcgen05, kind::f8f6f4), used for the
// MoE expert FFNs and for every dense fp8 projection.
//
//   Y[m, n] = sum_kb ( sum_{k in block kb} X8[m, k] * W8[e, n, k] ) * sx[m, kb] * sw[e, n / 128, kb]
//
//   W8 [E, Nout, K] fp8 e4m3, sw [E, Nout/128, K/128] fp32   (128 x 128 weight blocks)
//   X8 [M, K]       fp8 e4m3, sx [M, K/128] fp32              (1 x 128 activation groups)
//   offs [E + 1]: rows offs[e] .. offs[e+1] of X belong to expert e (E = 1 for a dense layer)
//
// Weight-stationary like the bf16 GEMM: 128 output features of one expert are the
// MMA M side, the expert's tokens (padded to 16) the N side.  Every 128-wide K
// block is accumulated into a fresh TMEM buffer (double buffered) and promoted by
// the epilogue warps into fp32 registers with the two scales, so the scaling is
// exact block scaling rather than one scale per tensor.  Decode is bound by
// streaming the weights: the producer keeps a TMA ring of up to 12 stages full, and the
// weights are stored tile-major so that every stage is one contiguous 16 KB read.
//
// The reference library has no GEMM; the serving framework it patches uses
// DeepGEMM for this role.
#include <stdlib.h>
#include "ulc/launch.h"
#include "ulc/ptx.cuh"
#include "ulc/tmap.h"

namespace ulc {

constexpr int kF8BM = 128;            // output features per CTA
constexpr int kF8BK = 128;            // one scale block of K (128 fp8 = 128 bytes)
constexpr int kF8MaxAccBufs = 8;       // TMEM accumulators in flight: 8 of up to 32 columns, or 4 of up to 128
constexpr int kF8Threads = 64 + 8 * 32 + 32;                   // producer, MMA, 8 epilogue warps, second MMA issuer
constexpr int kF8SecondMmaWarp = 10;
constexpr int kF8MaxKB = 144;                                  // K <= 18432

// Ring geometry for a kernel that handles at most MAXN tokens per pass: the fewer
// tokens, the smaller a stage and the more weight bytes in flight per SM.
template <int MAXN>
struct F8Geom {
  static constexpr int kStageBytes = kF8BM * 128 + MAXN * 128;
  static constexpr int kPartBytes = MAXN <= 32 ? 128 * MAXN * 4 : 0;       // partial sums of the second epilogue group
  // Products sx[token][k block] * sw[k block] of the pass in flight (narrow geometries): the epilogue
  // is the critical stage of the pipeline there, and a shared-memory read per token and K block is
  // cheaper than a global load, a multiply and a register move.
  static constexpr int kScaleBytes = MAXN <= 32 ? MAXN * 144 * 4 : 0;
  // The finished bf16 tile [token][feature] of the pass, staged so that the global stores are
  // 16-byte vectors along the feature axis issued by all epilogue threads.
  static constexpr int kOutBytes = MAXN <= 32 ? MAXN * 128 * 2 : 0;
  // An EVEN number of stages: the two MMA issuers take alternate K blocks, and a stage must
  // always come back to the same issuer.  A thread that waited on only every other phase of a
  // stage's barrier could not tell "my phase completed" from "the phase before it is still
  // pending" (a parity wait distinguishes adjacent phases only).
  static constexpr int kFit = (200 * 1024 - kPartBytes - kScaleBytes - kOutBytes) / kStageBytes;
  static constexpr int kStages = (kFit > 12 ? 12 : kFit) & ~1;
  static_assert(kStages >= 2 && kStages % 2 == 0, "stage count must be even");
  static constexpr int kSmem = 1024 + kStages * kStageBytes + 512 + kPartBytes + kScaleBytes + kOutBytes;
  // The K slices of a block may be spread over kSlices independent TMEM accumulators
  // (summed by the epilogue) to break the accumulate-after-accumulate dependency.
  static constexpr int kSlices = 1;   // measured: more slices do not help, the issue rate of one thread does
  static constexpr int kBufCols = kSlices * MAXN;            // columns of one accumulator buffer
};
constexpr int kF8MaxStages = 12;

struct F8Params {
  const float* sw;            // [E, Nout/128, KB]
  const float* sx;            // [M, KB]
  const int32_t* offs;        // [E + 1] (nullable when E == 1: rows 0..M)
  const int32_t* active;      // [E] experts with at least one row, compacted (nullable: all experts)
  const int32_t* n_active;    // [1] entries of `active` (nullable: E)
  void* out;                  // bf16 [M, Nout] or fp32 [M, Nout] (split-K)
  void* out_peers[8];         // optional: the same bf16 tile is also stored to these (peer) buffers
  int n_peers;
  int32_t* status;
  int M, Nout, K, E, kb_per_split, splits, out_f32;
  // In-kernel split-K reduction (dense layers, all rows in one pass): every split leaves its fp32
  // partial tile in `part`, takes a ticket, and the last split of a tile to arrive sums them and
  // stores bf16 - no cleared accumulation buffer, no global atomics, no conversion kernel.
  float* part;                // [tiles * splits][MAXN][128] fp32 (nullable)
  uint32_t* tickets;          // [tiles], zero when the kernel starts, zero again when it ends
  int rows_per_peer;          // > 0: reduce-scatter, row m goes only to peer m / rows_per_peer at row m % rows_per_peer
};

struct F8Barriers {
  uint64_t full[kF8MaxStages];
  uint64_t empty[kF8MaxStages];
  uint64_t acc_full[kF8MaxAccBufs];
  uint64_t acc_empty[kF8MaxAccBufs];
  uint32_t tmem_base;
  int abort_flag;
  int reduce_last;            // split-K reduction: this CTA drew the last ticket of its tile
};

// Optional timeline of CTA 0, compiled in with -DULC_F8_TRACE (development only):
// f8_trace[role][slot][event] = clock64; roles: 0 producer, 1 first MMA issuer, 2 epilogue group 0.
#ifdef ULC_F8_TRACE
__device__ long long f8_trace[3][64][4];
#define F8_T(role, slot, ev)                                                                   \
  do {                                                                                         \
    if (blockIdx.x == 0 && (slot) < 64) f8_trace[role][slot][ev] = clock64();                   \
  } while (0)
#else
#define F8_T(role, slot, ev) do {} while (0)
#endif

struct F8Item {
  int e, n0, kb0, nkb, m_begin, m_end;
  int tile_id, split;         // (expert slot, feature tile) index and K split of the item
};

// Work item `idx` of the persistent loop: (active expert, feature tile, K split).
__device__ __forceinline__ F8Item f8_item(const F8Params& p, int idx) {
  const int tiles = p.Nout / kF8BM;
  const int split = idx % p.splits;
  const int tile = (idx / p.splits) % tiles;
  const int a = idx / (p.splits * tiles);
  F8Item it;
  it.e = p.active ? p.active[a] : a;
  it.tile_id = a * tiles + tile;
  it.split = split;
  it.n0 = tile * kF8BM;
  const int KB = p.K / kF8BK;
  it.kb0 = split * p.kb_per_split;
  it.nkb = max(0, min(KB, it.kb0 + p.kb_per_split) - it.kb0);
  it.m_begin = p.offs ? p.offs[it.e] : 0;
  it.m_end = p.offs ? p.offs[it.e + 1] : p.M;
  return it;
}

// Persistent: each CTA walks items blockIdx.x, blockIdx.x + gridDim.x, ...; the TMA ring,
// the TMEM accumulators and their phase counters run straight through item boundaries, so
// the weight stream never drains between tiles.
template <int MAXN>
__global__ void __launch_bounds__(kF8Threads, 1)
fp8_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const F8Params p) {
  constexpr int kF8MaxN = MAXN;
  constexpr int kF8Stages = F8Geom<MAXN>::kStages;
  constexpr int kF8StageBytes = F8Geom<MAXN>::kStageBytes;
  // More accumulators for narrow tiles: the end of an item (partial-sum exchange, global store)
  // stalls the epilogue warps for a while; the MMA issuers keep going as long as buffers are free.
  constexpr int kF8AccBufs = MAXN <= 32 ? 8 : 4;
  constexpr int kSlices = F8Geom<MAXN>::kSlices;
  constexpr int kBufCols = F8Geom<MAXN>::kBufCols;
  extern __shared__ uint8_t f8_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(f8_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  F8Barriers& bar = *reinterpret_cast<F8Barriers*>(smem + kF8Stages * kF8StageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / kF8BK;
  const int n_act = p.n_active ? *p.n_active : p.E;
  const int n_items = n_act * (p.Nout / kF8BM) * p.splits;
  if (static_cast<int>(blockIdx.x) >= n_items) return;      // nothing allocated yet: just leave

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) { ptx::mbar_init(&bar.full[s], 1); ptx::mbar_init(&bar.empty[s], 1); }
    for (int s = 0; s < kF8AccBufs; ++s) { ptx::mbar_init(&bar.acc_full[s], 1); ptx::mbar_init(&bar.acc_empty[s], MAXN <= 32 ? 4 : 8); }
    bar.abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_w);
    ptx::prefetch_tmap(&tmap_x);
  }
  if (warp == 1) { ptx::tmem_alloc<512>(&bar.tmem_base); ptx::tmem_relinquish(); }
  // Dense layers (one weight, no row offsets to look up): the scales of this CTA's first pass are
  // requested NOW.  Once the producers of all CTAs have started, some 35 MB of weight tiles are
  // queued in the memory system and a small load issued behind them waits microseconds; the
  // epilogue cannot consume its first K block without these values.
  constexpr int kPreJ = MAXN <= 32 ? MAXN / 8 : 1;
  float pre_sx[kPreJ][2], pre_sw[2];
  bool pre_valid = false;
  if constexpr (MAXN <= 32) {
    if (p.E == 1 && warp >= 2 && warp != kF8SecondMmaWarp) {
      const F8Item w0 = f8_item(p, blockIdx.x);
      const int nt0 = min(kF8MaxN, w0.m_end - w0.m_begin);
      const float* sxb = p.sx + static_cast<size_t>(w0.m_begin) * KB + w0.kb0;
      const float* swt = p.sw + (static_cast<size_t>(w0.e) * (p.Nout / kF8BM) + w0.n0 / kF8BM) * KB + w0.kb0;
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        const int i = lane + 32 * ii;
        pre_sw[ii] = i < w0.nkb ? swt[i] : 0.f;
#pragma unroll
        for (int jj = 0; jj < kPreJ; ++jj) {
          const int j = (warp - 2) + 8 * jj;
          pre_sx[jj][ii] = (i < w0.nkb && j < nt0) ? sxb[static_cast<size_t>(j) * KB + i] : 0.f;
        }
      }
      pre_valid = true;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = bar.tmem_base;
  volatile int* abort_flag = &bar.abort_flag;

  if (warp == 0) {
    if (ptx::elect_one()) {
      int it = 0, issued = 0;
      for (int idx = blockIdx.x; idx < n_items && !*abort_flag; idx += gridDim.x) {
        const F8Item w = f8_item(p, idx);
        const int tokens = w.m_end - w.m_begin;
        const int passes = tokens > 0 ? (tokens + kF8MaxN - 1) / kF8MaxN : 0;
        F8_T(0, (idx - blockIdx.x) / gridDim.x, 0);          // producer reaches this item
        for (int ps = 0; ps < passes && !*abort_flag; ++ps) {
          const int t0 = w.m_begin + ps * kF8MaxN;
          const int nt = min(kF8MaxN, w.m_end - t0);
          const int boxes = (nt + 15) / 16;
          for (int i = 0; i < w.nkb; ++i, ++it) {
            const int s = it % kF8Stages;
            if (*abort_flag || !ptx::mbar_wait(&bar.empty[s], ((it / kF8Stages) & 1) ^ 1)) {
              if (!*abort_flag) report(p.status, kErrPipeline, 100 + s);
              *abort_flag = 1;
              break;
            }
            uint8_t* a = smem + s * kF8StageBytes;
            ptx::mbar_expect_tx(&bar.full[s], kF8BM * 128 + boxes * 16 * 128);
            ptx::tma_load_2d(a, &tmap_w, &bar.full[s], 0,
                             ((w.e * (p.Nout / kF8BM) + w.n0 / kF8BM) * KB + w.kb0 + i) * kF8BM);
            for (int bx = 0; bx < boxes; ++bx)
              ptx::tma_load_2d(a + kF8BM * 128 + bx * 2048, &tmap_x, &bar.full[s], (w.kb0 + i) * kF8BK, t0 + bx * 16);
            issued = it + 1;
          }
        }
        F8_T(0, (idx - blockIdx.x) / gridDim.x, 1);          // ... has issued its last load
      }
      if (*abort_flag)
        for (int i = max(0, issued - kF8Stages); i < issued; ++i)
          ptx::mbar_wait(&bar.full[i % kF8Stages], (i / kF8Stages) & 1, 200000000LL);
    }
  } else if (warp == 1 || warp == kF8SecondMmaWarp) {
    // two issuing threads take alternate K blocks: one thread's wait / issue / commit
    // sequence is too slow to keep up with the weight stream on its own
    const int mma_id = warp == 1 ? 0 : 1;
    if (ptx::elect_one()) {        // elected thread of the converged warp (a `lane == 0` branch issues 3.5x slower)
      int it = 0;
      const uint64_t smem_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem));
      for (int idx = blockIdx.x; idx < n_items && !*abort_flag; idx += gridDim.x) {
        const F8Item w = f8_item(p, idx);
        const int tokens = w.m_end - w.m_begin;
        const int passes = tokens > 0 ? (tokens + kF8MaxN - 1) / kF8MaxN : 0;
        if (mma_id == 0) F8_T(1, (idx - blockIdx.x) / gridDim.x, 0);   // issuer reaches this item
        for (int ps = 0; ps < passes && !*abort_flag; ++ps) {
          const int nt = min(kF8MaxN, w.m_end - (w.m_begin + ps * kF8MaxN));
          const uint32_t n_mma = static_cast<uint32_t>((nt + 15) / 16 * 16);
          const uint32_t idesc = ptx::umma_idesc(kF8BM, n_mma, 0, 0, 0, 0);
          for (int i = 0; i < w.nkb; ++i, ++it) {
            if ((it & 1) != mma_id) continue;
            const int s = it % kF8Stages, ab = it % kF8AccBufs;
            if (*abort_flag || !ptx::mbar_wait(&bar.acc_empty[ab], ((it / kF8AccBufs) & 1) ^ 1) ||
                !ptx::mbar_wait(&bar.full[s], (it / kF8Stages) & 1)) {
              if (!*abort_flag) report(p.status, kErrPipeline, 200 + s);
              *abort_flag = 1;
              break;
            }
            ptx::tc_fence_after();
            const uint64_t a_desc = ptx::umma_desc_advance(smem_desc, s * kF8StageBytes);
            const uint64_t b_desc = ptx::umma_desc_advance(a_desc, kF8BM * 128);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              ptx::umma_fp8(tmem + ab * kBufCols + (kk % kSlices) * kF8MaxN, ptx::umma_desc_advance(a_desc, kk * 32),
                            ptx::umma_desc_advance(b_desc, kk * 32), idesc, kk >= kSlices);
            ptx::umma_commit(&bar.empty[s]);
            ptx::umma_commit(&bar.acc_full[ab]);
          }
        }
        if (mma_id == 0) F8_T(1, (idx - blockIdx.x) / gridDim.x, 1);   // ... has issued its last MMA
      }
    }
  } else {
    // Eight epilogue warps in two groups of four (one warp per TMEM lane quarter).
    //  * MAXN <= 32: the groups take alternate K blocks, so each has two block times to get
    //    through its wait -> tcgen05.ld -> FMA chain; their partial sums meet in shared memory.
    //  * MAXN  > 32: both groups take every K block, one per half of the token columns.
    constexpr bool kAlternate = MAXN <= 32;
    const int ew = warp - 2;
    const int qd = warp & 3;
    const int grp = ew >> 2;
    const int colh = kAlternate ? 0 : grp;
    float* s_part = reinterpret_cast<float*>(smem + kF8Stages * kF8StageBytes + 512);   // [128][MAXN] when alternating
    float* s_scale = s_part + 128 * (kAlternate ? MAXN : 0);                             // [MAXN][kF8MaxKB] when alternating
    __nv_bfloat16* s_out = reinterpret_cast<__nv_bfloat16*>(s_scale + (kAlternate ? MAXN * kF8MaxKB : 0));   // [MAXN][128]
    const int etid = ew * 32 + lane;                                                     // 0..255 over the epilogue warps
    int it = 0;
    for (int idx = blockIdx.x; idx < n_items && !*abort_flag; idx += gridDim.x) {
      const F8Item w = f8_item(p, idx);
      const int tokens = w.m_end - w.m_begin;
      const int passes = tokens > 0 ? (tokens + kF8MaxN - 1) / kF8MaxN : 0;
      const int f = w.n0 + qd * 32 + lane;           // output feature of this thread
      if (etid == 0) F8_T(2, (idx - blockIdx.x) / gridDim.x, 0);       // epilogue reaches this item
      const float* sw_tile = p.sw + (static_cast<size_t>(w.e) * (p.Nout / kF8BM) + w.n0 / kF8BM) * KB + w.kb0;
      for (int ps = 0; ps < passes && !*abort_flag; ++ps) {
        const int t0 = w.m_begin + ps * kF8MaxN;
        const int nt = min(kF8MaxN, w.m_end - t0);
        const int my_n = max(0, min(kAlternate ? MAXN : 64, nt - colh * 64));
        constexpr int kAcc = kAlternate ? MAXN : 64;
        float acc[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) acc[j] = 0.f;
        const float* sx_base = p.sx + static_cast<size_t>(t0 + colh * 64) * KB + w.kb0;
        if (kAlternate) {
          // (both groups have left the previous pass: its closing barriers are behind every warp)
          // a warp per token row, a lane per K block: every load of the table is independent of the
          // others and in flight at once (the epilogue cannot consume a block before its products exist)
          const bool from_regs = pre_valid && idx == static_cast<int>(blockIdx.x) && ps == 0;
#pragma unroll
          for (int jj = 0; jj < MAXN / 8; ++jj) {
            const int j = ew + 8 * jj;
            if (from_regs) {
#pragma unroll
              for (int ii = 0; ii < 2; ++ii)
                if (lane + 32 * ii < w.nkb) s_scale[j * kF8MaxKB + lane + 32 * ii] = pre_sx[jj < kPreJ ? jj : 0][ii] * pre_sw[ii];
            }
            for (int i = lane + (from_regs ? 64 : 0); i < w.nkb; i += 32)
              s_scale[j * kF8MaxKB + i] = j < nt ? sx_base[static_cast<size_t>(j) * KB + i] * sw_tile[i] : 0.f;
          }
          asm volatile("bar.sync 3, 256;" ::: "memory");
          if (etid == 0) F8_T(2, (idx - blockIdx.x) / gridDim.x, 1);   // scale table ready
        }
        // (wide geometries) scales of the first 16 tokens are fetched one turn ahead of their use
        float s_pref[16];
        auto prefetch = [&](int i) {
          const float wsc = i < w.nkb ? sw_tile[i] : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) s_pref[j] = (j < my_n && i < w.nkb) ? sx_base[static_cast<size_t>(j) * KB + i] * wsc : 0.f;
        };
        const int first = kAlternate ? ((grp - (it & 1)) & 1) : 0;   // first K block of this group
        if (!kAlternate) prefetch(first);
        for (int i = 0; i < w.nkb; ++i, ++it) {
          if (kAlternate && ((it & 1) != grp)) continue;
          const int ab = it % kF8AccBufs;
          if (*abort_flag || !ptx::mbar_wait(&bar.acc_full[ab], (it / kF8AccBufs) & 1)) {
            if (!*abort_flag && lane == 0) report(p.status, kErrPipeline, 300 + ew);
            *abort_flag = 1;
            break;
          }
          ptx::tc_fence_after();
          float s_now[16];
          if (!kAlternate) {
#pragma unroll
            for (int j = 0; j < 16; ++j) s_now[j] = s_pref[j];
            prefetch(i + 1);
          }
#pragma unroll
          for (int c = 0; c < kAcc; c += 16) {
            if (c < my_n) {                            // warp-uniform
              uint32_t ds[kSlices][16];
#pragma unroll
              for (int ks = 0; ks < kSlices; ++ks)
                ptx::tmem_ld16(tmem + (static_cast<uint32_t>(qd * 32) << 16) + ab * kBufCols + ks * kF8MaxN +
                                   colh * 64 + c, ds[ks]);
              ptx::tmem_ld_wait();
              float d[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                d[j] = __uint_as_float(ds[0][j]);
#pragma unroll
                for (int ks = 1; ks < kSlices; ++ks) d[j] += __uint_as_float(ds[ks][j]);
              }
              if (kAlternate) {
                // the table read overlaps nothing critical: issue it before waiting on TMEM would be
                // better still, but the compiler hoists these loads above the wait on its own
                const float* row = s_scale + c * kF8MaxKB + i;
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] = fmaf(d[j], row[j * kF8MaxKB], acc[c + j]);
              } else if (c == 0) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] = fmaf(d[j], s_now[j], acc[j]);
              } else {
                const float wscale = sw_tile[i];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float sc = c + j < my_n ? sx_base[static_cast<size_t>(c + j) * KB + i] * wscale : 0.f;
                  acc[c + j] = fmaf(d[j], sc, acc[c + j]);
                }
              }
            }
          }
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bar.acc_empty[ab]);
        }
        if (*abort_flag) break;
        if (etid == 0) F8_T(2, (idx - blockIdx.x) / gridDim.x, 2);     // last K block consumed
        if (kAlternate) {
          // group 1 parks its partial sums, group 0 adds them and stores
          // (token-major staging: the 32 lanes of a warp hold 32 consecutive features, so every
          // shared-memory access below is conflict free)
          const int row = qd * 32 + lane;
          if (grp == 1) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) s_part[j * 128 + row] = acc[j];
          }
          asm volatile("bar.sync 1, 256;" ::: "memory");
          if (grp == 0) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) acc[j] += s_part[j * 128 + row];
            if (p.part != nullptr) {
#pragma unroll
              for (int j = 0; j < kAcc; ++j) s_part[j * 128 + row] = acc[j];
            } else if (!p.out_f32) {
#pragma unroll
              for (int j = 0; j < kAcc; ++j) s_out[j * 128 + row] = __float2bfloat16(acc[j]);
            }
          }
          asm volatile("bar.sync 2, 256;" ::: "memory");    // s_part may be rewritten by the next pass
          if (p.part != nullptr) {
            // split-K: park the fp32 partial tile, take a ticket; the last split of the tile reduces
            const size_t slot = (static_cast<size_t>(w.tile_id) * p.splits + w.split) * (MAXN * 128);
            const float4* src4 = reinterpret_cast<const float4*>(s_part);
            float4* dst4 = reinterpret_cast<float4*>(p.part + slot);
            for (int u = etid; u < nt * 32; u += 256) __stcg(dst4 + u, src4[u]);
            __threadfence();
            asm volatile("bar.sync 3, 256;" ::: "memory");   // every partial of this CTA is out; s_part is free again
            if (etid == 0) {
              const uint32_t ticket = atomicAdd(p.tickets + w.tile_id, 1u);
              bar.reduce_last = ticket == static_cast<uint32_t>(p.splits - 1) ? 1 : 0;
              if (bar.reduce_last) p.tickets[w.tile_id] = 0;      // ready for the next launch
            }
            asm volatile("bar.sync 3, 256;" ::: "memory");
            if (bar.reduce_last) {
              __threadfence();
              const float4* base4 = reinterpret_cast<const float4*>(p.part + static_cast<size_t>(w.tile_id) * p.splits * (MAXN * 128));
              for (int u = etid; u < nt * 32; u += 256) {
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp = 0; sp < p.splits; ++sp) {
                  const float4 v = __ldcg(base4 + static_cast<size_t>(sp) * (MAXN * 32) + u);
                  sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                const int r = u >> 5, c4 = u & 31;
                const int grow = t0 + r;
                const size_t o = static_cast<size_t>(grow) * p.Nout + w.n0 + c4 * 4;
                if (p.out) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = pk;
                if (p.rows_per_peer > 0) {
                  const int pr = grow / p.rows_per_peer;
                  if (pr < p.n_peers)
                    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out_peers[pr]) +
                                              static_cast<size_t>(grow % p.rows_per_peer) * p.Nout + w.n0 + c4 * 4) = pk;
                } else {
                  for (int pr = 0; pr < p.n_peers; ++pr)
                    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out_peers[pr]) + o) = pk;
                }
              }
            }
          } else if (!p.out_f32) {
            // all 256 epilogue threads store the tile: 16 bytes (8 features) per thread and step
            const uint4* src = reinterpret_cast<const uint4*>(s_out);
            for (int u = etid; u < nt * 16; u += 256) {
              const int r = u >> 4, c = u & 15;
              const uint4 v = src[u];
              const int grow = t0 + r;
              const size_t o = static_cast<size_t>(grow) * p.Nout + w.n0 + c * 8;
              if (p.out) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = v;
              if (p.rows_per_peer > 0) {
                const int pr = grow / p.rows_per_peer;
                if (pr < p.n_peers)
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out_peers[pr]) +
                                            static_cast<size_t>(grow % p.rows_per_peer) * p.Nout + w.n0 + c * 8) = v;
              } else {
                for (int pr = 0; pr < p.n_peers; ++pr)
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out_peers[pr]) + o) = v;
              }
            }
          }
        }
        if (f < p.Nout && ((!kAlternate) || (grp == 0 && p.out_f32 && p.part == nullptr))) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) {
            if (j < my_n) {
              const size_t o = static_cast<size_t>(t0 + colh * 64 + j) * p.Nout + f;
              if (p.out_f32) {
                atomicAdd(reinterpret_cast<float*>(p.out) + o, acc[j]);
              } else {
                const __nv_bfloat16 v = __float2bfloat16(acc[j]);
                if (p.out) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = v;
                if (p.rows_per_peer > 0) {
                  const int row = t0 + colh * 64 + j, r = row / p.rows_per_peer;
                  if (r < p.n_peers)
                    reinterpret_cast<__nv_bfloat16*>(p.out_peers[r])[static_cast<size_t>(row % p.rows_per_peer) * p.Nout + f] = v;
                } else {
                  for (int r = 0; r < p.n_peers; ++r) reinterpret_cast<__nv_bfloat16*>(p.out_peers[r])[o] = v;
                }
              }
            }
          }
        }
        if (etid == 0) F8_T(2, (idx - blockIdx.x) / gridDim.x, 3);     // stored
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (p.n_peers > 0 && threadIdx.x == 0) __threadfence_system();      // one cumulative fence per CTA after the barrier
  if (warp == 1) ptx::tmem_dealloc<512>(tmem);
}

// Compact the experts that received rows: active[0..n) ascending, n in n_active[0].
__global__ void f8_active_experts_kernel(const int32_t* __restrict__ offs, int E, int32_t* __restrict__ active,
                                         int32_t* __restrict__ n_active) {
  __shared__ int s_count;
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  for (int base = 0; base < E; base += blockDim.x) {
    const int e = base + threadIdx.x;
    const bool on = e < E && offs[e + 1] > offs[e];
    const unsigned m = __ballot_sync(0xffffffffu, on);
    int warp_base = 0;
    if ((threadIdx.x & 31) == 0 && m) warp_base = atomicAdd(&s_count, __popc(m));
    warp_base = __shfl_sync(0xffffffffu, warp_base, 0);
    if (on) active[warp_base + __popc(m & ((1u << (threadIdx.x & 31)) - 1))] = e;
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_active = s_count;
}

// bf16 [M, K] -> fp8 e4m3 [M, K] with one fp32 scale per (row, 128 columns).
// mode 1: input is [M, 2K] = gate | up and the value quantised is silu(gate) * up.
// row_limit (nullable, device): only rows below *row_limit are touched (the rows a routing step
// actually filled in a buffer sized for the worst case).
__global__ void __launch_bounds__(128)
act_quant_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, float* __restrict__ s,
                 int M, int K, int mode, const int32_t* __restrict__ row_limit) {
  const int KB = K / 128;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= M * KB) return;
  const int m = wid / KB, kb = wid % KB;
  if (row_limit != nullptr && m >= *row_limit) return;
  const __nv_bfloat16* row = x + static_cast<size_t>(m) * ldx;
  const uint2 raw = *reinterpret_cast<const uint2*>(row + kb * 128 + lane * 4);
  const __nv_bfloat162* pr = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float v[4];
  { const float2 a = __bfloat1622float2(pr[0]), b = __bfloat1622float2(pr[1]); v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; }
  if (mode == 1) {
    const uint2 raw2 = *reinterpret_cast<const uint2*>(row + K + kb * 128 + lane * 4);
    const __nv_bfloat162* pu = reinterpret_cast<const __nv_bfloat162*>(&raw2);
    const float2 a = __bfloat1622float2(pu[0]), b = __bfloat1622float2(pu[1]);
    const float u[4] = {a.x, a.y, b.x, b.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = v[i] / (1.f + __expf(-v[i])) * u[i];
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-4f) / 448.f;
  const float inv = 1.f / scale;
  uint32_t pk = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) pk |= static_cast<uint32_t>(float_to_fp8_e4m3(v[i] * inv)) << (8 * i);
  reinterpret_cast<uint32_t*>(q + static_cast<size_t>(m) * K + kb * 128)[lane] = pk;
  if (lane == 0) s[static_cast<size_t>(m) * KB + kb] = scale;
}

// Weights are stored tile-major: [E, Nout/128, K/128, 128 rows, 128 bytes], so the 16 KB
// one CTA needs per K block is one contiguous run in HBM.
static int make_w_tmap(CUtensorMap* out, const void* w, int E, int Nout, int K) {
  const uint64_t rows = static_cast<uint64_t>(E) * (Nout / 128) * (K / 128) * 128;
  return make_tmap_2d(out, w, 1, rows, 128, 128, 128, 128, true);
}

template <int MAXN>
static int launch_f8(const CUtensorMap& tw, const CUtensorMap& tx, const F8Params& p, int grid, cudaStream_t stream) {
  static PerDeviceOnce once;
  const int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(fp8_grouped_gemm_kernel<MAXN>), F8Geom<MAXN>::kSmem, once);
  if (rc != 0) return rc;
  fp8_grouped_gemm_kernel<MAXN><<<grid, kF8Threads, F8Geom<MAXN>::kSmem, stream>>>(tw, tx, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// x8 [M,K] fp8, sx [M,K/128]; w8 TILE-MAJOR [E,Nout/128,K/128,128,128] fp8, sw [E,Nout/128,K/128];
// offs [E+1] or null (E==1).  y: bf16 [M,Nout] when splits == 1, otherwise fp32 [M,Nout]
// accumulated with red.add (the caller clears it).  K and Nout must be multiples of 128,
// K <= 18432.  work: int32 [E + 1] scratch for the list of active experts (required when E > 1).
// max_rows: upper bound on the rows of any one expert (a performance hint that picks the ring
// geometry; any value is correct).
int ulc_fp8_grouped_gemm_peers(const void* x8, const float* sx, const void* w8, const float* sw, const int32_t* offs,
                               int M, int Nout, int K, int E, int splits, int max_rows, void* y,
                               void* const* peer_out, int n_peers, int32_t* work, int32_t* status,
                               cudaStream_t stream);

#ifdef ULC_F8_TRACE
int ulc_f8_trace_read(long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, ulc::f8_trace, sizeof(long long) * 3 * 64 * 4));
}
#endif

int ulc_fp8_grouped_gemm(const void* x8, const float* sx, const void* w8, const float* sw, const int32_t* offs,
                         int M, int Nout, int K, int E, int splits, int max_rows, void* y, int32_t* work,
                         int32_t* status, cudaStream_t stream) {
  return ulc_fp8_grouped_gemm_peers(x8, sx, w8, sw, offs, M, Nout, K, E, splits, max_rows, y, nullptr, 0, work,
                                    status, stream);
}

// As above, and every output tile is additionally stored (bf16) to `n_peers` buffers given as HOST
// array `peer_out` of device pointers (peer GPUs' receive slots): the scatter phase of a one-shot
// all-reduce runs in the GEMM epilogue.  Requires splits == 1; `y` may be null.
static int f8_gemm_impl(const void* x8, const float* sx, const void* w8, const float* sw, const int32_t* offs,
                       int M, int Nout, int K, int E, int splits, int max_rows, void* y, void* const* peer_out,
                       int n_peers, int rows_per_peer, int32_t* work, int32_t* status, cudaStream_t stream,
                       bool work_ready = false, void* splitk_ws = nullptr, long long splitk_ws_bytes = 0) {
  if (M <= 0 || E <= 0) return 0;
  if ((K % 128) || (Nout % 128) || K / 128 > kF8MaxKB) return -kErrUnsupported;
  if (E > 1 && (offs == nullptr || work == nullptr)) return -kErrUnsupported;
  if (splits < 1) splits = 1;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sm_count = 148;
  }
  CUtensorMap tw, tx;
  int rc = make_w_tmap(&tw, w8, E, Nout, K);
  if (rc != 0) return rc;
  rc = make_tmap_2d(&tx, x8, 1, M, K, K, 16, 128, true);
  if (rc != 0) return rc;
  F8Params p;
  p.sw = sw; p.sx = sx; p.offs = offs; p.out = y; p.status = status;
  p.M = M; p.Nout = Nout; p.K = K; p.E = E;
  if (n_peers < 0 || n_peers > 8 || (n_peers > 0 && splits > 1 && splitk_ws == nullptr)) return -kErrUnsupported;
  p.n_peers = n_peers;
  for (int r = 0; r < 8; ++r) p.out_peers[r] = r < n_peers ? peer_out[r] : nullptr;
  const int KB = K / 128;
  p.kb_per_split = (KB + splits - 1) / splits;
  p.splits = (KB + p.kb_per_split - 1) / p.kb_per_split;
  p.out_f32 = splits > 1;
  p.part = nullptr;
  p.tickets = nullptr;
  if (max_rows <= 0 || max_rows > M) max_rows = M;
  if (splitk_ws != nullptr && p.splits > 1) {
    // tickets (one per feature tile, 4 KB reserved) then the partial tiles
    const int geom = max_rows <= 16 ? 16 : 32;
    const long long tiles = Nout / kF8BM;
    const long long need = 4096 + tiles * p.splits * geom * 128 * 4;
    if (E != 1 || M > geom || max_rows > 32 || tiles > 1024 || need > splitk_ws_bytes) return -kErrUnsupported;
    p.tickets = reinterpret_cast<uint32_t*>(splitk_ws);
    p.part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(splitk_ws) + 4096);
    p.out_f32 = 0;
  }
  p.active = nullptr;
  p.n_active = nullptr;
  p.rows_per_peer = rows_per_peer;
  if (E > 1) {
    // work = [count, active expert ids...]; the routing kernel can leave it ready
    if (!work_ready) f8_active_experts_kernel<<<1, 256, 0, stream>>>(offs, E, work + 1, work);
    p.active = work + 1;
    p.n_active = work;
  }
  const long long max_items = static_cast<long long>(E) * (Nout / kF8BM) * p.splits;
  const int grid = static_cast<int>(max_items < sm_count ? max_items : sm_count);
  if (max_rows <= 16) return launch_f8<16>(tw, tx, p, grid, stream);
  if (max_rows <= 32) return launch_f8<32>(tw, tx, p, grid, stream);
  if (max_rows <= 64) return launch_f8<64>(tw, tx, p, grid, stream);
  return launch_f8<128>(tw, tx, p, grid, stream);
}

int ulc_fp8_grouped_gemm_peers(const void* x8, const float* sx, const void* w8, const float* sw, const int32_t* offs,
                               int M, int Nout, int K, int E, int splits, int max_rows, void* y,
                               void* const* peer_out, int n_peers, int32_t* work, int32_t* status,
                               cudaStream_t stream) {
  return f8_gemm_impl(x8, sx, w8, sw, offs, M, Nout, K, E, splits, max_rows, y, peer_out, n_peers, 0, work, status, stream);
}

// As ulc_fp8_grouped_gemm for E > 1, with `work` = [number of experts that received rows, their ids
// ascending] already on the device (written by the routing sort), so no compaction kernel runs.
int ulc_fp8_grouped_gemm_prepared(const void* x8, const float* sx, const void* w8, const float* sw, const int32_t* offs,
                                  int M, int Nout, int K, int E, int max_rows, void* y, int32_t* work, int32_t* status,
                                  cudaStream_t stream) {
  if (E <= 1 || work == nullptr) return -kErrUnsupported;
  return f8_gemm_impl(x8, sx, w8, sw, offs, M, Nout, K, E, 1, max_rows, y, nullptr, 0, 0, work, status, stream, true);
}

// Dense split-K GEMM with the reduction inside the kernel: y (bf16 [M, Nout], nullable) and/or the
// peer buffers get the finished result; `workspace` (device memory, `ws_bytes` long, at least
// 4096 + (Nout / 128) * splits * 32 * 128 * 4 bytes, its first 4096 bytes zero before the first use)
// holds the partial tiles and the tickets and is left ready for the next call.  M <= 32.  Calls that
// share a workspace must not overlap on the GPU.
int ulc_fp8_gemm_splitk(const void* x8, const float* sx, const void* w8, const float* sw, int M, int Nout, int K,
                        int splits, int max_rows, void* y, void* const* peer_out, int n_peers, int rows_per_peer,
                        void* workspace, long long ws_bytes, int32_t* status, cudaStream_t stream) {
  if (workspace == nullptr) return -kErrUnsupported;
  return f8_gemm_impl(x8, sx, w8, sw, nullptr, M, Nout, K, 1, splits, max_rows, y, peer_out, n_peers, rows_per_peer,
                      nullptr, status, stream, false, workspace, ws_bytes);
}

// GEMM + reduce-scatter: as ulc_fp8_grouped_gemm_peers (one weight), but row m of the result is
// stored only to peer m / rows_per_peer, at its row m % rows_per_peer.  Every rank then sums the
// partial blocks it received (the o_proj of tensor-parallel attention feeding data-parallel layers).
int ulc_fp8_gemm_reduce_scatter(const void* x8, const float* sx, const void* w8, const float* sw, int M, int Nout,
                                int K, int rows_per_peer, void* const* peer_out, int n_peers, int32_t* status,
                                cudaStream_t stream) {
  if (rows_per_peer <= 0 || (M + rows_per_peer - 1) / rows_per_peer > n_peers) return -kErrUnsupported;
  return f8_gemm_impl(x8, sx, w8, sw, nullptr, M, Nout, K, 1, 1, M, nullptr, peer_out, n_peers, rows_per_peer, nullptr,
                      status, stream);
}

int ulc_act_quant_rows(const void* x, long long ldx, void* q, float* s, int M, int K, int mode,
                       const int32_t* row_limit, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K % 128) return -kErrUnsupported;
  const long long warps = static_cast<long long>(M) * (K / 128);
  act_quant_kernel<<<static_cast<int>((warps + 3) / 4), 128, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<uint8_t*>(q), s, M, K, mode, row_limit);
  return static_cast<int>(cudaGetLastError());
}

int ulc_act_quant(const void* x, long long ldx, void* q, float* s, int M, int K, int mode, cudaStream_t stream) {
  return ulc_act_quant_rows(x, ldx, q, s, M, K, mode, nullptr, stream);
}

}  // extern "C"
