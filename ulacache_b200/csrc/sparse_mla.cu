// Sparse MLA decode attention fused with the KV gather (tcgen05 + TMEM).
//
// For every query token the indexer selected up to 2048 KV records; their
// resolved locations (owner rank << 28 | HBM slot) arrive as int32 [B, K].  One
// CTA handles one (query, block of 64 heads, KV split).  Its producer warps
// fetch the selected 656-byte fp8 records STRAIGHT from the owners' page pools —
// this GPU's HBM or a peer's HBM over NVLink, with plain 16-byte loads issued by
// this CTA (no staging copy, no multicast) — dequantise them (4 fp32 group
// scales per token) into bf16 tiles in shared memory laid out for the tensor
// core, and the MMA warp runs S = Q K^T and O += P V with tcgen05.mma, both
// accumulators living in TMEM.  Softmax warps read S from TMEM, keep running
// row maxima / sums, and write P (bf16) back through shared memory.
//
//   Q   [B, H, 576] bf16 (512 latent-absorbed dims + 64 rotary), loaded by TMA
//   KV  records: 512 fp8 e4m3 | 4 fp32 scales | 64 bf16 rotary   (or 576 bf16)
//   out [B, H, 512] bf16,  lse [B, H] fp32 (natural log)
//
// Tile: 64 heads (MMA M = 64) x 64 tokens, double buffered.  TMEM: O is two
// 64x256 fp32 accumulators sharing columns [0,256) on interleaved lane halves;
// S is two 64x64 partial accumulators (even / odd 64-dim slabs of the contraction,
// one per MMA-issuing thread) per buffer at columns [256,512).
//
// CTA pair (template PAIR, used when the head blocks come in twos): the two CTAs that serve the two
// head blocks of one (query, KV split) need the SAME K tiles.  They run as a cluster of two; each CTA's
// producer warps gather and dequantise HALF of every tile (32 records) and store it into BOTH CTAs'
// shared memory (distributed shared memory), so the scattered record reads - the stage that bounds the
// tile rate - are halved per SM and every record crosses NVLink / HBM once instead of twice.  A stage's
// "full" barrier counts the producer warps of both CTAs; its "free" barrier counts the MMA issuers of
// both (their commits are delivered to both CTAs), since either CTA's producers write into both.
// Measured (one B200, 32 queries x 128 heads x 2048 records): 73.4 us per layer against 68.3 us for
// independent CTAs, and 116.6 against 108.5 us for the owner-side attention of the two-rank micro-benchmark.
// Halving the gather per SM does not shorten a tile, so the gather rate is not what bounds it: the period
// is set by the dependent chain store -> QK^T -> softmax -> PV of which two stages are in flight, and the
// pair adds distributed-shared-memory stores and cluster-scope barriers to that chain.  OFF by default
// (ulc_sparse_mla_set_pair / ULC_MLA_PAIR=1 switch it on).
//
// The reference library has no attention kernel (it hands rows to FlashMLA) and
// moves remote rows with record_pull_cached_impl
// (ulacache/csrc/cache/common.cuh:1037) into a local buffer first; this kernel
// replaces that pull + the external attention call.
#include "ulc/launch.h"
#include "ulc/pool.h"
#include "ulc/ptx.cuh"
#include "ulc/tmap.h"

namespace ulc {

constexpr int kMlaM = 64;            // heads per CTA
constexpr int kMlaTile = 64;         // tokens per tile
constexpr int kSlab = 64 * 128;      // one 64-row x 128-byte swizzled slab
constexpr int kSlabs = 9;            // 8 latent slabs (64 dims each) + 1 rotary slab
constexpr int kQBytes = kSlabs * kSlab;
constexpr int kKBytes = kSlabs * kSlab;
constexpr int kMlaStages = 2;
constexpr int kSoftmaxWarps = 4;
constexpr int kMmaIssuers = 2;
constexpr int kProducerWarps = 8;
constexpr int kMlaThreads = (kSoftmaxWarps + kMmaIssuers + kProducerWarps) * 32;   // 448
constexpr int kMlaSmem = 1024 + kQBytes + kMlaStages * kKBytes + 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0;
constexpr uint32_t kColS = 256;
constexpr float kRescaleThreshold = 8.0f;   // in log2 units

struct MlaParams {
  PoolView pv;
  const int32_t* loc;        // [B, K] resolved locations, -1 masked
  const int32_t* lens;       // [B] valid columns per row (nullable)
  __nv_bfloat16* out;        // [B, H, 512]
  float* lse;                // [B, H] (nullable)
  float* part_o;             // [splits, B, H, 512] when splits > 1
  float* part_lse;           // [splits, B, H]
  int32_t* status;
  long long loc_stride;
  int B, H, K, splits;
  long long out_sb, out_sh;  // element strides of `out` over queries and heads
  float scale_log2;          // softmax scale * log2(e)
  int format;                // 0 = scaled656 fp8, 2 = bf16 1152
};

struct MlaBarriers {
  uint64_t qfull;
  uint64_t kfull[kMlaStages];
  uint64_t kfree[kMlaStages];
  uint64_t sfull[2];
  uint64_t pready[kMlaStages];
  uint64_t odone;
  uint32_t tmem_base;
  int abort_flag;
  uint32_t mask[kMlaStages][2];   // valid-token bits of the tile in each stage
  uint8_t mask_pair[kMlaStages][16];   // PAIR: 4 valid bits per producer warp of the pair (CTA rank * 8 + warp)
};

// Optional per-tile timeline of CTA (0,0,0), compiled in with -DULC_MLA_TRACE (development only):
// mla_trace[role][tile][event] = clock64 at that point.
#ifdef ULC_MLA_TRACE
__device__ long long mla_trace[4][64][8];
#define MLA_T(role, tile, ev)                                                                   \
  do {                                                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (tile) < 64)                   \
      mla_trace[role][tile][ev] = clock64();                                                    \
  } while (0)
#else
#define MLA_T(role, tile, ev) do {} while (0)
#endif

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 16 fp8 values (one 16-byte chunk) * scale -> 16 bf16 (two 16-byte chunks)
__device__ __forceinline__ void dequant16(const uint4& in, float scale, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw h0 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffff), __NV_E4M3);
    const __half2_raw h1 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h0));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&h1));
    const __nv_bfloat162 x = __floats2bfloat162_rn(a.x * scale, a.y * scale);
    const __nv_bfloat162 y = __floats2bfloat162_rn(b.x * scale, b.y * scale);
    o[2 * i] = *reinterpret_cast<const uint32_t*>(&x);
    o[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&y);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

template <bool PAIR>
__global__ void __launch_bounds__(kMlaThreads, 1)
sparse_mla_decode_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_qr,
                         const MlaParams p) {
  extern __shared__ uint8_t mla_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mla_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;
  uint8_t* sk = smem + kQBytes;
  MlaBarriers& bar = *reinterpret_cast<MlaBarriers*>(smem + kQBytes + kMlaStages * kKBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int hb = blockIdx.x;           // head block
  const int b = blockIdx.y;            // query
  const int split = blockIdx.z;
  const int h0 = hb * kMlaM;
  const uint32_t crank = PAIR ? ptx::cluster_ctarank() : 0u;      // which half of every tile this CTA gathers

  // token range of this CTA, in whole tiles
  int n_valid = p.lens ? min(max(p.lens[b], 0), p.K) : p.K;
  const int per = ((p.K + p.splits - 1) / p.splits + kMlaTile - 1) / kMlaTile * kMlaTile;
  const int c0 = split * per;
  const int c1 = min(n_valid, c0 + per);
  const int ntiles = c1 > c0 ? (c1 - c0 + kMlaTile - 1) / kMlaTile : 0;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar.qfull, 1);
    for (int s = 0; s < kMlaStages; ++s) {
      ptx::mbar_init(&bar.kfull[s], PAIR ? 2 * kProducerWarps : kProducerWarps);
      ptx::mbar_init(&bar.kfree[s], PAIR ? 2 * kMmaIssuers : kMmaIssuers);
      ptx::mbar_init(&bar.sfull[s], kMmaIssuers);
      ptx::mbar_init(&bar.pready[s], kSoftmaxWarps);
    }
    ptx::mbar_init(&bar.odone, kMmaIssuers);
    bar.abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_qr);
  }
  if (warp == kSoftmaxWarps) {
    ptx::tmem_alloc<kTmemCols>(&bar.tmem_base);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) ptx::cluster_sync_all();      // the peer's barriers exist before anyone arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem = bar.tmem_base;
  volatile int* abort_flag = &bar.abort_flag;

  if (warp < kSoftmaxWarps) {
    // =============================================================== softmax ==
    // MMA M = 64 puts row r of an accumulator in lane (r % 16) of quarter r / 16, so a warp
    // sees 16 rows, and lanes 16..31 are free for a second accumulator of the same rows:
    //   S: even-slab partial on lanes 0..15, odd-slab partial on lanes 16..31 (one per issuer);
    //   O: dims [0,256) on lanes 0..15, dims [256,512) on lanes 16..31.
    // Both lanes of a row share the softmax work: lane < 16 takes tokens 0..31 of the tile,
    // lane >= 16 tokens 32..63.
    const int row = warp * 16 + (lane & 15);    // head row inside the block
    const int half = lane >> 4;                 // which 32 tokens of S / which 256 dims of O
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_run = -INFINITY;                    // running max of raw scores (same in both lanes of a row)
    float l_run = 0.f;                          // running sum over this lane's tokens
    bool ok = true;
    for (int i = 0; i < ntiles && ok; ++i) {
      const int st = i & 1;
      if (*abort_flag || !ptx::mbar_wait(&bar.sfull[st], (i >> 1) & 1)) {
        if (!*abort_flag && lane == 0) report(p.status, kErrPipeline, 1000 + i);
        *abort_flag = 1;
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      if (threadIdx.x == 0) MLA_T(0, i, 0);      // S ready
      // This lane's 32 scores: its own partial of its token half plus the partner lane's.
      float sv[32];
      {
        uint32_t a[32], c[32];
        ptx::tmem_ld32(tmem + lane_base + kColS + st * 64, a);        // tokens 0..31 of my partial
        ptx::tmem_ld32(tmem + lane_base + kColS + st * 64 + 32, c);   // tokens 32..63
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float keep = __uint_as_float(half ? c[j] : a[j]);
          const float give = __uint_as_float(half ? a[j] : c[j]);
          sv[j] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
        }
      }
      uint32_t mask;
      if constexpr (PAIR) {
        // tokens [32 half, 32 half + 32) were gathered by CTA `half` of the pair: 4 bits per producer warp
        const uint64_t nib = *reinterpret_cast<const volatile uint64_t*>(&bar.mask_pair[st][half * 8]);
        mask = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) mask |= static_cast<uint32_t>((nib >> (8 * w)) & 0xfu) << (4 * w);
      } else {
        mask = bar.mask[st][half];
      }
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        sv[j] = ((mask >> j) & 1u) ? sv[j] : -INFINITY;
        mx = fmaxf(mx, sv[j]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run, mx);
      if (threadIdx.x == 0) MLA_T(0, i, 1);      // S read, max known
      // Every tile waits for the previous PV before it may signal P: an mbarrier parity
      // wait can only tell adjacent phases apart, so this warp must never fall two
      // completions behind `odone`.
      if (i > 0) {
        if (!ptx::mbar_wait(&bar.odone, (i - 1) & 1)) {
          if (lane == 0) report(p.status, kErrPipeline, 2000 + i);
          *abort_flag = 1;
          ok = false;
        }
        ptx::tc_fence_after();
      }
      if (threadIdx.x == 0) MLA_T(0, i, 2);      // previous PV done
      // rescale lazily: only when the maximum moved by more than the threshold
      const bool need = (m_new - m_run) * p.scale_log2 > kRescaleThreshold || (m_run == -INFINITY && m_new > -INFINITY);
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = need ? (m_run == -INFINITY ? 0.f : exp2f((m_run - m_new) * p.scale_log2)) : 1.f;
        if (i > 0 && ok) {
#pragma unroll 1
          for (int c = 0; c < 256; c += 32) {
            uint32_t o[32];
            ptx::tmem_ld32(tmem + lane_base + kColO + c, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st32(tmem + lane_base + kColO + c, o);
          }
          tmem_st_wait();
        }
        if (need) { l_run *= alpha; m_run = m_new; }
      }
      if (threadIdx.x == 0) MLA_T(0, i, 3);      // rescale done
      // P = exp2((s - m) * scale), bf16, into the rotary slab of this stage (dead after QK^T)
      {
        uint8_t* pslab = sk + st * kKBytes + 8 * kSlab;
        const float mscaled = m_run == -INFINITY ? 0.f : m_run * p.scale_log2;
        float sum = 0.f;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float a = exp2f(sv[ch * 8 + 2 * q] * p.scale_log2 - mscaled);
            const float c = exp2f(sv[ch * 8 + 2 * q + 1] * p.scale_log2 - mscaled);
            const __nv_bfloat162 pb = __floats2bfloat162_rn(a, c);
            sum += __bfloat162float(pb.x) + __bfloat162float(pb.y);
            w[q] = *reinterpret_cast<const uint32_t*>(&pb);
          }
          *reinterpret_cast<uint4*>(pslab + ptx::sw128_offset(row, half * 4 + ch)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        l_run += sum;                           // (each lane sums its own 32 tokens)
      }
      ptx::fence_async_smem();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar.pready[st]);
      if (threadIdx.x == 0) MLA_T(0, i, 4);      // P published
    }
    // ------------------------------------------------------------- epilogue --
    if (ok && ntiles > 0) {
      if (!ptx::mbar_wait(&bar.odone, (ntiles - 1) & 1)) {
        if (lane == 0) report(p.status, kErrPipeline, 3000);
        *abort_flag = 1;
        ok = false;
      }
      ptx::tc_fence_after();
    }
    ok = __all_sync(0xffffffffu, ok);
    const float l_tot = l_run + __shfl_xor_sync(0xffffffffu, l_run, 16);
    const int h = h0 + row;
    if (ok) {
      // every lane runs the (warp-aligned) TMEM loads; only rows of real heads are stored
      const bool store = h < p.H;
      const bool have = ntiles > 0;
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      const float lse = l_tot > 0.f ? (m_run * p.scale_log2 + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      const size_t row_index = static_cast<size_t>(b) * p.H + (store ? h : 0);
      __nv_bfloat16* dst16 = p.out + static_cast<size_t>(b) * p.out_sb + static_cast<size_t>(store ? h : 0) * p.out_sh + half * 256;
      float* dst32 = p.splits > 1
                         ? p.part_o + (static_cast<size_t>(split) * p.B * p.H + row_index) * 512 + half * 256
                         : nullptr;
#pragma unroll 1
      for (int c = 0; c < 256; c += 32) {
        uint32_t o[32];
        if (have) {
          ptx::tmem_ld32(tmem + lane_base + kColO + c, o);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0;
        }
        if (!store) continue;
        if (p.splits == 1) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv,
                                                           __uint_as_float(o[2 * j + 1]) * inv);
            w[j] = *reinterpret_cast<const uint32_t*>(&v);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(dst16 + c + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
        } else {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float4 v;
            v.x = __uint_as_float(o[4 * q]) * inv;
            v.y = __uint_as_float(o[4 * q + 1]) * inv;
            v.z = __uint_as_float(o[4 * q + 2]) * inv;
            v.w = __uint_as_float(o[4 * q + 3]) * inv;
            *reinterpret_cast<float4*>(dst32 + c + q * 4) = v;
          }
        }
      }
      if (store && half == 0) {
        if (p.splits == 1) { if (p.lse) p.lse[row_index] = lse; }
        else p.part_lse[static_cast<size_t>(split) * p.B * p.H + row_index] = lse;
      }
    } else if (p.splits > 1 && h < p.H && half == 0) {
      // A CTA that gave up (a bounded wait expired; the status word says so) still marks its
      // cells as empty, so that the merge does not read what an earlier call left in the scratch.
      p.part_lse[static_cast<size_t>(split) * p.B * p.H + static_cast<size_t>(b) * p.H + h] = -INFINITY;
    }
  } else if (warp < kSoftmaxWarps + kMmaIssuers) {
    // =========================================================== MMA issuers ==
    // Two issuing threads: the rate at which ONE thread can issue tcgen05.mma is the
    // bottleneck for tiles this small.  Issuer 0 takes the even 64-dim slabs of QK^T and
    // the first 256 dims of PV, issuer 1 the odd slabs and the last 256 dims; each owns
    // its own S partial accumulator (summed by the softmax warps).
    const int me = warp - kSoftmaxWarps;
    // one elected thread of the converged warp issues: tcgen05.mma from a `lane == 0` branch
    // of a diverged warp was measured 3.5x slower to issue
    if (ntiles > 0 && ptx::elect_one()) {
      constexpr uint32_t idesc_qk = ptx::umma_idesc(kMlaM, kMlaTile, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = ptx::umma_idesc(kMlaM, 256, 1, 1, 0, 1);
      const uint64_t q_desc = ptx::umma_desc_sw128(ptx::smem_u32(sq));
      bool ok = true;
      if (me == 0) {
        // load Q with TMA: eight latent boxes and the rotary box, 64 rows x 64 columns each
        ptx::mbar_expect_tx(&bar.qfull, kQBytes);
        for (int s = 0; s < kSlabs - 1; ++s) ptx::tma_load_3d(sq + s * kSlab, &tmap_q, &bar.qfull, s * 64, h0, b);
        ptx::tma_load_3d(sq + (kSlabs - 1) * kSlab, &tmap_qr, &bar.qfull, 0, h0, b);
      }
      if (!ptx::mbar_wait(&bar.qfull, 0)) {
        report(p.status, kErrPipeline, 4000);
        *abort_flag = 1;
        ok = false;
      }
      auto issue_qk = [&](int i) {           // K tile i is known to be in shared memory
        const int st = i & 1;
        ptx::tc_fence_after();
        if (me == 0) MLA_T(1, i, 0);             // K tile ready
        const uint64_t k_desc = ptx::umma_desc_sw128(ptx::smem_u32(sk + st * kKBytes));
        const uint32_t d = tmem + (me ? (16u << 16) : 0u) + kColS + st * 64;   // odd-slab partial on lanes 16..31
#pragma unroll
        for (int s = 0; s < kSlabs; ++s) {
          if ((s & 1) != me) continue;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            ptx::umma_bf16(d, ptx::umma_desc_advance(q_desc, s * kSlab + kk * 32),
                           ptx::umma_desc_advance(k_desc, s * kSlab + kk * 32), idesc_qk, (s > me || kk > 0) ? 1u : 0u);
        }
        ptx::umma_commit(&bar.sfull[st]);
        if (me == 0) MLA_T(1, i, 1);             // QK^T issued
      };
      auto issue_pv = [&](int i) {           // P of tile i is known to be in shared memory
        const int st = i & 1;
        ptx::tc_fence_after();
        if (me == 0) MLA_T(1, i, 2);             // P ready
        const uint32_t k_addr = ptx::smem_u32(sk + st * kKBytes);
        const uint64_t p_desc = ptx::umma_desc_sw128(k_addr + 8 * kSlab);
        const uint64_t v_desc = ptx::umma_desc_sw128_mn(k_addr + me * 4 * kSlab, kSlab, 1024);
        const uint32_t d = tmem + (me ? (16u << 16) : 0u) + kColO;      // second half on lanes 16..31
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          ptx::umma_bf16(d, ptx::umma_desc_advance(p_desc, kk * 32), ptx::umma_desc_advance(v_desc, kk * 2048),
                         idesc_pv, (i | kk) != 0);
        if constexpr (PAIR) ptx::umma_commit_mc(&bar.kfree[st], 0x3);     // the stage is free in BOTH CTAs' eyes
        else ptx::umma_commit(&bar.kfree[st]);
        ptx::umma_commit(&bar.odone);
        if (me == 0) MLA_T(1, i, 3);             // PV issued
      };
      // Issue whatever is ready: PV(i) as soon as P(i) is published, QK^T(i+1) as soon as its
      // K tile is, in either order.  (A fixed QK(i+1)-then-PV(i) order puts the dequantisation
      // of tile i+1, which can only start when PV(i-1) has freed its stage, in front of PV(i)
      // and serialises the two stages.)  QK^T(i+2) overwrites the S buffer of tile i, so it
      // stays behind PV(i), whose P was written after S(i) had been read.
      int qk_next = 0, pv_next = 0;
      long long idle_since = 0;
      while (ok && pv_next < ntiles) {
        if (pv_next < qk_next && ptx::mbar_test_wait(&bar.pready[pv_next & 1], (pv_next >> 1) & 1)) {
          issue_pv(pv_next++);
          idle_since = 0;
        } else if (qk_next < ntiles && qk_next <= pv_next + 1 &&
                   (PAIR ? ptx::mbar_test_wait_cluster(&bar.kfull[qk_next & 1], (qk_next >> 1) & 1)
                         : ptx::mbar_test_wait(&bar.kfull[qk_next & 1], (qk_next >> 1) & 1))) {
          issue_qk(qk_next++);
          idle_since = 0;
        } else {
          const long long now = clock64();
          if (idle_since == 0) idle_since = now;
          if (*abort_flag || now - idle_since > ptx::kWaitCycles) {
            if (!*abort_flag) report(p.status, kErrPipeline, 5000 + pv_next);
            *abort_flag = 1;
            ok = false;
          }
          __nanosleep(32);
        }
      }
    }
  } else {
    // ============================================================= producers ==
    // Eight warps, eight tokens each per tile.  A lane owns (token, quarter of the record)
    // and keeps TWO tiles of loads in flight: the records of tile i+1 are requested before
    // tile i is dequantised, so the NVLink / HBM latency of one tile hides behind the
    // conversion and the MMAs of the previous one.  (Measured: the tile rate is bound by how many
    // scattered sector reads one SM keeps in flight through L1, about 9 B/clk, not by the math.)
    const int pw = warp - kSoftmaxWarps - kMmaIssuers;   // 0..7
    // alone: 8 tokens per warp, a lane owns a quarter of a record; pair: 4 tokens per warp out of this CTA's
    // 32, a lane owns an eighth of a record
    constexpr int kParts = PAIR ? 8 : 4;         // lanes per record
    constexpr int kLat = 32 / kParts;            // latent chunks (16 B) per lane
    constexpr int kRope = 8 / kParts;            // rotary chunks per lane
    const int tt = PAIR ? (lane & 3) : (lane & 7);       // token within the warp's group
    const int part = PAIR ? (lane >> 2) : (lane >> 3);   // which chunks of the record
    const int trow = PAIR ? static_cast<int>(crank) * 32 + pw * 4 + tt : pw * 8 + tt;   // row in the tile
    const uint32_t peer = crank ^ 1u;
    struct Regs { uint4 lat[8]; uint4 rope[2]; uint4 sc; const uint8_t* rec; };
    // Locations are read two tiles before the records they name, so that a fetch never
    // waits on the location load before it can issue its record loads.
    auto load_loc = [&](int i) -> int32_t {
      const int col = c0 + i * kMlaTile + trow;
      return (i < ntiles && col < c1) ? __ldg(p.loc + static_cast<size_t>(b) * p.loc_stride + col) : -1;
    };
    int32_t loc_q0 = load_loc(0), loc_q1 = load_loc(1);
    auto fetch = [&](int i, Regs& r) {      // called for i = 0, 1, 2, ... in order
      if (pw == 0 && lane == 0) MLA_T(2, i, 0);  // fetch begins
      const int32_t l = loc_q0;
      loc_q0 = loc_q1;
      loc_q1 = load_loc(i + 2);
      r.rec = nullptr;
      if (l >= 0) {
        const int slot = loc_slot(l);
        if (slot < p.pv.hbm_slots) r.rec = p.pv.hbm[loc_rank(l)] + static_cast<size_t>(slot) * p.pv.rec_bytes;
        else report(p.status, kErrBounds, l);
      }
      r.sc = make_uint4(0, 0, 0, 0);
      if (p.format == 0) {
#pragma unroll
        for (int j = 0; j < kLat; ++j)
          r.lat[j] = r.rec ? ptx::ld_nc16(r.rec + (part + kParts * j) * 16) : make_uint4(0, 0, 0, 0);
        if (r.rec) r.sc = ptx::ld_nc16(r.rec + kRec656ScaleOffset);
#pragma unroll
        for (int j = 0; j < kRope; ++j)
          r.rope[j] = r.rec ? ptx::ld_nc16(r.rec + kRec656RopeOffset + (part + kParts * j) * 16) : make_uint4(0, 0, 0, 0);
      }
    };
    auto store = [&](int i, const Regs& r) -> bool {
      const int st = i & 1;
      if (*abort_flag || !(PAIR ? ptx::mbar_wait_cluster(&bar.kfree[st], ((i >> 1) & 1) ^ 1)
                                : ptx::mbar_wait(&bar.kfree[st], ((i >> 1) & 1) ^ 1))) {
        if (!*abort_flag && lane == 0) report(p.status, kErrPipeline, 7000 + i);
        *abort_flag = 1;
        return false;
      }
      uint8_t* kt = sk + st * kKBytes;
      // one 16-byte chunk into the tile of this CTA and, in a pair, of the peer CTA as well
      auto put = [&](uint8_t* dst, const uint4& v) {
        *reinterpret_cast<uint4*>(dst) = v;
        if constexpr (PAIR) ptx::st_cluster16(ptx::mapa(ptx::smem_u32(dst), peer), v);
      };
      if (pw == 0 && lane == 0) MLA_T(2, i, 1);  // stage free
      if (p.format == 0) {
        const float scales[4] = {__uint_as_float(r.sc.x), __uint_as_float(r.sc.y), __uint_as_float(r.sc.z),
                                 __uint_as_float(r.sc.w)};
#pragma unroll
        for (int j = 0; j < kLat; ++j) {
          const int ch = part + kParts * j;      // 16-value chunk 0..31 of the latent
          uint4 lo, hi;
          dequant16(r.lat[j], scales[ch >> 3], lo, hi);
          uint8_t* slab = kt + (ch >> 2) * kSlab;
          put(slab + ptx::sw128_offset(trow, (ch & 3) * 2), lo);
          put(slab + ptx::sw128_offset(trow, (ch & 3) * 2 + 1), hi);
        }
#pragma unroll
        for (int j = 0; j < kRope; ++j)
          put(kt + 8 * kSlab + ptx::sw128_offset(trow, part + kParts * j), r.rope[j]);
      } else {
        // 576 bf16 = 72 chunks: latent chunks 0..63 then rotary 64..71; 18 per lane
        constexpr int kPer = 72 / kParts;        // chunks per lane: 18 alone, 9 in a pair
        constexpr int kStep = kPer / 3;
#pragma unroll 1
        for (int j0 = 0; j0 < kPer; j0 += kStep) {
          uint4 v[kStep];
#pragma unroll
          for (int j = 0; j < kStep; ++j)
            v[j] = r.rec ? ptx::ld_nc16(r.rec + (part + kParts * (j0 + j)) * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int j = 0; j < kStep; ++j) {
            const int ch = part + kParts * (j0 + j);
            put(kt + (ch >> 3) * kSlab + ptx::sw128_offset(trow, ch & 7), v[j]);
          }
        }
      }
      if constexpr (PAIR) {
        const uint32_t bits = __ballot_sync(0xffffffffu, r.rec != nullptr) & 0xfu;
        if (lane == 0) {
          uint8_t* cell = &bar.mask_pair[st][crank * 8 + pw];
          *reinterpret_cast<volatile uint8_t*>(cell) = static_cast<uint8_t>(bits);
          ptx::st_cluster_u8(ptx::mapa(ptx::smem_u32(cell), peer), bits);
        }
        ptx::fence_async_all();                 // both CTAs' tensor cores read what this warp stored
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&bar.kfull[st]), crank));
          ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&bar.kfull[st]), peer));
        }
      } else {
        const uint32_t bits = __ballot_sync(0xffffffffu, r.rec != nullptr) & 0xffu;
        if (lane == 0) reinterpret_cast<volatile uint8_t*>(&bar.mask[st][0])[pw] = static_cast<uint8_t>(bits);
        ptx::fence_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bar.kfull[st]);
      }
      if (pw == 0 && lane == 0) MLA_T(2, i, 2);  // tile published
      if (lane == 0) MLA_T(3, i, pw);            // ... by each producer warp
      return true;
    };
    Regs ra, rb;
    if (ntiles > 0) fetch(0, ra);
    for (int i = 0; i < ntiles; i += 2) {
      fetch(i + 1, rb);                 // (a fetch past the last tile loads nothing)
      if (!store(i, ra)) break;
      if (i + 1 >= ntiles) break;
      fetch(i + 2, ra);
      if (!store(i + 1, rb)) break;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  // neither CTA of a pair may leave while the other can still store into its shared memory or arrive on
  // its barriers (every wait above is bounded, so both get here even after a failure)
  if constexpr (PAIR) ptx::cluster_sync_all();
  if (warp == kSoftmaxWarps) ptx::tmem_dealloc<kTmemCols>(tmem);
}

// Merge KV splits: out = sum_s w_s * O_s with w_s = exp(lse_s - max) / sum.
// One WARP per (query, head) row: lane s reads split s's log-sum-exp once and the weights travel by
// shuffle; a lane owns 16 output dims and has every split's 16-byte loads of a step in flight before it
// uses one (two dependent memory round trips per row instead of four).  A split whose LSE is -inf saw no
// token and its partial O is not read.
constexpr int kCombineWarps = 8;
__global__ void __launch_bounds__(kCombineWarps * 32)
mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int rows, int splits) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float mine = lane < splits ? part_lse[static_cast<size_t>(lane) * rows + row] : -INFINITY;
  float m = mine;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float wgt = mine > -INFINITY ? expf(mine - m) : 0.f;
  float denom = wgt;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll
  for (int step = 0; step < 4; ++step) {
    const int d = step * 128 + lane * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 4) {
      float4 v[4];
      float w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int s = s0 + j;
        w[j] = __shfl_sync(0xffffffffu, wgt, s & 31);
        if (s >= splits) w[j] = 0.f;
        v[j] = w[j] > 0.f
                   ? *reinterpret_cast<const float4*>(part_o + (static_cast<size_t>(s) * rows + row) * 512 + d)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc.x = fmaf(w[j], v[j].x, acc.x);
        acc.y = fmaf(w[j], v[j].y, acc.y);
        acc.z = fmaf(w[j], v[j].z, acc.z);
        acc.w = fmaf(w[j], v[j].w, acc.w);
      }
    }
    const __nv_bfloat162 o0 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    const __nv_bfloat162 o1 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 ow;
    ow.x = *reinterpret_cast<const uint32_t*>(&o0);
    ow.y = *reinterpret_cast<const uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(row) * 512 + d) = ow;
  }
  if (lse && lane == 0) lse[row] = denom > 0.f ? m + logf(denom) : -INFINITY;
}

// 3-D map over a query tensor addressed as [query b][head h][dim]: box = 64 dims x 64 heads.
static int make_q_tmap(CUtensorMap* out, const void* q, int B, int H, int dims, long long sb, long long sh) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -1;
  if ((sb & 7) || (sh & 7) || (reinterpret_cast<uintptr_t>(q) & 15)) return -kErrAlignment;
  cuuint64_t dimv[3] = {static_cast<cuuint64_t>(dims), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(sh) * 2, static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[3] = {64, 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dimv, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// Bytes of fp32 scratch needed for `splits` > 1: partial outputs then partial LSEs.
#ifdef ULC_MLA_TRACE
int ulc_mla_trace_read(long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, ulc::mla_trace, sizeof(long long) * 4 * 64 * 8));
}
#endif

// CTA-pair launch (see the file comment): off unless switched on, it measured slower.
static int g_mla_pair = 0;
void ulc_sparse_mla_set_pair(int on) { g_mla_pair = on ? 1 : 0; }

long long ulc_sparse_mla_scratch_bytes(int B, int H, int splits) {
  if (splits <= 1) return 0;
  return static_cast<long long>(splits) * B * H * (512 + 1) * 4;
}

// General form.  The query comes in two strided pieces (element strides over queries / heads):
// q_lat[b][h][0..512) the latent-absorbed part and q_rope[b][h][0..64) the rotary part, so that the
// output of a head-batched absorb GEMM ([H, B, 512]) can be consumed without a transpose.  The
// output is written as out[b * out_sb + h * out_sh + d].  loc [B,K] int32 (row pitch loc_stride);
// lse [B,H] fp32 or null; scratch: ulc_sparse_mla_scratch_bytes() bytes when splits > 1 (the split
// merge always writes a dense [B,H,512] result, so splits > 1 needs out_sb = H*512, out_sh = 512).
int ulc_sparse_mla_decode_ex(const PoolView* pv, const void* q_lat, long long lat_sb, long long lat_sh,
                             const void* q_rope, long long rope_sb, long long rope_sh, const int32_t* loc,
                             long long loc_stride, const int32_t* lens, int B, int H, int K, float sm_scale,
                             int format, int splits, void* out, long long out_sb, long long out_sh, float* lse,
                             void* scratch, int32_t* status, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || K <= 0) return 0;
  if (format != 0 && format != 2) return -kErrUnsupported;
  if (pv->rec_bytes != (format == 0 ? kRec656Bytes : kRecBf16Bytes)) return -kErrUnsupported;
  if (splits < 1) splits = 1;
  if (splits > 1 && scratch == nullptr) return -kErrUnsupported;
  if (splits > 1 && (out_sb != static_cast<long long>(H) * 512 || out_sh != 512)) return -kErrUnsupported;
  if ((out_sb & 7) || (out_sh & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return -kErrAlignment;
  static PerDeviceOnce once, once_pair;
  int attr_rc = ensure_dynamic_smem(reinterpret_cast<const void*>(sparse_mla_decode_kernel<false>), kMlaSmem, once);
  if (attr_rc != 0) return attr_rc;
  attr_rc = ensure_dynamic_smem(reinterpret_cast<const void*>(sparse_mla_decode_kernel<true>), kMlaSmem, once_pair);
  if (attr_rc != 0) return attr_rc;
  CUtensorMap tq, tr;
  int r = make_q_tmap(&tq, q_lat, B, H, 512, lat_sb, lat_sh);
  if (r != 0) return r;
  r = make_q_tmap(&tr, q_rope, B, H, 64, rope_sb, rope_sh);
  if (r != 0) return r;
  MlaParams p;
  p.pv = *pv;
  p.loc = loc; p.lens = lens; p.loc_stride = loc_stride;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_sb = out_sb; p.out_sh = out_sh;
  p.lse = lse;
  p.part_o = reinterpret_cast<float*>(scratch);
  p.part_lse = p.part_o ? p.part_o + static_cast<size_t>(splits) * B * H * 512 : nullptr;
  p.status = status;
  p.B = B; p.H = H; p.K = K; p.splits = splits;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.format = format;
  dim3 grid((H + kMlaM - 1) / kMlaM, B, splits);
  if (g_mla_pair && grid.x % 2 == 0) {
    // the two head blocks of a (query, split) as a cluster of two CTAs sharing every K tile
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kMlaThreads);
    cfg.dynamicSmemBytes = kMlaSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    r = static_cast<int>(cudaLaunchKernelEx(&cfg, sparse_mla_decode_kernel<true>, tq, tr, p));
  } else {
    sparse_mla_decode_kernel<false><<<grid, kMlaThreads, kMlaSmem, stream>>>(tq, tr, p);
    r = static_cast<int>(cudaGetLastError());
  }
  if (r != 0) return r;
  if (splits > 1) {
    mla_combine_kernel<<<(B * H + kCombineWarps - 1) / kCombineWarps, kCombineWarps * 32, 0, stream>>>(
        p.part_o, p.part_lse, p.out, lse, B * H, splits);
    r = static_cast<int>(cudaGetLastError());
  }
  return r;
}

// Merge `parts` partial attention results of the same rows (context-parallel ranks, or KV splits
// computed elsewhere): part_o fp32 [parts, rows, 512], part_lse fp32 [parts, rows] (natural log,
// -inf where a part saw no token) -> out bf16 [rows, 512], lse fp32 [rows] (nullable).
int ulc_merge_partial_attention(const float* part_o, const float* part_lse, void* out, float* lse, int rows,
                                int parts, cudaStream_t stream) {
  if (rows <= 0 || parts <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(part_o) & 15) || (reinterpret_cast<uintptr_t>(out) & 7)) return -kErrAlignment;
  if (parts > 32) return -kErrUnsupported;
  mla_combine_kernel<<<(rows + kCombineWarps - 1) / kCombineWarps, kCombineWarps * 32, 0, stream>>>(
      part_o, part_lse, reinterpret_cast<__nv_bfloat16*>(out), lse, rows, parts);
  return static_cast<int>(cudaGetLastError());
}

// Packed form: q [B,H,576] bf16 contiguous (512 latent dims then 64 rotary), out [B,H,512] bf16.
int ulc_sparse_mla_decode(const PoolView* pv, const void* q, const int32_t* loc, long long loc_stride,
                          const int32_t* lens, int B, int H, int K, float sm_scale, int format, int splits,
                          void* out, float* lse, void* scratch, int32_t* status, cudaStream_t stream) {
  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(q);
  return ulc_sparse_mla_decode_ex(pv, qp, static_cast<long long>(H) * 576, 576, qp + 512,
                                  static_cast<long long>(H) * 576, 576, loc, loc_stride, lens, B, H, K, sm_scale,
                                  format, splits, out, static_cast<long long>(H) * 512, 512, lse, scratch, status,
                                  stream);
}

}  // extern "C"
