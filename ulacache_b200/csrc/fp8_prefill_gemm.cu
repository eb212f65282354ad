// Block-scaled fp8 GEMM for MANY token rows (prefill chunks): y[M, Nout] = x[M, K] * W[e]^T per expert.
//
// The decode GEMM (fp8_gemm.cu) keeps a weight tile stationary and streams at most 128 token rows past
// it as the MMA's N dimension; its epilogue then needs one scale per token COLUMN and K block.  With
// hundreds of rows per expert the roles are swapped here: tokens are the MMA's M dimension (TMEM lanes),
// a 128-feature weight tile is its N dimension.  A thread of the epilogue owns one token row, so the
// block scale of a (token, K block) - sx[token][kb] * sw[feature tile][kb] - is ONE scalar per thread and
// K block, and the 128 partial sums of a K block are folded into 128 register accumulators with it.
//
//   x8 [M, K] fp8 e4m3 row-major, sx [M, K/128] fp32 (one scale per token and 128-deep K block)
//   w8 tile-major [E, Nout/128, K/128, 128, 128], sw [E, Nout/128, K/128]
//   offs [E + 1] rows of expert e = offs[e] .. offs[e+1] (null: one expert, rows 0 .. M)
//   out bf16 [M, Nout]
//
// Persistent CTAs walk the items (expert, feature tile, 128-row tile), row tiles fastest so that
// neighbouring CTAs read the same weight tile out of L2.  Roles: one TMA producer warp (a 128 x 128 x-tile
// and a 128 x 128 weight tile per K block, six 32 KB stages), one MMA warp (four tcgen05.mma of K = 32 per
// K block into one of two TMEM accumulators), four epilogue warps (tcgen05.ld of the finished K block,
// scaled accumulation, bf16 store of the rows that belong to the expert).  Every wait is bounded.
//
// Reference role: the grouped fp8 GEMMs the reference gets from DeepGEMM (README.md:42-59); no code shared.
#include "ulc/launch.h"
#include "ulc/ptx.cuh"
#include "ulc/status.h"
#include "ulc/tmap.h"

#include <cuda_bf16.h>

namespace ulc {

constexpr int kPgTile = 128;                     // rows, features and K bytes of a tile
constexpr int kPgStageBytes = 2 * kPgTile * kPgTile;
constexpr int kPgStages = 6;
constexpr int kPgThreads = 192;                  // producer, MMA, 4 epilogue warps
constexpr int kPgMaxExperts = 320;
constexpr int kPgSmem = 1024 + kPgStages * kPgStageBytes + 2048;

struct PgParams {
  const float* sw;
  const float* sx;
  const int32_t* offs;
  __nv_bfloat16* out;
  int32_t* status;
  int M, Nout, K, E;
};

struct PgBarriers {
  uint64_t full[kPgStages];
  uint64_t empty[kPgStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int32_t n_items;
  int32_t tile_start[kPgMaxExperts + 1];         // first item of every expert
};
static_assert(sizeof(PgBarriers) <= 2048, "barrier block outgrew its reservation");

struct PgItem { int e, n, row0, row_end; };

// item -> (expert, feature tile, first row, end of the expert's rows); row tiles run fastest
__device__ __forceinline__ PgItem pg_item(const PgBarriers& bar, const PgParams& p, int t) {
  int lo = 0, hi = p.E;                          // tile_start[lo] <= t < tile_start[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (bar.tile_start[mid] <= t) lo = mid; else hi = mid;
  }
  const int begin = p.offs ? p.offs[lo] : 0;
  const int end = p.offs ? p.offs[lo + 1] : p.M;
  const int mt = (end - begin + kPgTile - 1) / kPgTile;
  const int local = t - bar.tile_start[lo];
  PgItem it;
  it.e = lo;
  it.n = local / mt;
  it.row0 = begin + (local - it.n * mt) * kPgTile;
  it.row_end = end;
  return it;
}

__global__ void __launch_bounds__(kPgThreads, 1)
fp8_prefill_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                        const PgParams p) {
  extern __shared__ uint8_t pg_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pg_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  PgBarriers& bar = *reinterpret_cast<PgBarriers*>(smem + kPgStages * kPgStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / kPgTile, NT = p.Nout / kPgTile;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPgStages; ++s) { ptx::mbar_init(&bar.full[s], 1); ptx::mbar_init(&bar.empty[s], 1); }
    for (int s = 0; s < 2; ++s) { ptx::mbar_init(&bar.acc_full[s], 1); ptx::mbar_init(&bar.acc_empty[s], 4); }
    bar.abort_flag = 0;
    int run = 0;
    for (int e = 0; e < p.E; ++e) {
      bar.tile_start[e] = run;
      const int rows = p.offs ? max(p.offs[e + 1] - p.offs[e], 0) : p.M;
      run += (rows + kPgTile - 1) / kPgTile * NT;
    }
    bar.tile_start[p.E] = run;
    bar.n_items = run;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_x);
    ptx::prefetch_tmap(&tmap_w);
  }
  if (warp == 1) { ptx::tmem_alloc<256>(&bar.tmem_base); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = bar.tmem_base;
  const int n_items = bar.n_items;
  volatile int* abort_flag = &bar.abort_flag;

  if (warp == 0) {
    // ================================================================ producer ==
    if (ptx::elect_one()) {
      int it = 0, issued = 0;
      for (int t = blockIdx.x; t < n_items && !*abort_flag; t += gridDim.x) {
        const PgItem w = pg_item(bar, p, t);
        const int wrow = (w.e * NT + w.n) * KB;            // first 128-row block of this weight tile
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kPgStages;
          if (*abort_flag || !ptx::mbar_wait(&bar.empty[s], ((it / kPgStages) & 1) ^ 1)) {
            if (!*abort_flag) report(p.status, kErrPipeline, 100 + s);
            *abort_flag = 1;
            break;
          }
          uint8_t* a = smem + s * kPgStageBytes;
          ptx::mbar_expect_tx(&bar.full[s], kPgStageBytes);
          // rows past M read as zeros; rows past the expert's end belong to the next expert and are not stored
          ptx::tma_load_2d(a, &tmap_x, &bar.full[s], kb * kPgTile, w.row0);
          ptx::tma_load_2d(a + kPgTile * kPgTile, &tmap_w, &bar.full[s], 0, (wrow + kb) * kPgTile);
          issued = it + 1;
        }
      }
      if (*abort_flag)                                      // let the copies in flight land before the CTA leaves
        for (int i = max(0, issued - kPgStages); i < issued; ++i)
          ptx::mbar_wait(&bar.full[i % kPgStages], (i / kPgStages) & 1, 200000000LL);
    }
  } else if (warp == 1) {
    // ===================================================================== MMA ==
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc(kPgTile, kPgTile, 0, 0, 0, 0);    // e4m3 x e4m3 -> f32
      const uint64_t smem_desc = ptx::umma_desc_sw128(ptx::smem_u32(smem));
      int it = 0;
      for (int t = blockIdx.x; t < n_items && !*abort_flag; t += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kPgStages, ab = it & 1;
          if (*abort_flag || !ptx::mbar_wait(&bar.acc_empty[ab], ((it >> 1) & 1) ^ 1) ||
              !ptx::mbar_wait(&bar.full[s], (it / kPgStages) & 1)) {
            if (!*abort_flag) report(p.status, kErrPipeline, 200 + s);
            *abort_flag = 1;
            break;
          }
          ptx::tc_fence_after();
          const uint64_t a_desc = ptx::umma_desc_advance(smem_desc, s * kPgStageBytes);           // x tile: M = tokens
          const uint64_t b_desc = ptx::umma_desc_advance(a_desc, kPgTile * kPgTile);              // w tile: N = features
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            ptx::umma_fp8(tmem + ab * kPgTile, ptx::umma_desc_advance(a_desc, kk * 32),
                          ptx::umma_desc_advance(b_desc, kk * 32), idesc, kk > 0);
          ptx::umma_commit(&bar.empty[s]);
          ptx::umma_commit(&bar.acc_full[ab]);
        }
      }
    }
  } else {
    // ================================================================ epilogue ==
    const int qd = warp & 3;                       // TMEM lane quarter of this warp
    const int r = qd * 32 + lane;                  // token row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(qd * 32) << 16;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_items && ok; t += gridDim.x) {
      const PgItem w = pg_item(bar, p, t);
      const int row = w.row0 + r;
      const float* sx_row = p.sx + static_cast<size_t>(min(row, p.M - 1)) * KB;
      const float* sw_tile = p.sw + static_cast<size_t>(w.e * NT + w.n) * KB;
      float acc[kPgTile];
#pragma unroll
      for (int j = 0; j < kPgTile; ++j) acc[j] = 0.f;
      float s_next = sx_row[0] * sw_tile[0];
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int ab = it & 1;
        const float s = s_next;
        if (kb + 1 < KB) s_next = sx_row[kb + 1] * sw_tile[kb + 1];
        if (*abort_flag || !ptx::mbar_wait(&bar.acc_full[ab], (it >> 1) & 1)) {
          if (!*abort_flag && lane == 0) report(p.status, kErrPipeline, 300 + qd);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < kPgTile; c += 32) {
          uint32_t d[32];
          ptx::tmem_ld32(tmem + lane_base + ab * kPgTile + c, d);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(s, __uint_as_float(d[j]), acc[c + j]);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bar.acc_empty[ab]);
      }
      if (ok && row < w.row_end) {
        __nv_bfloat16* dst = p.out + static_cast<size_t>(row) * p.Nout + w.n * kPgTile;
#pragma unroll
        for (int c = 0; c < kPgTile; c += 8) {
          uint32_t wv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(acc[c + 2 * j], acc[c + 2 * j + 1]);
            wv[j] = *reinterpret_cast<const uint32_t*>(&v);
          }
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc<256>(tmem);
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// x8 [M, K] fp8 bytes, sx [M, K/128]; w8 tile-major [E, Nout/128, K/128, 128, 128], sw [E, Nout/128, K/128];
// offs device int32 [E + 1] (null with E == 1); out bf16 [M, Nout].  tiles_bound: an upper bound of the number
// of 128-row tiles over all experts (sizes the grid; M / 128 + E is always one).
int ulc_fp8_prefill_gemm(const void* x8, const float* sx, const void* w8, const float* sw, const int32_t* offs, int M,
                         int Nout, int K, int E, int tiles_bound, void* out, int32_t* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (Nout <= 0 || K <= 0 || (Nout % kPgTile) || (K % kPgTile) || E < 1 || E > kPgMaxExperts || (E > 1 && offs == nullptr))
    return -kErrUnsupported;
  if ((reinterpret_cast<uintptr_t>(x8) & 15) || (reinterpret_cast<uintptr_t>(w8) & 127) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -kErrAlignment;
  static PerDeviceOnce once;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(fp8_prefill_gemm_kernel), kPgSmem, once);
  if (rc != 0) return rc;
  CUtensorMap tx, tw;
  rc = make_tmap_2d(&tx, x8, 1, static_cast<uint64_t>(M), static_cast<uint64_t>(K), static_cast<uint64_t>(K), kPgTile, kPgTile,
                    true);
  if (rc != 0) return rc;
  const uint64_t wrows = static_cast<uint64_t>(E) * (Nout / kPgTile) * (K / kPgTile) * kPgTile;
  rc = make_tmap_2d(&tw, w8, 1, wrows, kPgTile, kPgTile, kPgTile, kPgTile, true);
  if (rc != 0) return rc;
  PgParams p;
  p.sw = sw; p.sx = sx; p.offs = offs; p.out = reinterpret_cast<__nv_bfloat16*>(out); p.status = status;
  p.M = M; p.Nout = Nout; p.K = K; p.E = E;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (tiles_bound <= 0) tiles_bound = (M + kPgTile - 1) / kPgTile + E;
  long long items = static_cast<long long>(tiles_bound) * (Nout / kPgTile);
  int grid = static_cast<int>(items < sms ? items : sms);
  if (grid < 1) grid = 1;
  fp8_prefill_gemm_kernel<<<grid, kPgThreads, kPgSmem, stream>>>(tx, tw, p);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
