// Owner-side attention for a page pool striped over tensor-parallel ranks.
//
// With queries replicated on every rank, a rank does not have to pull the selected records it does
// not own: it attends, for ALL heads, over the selected records it does own, and the ranks then
// exchange partial outputs (O normalised per rank, plus its log-sum-exp) by head: rank q receives
// from every rank the partials of ITS heads and merges them.  Per query this moves
// heads * 513 values instead of 7/8 of top-k 656-byte records across NVLink.
//
//   owner_localize_kernel   keep the locations owned by this rank, compact them to the front
//   scatter_heads_kernel    peer-store each head block of (O, lse) into its owner's receive slot
//   merge_heads_kernel      log-sum-exp merge of the received partials (bf16 in, bf16 out)
//
// The reference has no counterpart: its tensor-parallel path pulls remote records into a local
// arena (ulacache/csrc/cache/common.cuh:1037) and its context-parallel merge is the serving
// framework's all-to-all (patches/sglang.patch:1983-2011).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ulc/layout.h"
#include "ulc/ptx.cuh"
#include "ulc/status.h"

namespace ulc {

struct PeerPtrs { void* p[kMaxRanks]; };

__global__ void __launch_bounds__(256)
owner_localize_kernel(const int32_t* __restrict__ loc, int K, int rank, int32_t* __restrict__ out,
                      int32_t* __restrict__ counts) {
  __shared__ int s_warp[8];
  __shared__ int s_base;
  const int q = blockIdx.x, t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int32_t* row = loc + static_cast<size_t>(q) * K;
  int32_t* o = out + static_cast<size_t>(q) * K;
  if (t == 0) s_base = 0;
  __syncthreads();
  for (int base = 0; base < K; base += 256) {
    const int j = base + t;
    const int32_t v = j < K ? row[j] : -1;
    const bool keep = v >= 0 && loc_rank(v) == rank;
    const unsigned int bal = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) s_warp[w] = __popc(bal);
    __syncthreads();
    int before = 0;
    for (int i = 0; i < w; ++i) before += s_warp[i];
    if (keep) o[s_base + before + __popc(bal & ((1u << lane) - 1u))] = v;
    __syncthreads();
    if (t == 0) {
      int tot = 0;
      for (int i = 0; i < 8; ++i) tot += s_warp[i];
      s_base += tot;
    }
    __syncthreads();
  }
  const int n = s_base;
  for (int j = n + t; j < K; j += 256) o[j] = -1;
  if (t == 0) counts[q] = n;
}

// o bf16 [B, H, 512], lse fp32 [B, H]; H = ranks * hs.  Receive layout on every rank:
// o_recv bf16 [ranks (source)][rows_max * hs][512], lse_recv fp32 [ranks][rows_max * hs].
// grid (B, ranks): block (b, q) sends head block q of query b to rank q.
__global__ void __launch_bounds__(256)
scatter_heads_kernel(const __nv_bfloat16* __restrict__ o, const float* __restrict__ lse, int H, int hs, int rows_max,
                     int my_rank, PeerPtrs o_dst, PeerPtrs lse_dst) {
  const int b = blockIdx.x, q = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(o + (static_cast<size_t>(b) * H + static_cast<size_t>(q) * hs) * 512);
  const size_t row0 = static_cast<size_t>(my_rank) * rows_max * hs + static_cast<size_t>(b) * hs;
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(o_dst.p[q]) + row0 * 512);
  const int units = hs * 512 * 2 / 16;
  for (int i = threadIdx.x; i < units; i += blockDim.x) dst[i] = src[i];
  float* ldst = reinterpret_cast<float*>(lse_dst.p[q]) + row0;
  for (int i = threadIdx.x; i < hs; i += blockDim.x) ldst[i] = lse[static_cast<size_t>(b) * H + q * hs + i];
  ptx::cta_release_peer_stores();
}

// out[row] = sum_p w_p * part[p][row], w_p = exp(lse_p - max) / sum; part stride = rows_max * hs rows.
__global__ void __launch_bounds__(128)
merge_heads_kernel(const __nv_bfloat16* __restrict__ part_o, const float* __restrict__ part_lse, int parts,
                   long long part_stride_rows, __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int rows) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  float w[kMaxRanks];
  float m = -INFINITY;
  for (int p = 0; p < parts; ++p) {
    w[p] = part_lse[p * part_stride_rows + row];
    m = fmaxf(m, w[p]);
  }
  float denom = 0.f;
  for (int p = 0; p < parts; ++p) {
    w[p] = w[p] > -INFINITY ? __expf(w[p] - m) : 0.f;
    denom += w[p];
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x * 4; d < 512; d += blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < parts; ++p) {
      if (w[p] == 0.f) continue;
      const uint2 raw = *reinterpret_cast<const uint2*>(part_o + (p * part_stride_rows + row) * 512 + d);
      const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(v[0]), c = __bfloat1622float2(v[1]);
      acc[0] = fmaf(w[p], a.x, acc[0]); acc[1] = fmaf(w[p], a.y, acc[1]);
      acc[2] = fmaf(w[p], c.x, acc[2]); acc[3] = fmaf(w[p], c.y, acc[3]);
    }
    __nv_bfloat162 o0 = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv), o1 = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
    uint2 ow;
    ow.x = *reinterpret_cast<uint32_t*>(&o0);
    ow.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(row) * 512 + d) = ow;
  }
  if (lse_out != nullptr && threadIdx.x == 0) lse_out[row] = denom > 0.f ? m + logf(denom) : -INFINITY;
}

}  // namespace ulc

extern "C" {
using namespace ulc;

int ulc_owner_localize(const int32_t* loc, int Q, int K, int rank, int32_t* out, int32_t* counts, cudaStream_t s) {
  if (Q <= 0 || K <= 0) return 0;
  if (rank < 0 || rank >= kMaxRanks) return -kErrUnsupported;
  owner_localize_kernel<<<Q, 256, 0, s>>>(loc, K, rank, out, counts);
  return static_cast<int>(cudaGetLastError());
}

int ulc_scatter_heads(const void* o, const float* lse, int B, int H, int ranks, int rows_max, int my_rank,
                      void* const* o_dst, void* const* lse_dst, cudaStream_t s) {
  if (B <= 0) return 0;
  if (ranks < 1 || ranks > kMaxRanks || H % ranks || B > rows_max) return -kErrUnsupported;
  PeerPtrs od, ld;
  for (int r = 0; r < kMaxRanks; ++r) { od.p[r] = r < ranks ? o_dst[r] : nullptr; ld.p[r] = r < ranks ? lse_dst[r] : nullptr; }
  scatter_heads_kernel<<<dim3(B, ranks), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(o), lse, H, H / ranks, rows_max,
                                                      my_rank, od, ld);
  return static_cast<int>(cudaGetLastError());
}

int ulc_merge_heads(const void* part_o, const float* part_lse, int parts, long long part_stride_rows, void* out,
                    float* lse_out, int rows, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (parts < 1 || parts > kMaxRanks) return -kErrUnsupported;
  merge_heads_kernel<<<rows, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(part_o), part_lse, parts, part_stride_rows,
                                          reinterpret_cast<__nv_bfloat16*>(out), lse_out, rows);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
