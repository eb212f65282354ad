// Ragged gather of Index keys for prefill scoring over an owner-striped Index.
//
// A prefill chunk scores every query against its own causal prefix.  With the Index striped over owners (logical
// page p lives on owner p % ranks as that owner's page p / ranks), the scoring kernel wants each query's prefix as
// one dense run of (128-byte fp8 key, fp32 scale) pairs.  This kernel builds those runs: query q's tokens
// [0, lengths[q]) go to rows [offsets[q], offsets[q] + lengths[q]) of the outputs, read page by page from whichever
// owner's pool holds the page (plain 16-byte loads, coherent at L2, from local or peer memory).  One warp per token:
// lanes 0..7 move the key, lane 8 the scale.  A page number that is padding (<= 0) gives zeros; one outside its
// owner's pool is reported through `status` and gives zeros.  Nothing here waits on another rank.
//
// Reference: ulacache/indexer/native_prefill.py:10-139 (gather of owner-sharded Index pages into the ragged prefill
// layout), ulacache/indexer/kernels/fp8_storage.py.
#include <cstdint>

#include "ulc/layout.h"
#include "ulc/ptx.cuh"
#include "ulc/status.h"

namespace ulc {

struct IndexGatherPools { const uint8_t* base[kMaxRanks]; };

__global__ void __launch_bounds__(256)
index_ragged_gather_kernel(IndexGatherPools pools, int ranks, int pool_pages, const int32_t* __restrict__ page_table,
                           long long table_stride, int table_width, const int32_t* __restrict__ lengths,
                           const int32_t* __restrict__ offsets, int total_rows, uint8_t* __restrict__ keys,
                           float* __restrict__ scales, int32_t* status) {
  const int q = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int len = lengths[q];
  const int out0 = offsets[q];
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < len; t += gridDim.x * warps) {
    const int row = out0 + t;
    if (row < 0 || row >= total_rows) { if (lane == 0) report(status, kErrBounds, row); continue; }
    const int col = t / kPageTokens;
    const int32_t page = col < table_width ? page_table[q * table_stride + col] : 0;
    const uint8_t* src = nullptr;
    if (page > 0) {
      const int owner = page % ranks, local = page / ranks;
      if (local < pool_pages) src = pools.base[owner] + static_cast<long long>(local) * kIndexPageBytes;
      else if (lane == 0) report(status, kErrBounds, page);
    }
    const int in_page = t % kPageTokens;
    if (lane < 8) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (src != nullptr) v = ptx::ld_cg16(src + in_page * kIndexDim + lane * 16);
      *reinterpret_cast<uint4*>(keys + static_cast<long long>(row) * kIndexDim + lane * 16) = v;
    } else if (lane == 8) {
      float s = 0.f;
      if (src != nullptr) s = *reinterpret_cast<const volatile float*>(src + kIndexPageKeyBytes + in_page * 4);
      scales[row] = s;
    }
  }
}

}  // namespace ulc

extern "C" int ulc_index_ragged_gather(const void* const* pool_bases, int ranks, int pool_pages, const int32_t* page_table,
                                       long long table_stride, int table_width, const int32_t* lengths,
                                       const int32_t* offsets, int queries, int max_length, int total_rows, void* keys,
                                       float* scales, int32_t* status, cudaStream_t stream) {
  using namespace ulc;
  if (queries <= 0 || max_length <= 0 || total_rows <= 0) return 0;
  if (ranks < 1 || ranks > kMaxRanks || pool_pages < 1 || table_width < 1 || queries > 65535 ||
      (reinterpret_cast<uintptr_t>(keys) & 15)) return -kErrUnsupported;
  IndexGatherPools pools{};
  for (int r = 0; r < ranks; ++r) {
    if (pool_bases[r] == nullptr || (reinterpret_cast<uintptr_t>(pool_bases[r]) & 15)) return -kErrUnsupported;
    pools.base[r] = static_cast<const uint8_t*>(pool_bases[r]);
  }
  int blocks_x = (max_length + 7) / 8;                 // 8 warps per block, one token per warp and turn
  if (blocks_x > 1024) blocks_x = 1024;
  index_ragged_gather_kernel<<<dim3(blocks_x, queries), 256, 0, stream>>>(
      pools, ranks, pool_pages, page_table, table_stride, table_width, lengths, offsets, total_rows,
      static_cast<uint8_t*>(keys), scales, status);
  return static_cast<int>(cudaGetLastError());
}
