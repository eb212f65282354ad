// Owner-side Index scoring for ranks with independent queries (data-parallel attention against an
// Index striped over all ranks).  Two transfer kernels over peer memory bracket the local score and
// select kernels:
//
//   export : every rank stores its queries (fp8 q, head weights, lengths) and, per owner, the page
//            table of its requests on that owner into slot [asker] of the owner's inbox;
//   (flag barrier, index_score + top-k over world * rows queries on every owner)
//   return : every owner stores the candidates (score, logical token) of asker a's rows into slot
//            [owner] of a's merge buffer, translating owner-local columns to logical tokens on the way;
//   (flag barrier, merge top-k over world * k candidates on the asker)
//
// Both kernels only store to peers (no remote loads, no waiting): the flag barrier of the symmetric
// heap orders them against the consumers.
//
// Reference roles: ulacache/indexer/native_owner.py:153-477 (export / collect / score / restore),
// ulacache/indexer/kernels/scoring.py:83-984.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ulc/layout.h"
#include "ulc/ptx.cuh"
#include "ulc/status.h"

namespace ulc {

constexpr int kOwnerComps = 4;       // q8 | w | lengths | page table

struct OwnerExportArgs {
  const uint8_t* src[kOwnerComps];   // component c of this rank; the page table is [owner][rows][pages]
  long long bytes[kOwnerComps];      // bytes this rank contributes per component (per owner for the table)
  long long slot_bytes[kOwnerComps]; // bytes of one asker's slot in the inbox (sized for rows_max)
  uint8_t* dst[kMaxRanks][kOwnerComps];
  int my_rank, ranks;
};

__global__ void __launch_bounds__(256) owner_export_kernel(OwnerExportArgs a) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int p = 0; p < a.ranks; ++p) {
    for (int c = 0; c < kOwnerComps; ++c) {
      const uint8_t* src = a.src[c] + (c == kOwnerComps - 1 ? a.bytes[c] * p : 0);
      uint8_t* dst = a.dst[p][c] + a.slot_bytes[c] * a.my_rank;
      const long long nvec = a.bytes[c] >> 4;
      for (long long v = tid; v < nvec; v += nthreads)
        ptx::st_cg16(dst + (v << 4), ptx::ld_nc16(src + (v << 4)));
      const long long tail_words = (a.bytes[c] & 15) >> 2;      // component sizes are multiples of 4
      if (tid < tail_words)
        reinterpret_cast<uint32_t*>(dst + (nvec << 4))[tid] = reinterpret_cast<const uint32_t*>(src + (nvec << 4))[tid];
    }
  }
}

struct OwnerReturnArgs {
  const float* vals;            // [ranks (asker)][rows][k] candidate scores of this owner's shard
  const int32_t* cols;          // same shape: owner-local columns, -1 = none
  float* dst_vals[kMaxRanks];   // asker's merge buffers: [rows][ranks (owner)][k]
  int32_t* dst_toks[kMaxRanks];
  int my_rank, ranks, rows, k, page_tokens;
};

// grid (rows, ranks): block (r, a) sends row r of asker a's candidates
__global__ void __launch_bounds__(128) owner_return_kernel(OwnerReturnArgs a) {
  const int r = blockIdx.x, asker = blockIdx.y;
  const size_t src = (static_cast<size_t>(asker) * a.rows + r) * a.k;
  const size_t dst = (static_cast<size_t>(r) * a.ranks + a.my_rank) * a.k;
  for (int j = threadIdx.x * 4; j < a.k; j += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(a.vals + src + j);
    const int4 c = *reinterpret_cast<const int4*>(a.cols + src + j);
    auto tok = [&](int col) {
      if (col < 0) return -1;
      const int page = col / a.page_tokens;
      return (page * a.ranks + a.my_rank) * a.page_tokens + (col - page * a.page_tokens);
    };
    int4 t = make_int4(tok(c.x), tok(c.y), tok(c.z), tok(c.w));
    float4 w = v;
    const float ninf = __int_as_float(0xff800000);
    if (c.x < 0) w.x = ninf;
    if (c.y < 0) w.y = ninf;
    if (c.z < 0) w.z = ninf;
    if (c.w < 0) w.w = ninf;
    ptx::st_cg16(a.dst_vals[asker] + dst + j, *reinterpret_cast<uint4*>(&w));
    ptx::st_cg16(a.dst_toks[asker] + dst + j, *reinterpret_cast<uint4*>(&t));
  }
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// src / bytes / slot_bytes: HOST arrays of 4 entries; dst: HOST array [ranks][4] of device addresses.
int ulc_owner_export(const void* const* src, const long long* bytes, const long long* slot_bytes, void* const* dst,
                     int my_rank, int ranks, cudaStream_t s) {
  if (ranks < 1 || ranks > kMaxRanks) return -kErrUnsupported;
  OwnerExportArgs a;
  long long most = 0;
  for (int c = 0; c < kOwnerComps; ++c) {
    if (bytes[c] < 0 || (bytes[c] & 3) || bytes[c] > slot_bytes[c] || (slot_bytes[c] & 15) ||
        (reinterpret_cast<uintptr_t>(src[c]) & 15))
      return -kErrUnsupported;
    // the table is read at src + bytes * owner: keep every owner's block 16-byte aligned
    if (c == kOwnerComps - 1 && (bytes[c] & 15)) return -kErrUnsupported;
    a.src[c] = static_cast<const uint8_t*>(src[c]);
    a.bytes[c] = bytes[c];
    a.slot_bytes[c] = slot_bytes[c];
    if (bytes[c] > most) most = bytes[c];
  }
  for (int p = 0; p < kMaxRanks; ++p)
    for (int c = 0; c < kOwnerComps; ++c)
      a.dst[p][c] = p < ranks ? static_cast<uint8_t*>(dst[p * kOwnerComps + c]) : nullptr;
  a.my_rank = my_rank; a.ranks = ranks;
  long long blocks = ((most >> 4) + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 296) blocks = 296;
  owner_export_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

int ulc_owner_return(const float* vals, const int32_t* cols, void* const* dst_vals, void* const* dst_toks, int my_rank,
                     int ranks, int rows, int k, int page_tokens, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (ranks < 1 || ranks > kMaxRanks || k <= 0 || (k & 3) || page_tokens <= 0) return -kErrUnsupported;
  OwnerReturnArgs a;
  a.vals = vals; a.cols = cols;
  for (int p = 0; p < kMaxRanks; ++p) {
    a.dst_vals[p] = p < ranks ? static_cast<float*>(dst_vals[p]) : nullptr;
    a.dst_toks[p] = p < ranks ? static_cast<int32_t*>(dst_toks[p]) : nullptr;
  }
  a.my_rank = my_rank; a.ranks = ranks; a.rows = rows; a.k = k; a.page_tokens = page_tokens;
  owner_return_kernel<<<dim3(rows, ranks), 128, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
