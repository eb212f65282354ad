// Telemetry kernels: a sampled classifier of where selected records live, and a bounded trace ring
// for selection addresses.  Both are read-only with respect to cache state and cheap enough to be
// captured inside the decode graph.
//
// Passive replay probes: unique historical lookups of a step partitioned by where the record lives
// (deduplicated per request through an open-addressing table), bytes the step's plan moves in each
// direction, bytes of rows written straight to the host tier; and a chunked trace of the rows a
// tensor-parallel rank found missing locally.
//
// Reference roles: ulacache/csrc/telemetry/cache_hits.cuh:62 (sample_cache_hits), sparse_replay.cuh:11-112
// (unique hits, plan bytes, current bytes), tp_sparse_trace.cuh:10-37 (local-miss frames) and the
// trace recorders of csrc/telemetry/*.cuh.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ulc/residency.h"
#include "ulc/status.h"

namespace ulc {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

// counts[0] device hits, [1] host hits, [2] unallocated, [3] out of range, [4] sampled entries.
// Entry i of the selection is sampled when the low `shift` bits of hash(i + salt) are zero.
__global__ void sample_cache_hits_kernel(const int32_t* __restrict__ dir, int dir_len, const int32_t* __restrict__ sel,
                                         long long n, int shift, uint32_t salt, unsigned long long* counts) {
  unsigned long long c[5] = {0, 0, 0, 0, 0};
  const uint32_t mask = shift >= 32 ? 0xffffffffu : ((1u << shift) - 1u);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (mix32(static_cast<uint32_t>(i) + salt) & mask) continue;
    const int id = sel[i];
    if (id < 0) continue;                  // padding of a short selection
    ++c[4];
    if (id >= dir_len) { ++c[3]; continue; }
    const int e = dir[id];
    if (e >= 0) ++c[0]; else if (e <= -2) ++c[1]; else ++c[2];
  }
#pragma unroll
  for (int k = 0; k < 5; ++k) {
    for (int o = 16; o > 0; o >>= 1) c[k] += __shfl_xor_sync(0xffffffffu, c[k], o);
    if ((threadIdx.x & 31) == 0 && c[k]) atomicAdd(&counts[k], c[k]);
  }
}

// Trace ring of (step, layer, id) int32 triples.  header[0] = write cursor (triples), header[1] =
// dropped triples, header[2] = capacity.  A chunk that does not fit is dropped whole and counted,
// so the host drains complete chunks only.
__global__ void trace_append_kernel(int32_t* __restrict__ ring, unsigned long long* __restrict__ header,
                                    int step, int layer, const int32_t* __restrict__ sel, long long n) {
  __shared__ unsigned long long s_base;
  __shared__ int s_ok;
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    // one CTA reserves for the whole grid: the kernel is launched with a single CTA per chunk
    const unsigned long long cap = header[2];
    const unsigned long long cur = header[0];
    if (cur + static_cast<unsigned long long>(n) <= cap) {
      header[0] = cur + n;
      s_base = cur;
      s_ok = 1;
    } else {
      header[1] += n;
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) return;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    int32_t* dst = ring + (s_base + i) * 3;
    dst[0] = step; dst[1] = layer; dst[2] = sel[i];
  }
}


// counts (uint64[8]): [0] unique lookups, [1] on device, [2] on host, [3] unallocated, [4] errors
// (id out of range, table full), [5] host->device bytes of the plan, [6] device->host bytes of the
// plan, [7] bytes of this step's rows that were written to the host tier.
// sel int32 [queries, topk]; query q belongs to request requests[q / width] and wrote row
// current[q] this step (not a historical lookup).  keys: table of `table_size` (power of two) uint64,
// all ones = empty.
__global__ void replay_unique_hits_kernel(const int32_t* __restrict__ sel, const int32_t* __restrict__ current,
                                          const int32_t* __restrict__ requests, const int32_t* __restrict__ dir,
                                          int dir_len, unsigned long long* keys, unsigned int table_size,
                                          unsigned long long* counts, int queries, int width, int topk) {
  const long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= static_cast<long long>(queries) * topk) return;
  const int query = static_cast<int>(item / topk), request = query / width;
  const int id = sel[item];
  if (id < 0) return;
  if (id >= dir_len || requests[request] < 0) { atomicAdd(counts + 4, 1ULL); return; }
  for (int l = 0; l < width; ++l)
    if (current[request * width + l] == id) return;
  const unsigned long long key = (static_cast<unsigned long long>(static_cast<uint32_t>(requests[request])) << 32) |
                                 static_cast<uint32_t>(id);
  unsigned int at = mix32(static_cast<uint32_t>(key) ^ mix32(static_cast<uint32_t>(key >> 32))) & (table_size - 1);
  for (unsigned int probe = 0; probe < table_size; ++probe) {
    const unsigned long long prev = atomicCAS(keys + at, ~0ULL, key);
    if (prev == key) return;                      // another query of the request already counted it
    if (prev == ~0ULL) {
      const int e = dir[id];
      atomicAdd(counts, 1ULL);
      atomicAdd(counts + (e >= 0 ? 1 : e <= -2 ? 2 : 3), 1ULL);
      return;
    }
    at = (at + 1) & (table_size - 1);
  }
  atomicAdd(counts + 4, 1ULL);
}

// plan: the residency plan [kPlanRows, capacity]; plan_count: device pointer to the number of items.
__global__ void replay_plan_bytes_kernel(const int32_t* __restrict__ plan, const int32_t* __restrict__ plan_count,
                                         int capacity, unsigned long long bytes_per_item, unsigned long long* counts) {
  const int n = min(*plan_count, capacity);
  unsigned long long h2d = 0, d2h = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if (plan[kPlanHostSrc * capacity + i] >= 0) h2d += bytes_per_item;
    if (plan[kPlanHostDst * capacity + i] >= 0) d2h += bytes_per_item;
  }
  for (int o = 16; o > 0; o >>= 1) {
    h2d += __shfl_xor_sync(0xffffffffu, h2d, o);
    d2h += __shfl_xor_sync(0xffffffffu, d2h, o);
  }
  if ((threadIdx.x & 31) == 0) {
    if (h2d) atomicAdd(counts + 5, h2d);
    if (d2h) atomicAdd(counts + 6, d2h);
  }
}

__global__ void replay_current_bytes_kernel(const int32_t* __restrict__ current, int n, const int32_t* __restrict__ dir,
                                            int dir_len, unsigned long long bytes_per_item, unsigned long long* counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = current[i];
  if (id >= 0 && id < dir_len && dir[id] <= -2) atomicAdd(counts + 7, bytes_per_item);
}

// Local-miss trace of a tensor-parallel rank.  control (int64[4]): [0] enabled, [1] frame number,
// [2] valid query rows of the frame, [3] error bits (1 = bad valid count, 2 = bad row count,
// 4 = bad id).  Frame f of group g lands in chunk slot (f % chunk_frames) * groups + g:
// out_rows int32 [slots, bound, topk] (-1 padded), out_counts int32 [slots, bound],
// out_source int32 [slots] (rows the planner's source bucket held).
__global__ void tp_miss_trace_kernel(const int32_t* __restrict__ rows, long long stride,
                                     const int32_t* __restrict__ counts, int source_rows, long long* control,
                                     int32_t* __restrict__ out_rows, int32_t* __restrict__ out_counts,
                                     int32_t* __restrict__ out_source, int group, int frames, int chunk_frames,
                                     int groups, int bound, int topk) {
  if (!control[0] || control[1] < 0 || control[1] >= frames) return;
  const int valid = static_cast<int>(control[2]);
  if (valid < 0 || valid > source_rows || valid > bound) {
    if (!blockIdx.x && !threadIdx.x) atomicOr(reinterpret_cast<unsigned long long*>(control + 3), 1ULL);
    return;
  }
  const long long slot = (control[1] % chunk_frames) * groups + group;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < static_cast<long long>(bound) * topk) {
    const int q = static_cast<int>(i / topk), c = static_cast<int>(i - static_cast<long long>(q) * topk);
    const int count = q < valid ? counts[q] : -1;
    if (q < valid && (count < 0 || count > topk)) atomicOr(reinterpret_cast<unsigned long long*>(control + 3), 2ULL);
    const int id = (q < valid && c < count) ? rows[q * stride + c] : -1;
    if (id < -1) atomicOr(reinterpret_cast<unsigned long long*>(control + 3), 4ULL);
    out_rows[slot * bound * topk + i] = id;
    if (c == 0) out_counts[slot * bound + q] = count;
  }
  if (!blockIdx.x && !threadIdx.x) out_source[slot] = source_rows;
}

}  // namespace ulc

extern "C" {
using namespace ulc;

int ulc_sample_cache_hits(const int32_t* dir, int dir_len, const int32_t* sel, long long n, int shift,
                          unsigned int salt, unsigned long long* counts, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (shift < 0 || shift > 32) return -kErrUnsupported;
  long long blocks = (n + 255) / 256;
  if (blocks > 148) blocks = 148;
  sample_cache_hits_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(dir, dir_len, sel, n, shift, salt, counts);
  return static_cast<int>(cudaGetLastError());
}

int ulc_trace_append(int32_t* ring, unsigned long long* header, int step, int layer, const int32_t* sel,
                     long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  trace_append_kernel<<<1, 1024, 0, stream>>>(ring, header, step, layer, sel, n);
  return static_cast<int>(cudaGetLastError());
}

int ulc_replay_unique_hits(const int32_t* sel, const int32_t* current, const int32_t* requests, const int32_t* dir,
                           int dir_len, unsigned long long* keys, long long table_size, unsigned long long* counts,
                           int queries, int width, int topk, cudaStream_t stream) {
  if (queries <= 0 || topk <= 0) return 0;
  if (width <= 0 || queries % width || table_size <= 0 || (table_size & (table_size - 1)) ||
      table_size > (1LL << 31) || table_size < 2LL * queries * topk)
    return -kErrUnsupported;
  const long long items = static_cast<long long>(queries) * topk;
  replay_unique_hits_kernel<<<static_cast<int>((items + 255) / 256), 256, 0, stream>>>(
      sel, current, requests, dir, dir_len, keys, static_cast<unsigned int>(table_size), counts, queries, width, topk);
  return static_cast<int>(cudaGetLastError());
}

int ulc_replay_plan_bytes(const int32_t* plan, const int32_t* plan_count, int capacity, long long bytes_per_item,
                          unsigned long long* counts, cudaStream_t stream) {
  if (capacity <= 0 || bytes_per_item < 0) return -kErrUnsupported;
  int blocks = (capacity + 255) / 256;
  if (blocks > 148) blocks = 148;
  replay_plan_bytes_kernel<<<blocks, 256, 0, stream>>>(plan, plan_count, capacity,
                                                       static_cast<unsigned long long>(bytes_per_item), counts);
  return static_cast<int>(cudaGetLastError());
}

int ulc_replay_current_bytes(const int32_t* current, int n, const int32_t* dir, int dir_len, long long bytes_per_item,
                             unsigned long long* counts, cudaStream_t stream) {
  if (n <= 0) return 0;
  replay_current_bytes_kernel<<<(n + 255) / 256, 256, 0, stream>>>(current, n, dir, dir_len,
                                                                   static_cast<unsigned long long>(bytes_per_item), counts);
  return static_cast<int>(cudaGetLastError());
}

int ulc_tp_miss_trace(const int32_t* rows, long long stride, const int32_t* counts, int source_rows, long long* control,
                      int32_t* out_rows, int32_t* out_counts, int32_t* out_source, int group, int frames,
                      int chunk_frames, int groups, int bound, int topk, cudaStream_t stream) {
  if (group < 0 || group >= groups || frames <= 0 || chunk_frames <= 0 || bound <= 0 || topk <= 0)
    return -kErrUnsupported;
  const long long items = static_cast<long long>(bound) * topk;
  tp_miss_trace_kernel<<<static_cast<int>((items + 255) / 256), 256, 0, stream>>>(
      rows, stride, counts, source_rows, control, out_rows, out_counts, out_source, group, frames, chunk_frames, groups,
      bound, topk);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
