// Device side of a prefill -> decode hand-over: while a remote writer fills records of this cache,
// their device slots are LEASED: a leased slot leaves the recency ring (no plan can pick it as a
// victim) until the last lease on it is released, when it re-enters the ring as touched now.
//
//   acquire : ids -> locations (device slot, or -slot-2 for a host slot); first lease on a device slot
//             takes it out of its recency bucket;
//   release : drops the leases; the last one stamps the slot with the current epoch;
//   publish : copies complete records from a registered staging buffer to the locations acquired
//             (device planes or pinned host planes), one warp per (record, layer).
//
// Nothing here traps: a row that is out of range, unallocated or whose location changed between acquire
// and release is reported through `status` and skipped.
//
// Reference: ulacache/csrc/cache/local_cache.cuh:79-133 (acquire / release receive locations),
// ulacache/transfer/kernels/receive_publication.py:15-90 (publish records / sidecar),
// ulacache/transfer/receive_window.py:159.
#include "ulc/pool.h"
#include "ulc/ptx.cuh"
#include "ulc/residency.h"

namespace ulc {

constexpr int32_t kStampLeased = -2;        // stamps[]: -1 free, -2 leased (both skipped by the victim scan)

__global__ void receive_acquire_kernel(ResidencyState st, OwnerMap map, int my_rank, const int32_t* __restrict__ ids,
                                       int n, int32_t* __restrict__ leases, int32_t* __restrict__ locations,
                                       int32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t id = ids[i];
  locations[i] = kDirUnallocated;
  if (!id_valid(id) || map.owner(id) != my_rank) { report(status, kErrBounds, id); return; }
  const int32_t local = map.local(id);
  if (local >= st.dir_len) { report(status, kErrBounds, id); return; }
  const int32_t e = st.directory[local];
  if (e == kDirUnallocated) { report(status, kErrInvariant, id); return; }
  if (dir_on_device(e)) {
    if (e >= st.hbm_slots || st.hbm_tags[e] != local) { report(status, kErrInvariant, id); return; }
    if (atomicAdd(&leases[e], 1) == 0) {
      const int32_t epoch = st.counters[kCntEpoch];
      const int32_t old = atomicExch(&st.stamps[e], kStampLeased);
      if (old >= 0) {
        atomicSub(&st.ring[bucket_of(old, epoch)], 1);
        bm_clear(st, bucket_of(old, epoch), e);
      }
    }
  }
  locations[i] = e;
}

__global__ void receive_release_kernel(ResidencyState st, OwnerMap map, int my_rank, const int32_t* __restrict__ ids,
                                       int n, int32_t* __restrict__ leases, const int32_t* __restrict__ locations,
                                       int32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t id = ids[i];
  const int32_t e = locations[i];
  if (e == kDirUnallocated) return;                         // acquire refused this row
  const int32_t local = map.local(id);
  if (!id_valid(id) || local >= st.dir_len || st.directory[local] != e) { report(status, kErrInvariant, id); return; }
  if (!dir_on_device(e)) return;
  const int32_t before = atomicSub(&leases[e], 1);
  if (before <= 0) { atomicAdd(&leases[e], 1); report(status, kErrInvariant, id); return; }
  if (before == 1) {
    const int32_t epoch = st.counters[kCntEpoch];
    st.stamps[e] = epoch;
    atomicAdd(&st.ring[epoch % kRecentBuckets], 1);
    bm_set(st, epoch % kRecentBuckets, e);
    st.access_time[local] = epoch;
  }
}

// staging: [layers][staging_rows][row_bytes]; device planes: base + layer * device_layer_stride + slot * row_bytes;
// host planes likewise.  row_bytes is a multiple of 16.  One warp per (record, layer): blockIdx.y = layer.
__global__ void __launch_bounds__(256)
receive_publish_kernel(const uint8_t* __restrict__ staging, long long staging_layer_stride,
                       const int32_t* __restrict__ source_rows, const int32_t* __restrict__ locations, int n,
                       uint8_t* device_base, long long device_layer_stride, int device_slots, uint8_t* host_base,
                       long long host_layer_stride, int host_slots, int row_bytes, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  const int layer = blockIdx.y;
  for (int i = warp; i < n; i += nwarps) {
    const int32_t e = locations[i];
    if (e == kDirUnallocated) continue;
    uint8_t* dst;
    if (e >= 0) {
      if (e >= device_slots) { if (lane == 0) report(status, kErrBounds, e); continue; }
      dst = device_base + layer * device_layer_stride + static_cast<long long>(e) * row_bytes;
    } else {
      const int32_t h = dir_host_slot(e);
      if (h < 0 || h >= host_slots || host_base == nullptr) { if (lane == 0) report(status, kErrBounds, e); continue; }
      dst = host_base + layer * host_layer_stride + static_cast<long long>(h) * row_bytes;
    }
    const uint8_t* src = staging + layer * staging_layer_stride + static_cast<long long>(source_rows[i]) * row_bytes;
    for (int v = lane; v < row_bytes / 16; v += 32) ptx::st_cg16(dst + v * 16, ptx::ld_nc16(src + v * 16));
  }
}

}  // namespace ulc

extern "C" {
using namespace ulc;

int ulc_receive_acquire(const ResidencyState* st, const OwnerMap* map, int my_rank, const int32_t* ids, int n,
                        int32_t* leases, int32_t* locations, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  receive_acquire_kernel<<<(n + 255) / 256, 256, 0, s>>>(*st, *map, my_rank, ids, n, leases, locations, status);
  return static_cast<int>(cudaGetLastError());
}

int ulc_receive_release(const ResidencyState* st, const OwnerMap* map, int my_rank, const int32_t* ids, int n,
                        int32_t* leases, const int32_t* locations, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  receive_release_kernel<<<(n + 255) / 256, 256, 0, s>>>(*st, *map, my_rank, ids, n, leases, locations, status);
  return static_cast<int>(cudaGetLastError());
}

int ulc_receive_publish(const void* staging, long long staging_layer_stride, const int32_t* source_rows,
                        const int32_t* locations, int n, int layers, void* device_base, long long device_layer_stride,
                        int device_slots, void* host_base, long long host_layer_stride, int host_slots, int row_bytes,
                        int32_t* status, cudaStream_t s) {
  if (n <= 0 || layers <= 0) return 0;
  if (row_bytes <= 0 || (row_bytes & 15) || (reinterpret_cast<uintptr_t>(staging) & 15) ||
      (reinterpret_cast<uintptr_t>(device_base) & 15) || (reinterpret_cast<uintptr_t>(host_base) & 15) ||
      (staging_layer_stride & 15) || (device_layer_stride & 15) || (host_layer_stride & 15))
    return -kErrUnsupported;
  int blocks = (n + 7) / 8;
  if (blocks > 148) blocks = 148;
  receive_publish_kernel<<<dim3(blocks, layers), 256, 0, s>>>(
      static_cast<const uint8_t*>(staging), staging_layer_stride, source_rows, locations, n,
      static_cast<uint8_t*>(device_base), device_layer_stride, device_slots, static_cast<uint8_t*>(host_base),
      host_layer_stride, host_slots, row_bytes, status);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
