// Kernels for caches whose records are PAIRS of planes (separate K and V pages of a grouped-query model) and for
// receive-side slot ordering.
//
//  * compose_record_ids: a request table [requests, context] maps a token position to its record; a selection of
//    positions [rows, width] becomes record ids (-1 for padding, positions at or beyond the row's length or the
//    table's context).
//  * gather_pairs: the selected records' K and V rows (one row per record and plane, heads x dim elements) are copied
//    head by head into ragged outputs [total, heads, dim]: row r owns output rows offsets[r] .. offsets[r + 1].
//    A selected column whose position is valid but whose record is not resident (slot < 0) yields zeros; with
//    `padded` every column below `columns` is written (zeros where invalid), without it only the valid columns.
//  * sort_free_tail: the top `window` entries of a free-slot stack are sorted descending, so that the following pops
//    return ascending, mostly adjacent slots: a receive of n records then lands in a few contiguous extents instead
//    of n scattered rows.  The set of free slots and the count are unchanged.
//
// Reference: ulacache/storage/kernels/paired_records.py:8 (compose_record_ids_kernel), :37 (gather_pairs_kernel);
// ulacache/cache/kernels/local_cache.py:50 (_order_free_cpu_receive_tail).
#include <cuda_runtime.h>
#include <limits.h>
#include <stdint.h>

#include "ulc/launch.h"
#include "ulc/status.h"

namespace ulc {

__global__ void compose_record_ids_kernel(const int32_t* __restrict__ table, long long request_stride, int context,
                                          const int32_t* __restrict__ requests, const int32_t* __restrict__ positions,
                                          long long position_stride, const int32_t* __restrict__ lengths, int width,
                                          int32_t* __restrict__ out) {
  const int row = blockIdx.x;
  const long long request = requests[row];
  const int length = lengths[row];
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    const int p = positions[static_cast<long long>(row) * position_stride + c];
    const bool valid = p >= 0 && p < length && p < context;
    out[static_cast<long long>(row) * width + c] = valid ? table[request * request_stride + p] : -1;
  }
}

struct PairArgs {
  const uint8_t* key; const uint8_t* value;
  long long key_stride, value_stride;       // bytes between records of a plane
  const int32_t* records;                   // [rows, selected] slots, -1 not resident
  const int32_t* positions; long long position_stride;
  const int32_t* lengths;                   // [rows]
  const int32_t* offsets;                   // [rows + 1] output row starts
  uint8_t* out_key; uint8_t* out_value;     // [total, heads, head_bytes]
  int selected, heads, head_bytes, columns, padded;
};

// grid (rows, heads, column tiles of 16); a warp moves one (column, head) row of head_bytes in 16-byte pieces
__global__ void __launch_bounds__(256)
gather_pairs_kernel(const PairArgs a) {
  const int row = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int start = a.offsets[row];
  const int span = a.offsets[row + 1] - start;
  const int length = a.lengths[row];
  for (int c = blockIdx.z * 8 + warp; c < a.selected; c += gridDim.z * 8) {
    const int p = a.positions[static_cast<long long>(row) * a.position_stride + c];
    const int slot = a.records[static_cast<long long>(row) * a.selected + c];
    const bool native_valid = c < span && p >= 0 && p < length;
    const bool valid = native_valid && slot >= 0;
    const bool store = a.padded ? c < a.columns : native_valid;
    if (!store) continue;
    const size_t dst = (static_cast<size_t>(start + c) * a.heads + head) * a.head_bytes;
    const size_t sk = static_cast<size_t>(max(slot, 0)) * a.key_stride + static_cast<size_t>(head) * a.head_bytes;
    const size_t sv = static_cast<size_t>(max(slot, 0)) * a.value_stride + static_cast<size_t>(head) * a.head_bytes;
    const bool vec = ((reinterpret_cast<uintptr_t>(a.key + sk) | reinterpret_cast<uintptr_t>(a.value + sv) |
                       reinterpret_cast<uintptr_t>(a.out_key + dst) | reinterpret_cast<uintptr_t>(a.out_value + dst) |
                       static_cast<uintptr_t>(a.head_bytes)) & 15) == 0;
    if (vec) {
      for (int b = lane * 16; b < a.head_bytes; b += 32 * 16) {
        const uint4 zero = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(a.out_key + dst + b) = valid ? *reinterpret_cast<const uint4*>(a.key + sk + b) : zero;
        *reinterpret_cast<uint4*>(a.out_value + dst + b) = valid ? *reinterpret_cast<const uint4*>(a.value + sv + b) : zero;
      }
    } else {
      for (int b = lane; b < a.head_bytes; b += 32) {
        a.out_key[dst + b] = valid ? a.key[sk + b] : 0;
        a.out_value[dst + b] = valid ? a.value[sv + b] : 0;
      }
    }
  }
}

// One CTA: bitonic sort (descending) of the top `window` (power of two, <= 32768) entries of the stack in shared memory.
__global__ void __launch_bounds__(1024)
sort_free_tail_kernel(int32_t* __restrict__ stack, const int32_t* __restrict__ count_ptr, int window) {
  extern __shared__ int32_t tail[];
  const int count = *count_ptr;
  const int start = max(count - window, 0);
  for (int i = threadIdx.x; i < window; i += blockDim.x) tail[i] = start + i < count ? stack[start + i] : INT_MIN;
  __syncthreads();
  for (int k = 2; k <= window; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < window; i += blockDim.x) {
        const int partner = i ^ j;
        if (partner > i) {
          const bool descending = (i & k) == 0;
          const int32_t x = tail[i], y = tail[partner];
          if (descending ? x < y : x > y) { tail[i] = y; tail[partner] = x; }
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < window; i += blockDim.x)
    if (start + i < count) stack[start + i] = tail[i];
}

}  // namespace ulc

extern "C" {
using namespace ulc;

int ulc_compose_record_ids(const int32_t* table, long long request_stride, int context, const int32_t* requests,
                           const int32_t* positions, long long position_stride, const int32_t* lengths, int rows, int width,
                           int32_t* out, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  const int tiles = (width + 255) / 256;
  compose_record_ids_kernel<<<dim3(rows, tiles < 64 ? tiles : 64), 256, 0, stream>>>(table, request_stride, context, requests,
                                                                                     positions, position_stride, lengths,
                                                                                     width, out);
  return static_cast<int>(cudaGetLastError());
}

int ulc_gather_pairs(const void* key, const void* value, long long key_stride, long long value_stride, const int32_t* records,
                     const int32_t* positions, long long position_stride, const int32_t* lengths, const int32_t* offsets,
                     void* out_key, void* out_value, int rows, int selected, int heads, int head_bytes, int columns, int padded,
                     cudaStream_t stream) {
  if (rows <= 0 || selected <= 0 || heads <= 0) return 0;
  if (head_bytes <= 0 || heads > 65535) return -kErrUnsupported;
  PairArgs a;
  a.key = static_cast<const uint8_t*>(key); a.value = static_cast<const uint8_t*>(value);
  a.key_stride = key_stride; a.value_stride = value_stride; a.records = records; a.positions = positions;
  a.position_stride = position_stride; a.lengths = lengths; a.offsets = offsets;
  a.out_key = static_cast<uint8_t*>(out_key); a.out_value = static_cast<uint8_t*>(out_value);
  a.selected = selected; a.heads = heads; a.head_bytes = head_bytes; a.columns = columns; a.padded = padded;
  int tiles = (selected + 7) / 8;
  if (tiles > 64) tiles = 64;
  gather_pairs_kernel<<<dim3(rows, heads, tiles), 256, 0, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// stack: device int32 free-slot stack whose top is stack[*count - 1]; window: 16384 or 32768 (any power of two <= 32768).
int ulc_sort_free_tail(int32_t* stack, const int32_t* count_ptr, int window, cudaStream_t stream) {
  if (window < 2 || window > 32768 || (window & (window - 1))) return -kErrUnsupported;
  static PerDeviceOnce once;
  const int bytes = window * 4;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(sort_free_tail_kernel), 32768 * 4, once);
  if (rc != 0) return rc;
  sort_free_tail_kernel<<<1, 1024, bytes, stream>>>(stack, count_ptr, window);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
