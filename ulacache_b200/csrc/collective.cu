// Small peer-memory protocols that are not fused into a compute kernel:
//
//  * reader-lifetime publication: three monotonically increasing epochs per rank and domain
//    (SelectionsReady -> ResidencyReady -> ReadersRetired), written with system-scope release
//    stores into every rank's flag page and waited for with a bound;
//  * tagged all-gather of fp32 rows: every 8-byte word on the wire carries 4 payload bytes and the
//    4-byte call index, so the receiver needs no barrier: it polls each word until the tag matches.
//    Four slots rotate, the call index comes from a device counter (CUDA-graph replay safe).
//
//  * line all-gather of (ragged) fp32 rows: 128-byte lines of 31 payload words and one tag word
//    (96.9 % of the wire is payload), each line leaving as one aligned 128-byte store of eight
//    lanes x 16 bytes (`st.relaxed.sys.v4`), the way NCCL's LL128 protocol relies on NVLink
//    delivering an aligned 128-byte store whole.  A message starts with header lines carrying the
//    sender's device-side payload length and per-row lengths, so rows are packed on the wire and
//    unpacked (with a fill value past each row's end) by the receiver.
//
// Every wait has a cycle limit; on expiry the kernel records kErrTimeout in `status` and returns.
//
// Reference roles: ulacache/csrc/cache/reader_lifetime.cuh:14-44,86-149 and the FlashAG tagged
// all-gather ulacache/csrc/flashag/b300/ag_kernels_dynamic.cuh:143-145,250-267,375 (31+1 lines,
// dynamic payload length), packed_adapter.cuh:23-107 (ragged pack / unpack), common.cuh:328-349.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ulc/layout.h"
#include "ulc/ptx.cuh"
#include "ulc/status.h"

namespace ulc {

constexpr int kPhases = 3;
constexpr int kAgSlots = 4;

// flag page of a domain (int32): [phase][rank] at phase * 16 + rank
__global__ void lifetime_publish_kernel(int32_t* const* pages, int my_rank, int ranks, int phase, int epoch) {
  const int r = threadIdx.x;
  if (r < ranks) {
    __threadfence_system();
    ptx::st_release_sys(pages[r] + phase * 16 + my_rank, epoch);
  }
}

__global__ void lifetime_wait_kernel(const int32_t* page, int ranks, int phase, int epoch, long long limit,
                                     int32_t* status) {
  const int r = threadIdx.x;
  if (r < ranks && !ptx::wait_flag_ge(page + phase * 16 + r, epoch, limit)) report(status, kErrTimeout, phase * 16 + r);
}

struct AgPeers { uint2* slab[kMaxRanks]; };

// src: fp32 [n] of this rank.  Slab layout on every rank: [slot][source rank][n] of (value, tag).
// out: fp32 [ranks, n] in rank order.  counter[0] is the call index of the previous call.
__global__ void __launch_bounds__(256)
tagged_all_gather_kernel(const float* __restrict__ src, int n, int n_max, AgPeers peers, int my_rank, int ranks,
                         unsigned int* counter, float* __restrict__ out, long long limit, int32_t* status) {
  __shared__ unsigned int s_idx;
  __shared__ int s_abort;
  // every CTA reads the same pre-increment value; the last CTA to finish bumps it (ticket at counter[1])
  if (threadIdx.x == 0) { s_idx = counter[0] + 1; s_abort = 0; }
  __syncthreads();
  const unsigned int idx = s_idx;
  const int slot = static_cast<int>((idx - 1) & (kAgSlots - 1));
  const size_t slot_base = static_cast<size_t>(slot) * ranks * n_max;
  // send: my row into slot [slot][my_rank] of every rank
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint2 w = make_uint2(__float_as_uint(src[i]), idx);
    // one explicit 8-byte system-scope store per peer: value and tag can never be split
    for (int p = 0; p < ranks; ++p)
      ptx::st_relaxed_sys_v2(&peers.slab[p][slot_base + static_cast<size_t>(my_rank) * n_max + i], w);
  }
  // receive: poll my own slab
  const volatile uint2* mine = peers.slab[my_rank] + slot_base;
  for (int r = 0; r < ranks; ++r) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
      const volatile uint2* w = mine + static_cast<size_t>(r) * n_max + i;
      uint2 v;
      v.x = w->x; v.y = w->y;
      if (v.y != idx) {
        const long long t0 = clock64();
        bool ok = false;
        while (!s_abort) {
          // 8-byte load: value and tag come from one access
          const unsigned long long raw = *reinterpret_cast<const volatile unsigned long long*>(w);
          v.x = static_cast<unsigned int>(raw);
          v.y = static_cast<unsigned int>(raw >> 32);
          if (v.y == idx) { ok = true; break; }
          if (clock64() - t0 > limit) break;
          __nanosleep(40);
        }
        if (!ok) {
          if (!s_abort) report(status, kErrTimeout, r);
          s_abort = 1;
          continue;
        }
      } else {
        const unsigned long long raw = *reinterpret_cast<const volatile unsigned long long*>(w);
        v.x = static_cast<unsigned int>(raw);
      }
      out[static_cast<size_t>(r) * n + i] = __uint_as_float(v.x);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(&counter[1], 1u) + 1;
    if (done == gridDim.x) { counter[1] = 0; counter[0] = idx; }
  }
}


// ------------------------------------------------------------------------------------------------
// Line all-gather.  Slab on every rank: [slot][source rank][lines_max] lines of 8 x uint4.
// A message of `rows` rows: header lines hold word 0 = packed payload words, words 1..rows = row
// lengths; payload lines hold the rows' valid prefixes back to back.  Word 31 of every line is the
// call index.  out: fp32 [ranks, rows, cols]; out_len: int32 [ranks, rows] (may be null).
constexpr int kLineWords = 31;
constexpr int kLineMaxRows = 4096;
constexpr int kLineThreads = 512;
constexpr int kLineUnroll = 4;

struct LinePeers { uint4* slab[kMaxRanks]; };

struct LineArgs {
  const float* src;
  long long src_stride;
  const int32_t* row_len;      // device lengths of my rows, or null = every row has `cols` words
  int rows, cols;
  LinePeers peers;
  int my_rank, ranks, lines_max, slots;
  unsigned int* counter;       // [0] previous call index, [1] ticket
  float* out;
  int32_t* out_len;
  float fill;
  long long limit;
  int32_t* status;
};

// exclusive prefix of s_len[0..rows) into s_pre[0..rows]; every thread of the CTA calls it
__device__ __forceinline__ void line_block_prefix(const int32_t* s_len, int32_t* s_pre, int rows, int32_t* s_warp) {
  const int per = (rows + kLineThreads - 1) / kLineThreads;
  const int lo = min(rows, static_cast<int>(threadIdx.x) * per), hi = min(rows, lo + per);
  int sum = 0;
  for (int r = lo; r < hi; ++r) sum += s_len[r];
  int incl = sum;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < kLineThreads / 32 ? s_warp[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += o;
    }
    if (lane < kLineThreads / 32) s_warp[lane] = w;        // inclusive over warps
  }
  __syncthreads();
  int run = incl - sum + (warp ? s_warp[warp - 1] : 0);
  for (int r = lo; r < hi; ++r) { s_pre[r] = run; run += s_len[r]; }
  if (threadIdx.x == kLineThreads - 1) s_pre[rows] = run;
  __syncthreads();
}

// row that holds packed word w: the largest r with s_pre[r] <= w (rows with length 0 are skipped)
__device__ __forceinline__ int line_row_of(const int32_t* s_pre, int rows, int w) {
  int lo = 0, hi = rows;                 // invariant: s_pre[lo] <= w < s_pre[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_pre[mid] <= w) lo = mid; else hi = mid;
  }
  return lo;
}

// Polls one line of this rank's own slab until its tag is `idx`; lane l returns word l.
__device__ __forceinline__ bool line_poll(const uint4* line, unsigned int idx, long long limit, volatile int* s_abort,
                                          unsigned int& word) {
  const int lane = threadIdx.x & 31;
  const unsigned int* w = reinterpret_cast<const unsigned int*>(line) + lane;
  unsigned int v = ptx::ld_relaxed_sys_u32(w);
  if (__shfl_sync(0xffffffffu, v, 31) == idx) { word = v; return true; }
  const long long t0 = clock64();
  for (;;) {
    v = ptx::ld_relaxed_sys_u32(w);
    if (__shfl_sync(0xffffffffu, v, 31) == idx) { word = v; return true; }
    const int stop = (*s_abort != 0) || (clock64() - t0 > limit);
    if (__any_sync(0xffffffffu, stop)) return false;
    __nanosleep(32);
  }
}

__global__ void __launch_bounds__(kLineThreads)
line_all_gather_kernel(LineArgs a) {
  __shared__ int32_t s_len[kLineMaxRows];
  __shared__ int32_t s_pre[kLineMaxRows + 1];
  __shared__ int32_t s_warp[kLineThreads / 32];
  __shared__ unsigned int s_idx;
  __shared__ int s_abort;
  if (threadIdx.x == 0) { s_idx = a.counter[0] + 1; s_abort = 0; }
  for (int r = threadIdx.x; r < a.rows; r += kLineThreads) {
    int len = a.row_len ? a.row_len[r] : a.cols;
    s_len[r] = max(0, min(len, a.cols));
  }
  __syncthreads();
  const unsigned int idx = s_idx;
  const int slot = static_cast<int>((idx - 1) % static_cast<unsigned int>(a.slots));
  const int lane = threadIdx.x & 31;
  const int gwarp = blockIdx.x * (kLineThreads / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (kLineThreads / 32);
  const int header_lines = (a.rows + 1 + kLineWords - 1) / kLineWords;
  const size_t rank_lines = static_cast<size_t>(a.lines_max);
  const size_t slot_lines = static_cast<size_t>(slot) * a.ranks * rank_lines;

  // ---- send: my message into region [slot][my_rank] of every peer ----
  line_block_prefix(s_len, s_pre, a.rows, s_warp);
  const int total = s_pre[a.rows];
  const int my_lines = header_lines + (total + kLineWords - 1) / kLineWords;
  const int sub = lane & 7, grp = lane >> 3;
  const bool flat = a.row_len == nullptr && a.src_stride == a.cols;      // packed word w is src[w]
  // kLineUnroll lines per warp and iteration: their loads are in flight together
  for (int line0 = gwarp * kLineUnroll; line0 < my_lines; line0 += nwarps * kLineUnroll) {
    unsigned int word[kLineUnroll];
#pragma unroll
    for (int u = 0; u < kLineUnroll; ++u) {
      const int line = line0 + u;
      word[u] = 0;
      if (line >= my_lines) continue;
      if (lane == 31) {
        word[u] = idx;
      } else if (line < header_lines) {
        const int h = line * kLineWords + lane;               // header word index
        if (h == 0) word[u] = static_cast<unsigned int>(total);
        else if (h <= a.rows) word[u] = static_cast<unsigned int>(s_len[h - 1]);
      } else {
        const int w = (line - header_lines) * kLineWords + lane;
        if (w < total) {
          if (flat) {
            word[u] = __float_as_uint(__ldg(a.src + w));
          } else {
            const int r = a.row_len ? line_row_of(s_pre, a.rows, w) : w / a.cols;
            word[u] = __float_as_uint(__ldg(a.src + static_cast<long long>(r) * a.src_stride + (w - s_pre[r])));
          }
        }
      }
    }
    // lanes with the same (lane & 7) hold words 4*sub .. 4*sub+3 of the line as one uint4; lane group
    // `grp` stores the whole line (8 lanes x 16 bytes, one aligned 128-byte store) to peers grp, grp+4
#pragma unroll
    for (int u = 0; u < kLineUnroll; ++u) {
      const int line = line0 + u;
      if (line >= my_lines) break;
      uint4 v;
      v.x = __shfl_sync(0xffffffffu, word[u], 4 * sub);
      v.y = __shfl_sync(0xffffffffu, word[u], 4 * sub + 1);
      v.z = __shfl_sync(0xffffffffu, word[u], 4 * sub + 2);
      v.w = __shfl_sync(0xffffffffu, word[u], 4 * sub + 3);
      const size_t at = (slot_lines + static_cast<size_t>(a.my_rank) * rank_lines + line) * 8 + sub;
      for (int p = grp; p < a.ranks; p += 4)
        if (p != a.my_rank) ptx::st_relaxed_sys_v4(a.peers.slab[p] + at, v);
    }
  }

  // ---- my own rows go straight to the output ----
  {
    float* dst = a.out + static_cast<size_t>(a.my_rank) * a.rows * a.cols;
    const long long n = static_cast<long long>(a.rows) * a.cols;
    for (long long i = static_cast<long long>(blockIdx.x) * kLineThreads + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * kLineThreads) {
      const int r = static_cast<int>(i / a.cols), c = static_cast<int>(i - static_cast<long long>(r) * a.cols);
      dst[i] = c < s_len[r] ? a.src[static_cast<long long>(r) * a.src_stride + c] : a.fill;
    }
    if (a.out_len && blockIdx.x == 0)
      for (int r = threadIdx.x; r < a.rows; r += kLineThreads) a.out_len[a.my_rank * a.rows + r] = s_len[r];
  }

  // ---- receive: one source after the other, starting after my own rank ----
  const uint4* mine = a.peers.slab[a.my_rank] + slot_lines * 8;
  for (int step = 1; step < a.ranks; ++step) {
    const int src_rank = (a.my_rank + step) % a.ranks;
    const uint4* region = mine + static_cast<size_t>(src_rank) * rank_lines * 8;
    __syncthreads();                                       // s_len / s_pre of the previous source are done with
    __shared__ int s_total;
    for (int line = threadIdx.x >> 5; line < header_lines; line += kLineThreads / 32) {
      unsigned int word = 0;
      const bool ok = line_poll(region + static_cast<size_t>(line) * 8, idx, a.limit, &s_abort, word);
      if (!ok) {
        if (lane == 0 && !s_abort) { report(a.status, kErrTimeout, src_rank); s_abort = 1; }
        word = 0;
      }
      const int h = line * kLineWords + lane;
      if (lane < kLineWords) {
        if (h == 0) s_total = static_cast<int>(word);
        else if (h <= a.rows) s_len[h - 1] = max(0, min(static_cast<int>(word), a.cols));
      }
    }
    __syncthreads();
    line_block_prefix(s_len, s_pre, a.rows, s_warp);
    const int r_total = s_abort ? 0 : min(s_total, s_pre[a.rows]);
    const int r_lines = (r_total + kLineWords - 1) / kLineWords;
    float* dst = a.out + static_cast<size_t>(src_rank) * a.rows * a.cols;
    const bool dense = r_total == a.rows * a.cols;
    bool failed = false;
    for (int line0 = gwarp * kLineUnroll; line0 < r_lines && !failed; line0 += nwarps * kLineUnroll) {
      unsigned int word[kLineUnroll];
#pragma unroll
      for (int u = 0; u < kLineUnroll; ++u) {               // first look at all lines at once
        word[u] = 0;
        if (line0 + u < r_lines)
          word[u] = ptx::ld_relaxed_sys_u32(
              reinterpret_cast<const unsigned int*>(region + static_cast<size_t>(header_lines + line0 + u) * 8) + lane);
      }
#pragma unroll
      for (int u = 0; u < kLineUnroll; ++u) {
        const int line = line0 + u;
        if (line >= r_lines) break;
        if (__shfl_sync(0xffffffffu, word[u], 31) != idx &&
            !line_poll(region + static_cast<size_t>(header_lines + line) * 8, idx, a.limit, &s_abort, word[u])) {
          if (lane == 0 && !s_abort) { report(a.status, kErrTimeout, src_rank); s_abort = 1; }
          failed = true;
          break;
        }
        const int w = line * kLineWords + lane;
        if (lane < kLineWords && w < r_total) {
          if (dense) {
            dst[w] = __uint_as_float(word[u]);
          } else {
            const int r = line_row_of(s_pre, a.rows, w);
            dst[static_cast<size_t>(r) * a.cols + (w - s_pre[r])] = __uint_as_float(word[u]);
          }
        }
      }
    }
    if (!dense) {                                           // fill past each row's end
      const long long n = static_cast<long long>(a.rows) * a.cols;
      for (long long i = static_cast<long long>(blockIdx.x) * kLineThreads + threadIdx.x; i < n;
           i += static_cast<long long>(gridDim.x) * kLineThreads) {
        const int r = static_cast<int>(i / a.cols), c = static_cast<int>(i - static_cast<long long>(r) * a.cols);
        if (c >= s_len[r]) dst[i] = a.fill;
      }
    }
    if (a.out_len && blockIdx.x == 0)
      for (int r = threadIdx.x; r < a.rows; r += kLineThreads) a.out_len[src_rank * a.rows + r] = s_len[r];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(&a.counter[1], 1u) + 1;
    if (done == gridDim.x) { a.counter[1] = 0; a.counter[0] = idx; }
  }
}

}  // namespace ulc

extern "C" {
using namespace ulc;

int ulc_lifetime_publish(int32_t* const* pages, int my_rank, int ranks, int phase, int epoch, cudaStream_t s) {
  if (ranks < 1 || ranks > kMaxRanks || phase < 0 || phase >= kPhases) return -kErrUnsupported;
  lifetime_publish_kernel<<<1, 32, 0, s>>>(pages, my_rank, ranks, phase, epoch);
  return static_cast<int>(cudaGetLastError());
}

int ulc_lifetime_wait(const int32_t* page, int ranks, int phase, int epoch, long long limit_cycles, int32_t* status,
                      cudaStream_t s) {
  if (ranks < 1 || ranks > kMaxRanks || phase < 0 || phase >= kPhases) return -kErrUnsupported;
  if (limit_cycles <= 0) limit_cycles = 2000000000LL;
  lifetime_wait_kernel<<<1, 32, 0, s>>>(page, ranks, phase, epoch, limit_cycles, status);
  return static_cast<int>(cudaGetLastError());
}

// slabs: HOST array of `ranks` device pointers (each rank's slab, peer mapped), each holding
// 4 * ranks * n_max 8-byte words, zero-initialised.  counter: device uint32[2], zero-initialised.
// The grid is at most one CTA per SM, so every CTA is resident while it polls.
int ulc_tagged_all_gather(const float* src, int n, int n_max, void* const* slabs, int my_rank, int ranks,
                          unsigned int* counter, float* out, long long limit_cycles, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  if (ranks < 1 || ranks > kMaxRanks || n > n_max) return -kErrUnsupported;
  if (limit_cycles <= 0) limit_cycles = 2000000000LL;
  AgPeers peers;
  for (int r = 0; r < kMaxRanks; ++r) peers.slab[r] = r < ranks ? reinterpret_cast<uint2*>(slabs[r]) : nullptr;
  int blocks = (n + 255) / 256;
  if (blocks > 128) blocks = 128;
  tagged_all_gather_kernel<<<blocks, 256, 0, s>>>(src, n, n_max, peers, my_rank, ranks, counter, out, limit_cycles, status);
  return static_cast<int>(cudaGetLastError());
}

// Lines one rank's message needs at most: header + payload of `rows` full rows.
long long ulc_line_all_gather_lines(int rows, int cols) {
  const long long header = (rows + 1 + kLineWords - 1) / kLineWords;
  return header + (static_cast<long long>(rows) * cols + kLineWords - 1) / kLineWords;
}

// slabs: HOST array of `ranks` device pointers, each slots * ranks * lines_max * 128 bytes, zeroed
// before the first call.  row_len: device int32 [rows] or null.  counter: device uint32[2], zeroed.
// out fp32 [ranks, rows, cols]; out_len int32 [ranks, rows] or null.
int ulc_line_all_gather(const float* src, long long src_stride, const int32_t* row_len, int rows, int cols,
                        void* const* slabs, int my_rank, int ranks, int lines_max, int slots, unsigned int* counter,
                        float* out, int32_t* out_len, float fill, int max_ctas, long long limit_cycles, int32_t* status,
                        cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return 0;
  if (ranks < 1 || ranks > kMaxRanks || rows > kLineMaxRows || slots < 2 ||
      ulc_line_all_gather_lines(rows, cols) > lines_max)
    return -kErrUnsupported;
  if (limit_cycles <= 0) limit_cycles = 2000000000LL;
  LineArgs a;
  a.src = src; a.src_stride = src_stride; a.row_len = row_len; a.rows = rows; a.cols = cols;
  for (int r = 0; r < kMaxRanks; ++r) a.peers.slab[r] = r < ranks ? static_cast<uint4*>(slabs[r]) : nullptr;
  a.my_rank = my_rank; a.ranks = ranks; a.lines_max = lines_max; a.slots = slots; a.counter = counter;
  a.out = out; a.out_len = out_len; a.fill = fill; a.limit = limit_cycles; a.status = status;
  // every CTA polls, so all of them must be resident at once: at most one per SM
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long lines = ulc_line_all_gather_lines(rows, cols);
  const long long per_cta = static_cast<long long>(kLineThreads / 32) * kLineUnroll;
  long long blocks = (lines + per_cta - 1) / per_cta;
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;
  if (blocks > max_ctas) blocks = max_ctas;
  line_all_gather_kernel<<<static_cast<int>(blocks), kLineThreads, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
