// Symmetric heap plumbing (host code): slab allocation, CUDA IPC handle export /
// import with a handle cache, peer-access checks, and the cross-rank step
// barrier kernel built on system-scope flags with bounded waits.
//
// Every rank allocates one slab with cudaMalloc, exports its IPC handle, and
// opens every peer's slab; all pools (KV planes, index pages, directories,
// flags, exchange buffers) are carved out of the slab so any kernel can address
// (rank, offset).  The slab is plain cudaMalloc memory: no multicast object is
// bound to it, so a rank that dies leaves its peers' GPUs healthy.
//
// Reference counterparts: IPCManager (ulacache/csrc/transfer/ipc.cuh:54, handle
// cache and cuMemGetAddressRange), step publication and the P2P atomic check
// (ulacache/csrc/storage/records.cuh:327-377).  Unlike the reference's
// begin_global_step (ulacache/csrc/cache/common.cuh:119-127) the barrier here
// gives up after a limit and reports kErrTimeout.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>
#include <map>
#include <mutex>
#include <string>
#include "ulc/layout.h"
#include "ulc/ptx.cuh"

namespace ulc {

static std::mutex g_ipc_mutex;
static std::map<std::string, void*> g_open_handles;   // handle bytes -> mapped base

// Flags page layout (int32): [0..7] arrival flag written by rank r, [16] this rank's
// barrier count.  The count lives on the device so that a captured CUDA graph,
// whose kernel arguments are frozen, still advances it on every replay (all ranks
// run the same sequence of barriers, so their counts agree).
__global__ void step_barrier_kernel(int32_t* const* flag_pages, int my_rank, int ranks,
                                    long long limit_cycles, int32_t* status) {
  __shared__ int32_t s_epoch;
  const int r = threadIdx.x;
  if (r == 0) {
    int32_t* mine = flag_pages[my_rank];
    s_epoch = mine[16] + 1;
    mine[16] = s_epoch;
  }
  __syncthreads();
  const int32_t epoch = s_epoch;
  if (r < ranks) {
    // announce: write my count into slot [my_rank] of every rank's page
    __threadfence_system();
    ptx::st_release_sys(flag_pages[r] + my_rank, epoch);
  }
  __syncthreads();
  if (r < ranks) {
    if (!ptx::wait_flag_ge(flag_pages[my_rank] + r, epoch, limit_cycles)) report(status, kErrTimeout, r);
  }
}

__global__ void p2p_atomic_probe_kernel(int32_t* remote_word, int32_t* out) {
  // one relaxed system-scope add on a peer's word; the host checks the result arrives
  out[0] = atomicAdd_system(remote_word, 1);
}

}  // namespace ulc

extern "C" {
using namespace ulc;

// Plain device allocation outside any framework allocator (IPC-exportable).
int ulc_slab_alloc(void** out, unsigned long long bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*out, 0, bytes));
}
int ulc_slab_free(void* p) { return static_cast<int>(cudaFree(p)); }

// 64-byte IPC handle of the allocation containing `ptr`; *offset = ptr - allocation base.
int ulc_ipc_get_handle(const void* ptr, unsigned char* handle64, unsigned long long* offset) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  *offset = 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess && fn != nullptr) {
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    CUdeviceptr base = 0;
    size_t size = 0;
    if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS)
      *offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
  }
  return 0;
}

// Map a peer's allocation (cached: the same handle maps once per process).
int ulc_ipc_open_handle(const unsigned char* handle64, void** out_base) {
  std::lock_guard<std::mutex> lock(g_ipc_mutex);
  const std::string key(reinterpret_cast<const char*>(handle64), sizeof(cudaIpcMemHandle_t));
  auto it = g_open_handles.find(key);
  if (it != g_open_handles.end()) {
    *out_base = it->second;
    return 0;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return static_cast<int>(e);
  g_open_handles[key] = p;
  *out_base = p;
  return 0;
}

// Unmap ONE peer allocation opened with ulc_ipc_open_handle (by the base address it returned).
// A process may hold several symmetric heaps at once; closing one must leave the others mapped.
int ulc_ipc_close_handle(void* base) {
  std::lock_guard<std::mutex> lock(g_ipc_mutex);
  for (auto it = g_open_handles.begin(); it != g_open_handles.end(); ++it) {
    if (it->second == base) {
      const cudaError_t e = cudaIpcCloseMemHandle(base);
      g_open_handles.erase(it);
      return static_cast<int>(e);
    }
  }
  return 0;      // not (or no longer) mapped: nothing to do
}

int ulc_ipc_close_all() {
  std::lock_guard<std::mutex> lock(g_ipc_mutex);
  int rc = 0;
  for (auto& kv : g_open_handles) {
    cudaError_t e = cudaIpcCloseMemHandle(kv.second);
    if (e != cudaSuccess) rc = static_cast<int>(e);
  }
  g_open_handles.clear();
  return rc;
}

int ulc_p2p_native_atomics(int device, int peer, int* supported) {
  return static_cast<int>(cudaDeviceGetP2PAttribute(supported, cudaDevP2PAttrNativeAtomicSupported, device, peer));
}

int ulc_can_access_peer(int device, int peer, int* can) {
  return static_cast<int>(cudaDeviceCanAccessPeer(can, device, peer));
}

// flag_pages: device array of `ranks` pointers (each rank's flags page, peer-mapped).
int ulc_step_barrier(int32_t* const* flag_pages, int my_rank, int ranks, long long limit_cycles,
                     int32_t* status, cudaStream_t s) {
  if (ranks < 1 || ranks > kMaxRanks) return -kErrUnsupported;
  if (limit_cycles <= 0) limit_cycles = 2000000000LL;
  step_barrier_kernel<<<1, 32, 0, s>>>(flag_pages, my_rank, ranks, limit_cycles, status);
  return static_cast<int>(cudaGetLastError());
}

int ulc_p2p_atomic_probe(int32_t* remote_word, int32_t* out, cudaStream_t s) {
  p2p_atomic_probe_kernel<<<1, 1, 0, s>>>(remote_word, out);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
