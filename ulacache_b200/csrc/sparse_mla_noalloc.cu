// Sparse MLA decode for callers that may not allocate: the split-KV scratch lives
// in a file-scope device array of this library.  See ulc/no_alloc.h for who needs
// this and for the rules of use.
#include <atomic>
#include "ulc/no_alloc.h"
#include "ulc/status.h"

// Defined in sparse_mla.cu.
extern "C" long long ulc_sparse_mla_scratch_bytes(int B, int H, int splits);
extern "C" int ulc_sparse_mla_decode(const ulc::PoolView* pv, const void* q, const int32_t* loc,
                                     long long loc_stride, const int32_t* lens, int B, int H, int K,
                                     float sm_scale, int format, int splits, void* out, float* lse,
                                     void* scratch, int32_t* status, cudaStream_t stream);

namespace {

// The scratch itself.  In host code this name is only a stand-in for the symbol,
// not a device address: it must never be handed to a kernel directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[ULC_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_addr[kMaxDevices];      // zero-initialised; filled once per device, any thread

// Device address of the array on the current device, looked up once per device.
int scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -ulc::kErrUnsupported;
  void* p = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);      // threads that race here get the same address
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return 0;
}

}  // namespace

extern "C" {

long long ulc_noalloc_scratch_capacity(void) { return ULC_NOALLOC_SCRATCH_BYTES; }

int ulc_sparse_mla_decode_noalloc(const ulc::PoolView* pv, const void* q, const int32_t* loc,
                                  long long loc_stride, const int32_t* lens, int B, int H, int K,
                                  float sm_scale, int format, int splits, void* out, float* lse,
                                  int32_t* status, cudaStream_t stream) {
  if (splits < 1) splits = 1;
  if (B <= 0 || H <= 0 || K <= 0) return 0;
  const long long need = ulc_sparse_mla_scratch_bytes(B, H, splits);
  if (need > ULC_NOALLOC_SCRATCH_BYTES) return -ulc::kErrCapacity;   // too many splits * rows for the array
  void* scratch = nullptr;
  if (splits > 1) {
    const int rc = scratch_address(&scratch);
    if (rc != 0) return rc;
  }
  return ulc_sparse_mla_decode(pv, q, loc, loc_stride, lens, B, H, K, sm_scale, format, splits, out, lse,
                               scratch, status, stream);
}

}  // extern "C"
