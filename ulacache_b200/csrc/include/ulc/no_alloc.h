// Entry point for callers that cannot allocate device memory.
//
// This function has no counterpart in the reference library.
//
// Some users of this library run where cudaMalloc is off limits: inside a serving
// process whose memory pool was sized and frozen at start-up, inside a region that
// is being captured into a CUDA graph (allocation is illegal there), or in a
// sandboxed plugin that is handed a stream and nothing else.  The split-KV path of
// the sparse MLA decode kernel normally needs a scratch buffer (partial outputs and
// partial log-sum-exps of every KV split) that the caller allocates.  The function
// below runs the same kernel with that scratch placed in a fixed array inside the
// library image instead, so the caller passes only inputs and outputs.
//
// Limits and rules
//  * The array holds ULC_NOALLOC_SCRATCH_BYTES (32 MiB).  Every GPU that loads the
//    library keeps it resident until the process exits.
//  * splits * B * H * 513 * 4 bytes must fit; larger requests are rejected with
//    -2 (capacity) and nothing is launched.
//  * The first call on EACH device looks up the array's device address
//    (cudaGetSymbolAddress) and sets the kernel's shared-memory attribute, both with
//    that device current.  Make that first call, on every device you will use, before
//    starting any stream capture.
//  * All calls share the one array and it keeps whatever the previous call left.
//    Nothing in it has to start at zero: every (split, row) cell a call reads is
//    written by that call first.  A CTA that gives up on a bounded wait writes an
//    empty marker for its cells and reports through the status word; when the status
//    word is non-zero after a call, `out` and `lse` are undefined.  Two calls whose
//    kernels overlap on the GPU (other streams, other threads) race on the array;
//    serialise them.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "pool.h"

#define ULC_NOALLOC_SCRATCH_BYTES (32ll << 20)

extern "C" {

// Same arguments and result as ulc_sparse_mla_decode, minus the scratch pointer.
// Returns 0, a positive cudaError_t, or a negative ulc::Status (-2 when the split
// scratch would exceed ULC_NOALLOC_SCRATCH_BYTES, -6 for unsupported shapes).
int ulc_sparse_mla_decode_noalloc(const ulc::PoolView* pv, const void* q, const int32_t* loc,
                                  long long loc_stride, const int32_t* lens, int B, int H, int K,
                                  float sm_scale, int format, int splits, void* out, float* lse,
                                  int32_t* status, cudaStream_t stream);

// Bytes of the built-in scratch array (for callers that want to size their splits).
long long ulc_noalloc_scratch_capacity(void);

}  // extern "C"
