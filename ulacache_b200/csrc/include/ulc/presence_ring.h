// State of the parallel presence-bitmap ring (kernels in csrc/presence_ring.cu) and the view of it
// that the residency kernels use as a victim index over their stamp array.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ulc {

constexpr int kPrRecent = 255;
constexpr int kPrCold = 255;
constexpr int kPrChunks = 256;       // chunks of a bucket's summary that are counted / emitted in parallel

enum PrCtl : int { kPrEpoch = 0, kPrDrain = 1, kPrServed = 2, kPrListed = 3, kPrMissCursor = 4, kPrCtlWords = 8 };

struct PRing {
  uint32_t* bits;          // [256][w0]
  uint32_t* summary;       // [256][w1]
  int32_t* slot_bucket;    // [n]
  int32_t* count;          // [256]
  int32_t* bucket_epoch;   // [255], -1 = never used
  int32_t* ctl;            // [kPrCtlWords]
  int32_t* vlist;          // [256][3]: bucket, take, first output position
  int32_t* chunk_count;    // [256][kPrChunks]
  int32_t n, w0, w1;
};

}  // namespace ulc

extern "C" {
// Counts and emits the victims of the buckets listed in r->vlist[0 .. r->ctl[kPrListed]) into `victims`
// (two launches).  Used by ulc_pring_victims and by the residency plan when it keeps bitmaps.
int ulc_pring_count_emit(const ulc::PRing* r, int32_t* victims, int capacity, cudaStream_t s);
// Moves the bits of bucket r->ctl[kPrDrain] (if >= 0) into the cold bucket; `relabel` also rewrites
// slot_bucket (the stand-alone ring keeps an inverse map, the residency kernels derive it from stamps).
int ulc_pring_drain(const ulc::PRing* r, int relabel, cudaStream_t s);
}
