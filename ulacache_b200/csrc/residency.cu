// GPU-side residency transaction for one rank's share of the logical address
// space: register -> begin_step -> pin -> plan (quota, enumerate, assign) ->
// exchange (see exchange.cu) -> commit -> resolve -> release.
//
// All kernels are integer metadata work.  They never trap: inconsistencies and
// capacity shortfalls are written to the status buffer / counters and the
// affected rows are simply left where they were (resolve() then reports them as
// masked and the host decides what to do).
//
// Reference counterparts: ulacache/csrc/cache/cpu_residency.cuh:107-343
// (register_rows, begin_current, pin_rows, reserve, commit, release_rows),
// ulacache/csrc/eviction/victims.cuh:53-194 (victim selection) and the Triton
// `_remap` kernel (ulacache/cache/kernels/local_cache.py:149).
#include "ulc/pool.h"
#include "ulc/presence_ring.h"
#include "ulc/ptx.cuh"
#include "ulc/residency.h"

namespace ulc {

__global__ void register_rows_kernel(ResidencyState st, OwnerMap map, int my_rank,
                                     const int32_t* __restrict__ ids, int n, int prefer_device,
                                     int32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t id = ids[i];
  if (!id_valid(id) || map.owner(id) != my_rank) return;
  const int32_t local = map.local(id);
  if (local >= st.dir_len) { report(status, kErrBounds, id); return; }
  if (st.directory[local] != kDirUnallocated) { report(status, kErrInvariant, id); return; }
  const int32_t epoch = st.counters[kCntEpoch];
  if (prefer_device) {
    const int32_t c = atomicSub(&st.counters[kCntHbmFree], 1);
    if (c > 0) {
      const int32_t slot = st.hbm_free[c - 1];
      st.directory[local] = slot;
      st.hbm_tags[slot] = local;
      st.stamps[slot] = epoch;
      atomicAdd(&st.ring[epoch % kRecentBuckets], 1);
      bm_set(st, epoch % kRecentBuckets, slot);
      atomicAdd(&st.counters[kCntRegistered], 1);
      return;
    }
    atomicAdd(&st.counters[kCntHbmFree], 1);
  }
  const int32_t c = atomicSub(&st.counters[kCntHostFree], 1);
  if (c > 0) {
    const int32_t slot = st.host_free[c - 1];
    st.directory[local] = dir_encode_host(slot);
    st.host_tags[slot] = local;
    atomicAdd(&st.counters[kCntRegistered], 1);
    return;
  }
  atomicAdd(&st.counters[kCntHostFree], 1);
  if (!prefer_device) {   // host full: fall back to HBM
    const int32_t d = atomicSub(&st.counters[kCntHbmFree], 1);
    if (d > 0) {
      const int32_t slot = st.hbm_free[d - 1];
      st.directory[local] = slot;
      st.hbm_tags[slot] = local;
      st.stamps[slot] = epoch;
      atomicAdd(&st.ring[epoch % kRecentBuckets], 1);
      bm_set(st, epoch % kRecentBuckets, slot);
      atomicAdd(&st.counters[kCntRegistered], 1);
      return;
    }
    atomicAdd(&st.counters[kCntHbmFree], 1);
  }
  report(status, kErrCapacity, id);
}

__global__ void release_rows_kernel(ResidencyState st, OwnerMap map, int my_rank,
                                    const int32_t* __restrict__ ids, int n, int32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t id = ids[i];
  if (!id_valid(id) || map.owner(id) != my_rank) return;
  const int32_t local = map.local(id);
  if (local >= st.dir_len) { report(status, kErrBounds, id); return; }
  const int32_t e = atomicExch(&st.directory[local], kDirUnallocated);
  if (e == kDirUnallocated) return;   // double free is ignored
  const int32_t epoch = st.counters[kCntEpoch];
  if (dir_on_device(e)) {
    const int32_t stamp = st.stamps[e];
    if (stamp >= 0) {
      atomicSub(&st.ring[bucket_of(stamp, epoch)], 1);
      bm_clear(st, bucket_of(stamp, epoch), e);
    }
    st.stamps[e] = -1;
    st.hbm_tags[e] = -1;
    st.hbm_free[atomicAdd(&st.counters[kCntHbmFree], 1)] = e;
  } else {
    const int32_t s = dir_host_slot(e);
    st.host_tags[s] = -1;
    st.host_free[atomicAdd(&st.counters[kCntHostFree], 1)] = s;
  }
  atomicSub(&st.counters[kCntRegistered], 1);
}

__global__ void begin_step_kernel(ResidencyState st) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int32_t epoch = st.counters[kCntEpoch] + 1;
  st.counters[kCntEpoch] = epoch;
  // the bucket being reused still counts slots last touched 255 epochs ago: they turn cold
  const int b = epoch % kRecentBuckets;
  st.ring[kColdBucket] += st.ring[b];
  st.ring[b] = 0;
  // with a bitmap index the bits of the reused bucket (slots last touched 255 epochs ago) move to the
  // cold bucket in the launch that follows
  st.counters[kCntRingCtl + kPrDrain] = (st.bits != nullptr && epoch >= kRecentBuckets) ? b : -1;
  st.counters[kCntPromote] = 0;
  st.counters[kCntPlan] = 0;
  st.counters[kCntVictims] = 0;
  st.counters[kCntNeedVictims] = 0;
  st.counters[kCntFromFree] = 0;
  st.counters[kCntBoundaryTaken] = 0;
  st.counters[kCntUnserved] = 0;
}

// Touch every selected row this rank owns; queue host-resident ones for promotion.
__global__ void pin_rows_kernel(ResidencyState st, OwnerMap map, int my_rank,
                                const int32_t* __restrict__ sel, int n, int32_t* status) {
  const int32_t epoch = st.counters[kCntEpoch];
  int hits = 0, misses = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t id = sel[i];
    if (!id_valid(id) || map.owner(id) != my_rank) continue;
    const int32_t local = map.local(id);
    if (local >= st.dir_len) { report(status, kErrBounds, id); continue; }
    const int32_t e = st.directory[local];
    if (dir_on_device(e)) {
      const int32_t old = atomicExch(&st.stamps[e], epoch);
      if (old != epoch) {
        if (old >= 0) {
          atomicSub(&st.ring[bucket_of(old, epoch)], 1);
          bm_clear(st, bucket_of(old, epoch), e);
        }
        atomicAdd(&st.ring[epoch % kRecentBuckets], 1);
        bm_set(st, epoch % kRecentBuckets, e);
      }
      ++hits;
    } else if (dir_on_host(e)) {
      if (atomicExch(&st.access_time[local], epoch) != epoch) {
        const int32_t at = atomicAdd(&st.counters[kCntPromote], 1);
        if (at < st.plan_capacity) st.promote[at] = local;
        ++misses;
      }
    }
  }
  hits = __reduce_add_sync(0xffffffffu, hits);
  misses = __reduce_add_sync(0xffffffffu, misses);
  if ((threadIdx.x & 31) == 0) {
    if (hits) atomicAdd(&st.counters[kCntHits], hits);
    if (misses) atomicAdd(&st.counters[kCntMisses], misses);
  }
}

__global__ void plan_quota_kernel(ResidencyState st, int32_t* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int32_t* c = st.counters;
  int32_t want = c[kCntPromote];
  if (want > st.plan_capacity) {
    report(status, kErrCapacity, want);
    c[kCntUnserved] += want - st.plan_capacity;
    want = st.plan_capacity;
    c[kCntPromote] = want;
  }
  const int32_t from_free = min(want, c[kCntHbmFree]);
  c[kCntFromFree] = from_free;
  int32_t cutoff, quota;
  const int32_t served = victim_cutoff(st.ring, c[kCntEpoch], want - from_free, &cutoff, &quota);
  c[kCntNeedVictims] = served;
  c[kCntCutoffEpoch] = cutoff;
  c[kCntBoundaryQuota] = quota;
  if (served < want - from_free) {
    report(status, kErrCapacity, want - from_free - served);
    c[kCntUnserved] += want - from_free - served;
  }
  if (st.bits != nullptr) {
    // the same decision as a list of (bucket, take, first output position) for the bitmap emit: the cold
    // bucket, then recent buckets from the oldest epoch up to the cutoff epoch (which gives `quota`)
    int listed = 0, got = 0;
    auto add = [&](int bucket, int take) {
      if (take <= 0) return;
      st.vlist[listed * 3] = bucket; st.vlist[listed * 3 + 1] = take; st.vlist[listed * 3 + 2] = got;
      got += take; ++listed;
    };
    if (served > 0) {
      const int32_t epoch = c[kCntEpoch];
      if (cutoff == -0x7fffffff) {
        add(kColdBucket, quota);
      } else {
        add(kColdBucket, st.ring[kColdBucket]);
        for (int32_t e = epoch - kRecentBuckets + 1; e < cutoff && e < epoch; ++e)
          if (e >= 0) add(e % kRecentBuckets, st.ring[e % kRecentBuckets]);
        if (cutoff < epoch && cutoff >= 0) add(cutoff % kRecentBuckets, quota);
      }
    }
    c[kCntRingCtl + kPrListed] = listed;
    c[kCntVictims] = got;
  }
}

__global__ void plan_enumerate_kernel(ResidencyState st) {
  const int32_t need = st.counters[kCntNeedVictims];
  if (need <= 0) return;
  const int32_t epoch = st.counters[kCntEpoch];
  const int32_t cutoff = st.counters[kCntCutoffEpoch];
  const int32_t quota = st.counters[kCntBoundaryQuota];
  const bool cold_boundary = cutoff == -0x7fffffff;
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < st.hbm_slots; s += gridDim.x * blockDim.x) {
    const int32_t stamp = st.stamps[s];
    if (stamp < 0 || stamp == epoch) continue;
    bool take = false;
    if (cold_boundary) {
      if (epoch - stamp >= kRecentBuckets) take = atomicAdd(&st.counters[kCntBoundaryTaken], 1) < quota;
    } else if (stamp < cutoff) {
      take = true;
    } else if (stamp == cutoff && quota > 0) {
      take = atomicAdd(&st.counters[kCntBoundaryTaken], 1) < quota;
    }
    if (take) {
      const int32_t at = atomicAdd(&st.counters[kCntVictims], 1);
      if (at < st.plan_capacity) st.victims[at] = s;
    }
  }
}

__global__ void plan_assign_kernel(ResidencyState st, int32_t* status) {
  const int32_t want = st.counters[kCntPromote];
  const int32_t from_free = st.counters[kCntFromFree];
  const int32_t victims = min(st.counters[kCntVictims], st.counters[kCntNeedVictims]);
  const int32_t served = min(want, from_free + victims);
  const int32_t free_before = st.counters[kCntHbmFree];
  const int cap = st.plan_capacity;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < served; i += gridDim.x * blockDim.x) {
    const int32_t row = st.promote[i];
    const int32_t host_src = dir_host_slot(st.directory[row]);
    int32_t gpu, old_row = -1, host_dst = -1;
    if (i < from_free) {
      gpu = st.hbm_free[free_before - 1 - i];
    } else {
      gpu = st.victims[i - from_free];
      old_row = st.hbm_tags[gpu];
      host_dst = host_src;   // the evicted record takes the promoted record's host slot
      if (old_row < 0) report(status, kErrInvariant, gpu);
    }
    st.plan[kPlanRow * cap + i] = row;
    st.plan[kPlanGpu * cap + i] = gpu;
    st.plan[kPlanHostSrc * cap + i] = host_src;
    st.plan[kPlanHostDst * cap + i] = host_dst;
    st.plan[kPlanOldRow * cap + i] = old_row;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) st.counters[kCntPlan] = served;
}

__global__ void commit_kernel(ResidencyState st) {
  const int32_t n = st.counters[kCntPlan];
  const int32_t epoch = st.counters[kCntEpoch];
  const int cap = st.plan_capacity;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t row = st.plan[kPlanRow * cap + i];
    const int32_t gpu = st.plan[kPlanGpu * cap + i];
    const int32_t host_src = st.plan[kPlanHostSrc * cap + i];
    const int32_t host_dst = st.plan[kPlanHostDst * cap + i];
    const int32_t old_row = st.plan[kPlanOldRow * cap + i];
    if (old_row >= 0) {
      const int32_t old_stamp = st.stamps[gpu];
      if (old_stamp >= 0) {
        atomicSub(&st.ring[bucket_of(old_stamp, epoch)], 1);
        bm_clear(st, bucket_of(old_stamp, epoch), gpu);
      }
      st.directory[old_row] = dir_encode_host(host_dst);
      st.host_tags[host_dst] = old_row;
      atomicAdd(&st.counters[kCntEvictions], 1);
    } else {
      st.host_tags[host_src] = -1;
      st.host_free[atomicAdd(&st.counters[kCntHostFree], 1)] = host_src;
    }
    st.directory[row] = gpu;
    st.hbm_tags[gpu] = row;
    st.stamps[gpu] = epoch;
    atomicAdd(&st.ring[epoch % kRecentBuckets], 1);
    bm_set(st, epoch % kRecentBuckets, gpu);
    atomicAdd(&st.counters[kCntPromotions], 1);
  }
}

// Pop the HBM free-stack entries consumed by the plan.  Runs after commit so that
// plan_assign could still read the stack.
__global__ void commit_finish_kernel(ResidencyState st) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int32_t used = min(st.counters[kCntFromFree], st.counters[kCntPlan]);
  st.counters[kCntHbmFree] -= used;
  st.counters[kCntFromFree] = 0;
  st.counters[kCntPromote] = 0;
}

// Logical IDs -> physical locations (rank << 28 | slot), -1 when masked or not
// resident in HBM.  Peer directories are read through their mapped pointers.
__global__ void resolve_kernel(PoolView pv, const int32_t* __restrict__ sel, int32_t* __restrict__ loc,
                               int n, int32_t* __restrict__ not_resident, int32_t* status) {
  int bad = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t id = sel[i];
    int32_t out = kLocMasked;
    if (id_valid(id)) {
      const int32_t owner = pv.map.owner(id);
      const int32_t local = pv.map.local(id);
      if (local < pv.dir_len) {
        const int32_t e = owner == pv.my_rank ? pv.dir[owner][local]
                                              : ptx::ld_relaxed_sys(pv.dir[owner] + local);
        if (dir_on_device(e) && e < pv.hbm_slots) out = loc_encode(owner, e);
        else ++bad;
      } else {
        report(status, kErrBounds, id);
      }
    }
    loc[i] = out;
  }
  bad = __reduce_add_sync(0xffffffffu, bad);
  if (bad && not_resident && (threadIdx.x & 31) == 0) atomicAdd(not_resident, bad);
}

}  // namespace ulc

extern "C" {
using namespace ulc;

static inline int grid_for(int n, int threads, int cap) {
  int g = (n + threads - 1) / threads;
  return g < 1 ? 1 : (g > cap ? cap : g);
}

int ulc_res_register(const ResidencyState* st, const OwnerMap* map, int my_rank, const int32_t* ids,
                     int n, int prefer_device, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  register_rows_kernel<<<(n + 255) / 256, 256, 0, s>>>(*st, *map, my_rank, ids, n, prefer_device, status);
  return static_cast<int>(cudaGetLastError());
}
int ulc_res_release(const ResidencyState* st, const OwnerMap* map, int my_rank, const int32_t* ids,
                    int n, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  release_rows_kernel<<<(n + 255) / 256, 256, 0, s>>>(*st, *map, my_rank, ids, n, status);
  return static_cast<int>(cudaGetLastError());
}
// The residency state seen as a presence ring (bitmaps, bucket list, control words in the counters).
static inline PRing ring_view(const ResidencyState* st) {
  PRing r;
  r.bits = st->bits; r.summary = st->summary; r.slot_bucket = nullptr; r.count = st->ring; r.bucket_epoch = nullptr;
  r.ctl = st->counters + kCntRingCtl; r.vlist = st->vlist; r.chunk_count = st->chunk_count;
  r.n = st->hbm_slots; r.w0 = st->w0; r.w1 = st->w1;
  return r;
}

int ulc_res_begin_step(const ResidencyState* st, cudaStream_t s) {
  begin_step_kernel<<<1, 32, 0, s>>>(*st);
  if (st->bits != nullptr) {
    const PRing r = ring_view(st);
    return ulc_pring_drain(&r, 0, s);
  }
  return static_cast<int>(cudaGetLastError());
}
int ulc_res_pin(const ResidencyState* st, const OwnerMap* map, int my_rank, const int32_t* sel, int n,
                int blocks, int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  pin_rows_kernel<<<grid_for(n, 256, blocks > 0 ? blocks : 512), 256, 0, s>>>(*st, *map, my_rank, sel, n, status);
  return static_cast<int>(cudaGetLastError());
}
// quota -> enumerate -> assign, three dependent launches on one stream
int ulc_res_plan(const ResidencyState* st, int victim_blocks, int assign_blocks, int32_t* status,
                 cudaStream_t s) {
  plan_quota_kernel<<<1, 32, 0, s>>>(*st, status);
  if (st->bits != nullptr) {
    const PRing r = ring_view(st);
    const int rc = ulc_pring_count_emit(&r, st->victims, st->plan_capacity, s);
    if (rc != 0) return rc;
  } else {
    plan_enumerate_kernel<<<grid_for(st->hbm_slots, 256, victim_blocks > 0 ? victim_blocks : 296), 256, 0, s>>>(*st);
  }
  plan_assign_kernel<<<grid_for(st->plan_capacity, 256, assign_blocks > 0 ? assign_blocks : 128), 256, 0, s>>>(*st, status);
  return static_cast<int>(cudaGetLastError());
}
int ulc_res_commit(const ResidencyState* st, cudaStream_t s) {
  commit_kernel<<<grid_for(st->plan_capacity, 256, 128), 256, 0, s>>>(*st);
  commit_finish_kernel<<<1, 32, 0, s>>>(*st);
  return static_cast<int>(cudaGetLastError());
}
int ulc_res_resolve(const PoolView* pv, const int32_t* sel, int32_t* loc, int n, int32_t* not_resident,
                    int32_t* status, cudaStream_t s) {
  if (n <= 0) return 0;
  resolve_kernel<<<grid_for(n, 256, 1024), 256, 0, s>>>(*pv, sel, loc, n, not_resident, status);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
