"""Victim selection at a large device tier: the stamp scan of the residency kernels against the
parallel presence-bitmap ring, same recency distribution, same number of victims.

    python -m ulacache_b200.benchmarks.residency_plan --slots 1048576 --need 256,4096,65536

State: every slot holds a record last touched in one of ``--epochs`` epochs (uniformly), the current
epoch touched ``--touched`` slots.  Timed (CUDA-graph replay, device time per call):

* ``stamp_plan``    ``ulc_res_plan``: quota from the 256 bucket counts, one coalesced scan of the
                    per-slot stamps that claims victims with an atomic counter, plan assignment;
* ``bitmap_victims`` ``ulc_pring_victims``: bucket list from the counts, set bits counted per (bucket,
                    chunk), ordered emit through the level-1 summaries;
* ``stamp_touch`` / ``bitmap_touch``  the step's pin of ``--touched`` slots in either structure
                    (``ulc_res_pin`` against ``ulc_pring_touch``), since a structure that is cheaper to
                    search and dearer to maintain is no gain;
* ``bitmap_advance`` the ring's step (drain of the expiring bucket into the cold one).

Both select the same number of victims from the same buckets (the scan takes any slots of the boundary
bucket, the bitmap ring the lowest ones).

Reference: ulacache/csrc/eviction/victims.cuh:53-194, scripts/7_5_scheduler/pb_config.json (tuned launch).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json


def main(argv=None):
    import torch
    from ..cache.residency import (CNT_EPOCH, CNT_HBM_FREE, CNT_HOST_FREE, CNT_NEED, CNT_PLAN, CNT_PROMOTE, COLD, RECENT,
                                   ResidencyGeometry, make_residency)
    from ..eviction import ParallelPresenceRing
    from ..ops import _native as N
    from ..storage.layout import OwnerMap
    from .common import time_cuda_graph

    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=1 << 20)
    ap.add_argument("--need", default="256,4096,65536")
    ap.add_argument("--epochs", type=int, default=300, help="distinct last-touch epochs of the resident records")
    ap.add_argument("--touched", type=int, default=65536, help="slots touched by the current step")
    args = ap.parse_args(argv)
    dev = torch.device("cuda")
    n = args.slots
    needs = [int(x) for x in args.need.split(",")]
    cap = max(needs)
    g = torch.Generator(device=dev).manual_seed(3)
    epoch = args.epochs + 5
    stamps = torch.randint(epoch - args.epochs, epoch, (n,), device=dev, generator=g, dtype=torch.int32)
    touched = torch.randperm(n, device=dev, generator=g)[: args.touched].to(torch.int32)
    stamps[touched.long()] = epoch
    # ---- stamp ring of the residency kernels ----
    geometry = ResidencyGeometry(dir_len=n + cap + 64, hbm_slots=n, host_slots=cap, plan_capacity=cap)
    res = make_residency(geometry, OwnerMap(1, 6), 0, dev, victim_index="stamps")
    wired = make_residency(geometry, OwnerMap(1, 6), 0, dev, victim_index="bitmap")     # same plan through the bitmap index
    res.stamps.copy_(stamps)
    res.hbm_tags.copy_(torch.arange(n, device=dev, dtype=torch.int32))
    res.directory[:n] = torch.arange(n, device=dev, dtype=torch.int32)
    host_rows = torch.arange(n, n + cap, device=dev, dtype=torch.int32)
    res.directory[n: n + cap] = -(torch.arange(cap, device=dev, dtype=torch.int32)) - 2       # host slot s encoded as -s-2
    res.host_tags[:cap] = host_rows
    res.promote[:cap] = host_rows
    age = epoch - stamps
    bucket = torch.where(age >= RECENT, torch.full_like(stamps, COLD), stamps % RECENT)
    res.ring.copy_(torch.bincount(bucket.long(), minlength=256).to(torch.int32))
    res.counters[CNT_EPOCH] = epoch
    res.counters[CNT_HBM_FREE] = 0
    res.counters[CNT_HOST_FREE] = 0
    wired.load_state(res.state_dict())            # also builds its bitmaps from the stamps
    # ---- bitmap ring with the same membership ----
    ring = ParallelPresenceRing(n, dev)
    ring.slot_bucket.copy_(bucket)
    ring.count.copy_(res.ring)
    labels = torch.full((255,), -1, dtype=torch.int32, device=dev)
    for e in range(max(0, epoch - 254), epoch + 1):
        labels[e % 255] = e
    ring.bucket_epoch.copy_(labels)
    ring.ctl[0] = epoch
    import numpy as np

    bk = bucket.cpu().numpy().astype(np.int64)
    sl = np.arange(n, dtype=np.int64)
    bits = np.zeros((256, ring.w0), dtype=np.uint32)
    np.bitwise_or.at(bits, (bk, sl >> 5), (np.uint32(1) << (sl & 31).astype(np.uint32)))
    summary = np.zeros((256, ring.w1), dtype=np.uint32)
    bsel, wsel = np.nonzero(bits)
    np.bitwise_or.at(summary, (bsel, wsel >> 5), (np.uint32(1) << (wsel & 31).astype(np.uint32)))
    ring.bits.copy_(torch.from_numpy(bits.view(np.int32)).to(dev))
    ring.summary.copy_(torch.from_numpy(summary.view(np.int32)).to(dev))
    out = []
    victims = torch.empty(cap, dtype=torch.int32, device=dev)
    for need in needs:
        res.counters[CNT_PROMOTE] = need
        res.counters[5:8] = 0
        res.counters[15] = 0
        saved = res.counters.clone()

        def reset():                                    # the plan consumes its counters: put them back
            res.counters.copy_(saved)

        def stamp_plan():
            reset()
            res.plan_step()

        def wired_plan():
            wired.counters.copy_(saved)
            wired.plan_step()

        def bitmap_victims():
            ring.victims(need, victims)

        stamp_plan()
        bitmap_victims()
        wired_plan()
        torch.cuda.synchronize()
        wired.check_status("bitmap-indexed plan")
        assert int(wired.counters[CNT_PLAN]) == int(res.counters[CNT_PLAN])
        res.check_status("stamp plan")
        served_stamp = int(res.counters[CNT_PLAN])
        served_bits = ring.served
        got = victims[:served_bits].long()
        same_buckets = bool(torch.equal(torch.bincount(bucket[got].long(), minlength=256),
                                        torch.bincount(bucket[res.victims[:served_stamp].long()].long(), minlength=256)))
        fill_us = time_cuda_graph(reset)
        row = dict(kernel="victim_selection", slots=n, need=need, served_stamp=served_stamp, served_bitmap=served_bits,
                   same_bucket_histogram=same_buckets,
                   stamp_plan_us=round(time_cuda_graph(stamp_plan) - fill_us, 2),
                   bitmap_indexed_plan_us=round(time_cuda_graph(wired_plan) - fill_us, 2),
                   bitmap_victims_us=round(time_cuda_graph(bitmap_victims), 2))
        out.append(row)
        print(json.dumps(row), flush=True)
    # maintenance cost of a step: pin / touch of the step's slots, and the ring's advance
    ids = touched.clone()
    sel = torch.randperm(n, device=dev, generator=g)[: args.touched].to(torch.int32)

    def stamp_touch():
        res.pin(sel)

    def bitmap_touch():
        ring.touch(sel)

    row = dict(kernel="step_maintenance", slots=n, touched=args.touched,
               stamp_touch_us=round(time_cuda_graph(stamp_touch), 2), bitmap_touch_us=round(time_cuda_graph(bitmap_touch), 2),
               bitmap_advance_us=round(time_cuda_graph(ring.advance, iters=4, replays=1), 2),
               stamp_metadata_mb=round(res.metadata_bytes() / 2 ** 20, 1), bitmap_metadata_mb=round(ring.metadata_bytes / 2 ** 20, 1))
    print(json.dumps(row), flush=True)
    torch.cuda.synchronize()
    N.raise_on_status(ring.status, "bitmap ring")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
