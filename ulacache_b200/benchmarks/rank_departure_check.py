"""A rank that leaves between steps is noticed on the host before the next launch (run under torchrun,
one rank per GPU, two or more ranks):

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m ulacache_b200.benchmarks.rank_departure_check

Every rank runs a few steps of the peer-memory all-gather (plain peer stores, bounded flag waits), publishing a
heartbeat after each.  The last rank then leaves in order: it synchronises its device (none of its kernels in
flight), announces the departure in the rendezvous store, waits until the others have unmapped its memory, frees
it and exits.  The others check the heartbeats before their next launch, get :class:`PeerFailure` naming the
rank, launch nothing that touches it, unmap its slab and show that their own GPU and context still work.  No
collective of a library is used (the process group is gloo, for the store and the handle exchange only), no
multicast object is bound, nothing faults.  Rank 0 prints one JSON line.

Reference: the reference spins on peers' flags without a bound (csrc/cache/common.cuh:119-127) and has no
departure protocol; this is the host-side replacement for it.
"""
from __future__ import annotations

import datetime
import json
import os
import time


def main():
    import torch
    import torch.distributed as dist
    from ..ops import _native as N
    from ..parallel.health import PeerFailure, RankHeartbeat
    from ..parallel.peer_collectives import PeerAllGather
    from ..parallel.symmetric import SymmetricHeap

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    store = dist.distributed_c10d._get_default_store()
    cpu_group = dist.group.WORLD
    heap = SymmetricHeap(cpu_group=cpu_group, rank=rank, world_size=world, nbytes=16 << 20, device=dev)
    ag = PeerAllGather(heap, 8, [(64, torch.uint8)])
    hb = RankHeartbeat(store, rank, world)
    leaver = world - 1
    steps_ok = 0
    for step in range(1, 4):
        hb.check_peers(min_step=step - 1, stale_after_s=20.0)        # before every launch
        (got,) = ag.gather([torch.full((8, 64), 16 * step + rank, dtype=torch.uint8, device=dev)])
        torch.cuda.synchronize()
        N.raise_on_status(heap.status, "peer all-gather")
        want = torch.arange(world, device=dev, dtype=torch.uint8).repeat_interleave(8)[:, None] + 16 * step
        steps_ok += int(bool((got == want).all()))
        hb.beat(step)
        hb.wait_for_peers(min_step=step, stale_after_s=20.0)
    # everybody has seen step 3 complete everywhere before anyone leaves
    store.set(f"seen3/{rank}", b"1")
    store.wait([f"seen3/{r}" for r in range(world)], datetime.timedelta(seconds=30))

    if rank == leaver:
        torch.cuda.synchronize()                                   # nothing of this rank in flight
        hb.leave()
        store.wait([f"unmapped/{r}" for r in range(world) if r != leaver], datetime.timedelta(seconds=30))
        heap.close(collective=False)
        return

    t0 = time.monotonic()
    seen = None
    while seen is None and time.monotonic() - t0 < 20.0:
        try:
            hb.check_peers(min_step=4, stale_after_s=5.0)          # the check that precedes the step-4 launch
            time.sleep(0.01)
        except PeerFailure as exc:
            seen = exc.ranks
    launched_after = False                                         # the step-4 all-gather is NOT launched
    # this rank's device and context are intact: a local kernel of the library runs and the status word is clean
    from ..ops import fp8

    x = torch.randn(16, 256, device=dev, dtype=torch.bfloat16)
    q, s = fp8.act_quant(x)
    torch.cuda.synchronize()
    qr, sr = fp8.act_quant_reference(x)
    local_ok = bool(torch.allclose(s, sr)) and int(heap.status.abs().sum()) == 0
    heap.close(collective=False)                                   # unmap the leaver's slab, free ours
    store.set(f"unmapped/{rank}", b"1")
    res = dict(ranks=world, steps_before_departure_ok=steps_ok, departed=leaver, detected=seen,
               detect_s=round(time.monotonic() - t0, 3), launched_after_departure=launched_after,
               local_gpu_ok_after=local_ok)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if not (steps_ok == 3 and seen == [leaver] and local_ok):
        raise SystemExit(1)


if __name__ == "__main__":
    main()
