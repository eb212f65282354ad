"""Leases on the destinations of a receive in flight, and the publication copy.

While a remote writer (or a staged chunk) fills records of this cache, their device slots must not be
chosen as eviction victims.  ``acquire`` looks the rows up, counts a lease on every device slot and takes
a slot out of its recency bucket on the first lease; ``release`` drops the leases and stamps a slot as
touched now when its last lease goes; ``publish`` copies complete records from a staging buffer to the
acquired locations (HBM planes or pinned host planes), one warp per (record, layer).

CUDA residencies run the kernels of ``csrc/receive.cu``; CPU residencies run the same steps in torch (the
oracle of the GPU test).

Reference: ulacache/csrc/cache/local_cache.cuh:79-133 (acquire / release receive locations),
ulacache/transfer/kernels/receive_publication.py:15-90, ulacache/transfer/receive_window.py:159.
"""
from __future__ import annotations

import ctypes as C

STAMP_LEASED = -2


class ReceiveLeases:
    def __init__(self, residency):
        import torch

        self.res = residency
        self.leases = torch.zeros(residency.geometry.hbm_slots, dtype=torch.int32, device=residency.device)
        self.cuda = hasattr(residency, "native_state")

    def acquire(self, ids):
        """int32 ids -> int32 locations (device slot >= 0, host slot as -slot-2, -1 = refused and reported)."""
        import torch

        res = self.res
        ids = ids.reshape(-1).to(device=res.device, dtype=torch.int32).contiguous()
        loc = torch.full_like(ids, -1)
        if self.cuda:
            N = res._N
            N.check(N.cuda().ulc_receive_acquire(C.byref(res.native_state), C.byref(res._map), C.c_int(res.my_rank),
                                                 N.ptr(ids), C.c_int(ids.numel()), N.ptr(self.leases), N.ptr(loc),
                                                 N.ptr(res.status), N.stream()), "receive_acquire")
            return loc
        from ..cache.residency import CNT_EPOCH, COLD, RECENT

        mine, local = res._owned_locals(ids)
        epoch = int(res.counters[CNT_EPOCH])
        for i in range(ids.numel()):
            if not bool(mine[i]) or int(local[i]) >= res.geometry.dir_len:
                raise ValueError("a received row is not owned by this rank")
            e = int(res.directory[int(local[i])])
            if e == -1:
                raise RuntimeError("a received row has no slot")
            if e >= 0:
                if int(self.leases[e]) == 0:
                    old = int(res.stamps[e])
                    res.stamps[e] = STAMP_LEASED
                    if old >= 0:
                        res.ring[COLD if epoch - old >= RECENT else old % RECENT] -= 1
                self.leases[e] += 1
            loc[i] = e
        return loc

    def release(self, ids, locations):
        import torch

        res = self.res
        ids = ids.reshape(-1).to(device=res.device, dtype=torch.int32).contiguous()
        if self.cuda:
            N = res._N
            N.check(N.cuda().ulc_receive_release(C.byref(res.native_state), C.byref(res._map), C.c_int(res.my_rank),
                                                 N.ptr(ids), C.c_int(ids.numel()), N.ptr(self.leases), N.ptr(locations),
                                                 N.ptr(res.status), N.stream()), "receive_release")
            return
        from ..cache.residency import CNT_EPOCH, RECENT

        _, local = res._owned_locals(ids)
        epoch = int(res.counters[CNT_EPOCH])
        for i in range(ids.numel()):
            e = int(locations[i])
            if e < 0:
                continue
            if int(res.directory[int(local[i])]) != e or int(self.leases[e]) <= 0:
                raise RuntimeError("a lease is released on a row that moved or was never leased")
            self.leases[e] -= 1
            if int(self.leases[e]) == 0:
                res.stamps[e] = epoch
                res.ring[epoch % RECENT] += 1
                res.access_time[int(local[i])] = epoch

    def publish(self, staging, source_rows, locations, device_plane, host_plane=None):
        """``staging`` uint8 [layers, rows, row_bytes]; ``device_plane`` uint8 [layers, slots, row_bytes];
        ``host_plane`` the same over pinned host memory (or None).  Record ``source_rows[i]`` of every layer
        goes to ``locations[i]``."""
        import torch

        layers, _, rb = staging.shape
        if self.cuda:
            N = self.res._N
            src = source_rows.to(device=self.res.device, dtype=torch.int32).contiguous()
            hp = host_plane
            N.check(N.cuda().ulc_receive_publish(
                N.ptr(staging), C.c_longlong(staging.stride(0)), N.ptr(src), N.ptr(locations), C.c_int(src.numel()),
                C.c_int(layers), N.ptr(device_plane), C.c_longlong(device_plane.stride(0)), C.c_int(device_plane.shape[1]),
                N.ptr(hp), C.c_longlong(hp.stride(0) if hp is not None else 0), C.c_int(hp.shape[1] if hp is not None else 0),
                C.c_int(rb), N.ptr(self.res.status), N.stream()), "receive_publish")
            return
        for i in range(source_rows.numel()):
            e = int(locations[i])
            if e == -1:
                continue
            if e >= 0:
                device_plane[:, e] = staging[:, int(source_rows[i])]
            else:
                host_plane[:, -e - 2] = staging[:, int(source_rows[i])]
