"""Ablation policies that replay a selection trace on the GPU (CPU tensors fall back to the oracle).

* :class:`ExactLruPolicy` - per-slot timestamps; victims by a byte-radix select of the smallest
  (stamp, slot) keys (kernel ``exact_lru_victims_kernel``).
* :class:`LinkedListLruPolicy` - a doubly linked recency list walked by one device thread.
* :class:`HotBufferPolicy` - a fixed buffer per request, the HiSparse baseline's scheme.
* :func:`trace_hits` - read-only: how many selected ids are resident.

Reference: ulacache/csrc/eviction/naive_lru.cuh:61-139, csrc/kvcacheio/linked_list_lru.cuh:75,
hisparse_union.cuh:310, trace_hits.cuh:1-107 and their Python wrappers under ulacache/eviction/.
"""
from __future__ import annotations

import ctypes as C


def _n():
    from ..ops import _native as N

    return N


class ExactLruPolicy:
    """State: dir[id] -> slot | -1, id_of[slot], stamp[slot].  ``step`` touches hits, places
    misses into free slots and then into the least recently used slots."""

    def __init__(self, capacity: int, id_space: int, device):
        import torch

        self.capacity, self.id_space = capacity, id_space
        self.dir = torch.full((id_space,), -1, dtype=torch.int32, device=device)
        self.id_of = torch.full((capacity,), -1, dtype=torch.int32, device=device)
        self.stamp = torch.full((capacity,), -1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.totals = dict(hits=0, misses=0, evictions=0, overflow=0)

    def victims(self, need: int):
        """Slots holding the ``need`` least recently used records not touched in this step."""
        import torch

        if need <= 0:
            return torch.empty(0, dtype=torch.int32, device=self.dir.device)
        if not self.dir.is_cuda:
            live = ((self.id_of >= 0) & (self.stamp != self.epoch)).nonzero().flatten()
            key = self.stamp[live].long() * (self.capacity + 1) + live
            return live[key.argsort()[:need]].to(torch.int32)
        N = _n()
        out = torch.empty(need, dtype=torch.int32, device=self.dir.device)
        cnt = torch.zeros(1, dtype=torch.int32, device=self.dir.device)
        N.check(N.cuda().ulc_ablate_exact_lru_victims(N.ptr(self.stamp), N.ptr(self.id_of), C.c_int(self.capacity),
                                                      C.c_int(self.epoch), C.c_int(need), N.ptr(out), N.ptr(cnt),
                                                      N.stream()), "exact_lru_victims")
        return out[: int(cnt)]

    def step(self, ids):
        """``ids``: int tensor of distinct record ids accessed this step.  Returns (hits, misses, evicted ids)."""
        import torch

        self.epoch += 1
        ids = ids.to(self.dir.device).long()
        slots = self.dir[ids]
        hit = slots >= 0
        self.stamp[slots[hit].long()] = self.epoch
        miss_ids = ids[~hit]
        n_miss = int(miss_ids.numel())
        free = (self.id_of < 0).nonzero().flatten()[:n_miss]
        need = n_miss - int(free.numel())
        vict = self.victims(need).long()
        evicted = self.id_of[vict].clone()
        self.dir[evicted.long()] = -1
        target = torch.cat([free, vict])
        placed = miss_ids[: target.numel()]
        self.id_of[target] = placed.to(torch.int32)
        self.stamp[target] = self.epoch
        self.dir[placed] = target.to(torch.int32)
        over = n_miss - int(target.numel())
        h = int(hit.sum())
        self.totals["hits"] += h
        self.totals["misses"] += n_miss
        self.totals["evictions"] += int(evicted.numel())
        self.totals["overflow"] += over
        return h, n_miss, evicted


class LinkedListLruPolicy:
    def __init__(self, capacity: int, id_space: int, device):
        import torch

        i32 = dict(dtype=torch.int32, device=device)
        self.capacity = capacity
        self.dir = torch.full((id_space,), -1, **i32)
        self.id_of = torch.full((capacity,), -1, **i32)
        self.stamp = torch.full((capacity,), -1, **i32)
        self.next = torch.full((capacity,), -1, **i32)
        self.prev = torch.full((capacity,), -1, **i32)
        self.list = torch.tensor([-1, -1, capacity, 0], **i32)                 # head, tail, free height, epoch
        self.free_stack = torch.arange(capacity - 1, -1, -1, **i32)            # lowest slot on top
        self.totals = dict(hits=0, misses=0, evictions=0, overflow=0)
        self._oracle = None
        if torch.device(device).type != "cuda":
            from .oracle import PolicyOracle

            self._oracle = PolicyOracle("linked_list", capacity)

    def step(self, ids):
        import torch

        if self._oracle is not None:
            h, m, ev, over = self._oracle.step([int(x) for x in ids.tolist()])
            evicted = torch.tensor(ev, dtype=torch.int32)
        else:
            N = _n()
            ids32 = ids.to(self.dir.device).to(torch.int32).contiguous()
            n = int(ids32.numel())
            evicted_buf = torch.empty(max(n, 1), dtype=torch.int32, device=self.dir.device)
            cnt = torch.zeros(4, dtype=torch.int32, device=self.dir.device)
            N.check(N.cuda().ulc_ablate_linked_lru_step(N.ptr(self.dir), N.ptr(self.id_of), N.ptr(self.stamp),
                                                        N.ptr(self.next), N.ptr(self.prev), N.ptr(self.list),
                                                        N.ptr(self.free_stack), N.ptr(ids32), C.c_int(n),
                                                        N.ptr(evicted_buf), N.ptr(cnt), N.stream()), "linked_lru_step")
            h, m, e, over = (int(x) for x in cnt.tolist())
            evicted = evicted_buf[:e]
        self.totals["hits"] += h
        self.totals["misses"] += m
        self.totals["evictions"] += int(evicted.numel())
        self.totals["overflow"] += over
        return h, m, evicted


class PresenceRingPolicy:
    """The bucket-ring policy taken from hierarchical presence bitmaps (``csrc/include/ulc/presence_bitmap.h``:
    255 recent buckets + a cold one, each a 32-ary bitmap tree over the slots).  The same header runs in the
    CPU oracle (policy ``bitmap_ring``) and, here, in a one-thread device kernel that replays a step; its
    decisions equal those of the stamp-based ring of the residency kernels.

    Reference: ulacache/csrc/eviction/presence_recent.cuh:52-229."""

    def __init__(self, capacity: int, id_space: int, device):
        import torch

        self.capacity = capacity
        self.totals = dict(hits=0, misses=0, evictions=0, overflow=0)
        self._oracle = None
        if torch.device(device).type != "cuda":
            from .oracle import PolicyOracle

            self._oracle = PolicyOracle("bitmap_ring", capacity)
            return
        N = _n()
        lib = N.cuda()
        lib.ulc_presence_ring_bytes.restype = C.c_longlong
        lib.ulc_presence_ring_words.restype = C.c_longlong
        i32 = dict(dtype=torch.int32, device=device)
        self.ring = torch.zeros(int(lib.ulc_presence_ring_bytes()), dtype=torch.uint8, device=device)
        self.bits = torch.zeros(int(lib.ulc_presence_ring_words(C.c_int(capacity))), **i32)
        self.inverse = torch.zeros(capacity, dtype=torch.int16, device=device)
        self.dir = torch.full((id_space,), -1, **i32)
        self.id_of = torch.full((capacity,), -1, **i32)
        self.free_stack = torch.arange(capacity - 1, -1, -1, **i32)            # lowest slot on top
        self.state = torch.tensor([capacity, 0], **i32)                        # free height, initialised flag
        self.status = N.new_status(device)

    def step(self, ids):
        import torch

        if self._oracle is not None:
            h, m, ev, over = self._oracle.step([int(x) for x in ids.tolist()])
            evicted = torch.tensor(ev, dtype=torch.int32)
        else:
            N = _n()
            ids32 = ids.to(self.dir.device).to(torch.int32).contiguous()
            n = int(ids32.numel())
            evicted_buf = torch.empty(max(n, 1), dtype=torch.int32, device=self.dir.device)
            cnt = torch.zeros(4, dtype=torch.int32, device=self.dir.device)
            N.check(N.cuda().ulc_ablate_presence_ring_step(
                N.ptr(self.ring), N.ptr(self.bits), N.ptr(self.inverse), C.c_int(self.capacity), N.ptr(self.dir),
                C.c_int(self.dir.numel()), N.ptr(self.id_of), N.ptr(self.free_stack), N.ptr(self.state), N.ptr(ids32),
                C.c_int(n), N.ptr(evicted_buf), N.ptr(cnt), N.ptr(self.status), N.stream()), "presence_ring_step")
            h, m, e, over = (int(x) for x in cnt.tolist())
            N.raise_on_status(self.status, "presence ring step")
            evicted = evicted_buf[:e]
        self.totals["hits"] += h
        self.totals["misses"] += m
        self.totals["evictions"] += int(evicted.numel())
        self.totals["overflow"] += over
        return h, m, evicted


class _PRing(C.Structure):
    _fields_ = [("bits", C.c_void_p), ("summary", C.c_void_p), ("slot_bucket", C.c_void_p), ("count", C.c_void_p),
                ("bucket_epoch", C.c_void_p), ("ctl", C.c_void_p), ("vlist", C.c_void_p), ("chunk_count", C.c_void_p),
                ("n", C.c_int32), ("w0", C.c_int32), ("w1", C.c_int32)]


class ParallelPresenceRing:
    """Device state and launches of the parallel presence-bitmap ring (``csrc/presence_ring.cu``):
    ``advance`` / ``touch`` / ``detach`` / ``victims`` on slot numbers, usable by any directory.

    Reference: ulacache/eviction/lru.py:132 (create_presence_ring), csrc/eviction/presence_recent.cuh:52-229,
    presence_warp.cuh:11-133, victims.cuh:81-194."""

    def __init__(self, slots: int, device):
        import torch

        N = _n()
        w0, w1 = C.c_int(0), C.c_int(0)
        N.check(N.cuda().ulc_pring_words(C.c_int(slots), C.byref(w0), C.byref(w1)), "pring_words")
        self.slots, self.w0, self.w1 = slots, w0.value, w1.value
        i32 = dict(dtype=torch.int32, device=device)
        self.bits = torch.zeros((256, self.w0), **i32)
        self.summary = torch.zeros((256, self.w1), **i32)
        self.slot_bucket = torch.full((slots,), -1, **i32)
        self.count = torch.zeros(256, **i32)
        self.bucket_epoch = torch.full((255,), -1, **i32)
        self.bucket_epoch[0] = 0                      # slots touched before the first advance belong to epoch 0
        self.ctl = torch.zeros(8, **i32)
        self.vlist = torch.zeros((256, 3), **i32)
        self.chunk_count = torch.zeros((256, 256), **i32)          # [bucket list entry][chunk]
        self.status = N.new_status(device)
        self.struct = _PRing(self.bits.data_ptr(), self.summary.data_ptr(), self.slot_bucket.data_ptr(),
                             self.count.data_ptr(), self.bucket_epoch.data_ptr(), self.ctl.data_ptr(),
                             self.vlist.data_ptr(), self.chunk_count.data_ptr(), slots, self.w0, self.w1)

    @property
    def metadata_bytes(self) -> int:
        return sum(t.numel() * 4 for t in (self.bits, self.summary, self.slot_bucket, self.count, self.bucket_epoch,
                                           self.ctl, self.vlist, self.chunk_count))

    def advance(self):
        N = _n()
        N.check(N.cuda().ulc_pring_advance(C.byref(self.struct), N.stream()), "pring_advance")

    def touch(self, slots, detach: bool = False):
        N = _n()
        N.check(N.cuda().ulc_pring_touch(C.byref(self.struct), N.ptr(slots), C.c_int(slots.numel()), C.c_int(int(detach)),
                                         N.ptr(self.status), N.stream()), "pring_touch")

    def victims(self, need: int, out):
        """Writes the victims (eviction order: cold bucket first, then the oldest recent buckets, lowest slot
        first inside a bucket; never a slot of the current epoch) to ``out``; ``ctl[2]`` holds how many."""
        N = _n()
        N.check(N.cuda().ulc_pring_victims(C.byref(self.struct), C.c_int(need), N.ptr(out), C.c_int(out.numel()),
                                           N.stream()), "pring_victims")

    @property
    def served(self) -> int:
        return int(self.ctl[2])


class ParallelPresenceRingPolicy:
    """Replay policy on the parallel presence-bitmap ring.  A step is a transaction, as in the residency
    kernels: every hit is touched first, then the misses are placed in input order (free slots, then
    victims), so a record accessed in this step is never evicted by it.  CPU tensors run the same
    semantics in Python (the oracle of the GPU test)."""

    def __init__(self, capacity: int, id_space: int, device):
        import torch

        self.capacity, self.id_space = capacity, id_space
        self.device = torch.device(device)
        self.totals = dict(hits=0, misses=0, evictions=0, overflow=0)
        i32 = dict(dtype=torch.int32, device=device)
        self.dir = torch.full((id_space,), -1, **i32)
        self.id_of = torch.full((capacity,), -1, **i32)
        self.free_stack = torch.arange(capacity - 1, -1, -1, **i32)            # lowest slot on top
        self.nfree = capacity
        self.epoch = 0
        if self.device.type == "cuda":
            self.ring = ParallelPresenceRing(capacity, device)
        else:
            self.stamp = [-1] * capacity

    def _cpu_step(self, ids):
        import torch

        self.epoch += 1
        dir_, id_of = self.dir, self.id_of
        misses = []
        hits = 0
        for rid in ids.tolist():
            s = int(dir_[rid])
            if s >= 0:
                hits += 1
                self.stamp[s] = self.epoch
            else:
                misses.append(rid)
        from_free = min(len(misses), self.nfree)
        need = len(misses) - from_free
        live = [s for s in range(self.capacity) if int(id_of[s]) >= 0 and self.stamp[s] != self.epoch]
        live.sort(key=lambda s: (-min(self.epoch - self.stamp[s], 255), s))
        victims = live[:need]
        evicted = []
        for i, rid in enumerate(misses[: from_free + len(victims)]):
            if i < from_free:
                s = int(self.free_stack[self.nfree - 1 - i])
            else:
                s = victims[i - from_free]
                evicted.append(int(id_of[s]))
                dir_[int(id_of[s])] = -1
            id_of[s] = rid
            dir_[rid] = s
            self.stamp[s] = self.epoch
        self.nfree -= from_free
        return hits, len(misses), torch.tensor(evicted, dtype=torch.int32), len(misses) - from_free - len(victims)

    def step(self, ids):
        """``ids``: distinct record ids accessed this step -> (hits, misses, evicted ids in eviction order)."""
        import torch

        if self.device.type != "cuda":
            h, m, evicted, over = self._cpu_step(ids)
        else:
            N = _n()
            ring = self.ring
            ids32 = ids.to(self.device).to(torch.int32).contiguous()
            n = int(ids32.numel())
            self.epoch += 1
            ring.advance()
            flags = torch.empty(n, dtype=torch.int32, device=self.device)
            N.check(N.cuda().ulc_pring_lookup_touch(C.byref(ring.struct), N.ptr(ids32), C.c_int(n), N.ptr(self.dir),
                                                    C.c_int(self.id_space), N.ptr(flags), N.ptr(ring.status), N.stream()),
                    "pring_lookup_touch")
            miss_ids = ids32[flags.bool()].contiguous()            # input order (stable compaction)
            m = int(miss_ids.numel())
            h = n - m
            from_free = min(m, self.nfree)
            need = m - from_free
            victims = torch.empty(max(need, 1), dtype=torch.int32, device=self.device)
            ring.victims(need, victims)
            served = ring.served if need else 0
            evicted = torch.empty(max(served, 1), dtype=torch.int32, device=self.device)
            N.check(N.cuda().ulc_pring_place(C.byref(ring.struct), N.ptr(miss_ids), C.c_int(from_free + served),
                                             C.c_int(from_free), N.ptr(self.free_stack), C.c_int(self.nfree),
                                             N.ptr(victims), N.ptr(self.dir), N.ptr(self.id_of), N.ptr(evicted),
                                             N.stream()), "pring_place")
            self.nfree -= from_free
            evicted = evicted[:served]
            over = need - served
            N.raise_on_status(ring.status, "presence ring")
        self.totals["hits"] += h
        self.totals["misses"] += m
        self.totals["evictions"] += int(evicted.numel())
        self.totals["overflow"] += over
        return h, m, evicted


class HotBufferPolicy:
    """``requests`` buffers of ``width`` entries each."""

    def __init__(self, requests: int, width: int, device):
        import torch

        self.requests, self.width = requests, width
        self.tags = torch.full((requests, width), -1, dtype=torch.int32, device=device)
        self.stamps = torch.full((requests, width), -1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.totals = dict(hits=0, misses=0)

    def step(self, ids, row_offsets):
        """``ids`` int32 [n] accesses grouped by request, ``row_offsets`` int32 [requests + 1]."""
        import torch

        self.epoch += 1
        if not self.tags.is_cuda:
            hits = misses = 0
            offs = row_offsets.tolist()
            for r in range(self.requests):
                for rid in ids[offs[r]:offs[r + 1]].tolist():
                    row = self.tags[r]
                    where = (row == rid).nonzero().flatten()
                    if where.numel():
                        self.stamps[r, int(where.max())] = self.epoch
                        hits += 1
                        continue
                    misses += 1
                    cand = (self.stamps[r] != self.epoch).nonzero().flatten()
                    if cand.numel():
                        key = (self.stamps[r, cand].long() + 1) * (self.width + 1) + cand
                        j = int(cand[int(key.argmin())])
                        self.tags[r, j] = rid
                        self.stamps[r, j] = self.epoch
            out = (hits, misses)
        else:
            N = _n()
            cnt = torch.zeros((self.requests, 2), dtype=torch.int32, device=self.tags.device)
            N.check(N.cuda().ulc_ablate_hot_buffer_step(N.ptr(self.tags), N.ptr(self.stamps), C.c_int(self.requests),
                                                        C.c_int(self.width), N.ptr(ids.to(torch.int32).contiguous()),
                                                        N.ptr(row_offsets.to(torch.int32).contiguous()),
                                                        C.c_int(self.epoch), N.ptr(cnt), N.stream()), "hot_buffer_step")
            s = cnt.sum(0).tolist()
            out = (int(s[0]), int(s[1]))
        self.totals["hits"] += out[0]
        self.totals["misses"] += out[1]
        return out


def trace_hits(directory, selection):
    """(resident, valid) counts of a selection against a directory (entry >= 0 = in HBM); changes nothing."""
    import torch

    sel = selection.reshape(-1)
    if not directory.is_cuda:
        ok = (sel >= 0) & (sel < directory.numel())
        return int((directory[sel[ok].long()] >= 0).sum()), int(ok.sum())
    N = _n()
    cnt = torch.zeros(2, dtype=torch.int64, device=directory.device)
    N.check(N.cuda().ulc_trace_hits(N.ptr(directory), C.c_int(directory.numel()), N.ptr(sel.to(torch.int32).contiguous()),
                                    C.c_longlong(sel.numel()), N.ptr(cnt), N.stream()), "trace_hits")
    return int(cnt[0]), int(cnt[1])
