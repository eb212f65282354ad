"""One residency group: directory, free stacks, recency ring and the promotion plan.

Two interchangeable implementations of the same transaction

    register -> begin_step -> pin -> plan -> (exchange) -> commit -> resolve -> release

* :class:`TorchResidency` — plain PyTorch on whatever device the tensors live
  on (CPU in the test-suite).  It is the executable specification and the oracle
  for the kernels.
* :class:`CudaResidency` — launches the sm_100a kernels in ``csrc/residency.cu``.

Both keep the same int32 state tensors (see ``csrc/include/ulc/residency.h``), so
a test can copy state from one to the other and compare.

Reference: the host-tier transaction of ulacache/csrc/cache/cpu_residency.cuh
(register_rows :107, pin_rows :153, reserve :182, commit :268, release_rows :317)
with its state tensors in ulacache/cache/directory.py:9-18.  Victim choice follows
the bucketed-recency rule of ulacache/csrc/eviction/presence_recent.cuh:199-229.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from ..storage.layout import DIR_UNALLOCATED, OwnerMap

RECENT = 255
COLD = 255
RING = 256
NUM_COUNTERS = 32
PLAN_ROWS = 5
(CNT_EPOCH, CNT_HBM_FREE, CNT_HOST_FREE, CNT_PROMOTE, CNT_PLAN, CNT_VICTIMS, CNT_NEED, CNT_FROM_FREE,
 CNT_HITS, CNT_MISSES, CNT_PROMOTIONS, CNT_EVICTIONS, CNT_REGISTERED, CNT_BBUCKET, CNT_BQUOTA,
 CNT_BTAKEN, CNT_CUTOFF, CNT_UNSERVED) = range(18)
COLD_MARK = -0x7FFFFFFF


@dataclass
class ResidencyGeometry:
    dir_len: int
    hbm_slots: int
    host_slots: int
    plan_capacity: int


def victim_cutoff(ring, epoch: int, need: int):
    """Python twin of ``ulc::victim_cutoff``: returns (served, cutoff, quota)."""
    if need <= 0:
        return 0, COLD_MARK, 0
    cold = int(ring[COLD])
    if cold >= need:
        return need, COLD_MARK, need
    got = cold
    for e in range(epoch - RECENT + 1, epoch):
        if e < 0:
            continue
        c = int(ring[e % RECENT])
        if got + c >= need:
            return need, e, need - got
        got += c
    return got, epoch, 0


class _ResidencyBase:
    def __init__(self, geometry: ResidencyGeometry, owners: OwnerMap, my_rank: int, device):
        import torch

        g = geometry
        self.geometry, self.owners, self.my_rank, self.device = g, owners, my_rank, device
        i32 = dict(dtype=torch.int32, device=device)
        self.directory = torch.full((g.dir_len,), DIR_UNALLOCATED, **i32)
        self.hbm_tags = torch.full((g.hbm_slots,), -1, **i32)
        self.host_tags = torch.full((max(g.host_slots, 1),), -1, **i32)
        self.stamps = torch.full((g.hbm_slots,), -1, **i32)
        self.access_time = torch.full((g.dir_len,), -1, **i32)
        # stacks pop from the top, so store descending to hand out low slots first
        self.hbm_free = torch.arange(g.hbm_slots - 1, -1, -1, **i32)
        self.host_free = torch.arange(max(g.host_slots, 1) - 1, -1, -1, **i32)
        self.counters = torch.zeros(NUM_COUNTERS, **i32)
        self.counters[CNT_HBM_FREE] = g.hbm_slots
        self.counters[CNT_HOST_FREE] = g.host_slots
        self.ring = torch.zeros(RING, **i32)
        self.promote = torch.zeros(max(g.plan_capacity, 1), **i32)
        self.plan = torch.full((PLAN_ROWS, max(g.plan_capacity, 1)), -1, **i32)
        self.victims = torch.zeros(max(g.plan_capacity, 1), **i32)

    STATE = ("directory", "hbm_tags", "host_tags", "stamps", "access_time", "hbm_free", "host_free",
             "counters", "ring", "promote", "plan", "victims")

    def state_dict(self):
        return {k: getattr(self, k).detach().cpu().clone() for k in self.STATE}

    def load_state(self, state):
        for k in self.STATE:
            getattr(self, k).copy_(state[k].to(self.device))

    def metadata_bytes(self) -> int:
        return sum(getattr(self, k).numel() * 4 for k in self.STATE)

    def order_host_free_tail(self, records: int) -> bool:
        """Before a receive of ``records`` records: sort the top of the host free stack so that the slots handed out
        next are ascending and mostly adjacent (contiguous receive extents).  Only a bounded tail is permuted; the
        set of free slots, the count and every live entry stay as they are.  Call between forwards, on the stream
        that allocates."""
        from ..ops import paired

        return paired.sort_free_tail(self.host_free, self.counters[CNT_HOST_FREE:CNT_HOST_FREE + 1], records)

    def stats(self) -> dict:
        c = self.counters.tolist()
        return {"epoch": c[CNT_EPOCH], "hbm_free": c[CNT_HBM_FREE], "host_free": c[CNT_HOST_FREE],
                "hits": c[CNT_HITS], "misses": c[CNT_MISSES], "promotions": c[CNT_PROMOTIONS],
                "evictions": c[CNT_EVICTIONS], "registered": c[CNT_REGISTERED],
                "unserved": c[CNT_UNSERVED]}

    def reset(self):
        fresh = type(self)(self.geometry, self.owners, self.my_rank, self.device)
        for k in self.STATE:
            getattr(self, k).copy_(getattr(fresh, k))

    # helpers shared by both implementations -----------------------------------
    def _owned_locals(self, ids):
        """(mask of IDs this rank owns, their owner-local IDs) for a flat int32 tensor."""
        m = self.owners
        valid = ids > 0
        stripe = ids >> m.stripe_shift
        mine = valid & ((stripe % m.ranks) == self.my_rank)
        local = ((stripe // m.ranks) << m.stripe_shift) | (ids & ((1 << m.stripe_shift) - 1))
        return mine, local


class TorchResidency(_ResidencyBase):
    """Reference implementation; sequential semantics, any device."""

    def register(self, ids, prefer_device=True):
        import torch

        ids = ids.reshape(-1).to(torch.int32)
        mine, local = self._owned_locals(ids)
        rows = local[mine].long()
        if rows.numel() == 0:
            return
        if (rows >= self.geometry.dir_len).any():
            raise IndexError("logical ID outside the directory")
        if (self.directory[rows] != DIR_UNALLOCATED).any():
            raise RuntimeError("registering a row that is already allocated")
        epoch = int(self.counters[CNT_EPOCH])
        n = rows.numel()
        hbm_free, host_free = int(self.counters[CNT_HBM_FREE]), int(self.counters[CNT_HOST_FREE])
        take_dev = min(n, hbm_free) if prefer_device else 0
        take_host = min(n - take_dev, host_free)
        if not prefer_device:
            take_dev = min(n - take_host, hbm_free)
        if take_dev + take_host < n:
            raise MemoryError("no free slot left in either tier")
        order = (rows[:take_dev], rows[take_dev:]) if prefer_device else (rows[take_host:], rows[:take_host])
        dev_rows, host_rows = order
        if take_dev:
            slots = self.hbm_free[hbm_free - take_dev:hbm_free].flip(0).long()
            self.directory[dev_rows] = slots.int()
            self.hbm_tags[slots] = dev_rows.int()
            self.stamps[slots] = epoch
            self.ring[epoch % RECENT] += take_dev
            self.counters[CNT_HBM_FREE] -= take_dev
        if take_host:
            slots = self.host_free[host_free - take_host:host_free].flip(0).long()
            self.directory[host_rows] = (-slots - 2).int()
            self.host_tags[slots] = host_rows.int()
            self.counters[CNT_HOST_FREE] -= take_host
        self.counters[CNT_REGISTERED] += n

    def release(self, ids):
        import torch

        ids = ids.reshape(-1).to(torch.int32)
        mine, local = self._owned_locals(ids)
        epoch = int(self.counters[CNT_EPOCH])
        for row in torch.unique(local[mine]).tolist():
            e = int(self.directory[row])
            if e == DIR_UNALLOCATED:
                continue
            self.directory[row] = DIR_UNALLOCATED
            if e >= 0:
                st = int(self.stamps[e])
                if st >= 0:
                    self.ring[COLD if epoch - st >= RECENT else st % RECENT] -= 1
                self.stamps[e] = -1
                self.hbm_tags[e] = -1
                top = int(self.counters[CNT_HBM_FREE])
                self.hbm_free[top] = e
                self.counters[CNT_HBM_FREE] = top + 1
            else:
                s = -e - 2
                self.host_tags[s] = -1
                top = int(self.counters[CNT_HOST_FREE])
                self.host_free[top] = s
                self.counters[CNT_HOST_FREE] = top + 1
            self.counters[CNT_REGISTERED] -= 1

    def begin_step(self):
        epoch = int(self.counters[CNT_EPOCH]) + 1
        self.counters[CNT_EPOCH] = epoch
        b = epoch % RECENT
        self.ring[COLD] += self.ring[b]
        self.ring[b] = 0
        for c in (CNT_PROMOTE, CNT_PLAN, CNT_VICTIMS, CNT_NEED, CNT_FROM_FREE, CNT_BTAKEN, CNT_UNSERVED):
            self.counters[c] = 0

    def pin(self, sel):
        import torch

        ids = sel.reshape(-1).to(torch.int32)
        mine, local = self._owned_locals(ids)
        rows = torch.unique(local[mine]).long()
        if rows.numel() == 0:
            return
        epoch = int(self.counters[CNT_EPOCH])
        e = self.directory[rows]
        dev = e >= 0
        slots = e[dev].long()
        old = self.stamps[slots]
        for st in old[(old != epoch) & (old >= 0)].tolist():
            self.ring[COLD if epoch - st >= RECENT else st % RECENT] -= 1
        self.ring[epoch % RECENT] += int((old != epoch).sum())
        self.stamps[slots] = epoch
        self.counters[CNT_HITS] += int(dev.sum())
        host_rows = rows[e <= -2]
        fresh = host_rows[self.access_time[host_rows] != epoch]
        self.access_time[fresh] = epoch
        at = int(self.counters[CNT_PROMOTE])
        room = max(0, self.geometry.plan_capacity - at)
        self.promote[at:at + min(room, fresh.numel())] = fresh[:room].int()
        self.counters[CNT_PROMOTE] = at + fresh.numel()
        self.counters[CNT_MISSES] += fresh.numel()

    def plan_step(self):
        import torch

        c = self.counters
        want = int(c[CNT_PROMOTE])
        cap = self.geometry.plan_capacity
        if want > cap:
            c[CNT_UNSERVED] += want - cap
            want = cap
            c[CNT_PROMOTE] = want
        free_before = int(c[CNT_HBM_FREE])
        from_free = min(want, free_before)
        epoch = int(c[CNT_EPOCH])
        served, cutoff, quota = victim_cutoff(self.ring.tolist(), epoch, want - from_free)
        c[CNT_FROM_FREE], c[CNT_NEED], c[CNT_CUTOFF], c[CNT_BQUOTA] = from_free, served, cutoff, quota
        if served < want - from_free:
            c[CNT_UNSERVED] += want - from_free - served
        victims = torch.empty(0, dtype=torch.long, device=self.device)
        if served > 0:
            st = self.stamps
            live = (st >= 0) & (st != epoch)
            if cutoff == COLD_MARK:
                victims = torch.nonzero(live & (epoch - st >= RECENT)).flatten()[:quota]
            else:
                sure = torch.nonzero(live & (st < cutoff)).flatten()
                edge = torch.nonzero(live & (st == cutoff)).flatten()[:quota]
                victims = torch.cat([sure, edge])
        c[CNT_VICTIMS] = victims.numel()
        self.victims[:victims.numel()] = victims.int()
        total = min(want, from_free + victims.numel())
        rows = self.promote[:total].long()
        host_src = (-self.directory[rows] - 2)
        gpu = torch.empty(total, dtype=torch.int32, device=self.device)
        old_row = torch.full((total,), -1, dtype=torch.int32, device=self.device)
        host_dst = torch.full((total,), -1, dtype=torch.int32, device=self.device)
        k = min(from_free, total)
        if k:
            gpu[:k] = self.hbm_free[free_before - k:free_before].flip(0)
        if total > k:
            v = victims[:total - k]
            gpu[k:] = v.int()
            old_row[k:] = self.hbm_tags[v]
            host_dst[k:] = host_src[k:]
        self.plan[0, :total], self.plan[1, :total] = rows.int(), gpu
        self.plan[2, :total], self.plan[3, :total], self.plan[4, :total] = host_src.int(), host_dst, old_row
        c[CNT_PLAN] = total

    def commit(self):
        c = self.counters
        n, epoch = int(c[CNT_PLAN]), int(c[CNT_EPOCH])
        for i in range(n):
            row, gpu, hs, hd, old = (int(self.plan[r, i]) for r in range(5))
            if old >= 0:
                st = int(self.stamps[gpu])
                if st >= 0:
                    self.ring[COLD if epoch - st >= RECENT else st % RECENT] -= 1
                self.directory[old] = -hd - 2
                self.host_tags[hd] = old
                c[CNT_EVICTIONS] += 1
            else:
                self.host_tags[hs] = -1
                top = int(c[CNT_HOST_FREE])
                self.host_free[top] = hs
                c[CNT_HOST_FREE] = top + 1
            self.directory[row] = gpu
            self.hbm_tags[gpu] = row
            self.stamps[gpu] = epoch
            self.ring[epoch % RECENT] += 1
            c[CNT_PROMOTIONS] += 1
        c[CNT_HBM_FREE] -= min(int(c[CNT_FROM_FREE]), n)
        c[CNT_FROM_FREE] = 0
        c[CNT_PROMOTE] = 0

    def plan_items(self):
        n = int(self.counters[CNT_PLAN])
        return self.plan[:, :n]


class CudaResidency(_ResidencyBase):
    """Kernel-backed implementation (sm_100a)."""

    def __init__(self, geometry, owners, my_rank, device, *, pin_blocks=512, victim_blocks=296,
                 assign_blocks=128, victim_index=None):
        """``victim_index``: "bitmap" keeps a presence bitmap per recency bucket beside the stamps and finds
        victims through it (cost follows the victims, 1.3 to 3.7 times faster than the scan at a million
        slots, 32 bytes of metadata per slot); "stamps" finds them with one scan of the stamps.  Default:
        ``ULC_VICTIM_INDEX`` if set, else bitmaps from 262144 device slots up."""
        super().__init__(geometry, owners, my_rank, device)
        import os

        import torch
        from ..ops import _native as N

        self._N = N
        self.status = N.new_status(device)
        self._map = N.OwnerMap(owners.ranks, owners.stripe_shift)
        self._launch = (pin_blocks, victim_blocks, assign_blocks)
        st = N.ResidencyState()
        for k in self.STATE:
            setattr(st, k, getattr(self, k).data_ptr())
        g = geometry
        st.dir_len, st.hbm_slots, st.host_slots, st.plan_capacity = g.dir_len, g.hbm_slots, g.host_slots, max(g.plan_capacity, 1)
        if victim_index is None:
            victim_index = os.environ.get("ULC_VICTIM_INDEX", "") or ("bitmap" if g.hbm_slots >= 262144 else "stamps")
        if victim_index not in ("bitmap", "stamps"):
            raise ValueError("victim_index must be bitmap or stamps")
        self.victim_index = victim_index
        if victim_index == "bitmap":
            self.w0 = (g.hbm_slots + 31) // 32
            self.w1 = (self.w0 + 31) // 32
            i32 = dict(dtype=torch.int32, device=device)
            self.bits = torch.zeros((RING, self.w0), **i32)
            self.summary = torch.zeros((RING, self.w1), **i32)
            self.vlist = torch.zeros((RING, 3), **i32)
            self.chunk_count = torch.zeros((RING, 256), **i32)
            st.bits, st.summary = self.bits.data_ptr(), self.summary.data_ptr()
            st.vlist, st.chunk_count = self.vlist.data_ptr(), self.chunk_count.data_ptr()
            st.w0, st.w1 = self.w0, self.w1
        self.native_state = st

    def metadata_bytes(self) -> int:
        extra = 0
        if self.victim_index == "bitmap":
            extra = sum(t.numel() * 4 for t in (self.bits, self.summary, self.vlist, self.chunk_count))
        return super().metadata_bytes() + extra

    def load_state(self, state):
        super().load_state(state)
        self.rebuild_victim_index()

    def reset(self):
        super().reset()
        self.rebuild_victim_index()

    def rebuild_victim_index(self):
        """Bitmaps and summaries from the stamps (after a state load; the kernels keep them in step)."""
        if self.victim_index != "bitmap":
            return
        import numpy as np
        import torch

        stamps = self.stamps.cpu().numpy().astype(np.int64)
        epoch = int(self.counters[CNT_EPOCH])
        live = np.nonzero(stamps >= 0)[0]
        bucket = np.where(epoch - stamps[live] >= RECENT, COLD, stamps[live] % RECENT)
        bits = np.zeros((RING, self.w0), dtype=np.uint32)
        np.bitwise_or.at(bits, (bucket, live >> 5), (np.uint32(1) << (live & 31).astype(np.uint32)))
        summary = np.zeros((RING, self.w1), dtype=np.uint32)
        b, w = np.nonzero(bits)
        np.bitwise_or.at(summary, (b, w >> 5), (np.uint32(1) << (w & 31).astype(np.uint32)))
        self.bits.copy_(torch.from_numpy(bits.view(np.int32)).to(self.device))
        self.summary.copy_(torch.from_numpy(summary.view(np.int32)).to(self.device))

    def _i32(self, t):
        import torch

        return t.reshape(-1).to(device=self.device, dtype=torch.int32).contiguous()

    def register(self, ids, prefer_device=True):
        N = self._N
        ids = self._i32(ids)
        N.check(N.cuda().ulc_res_register(C.byref(self.native_state), C.byref(self._map), C.c_int(self.my_rank),
                                          N.ptr(ids), C.c_int(ids.numel()), C.c_int(int(prefer_device)),
                                          N.ptr(self.status), N.stream()), "res_register")

    def release(self, ids):
        N = self._N
        ids = self._i32(ids)
        N.check(N.cuda().ulc_res_release(C.byref(self.native_state), C.byref(self._map), C.c_int(self.my_rank),
                                         N.ptr(ids), C.c_int(ids.numel()), N.ptr(self.status), N.stream()),
                "res_release")

    def begin_step(self):
        N = self._N
        N.check(N.cuda().ulc_res_begin_step(C.byref(self.native_state), N.stream()), "res_begin_step")

    def pin(self, sel):
        N = self._N
        sel = self._i32(sel)
        N.check(N.cuda().ulc_res_pin(C.byref(self.native_state), C.byref(self._map), C.c_int(self.my_rank),
                                     N.ptr(sel), C.c_int(sel.numel()), C.c_int(self._launch[0]),
                                     N.ptr(self.status), N.stream()), "res_pin")

    def plan_step(self):
        N = self._N
        N.check(N.cuda().ulc_res_plan(C.byref(self.native_state), C.c_int(self._launch[1]),
                                      C.c_int(self._launch[2]), N.ptr(self.status), N.stream()), "res_plan")

    def commit(self):
        N = self._N
        N.check(N.cuda().ulc_res_commit(C.byref(self.native_state), N.stream()), "res_commit")

    def plan_items(self):
        n = int(self.counters[CNT_PLAN])
        return self.plan[:, :n]

    def check_status(self, what="residency"):
        self._N.raise_on_status(self.status, what)


def make_residency(geometry, owners, my_rank, device, **kw):
    import torch

    dev = torch.device(device)
    if dev.type == "cuda":
        return CudaResidency(geometry, owners, my_rank, dev, **kw)
    return TorchResidency(geometry, owners, my_rank, dev)
