"""Whole-request page tier: residency at 64-token page granularity, decided on the host at step
boundaries (the ``cpu_policy="request"`` alternative to per-record residency).

A request is either fully resident in device pages while it is scheduled, or (partly) parked in
host pages.  ``reserve_request`` computes, under the device page budget, which pages of *other*,
idle requests have to be offloaded and which pages of this request have to be onloaded, grouped
into waves that never need more free device pages than exist when the wave starts.  The
transaction is applied with ``commit`` (after the executor moved the bytes) or dropped with
``cancel``.  ``attach`` / ``retire`` track readers: pages of an attached request are never chosen
as victims.  ``page_map`` (int32, logical page -> device page or -1) is what kernels consume.

Reference: ulacache/cache/request_pages.py:128-576 (FlowKVRequestPagePool, reserve_request :307,
commit :365, BoundaryTransaction), cache/request_storage.py:63-276, request_access.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

PAGE_TOKENS = 64


class PageBudgetError(MemoryError):
    pass


@dataclass
class Wave:
    offloads: List[Tuple[int, int, int]] = field(default_factory=list)   # (logical page, device page, host page)
    onloads: List[Tuple[int, int, int]] = field(default_factory=list)    # (logical page, host page, device page)


@dataclass
class BoundaryTransaction:
    request: int
    waves: List[Wave]
    new_pages: List[Tuple[int, int]]          # (logical page, device page) freshly allocated (no copy)
    state: str = "open"                       # open | committed | cancelled

    @property
    def moved_pages(self) -> int:
        return sum(len(w.offloads) + len(w.onloads) for w in self.waves)


class RequestPagePool:
    def __init__(self, device_pages: int, host_pages: int, logical_pages: int, reserved_device_pages=()):
        """``reserved_device_pages``: device pages that are never handed out (a sentinel page that padded
        page-table entries may point at, pages another allocator owns)."""
        if device_pages < 1 or host_pages < 0 or logical_pages < 1:
            raise ValueError("page counts must be positive")
        self.device_pages, self.host_pages, self.logical_pages = device_pages, host_pages, logical_pages
        self.reserved_device_pages = tuple(sorted(set(int(p) for p in reserved_device_pages)))
        if any(not 0 <= p < device_pages for p in self.reserved_device_pages):
            raise ValueError("reserved device pages must lie inside the device pool")
        self.free_device = [p for p in range(device_pages - 1, -1, -1) if p not in self.reserved_device_pages]
        self.free_host = list(range(host_pages - 1, -1, -1))
        self.free_logical = list(range(logical_pages - 1, -1, -1))
        self.where: Dict[int, Tuple[str, int]] = {}          # logical page -> ("d"|"h", physical page)
        self.pages_of: Dict[int, List[int]] = {}             # request -> logical pages in token order
        self.readers: Dict[int, int] = {}                    # request -> attached readers
        self.last_use: Dict[int, int] = {}
        self.clock = 0
        self._open: Optional[BoundaryTransaction] = None
        self.stats = dict(onloaded=0, offloaded=0, transactions=0)

    # ----------------------------------------------------------------- queries --
    def page_map(self):
        """int32 [logical_pages]: device page of every logical page, -1 when not on the device."""
        import torch

        m = torch.full((self.logical_pages,), -1, dtype=torch.int32)
        for lp, (tier, phys) in self.where.items():
            if tier == "d":
                m[lp] = phys
        return m

    @property
    def usable_device_pages(self) -> int:
        return self.device_pages - len(self.reserved_device_pages)

    def resident_pages(self, request: int) -> int:
        return sum(1 for lp in self.pages_of.get(request, ()) if self.where[lp][0] == "d")

    def is_resident(self, request: int) -> bool:
        return self.resident_pages(request) == len(self.pages_of.get(request, ()))

    # ------------------------------------------------------------- transactions --
    def reserve_request(self, request: int, total_tokens: int) -> BoundaryTransaction:
        """Make ``request`` fully device resident with room for ``total_tokens`` tokens."""
        if self._open is not None:
            raise RuntimeError("another boundary transaction is open")
        self.clock += 1
        have = self.pages_of.setdefault(request, [])
        need_total = (total_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        grow = max(0, need_total - len(have))
        parked = [lp for lp in have if self.where[lp][0] == "h"]
        demand = grow + len(parked)
        if grow > len(self.free_logical):
            raise PageBudgetError("logical page space exhausted")
        # victims: device pages of idle requests, least recently used request first, tail pages first
        shortfall = demand - len(self.free_device)
        victims: List[int] = []
        if shortfall > 0:
            idle = sorted((r for r in self.pages_of if r != request and not self.readers.get(r)),
                          key=lambda r: self.last_use.get(r, 0))
            for r in idle:
                for lp in reversed(self.pages_of[r]):
                    if self.where[lp][0] == "d":
                        victims.append(lp)
                        if len(victims) == shortfall:
                            break
                if len(victims) == shortfall:
                    break
            if len(victims) < shortfall:
                raise PageBudgetError(f"request {request} needs {demand} device pages; only "
                                      f"{len(self.free_device) + len(victims)} can be made free")
            if len(victims) > len(self.free_host):
                raise PageBudgetError("host tier cannot take the pages that must be offloaded")
        # waves: each wave first offloads up to `room` victims, then onloads into what is free
        free_d, free_h = list(self.free_device), list(self.free_host)
        waves: List[Wave] = []
        todo_on, todo_off = list(parked), list(victims)
        new_pages: List[Tuple[int, int]] = []
        # fresh pages take free device pages first (no copy needed)
        fresh_needed = grow
        while todo_on or todo_off or fresh_needed:
            wave = Wave()
            # offload enough victims for what this wave will place, bounded by free host pages
            want = max(0, min(len(todo_on) + fresh_needed, max(1, len(free_h))) - len(free_d))
            for _ in range(min(want, len(todo_off))):
                lp = todo_off.pop(0)
                hp = free_h.pop()
                dp = self.where[lp][1]
                wave.offloads.append((lp, dp, hp))
                free_d.append(dp)
            while todo_on and free_d:
                lp = todo_on.pop(0)
                dp = free_d.pop()
                hp = self.where[lp][1]
                wave.onloads.append((lp, hp, dp))
                free_h.append(hp)
            while fresh_needed and free_d:
                new_pages.append((-1, free_d.pop()))
                fresh_needed -= 1
            if not wave.offloads and not wave.onloads and (todo_on or todo_off or fresh_needed):
                if not todo_off:
                    raise PageBudgetError("no progress possible: nothing left to offload")
                continue
            if wave.offloads or wave.onloads:
                waves.append(wave)
        txn = BoundaryTransaction(request, waves, new_pages)
        self._open = txn
        return txn

    def commit(self, txn: BoundaryTransaction):
        if txn is not self._open or txn.state != "open":
            raise RuntimeError("transaction is not the open one")
        for wave in txn.waves:
            for lp, dp, hp in wave.offloads:
                self.where[lp] = ("h", hp)
                self.free_host.remove(hp)
                self.free_device.append(dp)
                self.stats["offloaded"] += 1
            for lp, hp, dp in wave.onloads:
                self.where[lp] = ("d", dp)
                self.free_device.remove(dp)
                self.free_host.append(hp)
                self.stats["onloaded"] += 1
        for _, dp in txn.new_pages:
            lp = self.free_logical.pop()
            self.free_device.remove(dp)
            self.where[lp] = ("d", dp)
            self.pages_of[txn.request].append(lp)
        self.last_use[txn.request] = self.clock
        self.stats["transactions"] += 1
        txn.state = "committed"
        self._open = None

    def cancel(self, txn: BoundaryTransaction):
        if txn is self._open:
            self._open = None
        if not self.pages_of.get(txn.request):
            self.pages_of.pop(txn.request, None)
        txn.state = "cancelled"

    # ------------------------------------------------------------ reader lifetime --
    def attach(self, request: int):
        if not self.is_resident(request):
            raise RuntimeError(f"request {request} is not fully device resident")
        self.readers[request] = self.readers.get(request, 0) + 1
        self.clock += 1
        self.last_use[request] = self.clock

    def retire(self, request: int):
        n = self.readers.get(request, 0)
        if n <= 0:
            raise RuntimeError("retire without attach")
        self.readers[request] = n - 1

    def free_request(self, request: int):
        if self.readers.get(request):
            raise RuntimeError("request still has readers")
        for lp in self.pages_of.pop(request, []):
            tier, phys = self.where.pop(lp)
            (self.free_device if tier == "d" else self.free_host).append(phys)
            self.free_logical.append(lp)
        self.readers.pop(request, None)
        self.last_use.pop(request, None)
