"""Receiver object of a prefill -> decode hand-over: reserves destination records in the cache,
turns them into byte extents a transport writes to, tracks completions and publishes.

    rx = DirectReceiver(cache, layers)
    ticket = rx.prepare(n_tokens)            # allocates ids, looks their slots up in the directory
    for tier, plan in ticket.plans.items():  # "device" / "host": DirectReceivePlan (address extents)
        transport.write(plan)                # RDMA in production; any byte copy in tests
        for seq in range(plan.chunk_count): ticket.windows[tier].accept(seq)
    ids = rx.publish(ticket)                 # refuses until every chunk of every tier has landed

Records go straight into the canonical record storage of the tier the cache assigned (HBM first,
then pinned host memory): nothing is staged and copied again.

Reference: ulacache/transfer/direct_receiver.py:1-417, native_paged_receive.py, owner_receive_window.py,
csrc/cache/local_cache.cuh:79-133 (acquire / release receive locations).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict

from .direct_receive import DirectReceivePlan, OrderedReceiveWindow, ReceiveNotComplete, plan_direct_receive


@dataclass
class ReceiveTicket:
    ids: object                                   # int32 [n] logical ids in token order
    positions: Dict[str, object]                  # tier -> index tensor into ids (which records go to that tier)
    plans: Dict[str, DirectReceivePlan] = field(default_factory=dict)
    windows: Dict[str, OrderedReceiveWindow] = field(default_factory=dict)
    published: bool = False
    reserved: object = None                       # every id that was allocated (whole pages), for cancel / free


class DirectReceiver:
    """Beside the ticket calls (:meth:`prepare` / :meth:`publish` / :meth:`cancel`), rooms give the scheduler's
    view of a hand-over: ``note_waiting`` -> ``can_accept`` -> ``reserve`` (destinations leave the eviction ring)
    -> ``metadata_sent`` -> ``complete`` (or ``logical_pages_freed`` after a drained abort).  Device destinations of
    open rooms are counted against a working-set reserve of ``max_queries * (topk + 1) + 1`` slots, so that
    receives can never starve the attention of the requests that are already decoding."""

    def __init__(self, cache, layers: int, *, chunk_records: int = 4096, audit=None, working_records=None):
        self.cache, self.layers, self.chunk = cache, layers, chunk_records
        self._audit = audit
        self._rooms: Dict[object, dict] = {}
        self._waiting: Dict[object, float] = {}
        self._page_owner: Dict[int, object] = {}
        self._leases = None
        self._leased_device = 0
        sparse = cache.cache_specification.sparse_access
        if working_records is None:
            working_records = sparse.maximum_padded_query_count * (sparse.maximum_selected_record_count + 1) + 1
        self.working_records = int(working_records)

    def prepare(self, n_tokens: int) -> ReceiveTicket:
        """Reserve ``n_tokens`` records and plan the extents.  Single-owner caches only (a striped
        pool plans per owner with that owner's engine)."""
        import torch

        ids = self.cache.alloc((n_tokens + 63) // 64 * 64)
        if ids is None:
            raise MemoryError("the cache cannot take the incoming request")
        reserved, ids = ids, ids[:n_tokens]            # ids come in whole 64-record pages
        eng = self.cache.engine
        if getattr(eng.owners, "ranks", 1) != 1:
            raise NotImplementedError("plan striped pools per owner")
        res = eng.residency[0]
        _, local = res._owned_locals(ids)
        entry = res.directory[local.long()].cpu()
        if bool((entry == -1).any()):
            raise RuntimeError("an allocated id has no slot")
        ticket = ReceiveTicket(ids=ids, positions={}, reserved=reserved)
        rb = eng.storages[0].plane.bytes_per_record
        for tier, mask, slots in (("device", entry >= 0, entry), ("host", entry <= -2, -entry - 2)):
            pos = mask.nonzero().flatten()
            if pos.numel() == 0:
                continue
            plane = eng.storages[0].gpu if tier == "device" else eng.storages[0].host
            stride = plane[1].data_ptr() - plane[0].data_ptr() if plane.shape[0] > 1 else 0
            plan = plan_direct_receive(slots[pos].tolist(), record_bytes=rb, layers=min(self.layers, plane.shape[0]),
                                       layer_stride=stride, base_address=plane.data_ptr(), tier=tier,
                                       chunk_records=self.chunk)
            ticket.positions[tier] = pos
            ticket.plans[tier] = plan
            ticket.windows[tier] = OrderedReceiveWindow(plan.chunk_count)
        return ticket

    def publish(self, ticket: ReceiveTicket):
        missing = {t: w.missing()[:4] for t, w in ticket.windows.items() if not w.complete}
        if missing:
            raise ReceiveNotComplete(f"chunks outstanding: {missing}")
        ticket.published = True
        return ticket.ids

    def cancel(self, ticket: ReceiveTicket):
        self.cache.free(ticket.reserved if ticket.reserved is not None else ticket.ids)

    # ------------------------------------------------------------------ rooms --
    def _residency(self):
        eng = self.cache.engine
        if getattr(eng.owners, "ranks", 1) != 1:
            raise NotImplementedError("plan striped pools per owner")
        if self._leases is None:
            from .receive_lease import ReceiveLeases

            self._leases = [ReceiveLeases(res) for res in eng.residency]
        return eng.residency

    @property
    def available_records(self) -> int:
        """Unbound destinations a new room may take: every free host slot, and the free device slots beyond
        the working-set reserve and the device destinations already leased to open rooms."""
        out = None
        for res in self._residency():
            st = res.stats()
            device = max(0, min(st["hbm_free"], res.geometry.hbm_slots - self.working_records - self._leased_device))
            room = st["host_free"] + device
            out = room if out is None else min(out, room)
        return int(out or 0)

    def note_waiting(self, key):
        import time

        self._waiting.setdefault(key, time.monotonic())

    def can_accept(self, records: int) -> bool:
        return records <= self.available_records

    def reserve(self, key, ids, *, request_id=None, prefix_records: int = 0):
        """``ids``: allocated record ids of the part of the request that is still to arrive, whole pages in token
        order.  Their device slots are leased (no eviction plan can take them), the tier plans are built against
        the frozen locations, and the pages are marked as having a remote writer."""
        import time

        import torch

        if key in self._rooms:
            raise ValueError(f"room {key!r} already advertises destinations")
        t0 = time.monotonic()
        flat = ids.reshape(-1).to(dtype=torch.int64, device="cpu")
        heads = flat[::64]
        if (flat.numel() % 64 or bool((heads % 64 != 0).any()) or bool((flat <= 0).any())
                or not torch.equal(flat, (heads[:, None] + torch.arange(64)).reshape(-1))
                or heads.unique().numel() != heads.numel()):
            raise ValueError("a room takes unique, complete pages of allocated ids")
        pages = set((heads // 64).tolist())
        if pages & self._page_owner.keys():
            raise ValueError("some of these pages already have a remote writer")
        residency = self._residency()
        dev_ids = ids.reshape(-1).to(device=residency[0].device, dtype=torch.int32)
        locations = [lease.acquire(dev_ids) for lease in self._leases]
        loc0 = locations[0].cpu()
        if bool((loc0 == -1).any()):
            for lease, loc in zip(self._leases, locations):
                lease.release(dev_ids, loc)
            raise RuntimeError("an id of the room has no slot")
        eng = self.cache.engine
        rb = eng.storages[0].plane.bytes_per_record
        plans, positions = {}, {}
        for tier, mask, slots in (("device", loc0 >= 0, loc0), ("host", loc0 <= -2, -loc0 - 2)):
            pos = mask.nonzero().flatten()
            if pos.numel() == 0:
                continue
            plane = eng.storages[0].gpu if tier == "device" else eng.storages[0].host
            stride = plane[1].data_ptr() - plane[0].data_ptr() if plane.shape[0] > 1 else 0
            plans[tier] = plan_direct_receive(slots[pos].tolist(), record_bytes=rb, layers=min(self.layers, plane.shape[0]),
                                              layer_stride=stride, base_address=plane.data_ptr(), tier=tier,
                                              chunk_records=self.chunk)
            positions[tier] = pos
        device_records = int((loc0 >= 0).sum())
        self._leased_device += device_records
        now = time.monotonic()
        self._rooms[key] = dict(ids=dev_ids, locations=locations, pages=pages, plans=plans, positions=positions,
                                device_records=device_records,
                                timing=dict(room=key, request_id=request_id, prefix_records=prefix_records,
                                            received_records=int(flat.numel()), device_records=device_records,
                                            admission_wait_seconds=t0 - self._waiting.pop(key, t0),
                                            reserve_seconds=now - t0, reserved_at=now, payload_staging_bytes=0))
        for page in pages:
            self._page_owner[page] = key
        return plans, positions

    def metadata_sent(self, key, *, encoding_seconds=None, metadata_bytes=None):
        import time

        timing = self._rooms[key]["timing"]
        timing["metadata_sent_at"] = time.monotonic()
        if encoding_seconds is not None:
            timing["metadata_encoding_seconds"] = encoding_seconds
        if metadata_bytes is not None:
            timing["metadata_bytes"] = metadata_bytes

    def _retire(self, key, *, transport_quiesced: bool) -> int:
        import time

        if transport_quiesced is not True:
            raise RuntimeError("remote writes must have drained before their destinations are retired")
        room = self._rooms.pop(key)
        for lease, loc in zip(self._leases, room["locations"]):
            lease.release(room["ids"], loc)
        self._leased_device -= room["device_records"]
        for page in room["pages"]:
            del self._page_owner[page]
        if self._audit is not None:
            now, timing = time.monotonic(), room["timing"]
            self._audit(dict(timing, retired_at=now, destination_lease_seconds=now - timing["reserved_at"],
                             advertised_to_retired_seconds=now - timing.get("metadata_sent_at", now),
                             transport_quiesced=True))
        return int(room["ids"].numel())

    def complete(self, key) -> int:
        """The sender confirmed every write of the room: the records become ordinary, touched-now records."""
        return self._retire(key, transport_quiesced=True)

    def logical_pages_freed(self, page_ids, *, transport_quiesced: bool):
        """An aborted request's pages were retired by the allocator.  A room is dropped only whole."""
        gone = {int(p) for p in page_ids}
        keys = {self._page_owner[p] for p in gone if p in self._page_owner}
        for key in keys:
            if not self._rooms[key]["pages"] <= gone:
                raise RuntimeError("an aborted receive must retire every page it advertised")
        for key in keys:
            self._retire(key, transport_quiesced=transport_quiesced)

    def metadata_inventory(self) -> dict:
        return dict(payload_staging_bytes=0, pending_rooms=len(self._rooms), waiting_rooms=len(self._waiting),
                    directory_bytes=sum(4 * r["ids"].numel() * (1 + len(r["locations"])) for r in self._rooms.values()),
                    leased_device_records=self._leased_device, working_records=self.working_records)
