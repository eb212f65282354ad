"""Bounded staging window of a prefill -> decode hand-over that cannot write canonical storage directly.

A remote writer only ever sees this window: ``record_capacity`` records of every layer in one pinned host
allocation, handed out in 64-record pages under leases.  When the transport reports a request complete, the
owning thread publishes it: the records' CURRENT locations are looked up (they may have moved between HBM and
host slots while the bytes were in flight), leased so that no eviction plan can take them during the copy,
filled by ``csrc/receive.cu:receive_publish_kernel`` (one warp per record and layer, reading the pinned window
through its mapped address) and released as touched-now.  Staging pages are reusable only after the transport
has been told to stop writing them (``transport_quiesced=True``).

Additional banks (draft-model state, Index records ...) ride under the same lease: ``add_sidecar`` gives each its
own pinned window rows and publication copies them to destinations addressed by the logical record id itself.

    window = StagedReceiveWindow(cache, record_capacity=4096)
    banks = window.registration()                      # (address, bytes, page bytes) per layer, for the transport
    lease = window.reserve("room-7", ids, record_count=n)
    ... transport writes window.staging[:, window.staging_rows("room-7")] ...
    window.publish("room-7")

Reference: ulacache/transfer/receive_window.py:15-502 (page leases, native page helpers,
``PinnedRecordReceiveWindow``), ulacache/transfer/kernels/receive_publication.py:15-90.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

PAGE = 64


def _is_count(x, lowest=0) -> bool:
    return type(x) is int and x >= lowest


@dataclass(frozen=True)
class StagingLease:
    key: object
    generation: int
    pages: Tuple[int, ...]


class StagingPages:
    """LIFO free list of staging pages; one live lease per key; generations expose stale leases."""

    def __init__(self, page_count: int):
        if not _is_count(page_count, 1):
            raise ValueError("a staging window holds at least one page")
        self._free = list(reversed(range(page_count)))
        self._live: Dict[object, StagingLease] = {}
        self._generation = 0

    @property
    def available_pages(self) -> int:
        return len(self._free)

    def reserve(self, key, page_count: int) -> StagingLease:
        if key in self._live:
            raise ValueError(f"{key!r} already holds staging pages")
        if not _is_count(page_count):
            raise ValueError("page count must be a non-negative integer")
        if page_count > len(self._free):
            raise BufferError(f"the staging window has {len(self._free)} free pages; {page_count} were asked for")
        self._generation += 1
        taken = tuple(self._free.pop() for _ in range(page_count))
        lease = self._live[key] = StagingLease(key, self._generation, taken)
        return lease

    def release(self, lease: StagingLease, *, transport_quiesced: bool):
        if transport_quiesced is not True:
            raise RuntimeError("staging pages are reusable only after the transport stopped writing them")
        if self._live.get(lease.key) != lease:
            raise ValueError("this lease is stale or was never granted")
        del self._live[lease.key]
        self._free.extend(reversed(lease.pages))


# ------------------------------------------------------------------------------------- page arithmetic --

def received_record_count(page_count: int, page_size: int, record_count=None) -> int:
    """Records a transfer of ``page_count`` pages carries: all of them, or ``record_count`` when the last page is
    only partly allocated (it must reach into that last page and not beyond it)."""
    if not _is_count(page_count) or not _is_count(page_size, 1):
        raise ValueError("page count >= 0 and page size >= 1")
    full = page_count * page_size
    if record_count is None:
        return full
    if not _is_count(record_count):
        raise ValueError("record count must be a non-negative integer")
    if full == 0 and record_count == 0:
        return 0
    if not full - page_size < record_count <= full:
        raise ValueError("valid records must end inside the last transferred page")
    return record_count


def drop_committed_prefix(source_pages, destination_pages, prefix_tokens: int, page_size: int):
    """The receiver already holds ``prefix_tokens`` (a whole number of pages): both page lists lose that head."""
    if not _is_count(prefix_tokens) or not _is_count(page_size, 1) or prefix_tokens % page_size:
        raise ValueError("the committed prefix is a whole number of pages")
    if len(source_pages) != len(destination_pages):
        raise ValueError("source and destination list a different number of pages")
    head = prefix_tokens // page_size
    if head > len(source_pages):
        raise ValueError("the committed prefix is longer than the payload")
    return source_pages[head:], destination_pages[head:]


def staged_state_pages(canonical_pages, staging_pages, *, prefix_tokens: int, page_size: int):
    """Destination list of a transfer whose suffix goes through the staging window: the canonical pages of the
    committed prefix stay as placeholders (the sender drops them), the rest is replaced by the lease's pages.
    Canonical pages are >= 1 (page 0 is padding); staging page 0 is a real page."""
    canonical, staged = tuple(canonical_pages), tuple(staging_pages)
    if not _is_count(prefix_tokens) or not _is_count(page_size, 1) or prefix_tokens % page_size:
        raise ValueError("the committed prefix is a whole number of pages")
    ok = (all(_is_count(p, 1) for p in canonical) and all(_is_count(p) for p in staged)
          and len(set(canonical)) == len(canonical) and len(set(staged)) == len(staged))
    if not ok:
        raise ValueError("pages must be unique integers (canonical >= 1, staging >= 0)")
    head = prefix_tokens // page_size
    if head > len(canonical) or len(staged) != len(canonical) - head:
        raise ValueError("the staging lease does not match the uncommitted suffix")
    return canonical[:head] + staged


def transfer_pages_of_allocation_pages(page_ids, *, allocation_page_size: int, transfer_page_size: int):
    """An allocation page of ``allocation_page_size`` records is ``ratio`` consecutive transfer pages."""
    if (not _is_count(allocation_page_size, 1) or not _is_count(transfer_page_size, 1)
            or allocation_page_size % transfer_page_size):
        raise ValueError("an allocation page holds a whole number of transfer pages")
    pages = tuple(page_ids)
    if any(not _is_count(p, 1) for p in pages) or len(set(pages)) != len(pages):
        raise ValueError("retired allocation pages are unique and >= 1")
    ratio = allocation_page_size // transfer_page_size
    if any((p + 1) * ratio > 2 ** 31 for p in pages):
        raise ValueError("transfer page numbers would leave int32")
    return tuple(p * ratio + k for p in pages for k in range(ratio))


# ------------------------------------------------------------------------------------------- the window --

def _layer_runs(layers, storage_index):
    """Split ``layers`` (ascending) into runs whose storage indices ascend by one as well: one kernel launch each."""
    runs, start = [], 0
    for i in range(1, len(layers) + 1):
        if (i == len(layers) or layers[i] != layers[i - 1] + 1
                or storage_index[layers[i]] != storage_index[layers[i - 1]] + 1):
            runs.append((layers[start], storage_index[layers[start]], i - start))
            start = i
    return runs


class StagedReceiveWindow:
    """``cache``: a rank-local client (one owner).  Incoming records are excluded from model execution by the
    caller until :meth:`publish` returns."""

    def __init__(self, cache, *, record_capacity: int, copy_chunk_records: int = 4096, pin: bool = True):
        import torch

        from .receive_lease import ReceiveLeases

        eng = cache.engine
        if getattr(eng.owners, "ranks", 1) != 1:
            raise NotImplementedError("a striped pool stages per owner with that owner's engine")
        if not _is_count(record_capacity, PAGE) or record_capacity % PAGE:
            raise ValueError("the window holds whole 64-record pages")
        if not _is_count(copy_chunk_records, 1):
            raise ValueError("publication copies at least one record per chunk")
        self.cache, self.engine = cache, eng
        self.record_capacity, self.chunk = record_capacity, copy_chunk_records
        self.layers = len(eng._storage_of_layer)
        self.row_bytes = eng.storages[0].plane.bytes_per_record
        self.pinned = bool(pin and torch.cuda.is_available())
        self.staging = self._host((self.layers, record_capacity, self.row_bytes))
        self.pages = StagingPages(record_capacity // PAGE)
        self.leases = [ReceiveLeases(res) for res in eng.residency]
        self._pending: Dict[object, dict] = {}
        self._sidecars: Dict[str, dict] = {}
        self._frozen = False
        self.published_records = 0

    def _host(self, shape):
        import torch

        t = torch.zeros(shape, dtype=torch.uint8)
        return t.pin_memory() if self.pinned else t

    # ------------------------------------------------------------- registration --
    @property
    def available_records(self) -> int:
        return self.pages.available_pages * PAGE

    @staticmethod
    def _banks(storage, width):
        return [(storage[l].data_ptr(), storage[l].numel(), PAGE * width) for l in range(storage.shape[0])]

    def registration(self):
        """Per layer: (address, bytes, bytes per page) of the window.  After this call no bank can be added:
        the transport has the addresses."""
        self._frozen = True
        return self._banks(self.staging, self.row_bytes)

    def add_sidecar(self, name: str, destinations):
        """``destinations``: tensors [rows, ...] on the engine's device, one per bank, all of one row width; row
        ``id`` of each is where record ``id`` of that bank finally lives.  Returns a callable that yields the
        bank's registration (and freezes the window)."""
        import torch

        if self._frozen or self._pending:
            raise RuntimeError("banks are fixed once addresses were handed out or a transfer was reserved")
        if not isinstance(name, str) or not name or name in self._sidecars:
            raise ValueError("a sidecar needs a unique non-empty name")
        dests = list(destinations)
        want = self.engine.device             # may carry no index ("cuda"): compare the type, and the index if given

        def elsewhere(d):
            return d.device.type != want.type or (want.index is not None and d.device.index != want.index)

        if not dests or any(d.ndim < 2 or not d.is_contiguous() or d.shape[0] < 1 or elsewhere(d) for d in dests):
            raise ValueError("sidecar destinations are contiguous [rows, ...] tensors on the cache's device")
        flat = [d.view(torch.uint8).reshape(d.shape[0], -1) for d in dests]
        width = flat[0].shape[1]
        if width < 1 or any(f.shape[1] != width for f in flat):
            raise ValueError("the banks of one sidecar share one row width")
        storage = self._host((len(flat), self.record_capacity, width))
        self._sidecars[name] = dict(storage=storage, destinations=flat, width=width)

        def registration():
            self._frozen = True
            return self._banks(storage, width)

        return registration

    # ---------------------------------------------------------------- transfers --
    def reserve(self, key, ids, *, record_count=None) -> StagingLease:
        """``ids``: the request's logical record ids in token order, whole pages (as ``cache.alloc`` returns
        them); ``record_count``: how many of them the sender fills (the last page may be partly used)."""
        import torch

        if key in self._pending:
            raise ValueError(f"{key!r} already has a transfer in flight")
        ids = ids.reshape(-1).to(device="cpu", dtype=torch.int64)
        if ids.numel() % PAGE:
            raise ValueError("incoming ids come in whole pages")
        heads = ids[::PAGE]
        if (bool((heads % PAGE != 0).any()) or bool((heads <= 0).any()) or heads.unique().numel() != heads.numel()
                or not torch.equal(ids, (heads[:, None] + torch.arange(PAGE)).reshape(-1))):
            raise ValueError("incoming pages must be unique, non-zero and complete")
        n = received_record_count(heads.numel(), PAGE, record_count)
        rows = ids[:n]
        if n and any(int(rows.max()) >= f.shape[0] for s in self._sidecars.values() for f in s["destinations"]):
            raise ValueError("a sidecar destination is too small for these records")
        self.validate_extra_destinations(rows)
        lease = self.pages.reserve(key, heads.numel())
        self._frozen = True
        src = (torch.tensor(lease.pages, dtype=torch.int64)[:, None] * PAGE + torch.arange(PAGE)).reshape(-1)[:n]
        self._pending[key] = dict(lease=lease, pages=set((heads // PAGE).tolist()), rows=rows, source_rows=src)
        return lease

    def transfer_pages(self, key) -> Tuple[int, ...]:
        return self._pending[key]["lease"].pages

    def staging_rows(self, key):
        """Window rows of the transfer's records, in token order."""
        return self._pending[key]["source_rows"]

    # hooks of windows that carry more state under the same lease
    def validate_extra_destinations(self, rows):
        pass

    def publish_extra_banks(self, item):
        pass

    def _publish_records(self, rows, src):
        import torch

        eng = self.engine
        dev = eng.device
        st = eng.storages[0]
        for g, leases in enumerate(self.leases):
            ids = rows.to(device=dev, dtype=torch.int32)
            loc = leases.acquire(ids)
            try:
                if bool((loc == -1).any()):
                    raise RuntimeError("incoming records were freed before their publication")
                src_dev = src.to(device=dev, dtype=torch.int32)
                layers = sorted(eng.groups.layers_of(g))
                for first_layer, first_storage, count in _layer_runs(layers, eng._storage_of_layer):
                    host = None if st.host is None else st.host[first_storage:first_storage + count]
                    leases.publish(self.staging[first_layer:first_layer + count], src_dev, loc,
                                   st.gpu[first_storage:first_storage + count], host)
            finally:
                leases.release(ids, loc)

    def _publish_sidecar(self, side, rows, src):
        import torch

        dev = self.engine.device
        for bank, dest in enumerate(side["destinations"]):
            if dev.type == "cuda" and side["width"] % 16 == 0:
                self.leases[0].publish(side["storage"][bank:bank + 1], src.to(device=dev, dtype=torch.int32),
                                       rows.to(device=dev, dtype=torch.int32), dest.unsqueeze(0), None)
            else:
                payload = side["storage"][bank].index_select(0, src)
                dest.index_copy_(0, rows.to(dev), payload.to(dev))

    def publish(self, key) -> int:
        """Copy a completed transfer to the records' current locations and free its staging pages."""
        import torch

        item = self._pending[key]
        rows_all, src_all = item["rows"], item["source_rows"]
        for a in range(0, rows_all.numel(), self.chunk):
            rows, src = rows_all[a:a + self.chunk], src_all[a:a + self.chunk]
            self._publish_records(rows, src)
            for side in self._sidecars.values():
                self._publish_sidecar(side, rows, src)
        self.publish_extra_banks(item)
        if self.engine.device.type == "cuda":
            torch.cuda.current_stream(self.engine.device).synchronize()      # the pages are about to be reused
            for leases in self.leases:
                leases.res.check_status("receive publication")
        self.pages.release(item["lease"], transport_quiesced=True)
        del self._pending[key]
        self.published_records += rows_all.numel()
        return rows_all.numel()

    def logical_pages_freed(self, logical_pages):
        """The allocator retired these pages after draining the remote writer: a transfer whose pages are all
        gone is dropped and its staging pages return."""
        gone = {int(p) for p in logical_pages}
        for key, item in list(self._pending.items()):
            item["pages"] -= gone
            if not item["pages"]:
                self.pages.release(item["lease"], transport_quiesced=True)
                del self._pending[key]

    def memory_inventory(self) -> dict:
        side = self._sidecars.values()
        return dict(
            cpu_receive_bytes=self.staging.numel() + sum(s["storage"].numel() for s in side),
            cpu_receive_metadata_bytes=sum(8 * (i["rows"].numel() + i["source_rows"].numel())
                                           for i in self._pending.values()),
            gpu_lease_bytes=sum(4 * l.leases.numel() for l in self.leases),
            record_capacity=self.record_capacity,
            sidecar_banks=sum(len(s["destinations"]) for s in side),
            pending_publications=len(self._pending),
            published_records=self.published_records,
            pinned=self.pinned,
        )


class IndexStagedReceiveWindow(StagedReceiveWindow):
    """A staged window that also carries the request's Index records under the same lease.  Index records keep
    their stable addresses (owner-local record = function of the logical id): only the KV records go through the
    residency directory.  The sender writes native Index pages (64 keys of 128 bytes, then 64 scales of 4) into the
    window's Index staging; publication copies the records THIS rank owns into the bound page banks.

    Reference: ulacache/transfer/owner_index_receive.py:12-151 (Index page banks under the KV receive lease)."""

    def __init__(self, cache, *, ranks: int = 1, rank: int = 0, **kw):
        super().__init__(cache, **kw)
        if type(ranks) is not int or ranks < 1 or not 0 <= rank < ranks:
            raise ValueError("Index ownership needs a positive owner count and a rank inside it")
        self.ranks, self.rank = ranks, rank
        self._index_banks: Dict[str, dict] = {}
        self.published_index_records = 0

    def add_index_page_banks(self, name: str, destinations, *, replicated: bool = False):
        """``destinations``: uint8 page pools (whole 8448-byte pages), one per Index layer.  ``replicated``: every
        rank keeps all records (a draft model's Index) instead of only its stripe."""
        import torch

        from .index_pages import PAGE_BYTES

        if self._frozen or self._pending:
            raise RuntimeError("banks are fixed once addresses were handed out or a transfer was reserved")
        if not isinstance(name, str) or not name or name in self._index_banks or name in self._sidecars \
                or type(replicated) is not bool:
            raise ValueError("an Index bank needs a unique name and an explicit ownership")
        banks = list(destinations)
        if not banks or any(not isinstance(b, torch.Tensor) or b.dtype != torch.uint8 or not b.is_contiguous()
                            or b.numel() == 0 or b.numel() % PAGE_BYTES for b in banks):
            raise ValueError("Index banks are contiguous uint8 tensors of whole pages")
        pages = self.record_capacity // PAGE
        staging = self._host((len(banks), pages, PAGE_BYTES))
        self._index_banks[name] = dict(staging=staging, destinations=banks, replicated=replicated)

        def registration():
            self._frozen = True
            return [(staging[l].data_ptr(), staging[l].numel(), PAGE_BYTES) for l in range(staging.shape[0])]

        return registration

    def validate_extra_destinations(self, rows):
        from .index_pages import PAGE_BYTES, owner_local_record

        if not rows.numel() or not self._index_banks:
            return
        for bank in self._index_banks.values():
            ranks = 1 if bank["replicated"] else self.ranks
            last = max(owner_local_record(int(r), ranks)[1] for r in (rows.max(), rows.min()))
            if any((last // PAGE + 1) * PAGE_BYTES > d.numel() for d in bank["destinations"]):
                raise ValueError("an Index bank is too small for these records")

    def publish_extra_banks(self, item):
        from .index_pages import plan_index_record_copies, publish_index_records

        rows, src = item["rows"].tolist(), item["source_rows"].tolist()
        for bank in self._index_banks.values():
            ranks, rank = (1, 0) if bank["replicated"] else (self.ranks, self.rank)
            keep = [(r, s) for r, s in zip(rows, src) if r >= ranks * PAGE]          # the first page is padding
            plan = plan_index_record_copies([r for r, _ in keep], [s for _, s in keep], ranks=ranks, rank=rank)
            for layer, dest in enumerate(bank["destinations"]):
                staged = bank["staging"][layer]
                self.published_index_records += publish_index_records(
                    staged.to(dest.device) if dest.device.type != "cpu" else staged, dest, plan, transport_quiesced=True)

    def memory_inventory(self) -> dict:
        out = super().memory_inventory()
        out["cpu_receive_bytes"] += sum(b["staging"].numel() for b in self._index_banks.values())
        out["index_banks"] = sum(len(b["destinations"]) for b in self._index_banks.values())
        out["published_index_records"] = self.published_index_records
        return out
