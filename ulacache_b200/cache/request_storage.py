"""Whole-request tier: physical storage, page-map publication and boundary execution around the page pool.

``cpu_policy="request"`` keeps a scheduled request fully device resident and parks idle requests in pinned
host pages.  :class:`~ulacache_b200.cache.request_pages.RequestPagePool` decides WHICH pages move;
this module owns everything physical:

* :class:`RequestPageStorage` - the record pages of every layer on the device and in pinned host memory,
  and (optionally) the Index pages of the anchor layers, which move with the same page numbers;
* :class:`PageMapPublisher` - the host mirror of the logical -> device page map and its device copy.  The
  device map changes only at step boundaries (``publish``), by a blocking copy that the model stream
  follows; bindings the allocator already scattered on the GPU are settled in the mirror only
  (``record_completed_bindings``) so a later publish keeps them;
* :class:`RequestTier` - sizes the host side against a memory budget before allocating anything, refuses
  to run until a runtime that can answer "have the readers retired?" is bound, executes boundary
  transactions (bytes first, publication after), tracks attached readers, and reports a capacity audit.

Reference: ulacache/cache/request_storage.py:18-276 (``request_workspace_rows``,
``LocalPageMapPublisher``, ``FlowKVRequestTier``).
"""
from __future__ import annotations

from .request_pages import PAGE_TOKENS, RequestPagePool

INDEX_PAGE_BYTES = PAGE_TOKENS * 132          # 64 keys of 128 fp8 bytes + one fp32 scale each


def request_workspace_rows(page_tokens: int, max_query_tokens: int, peers: int, topk: int) -> int:
    """Rows of the exchange workspace: every query may name ``topk`` records on every peer plus its own."""
    return max(page_tokens, max_query_tokens * (peers * topk + 1))


class _PagePlane:
    """[layers, pages, page_bytes] on the device and in (pinned) host memory."""

    def __init__(self, layers, device_pages, host_pages, page_bytes, device, pin_host):
        import torch

        self.layers, self.page_bytes = layers, page_bytes
        self.device_pool = torch.zeros((layers, device_pages, page_bytes), dtype=torch.uint8, device=device)
        host = torch.zeros((layers, max(host_pages, 1), page_bytes), dtype=torch.uint8)
        if pin_host and torch.cuda.is_available():
            host = host.pin_memory()
        self.host_pool = host


class RequestPageStorage(_PagePlane):
    def __init__(self, *, layers: int, device_pages: int, host_pages: int, record_bytes: int, device,
                 pin_host: bool = True, index_anchor_layers=()):
        super().__init__(layers, device_pages, host_pages, PAGE_TOKENS * record_bytes, device, pin_host)
        self.record_bytes = record_bytes
        self.index_anchor_layers = tuple(index_anchor_layers)
        self.index = (_PagePlane(len(self.index_anchor_layers), device_pages, host_pages, INDEX_PAGE_BYTES, device,
                                 pin_host) if self.index_anchor_layers else None)

    def record_view(self, layer: int):
        """Device pages of ``layer`` as records: uint8 [device_pages * 64, record_bytes]."""
        return self.device_pool[layer].view(-1, self.record_bytes)

    def index_view(self, layer: int):
        """Device Index pages of the group that ``layer`` anchors: uint8 [device_pages, 8448]."""
        if self.index is None or layer not in self.index_anchor_layers:
            raise KeyError("this layer anchors no Index pages in the request tier")
        return self.index.device_pool[self.index_anchor_layers.index(layer)]

    def plane_shapes(self) -> dict:
        out = {"record_gpu": tuple(self.device_pool.shape), "record_cpu": tuple(self.host_pool.shape)}
        if self.index is not None:
            out["index_gpu"] = tuple(self.index.device_pool.shape)
            out["index_cpu"] = tuple(self.index.host_pool.shape)
        return out

    @property
    def device_bytes(self) -> int:
        return self.device_pool.numel() + (self.index.device_pool.numel() if self.index is not None else 0)

    @property
    def host_bytes(self) -> int:
        return self.host_pool.numel() + (self.index.host_pool.numel() if self.index is not None else 0)


class PageMapPublisher:
    def __init__(self, pool: RequestPagePool, device):
        self.pool = pool
        self.host_map = pool.page_map()                    # int32 [logical pages], CPU
        self.device_map = self.host_map.to(device)
        self.pending_bindings = 0
        self.publications = 0

    def publish(self, updates=None):
        """Boundary publication: fold ``updates`` ((logical, device page) pairs; None = take the pool's
        whole map) into the mirror and copy the mirror to the device.  Refused while fresh bindings are
        still pending: their GPU scatter must be settled first or the copy would erase them."""
        if self.pending_bindings:
            raise RuntimeError("settle every pending page binding before a boundary publication")
        if updates is None:
            self.host_map.copy_(self.pool.page_map())
        else:
            for logical, physical in updates:
                self.host_map[logical] = physical
        self.device_map.copy_(self.host_map, non_blocking=False)      # the model stream follows this copy
        self.publications += 1

    def begin_binding(self, count: int = 1):
        """The allocator is scattering ``count`` fresh bindings into the device map itself."""
        self.pending_bindings += count

    def record_completed_bindings(self, updates):
        """Settle the mirror after the allocator's GPU scatter; the device map is neither copied nor read."""
        n = 0
        for logical, physical in updates:
            self.host_map[logical] = physical
            n += 1
        self.pending_bindings = max(0, self.pending_bindings - n)


class RequestTier:
    """``runtime`` objects (see :meth:`bind_runtime`) provide ``validate(tier)`` and ``readers_retired(tier)``."""

    def __init__(self, *, layers: int, device_pages: int, host_pages: int, logical_pages: int, record_bytes: int,
                 device, index_anchor_layers=(), host_memory_budget_bytes=None, pin_host: bool = True,
                 reserved_device_pages=(0,), max_query_tokens: int = 1, peers: int = 1, topk: int = 2048,
                 stream=None):
        from ..transfer.page_exchange import PageExchangeExecutor

        self.workspace_rows = request_workspace_rows(PAGE_TOKENS, max_query_tokens, peers, topk)
        anchors = tuple(index_anchor_layers)
        need = (layers * host_pages * PAGE_TOKENS * record_bytes + len(anchors) * host_pages * INDEX_PAGE_BYTES
                + 20 * self.workspace_rows + 4 * logical_pages + 256)
        self.host_bytes_required = need
        if host_memory_budget_bytes is not None and need > host_memory_budget_bytes:
            raise ValueError(f"the request tier's record and Index pages need {need} host bytes; "
                             f"the budget is {host_memory_budget_bytes}")
        self.pool = RequestPagePool(device_pages, host_pages, logical_pages, reserved_device_pages)
        self.storage = RequestPageStorage(layers=layers, device_pages=device_pages, host_pages=host_pages,
                                          record_bytes=record_bytes, device=device, pin_host=pin_host,
                                          index_anchor_layers=anchors)
        self.publisher = PageMapPublisher(self.pool, device)
        self.page_map = self.publisher.device_map
        self.executor = PageExchangeExecutor(self.storage, stream=stream,
                                             extra_storages=(self.storage.index,) if self.storage.index else ())
        self._runtime = None
        self._closed = False

    # ------------------------------------------------------------------- runtime --
    def bind_runtime(self, runtime):
        """Install the object that knows the model's streams: it certifies the tier's shapes
        (``validate``) and answers whether every reader of the previous step has retired."""
        if runtime is None:
            raise ValueError("a request tier needs a runtime that can vouch for reader retirement")
        runtime.validate(self)
        self._runtime = runtime

    def require_runtime(self):
        if self._runtime is None:
            raise NotImplementedError("the request tier's reader-retirement runtime is not connected")
        return self._runtime

    def _readers_retired(self) -> bool:
        return bool(self.require_runtime().readers_retired(self))

    # -------------------------------------------------------------- transactions --
    def check_gpu_capacity(self, total_tokens: int) -> bool:
        """Whether a request of ``total_tokens`` can ever be resident (ignoring who else is)."""
        return (total_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS <= self.pool.usable_device_pages

    def location(self, logical_page: int):
        return self.pool.where.get(logical_page)

    def reserve_request(self, request: int, total_tokens: int):
        return self.pool.reserve_request(request, total_tokens)

    def ensure_resident(self, txn):
        """Move the bytes of ``txn`` (records and Index pages, offloads before onloads in every wave).
        The previous step's readers must have retired: victims' pages are overwritten."""
        if txn.moved_pages and not self._readers_retired():
            raise RuntimeError("readers of the previous step have not retired; pages cannot move yet")
        return self.executor.move(txn)

    def commit(self, txn):
        """Apply ``txn`` to the pool and publish the new map (after :meth:`ensure_resident`)."""
        before = self.pool.page_map()
        self.pool.commit(txn)
        after = self.pool.page_map()
        changed = (before != after).nonzero().flatten().tolist()
        self.publisher.publish([(lp, int(after[lp])) for lp in changed])
        return len(changed)

    def cancel(self, txn):
        return self.pool.cancel(txn)

    def admit(self, request: int, total_tokens: int) -> int:
        """reserve -> move -> commit -> publish; returns the number of pages that moved."""
        txn = self.reserve_request(request, total_tokens)
        try:
            moved = self.ensure_resident(txn)
        except Exception:
            self.cancel(txn)
            raise
        self.commit(txn)
        return moved

    # ------------------------------------------------------------ reader lifetime --
    def attach_native_pages(self, request: int):
        self.require_runtime()
        self.pool.attach(request)
        return [self.pool.where[lp][1] for lp in self.pool.pages_of[request]]

    def retire_native_pages(self, request: int, *, readers_retired: bool):
        self.require_runtime()
        if not readers_retired:
            raise RuntimeError("retire pages only after their readers have finished on the stream")
        self.pool.retire(request)

    def free_request(self, request: int):
        pages = list(self.pool.pages_of.get(request, ()))
        self.pool.free_request(request)
        self.publisher.publish([(lp, -1) for lp in pages])

    def clear(self):
        if not self._readers_retired():
            raise RuntimeError("clear the request tier only after every reader has retired")
        if self.executor.stream is not None:
            self.executor.stream.synchronize()
        for r in list(self.pool.pages_of):
            self.pool.readers.pop(r, None)
            self.pool.free_request(r)
        self.publisher.publish()

    # ------------------------------------------------------------------- accounts --
    @property
    def gpu_free_pages(self) -> int:
        return len(self.pool.free_device)

    @property
    def metadata_bytes(self) -> int:
        return self.page_map.numel() * 4

    @property
    def host_payload_bytes(self) -> int:
        return self.storage.host_bytes

    @property
    def host_metadata_bytes(self) -> int:
        return self.publisher.host_map.numel() * 4 + 20 * self.workspace_rows

    def capacity_audit(self) -> dict:
        p = self.pool
        return {
            "policy": "request",
            "physical_gpu_rows": p.device_pages * PAGE_TOKENS,
            "physical_cpu_rows": p.host_pages * PAGE_TOKENS,
            "logical_rows": p.logical_pages * PAGE_TOKENS,
            "gpu_usable_pages": p.usable_device_pages,
            "cpu_usable_pages": p.host_pages,
            "gpu_free_pages": self.gpu_free_pages,
            "map_shape": tuple(self.page_map.shape),
            "plane_shapes": self.storage.plane_shapes(),
            "metadata_bytes": self.metadata_bytes,
            "host_payload_bytes": self.host_payload_bytes,
            "host_metadata_bytes": self.host_metadata_bytes,
            "host_bytes_required": self.host_bytes_required,
            "workspace_rows": self.workspace_rows,
            "moved_bytes": {"d2h": self.executor.bytes_d2h, "h2d": self.executor.bytes_h2d},
            "transactions": dict(p.stats),
            "runtime_connected": self._runtime is not None,
        }

    def close(self):
        if self._closed:
            return
        if self.executor.stream is not None:
            self.executor.stream.synchronize()
        self.storage = None
        self.page_map = None
        self.publisher = None
        self._closed = True
