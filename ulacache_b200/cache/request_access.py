"""Token -> device record row through the replicated page map of the whole-request tier.

Reference: ulacache/cache/request_access.py:1-62, csrc/include/sgl_kernel/flowkv/request_page_map.cuh:17-26.
"""
from __future__ import annotations

from .request_pages import PAGE_TOKENS


def request_physical_rows(page_map, request_pages, positions):
    """``request_pages`` int32 [R, max_pages] logical pages of each request, ``positions`` int32 [R, K]
    token positions (-1 padding) -> int32 [R, K] rows in ``RequestPageStorage.record_view`` (-1 when
    the page is not on the device or the position is padding)."""
    import torch

    pos = positions.long()
    valid = pos >= 0
    page_slot = (pos.clamp(min=0) // PAGE_TOKENS).clamp(max=request_pages.shape[1] - 1)
    lp = torch.gather(request_pages.long(), 1, page_slot)
    dp = torch.where(lp >= 0, page_map.to(pos.device)[lp.clamp(min=0)].long(), torch.full_like(lp, -1))
    rows = dp * PAGE_TOKENS + pos.clamp(min=0) % PAGE_TOKENS
    return torch.where(valid & (lp >= 0) & (dp >= 0), rows, torch.full_like(rows, -1)).to(torch.int32)


class RequestAddressRuntime:
    """The object a :class:`~ulacache_b200.cache.request_storage.RequestTier` asks "may pages move now?".

    Readers of the tier's pages are the kernels of a forward (decode step or prefill chunk) queued on the model's
    stream.  The runtime brackets every forward: ``begin_forward`` / ``finish_forward`` (``begin_prefill`` /
    ``finish_prefill`` are the same bracket for a chunk).  ``finish_forward`` records an event behind the last
    reader; ``readers_retired`` refuses inside a bracket, waits for that event at the admission / release
    boundary where it is called, and, in a group of ranks whose kernels read each other's pages, also for every
    peer's published phase (``publication``: a ``DistributedResidencyPublication``, domain ``domain``).

    Reference: ulacache/cache/request_access.py:5-62 (``RequestAddressRuntime``: validate, begin / finish prefill,
    reader retirement at request boundaries)."""

    def __init__(self, *, device, publication=None, domain: int = 0):
        import torch

        self.device = torch.device(device)
        self.publication, self.domain = publication, domain
        self._open = False
        self._event = None
        self.forwards = self.boundary_waits = 0

    def validate(self, tier):
        import torch

        pm = tier.page_map
        shapes = tier.storage.plane_shapes()
        ok = (pm.dtype == torch.int32 and pm.ndim == 1 and pm.is_contiguous() and pm.device.type == self.device.type
              and pm.numel() == tier.pool.logical_pages and shapes["record_gpu"][1] == tier.pool.device_pages
              and shapes["record_cpu"][1] >= tier.pool.host_pages
              and tier.storage.device_pool.device.type == self.device.type)
        if not ok:
            raise ValueError("the request tier's page map and planes do not match the pool this runtime serves")

    def begin_forward(self):
        if self._open:
            raise RuntimeError("the previous forward has not finished")
        self._open = True
        self.forwards += 1

    def finish_forward(self):
        """Call after the model has queued every read of the forward on the current stream."""
        import torch

        if not self._open:
            raise RuntimeError("no forward is open")
        if self.device.type == "cuda":
            self._event = torch.cuda.Event()
            self._event.record(torch.cuda.current_stream(self.device))
        if self.publication is not None:
            self.publication.publish(self.domain, 1)
        self._open = False

    begin_prefill, finish_prefill = begin_forward, finish_forward

    def readers_retired(self, tier) -> bool:
        """At an admission / release boundary only: blocks until the last forward's readers are done."""
        self.validate(tier)
        if self._open:
            return False
        if self._event is not None:
            self._event.synchronize()
            self._event = None
        if self.publication is not None and not self.publication.may_move_records(self.domain):
            return False
        self.boundary_waits += 1
        return True
