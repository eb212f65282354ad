"""Leases on window rows: a window may be refilled only when no reader holds it.

Reference: ulacache/cache/prefill/leases.py:1-101.
"""
from __future__ import annotations


class WindowLeaseError(RuntimeError):
    pass


class WindowLeases:
    def __init__(self):
        self._held = {}        # window id -> set of reader tokens
        self._next = 0

    def acquire(self, window) -> int:
        self._next += 1
        self._held.setdefault(id(window), set()).add(self._next)
        return self._next

    def release(self, window, token: int):
        held = self._held.get(id(window), set())
        if token not in held:
            raise WindowLeaseError("released a lease that is not held")
        held.discard(token)

    def readers(self, window) -> int:
        return len(self._held.get(id(window), ()))

    def check_refill(self, window):
        if self.readers(window):
            raise WindowLeaseError(f"window still has {self.readers(window)} reader(s); refill refused")


# ----------------------------------------------------------------------------------------------
# Page leases of prefill READERS.  A request that reuses a cached prefix reads its pages while it
# prefills; the allocator must not reclaim (or re-map) such a page until the last reader is gone.
# Leases are counted per logical page; a request holds each page at most once.
#
# Reference: ulacache/cache/prefill/leases.py:9-101 (PrefillPageLeases, prefill_physical_tokens).
# ----------------------------------------------------------------------------------------------
class PrefixPageLeases:
    def __init__(self):
        self._pages = {}        # logical page -> [physical page, readers]
        self._held = {}         # request -> set of logical pages

    def acquire(self, request, logical_to_physical) -> list:
        """Lease the pages of ``logical_to_physical`` ({logical: physical}, page 0 is padding) for ``request``.
        The whole update is validated before anything changes, so a page whose physical home moved under a live
        reader cannot leave a half-acquired request behind.  Returns the pages newly held by the request."""
        items = dict(logical_to_physical)
        for logical, physical in items.items():
            if type(logical) is not int or type(physical) is not int:
                raise ValueError("page identities must be integers")
            if logical <= 0 or physical <= 0:
                raise ValueError("page zero is reserved for padding")
            have = self._pages.get(logical)
            if have is not None and have[0] != physical:
                raise ValueError(f"logical page {logical} moved from physical page {have[0]} to {physical} under a reader")
        held = self._held.setdefault(request, set())
        fresh = []
        for logical, physical in items.items():
            if logical in held:
                continue
            self._pages.setdefault(logical, [physical, 0])[1] += 1
            held.add(logical)
            fresh.append(logical)
        return fresh

    def release(self, request, logical_pages=None) -> dict:
        """Drop ``request``'s leases (all of them, or the listed pages).  Returns {logical: physical} of the pages
        whose last reader this was: those may be reclaimed now."""
        held = self._held.get(request)
        if held is None:
            return {}
        chosen = set(held) if logical_pages is None else set(logical_pages)
        if not chosen <= held:
            raise ValueError("a request cannot release pages it does not hold")
        freed = {}
        for logical in chosen:
            entry = self._pages[logical]
            entry[1] -= 1
            held.discard(logical)
            if entry[1] == 0:
                freed[logical] = entry[0]
                del self._pages[logical]
        if not held:
            del self._held[request]
        return freed

    def readers(self, logical_page: int) -> int:
        entry = self._pages.get(logical_page)
        return 0 if entry is None else entry[1]

    def assert_reclaimable(self, logical_pages):
        busy = [p for p in logical_pages if p in self._pages]
        if busy:
            raise ValueError(f"logical prefix pages {busy[:8]} still have prefill readers")


def prefill_physical_tokens(*, prefix_tokens: int, held_prefix_tokens: int, extend_tokens: int, hot_tokens: int,
                            scratch_tokens: int, page_size: int) -> int:
    """Device tokens a prefill needs, whatever the host tier could still give back: the part of the prefix that
    is not already held, the new tokens (both rounded up to pages), the decode working set that must stay, scratch,
    and one spare page."""
    vals = (prefix_tokens, held_prefix_tokens, extend_tokens, hot_tokens, scratch_tokens)
    if page_size <= 0 or any(v < 0 for v in vals):
        raise ValueError("prefill memory geometry must be non-negative")

    def pages(n):
        return -(-n // page_size) * page_size

    return pages(max(prefix_tokens - held_prefix_tokens, 0)) + pages(extend_tokens) + hot_tokens + scratch_tokens + page_size
