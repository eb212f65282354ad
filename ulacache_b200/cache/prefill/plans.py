"""Chunking of a long prompt into prefill steps that fit the windows.

Reference: ulacache/cache/prefill/plans.py:1-154.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class PrefillChunkPlan:
    start: int            # first prompt token of the chunk
    tokens: int           # new tokens computed in this chunk
    history: int          # cached tokens the chunk attends to (prefix + earlier chunks)
    window_records: int   # upper bound on distinct records read: min(history + tokens, tokens * topk)


def plan_prefill_chunks(prompt_tokens: int, *, cached_prefix: int = 0, chunk_tokens: int = 8192, topk: int = 2048,
                        window_capacity: int = 1 << 20) -> List[PrefillChunkPlan]:
    """Split ``prompt_tokens`` (of which ``cached_prefix`` are already cached) so that no chunk can
    select more distinct records than one window holds."""
    if not 0 <= cached_prefix <= prompt_tokens:
        raise ValueError("cached_prefix must lie inside the prompt")
    if chunk_tokens < 1 or window_capacity < topk:
        raise ValueError("chunk_tokens >= 1 and a window of at least topk records")
    plans, pos = [], cached_prefix
    while pos < prompt_tokens:
        n = min(chunk_tokens, prompt_tokens - pos)
        # shrink the chunk until its worst-case union fits the window
        while n > 1 and min(pos + n, n * topk) > window_capacity:
            n = max(1, n // 2)
        if min(pos + n, n * topk) > window_capacity:
            raise MemoryError("a single token's selection does not fit the prefill window")
        plans.append(PrefillChunkPlan(pos, n, pos, min(pos + n, n * topk)))
        pos += n
    return plans


# ----------------------------------------------------------------------------------------------
# Admission against the reconstruction window, grouping of requests, and read plans that are
# computed once and reused by every layer of a forward.
#
# Reference: ulacache/cache/prefill/plans.py:14-154 (PrefillSequenceBudget, prefill_request_groups,
# NativePrefillReadPlans.read / read_selected).
# ----------------------------------------------------------------------------------------------
class PrefillSequenceBudget:
    """A prefill batch reconstructs the FULL history (cached prefix + new tokens) of every sequence it admits;
    the sum must fit one window."""

    def __init__(self, capacity: int = 1 << 20):
        if type(capacity) is not int or capacity < 1:
            raise ValueError("prefill sequence capacity must be a positive integer")
        self.capacity, self.used = capacity, 0

    def can_reserve(self, prefix_len: int, extend_len: int) -> bool:
        if any(type(n) is not int or n < 0 for n in (prefix_len, extend_len)):
            raise ValueError("prefix and extend lengths must be non-negative integers")
        if prefix_len + extend_len > self.capacity:
            raise ValueError("one sequence exceeds the reconstruction window")
        return self.used + prefix_len + extend_len <= self.capacity

    def reserve(self, prefix_len: int, extend_len: int):
        if not self.can_reserve(prefix_len, extend_len):
            raise RuntimeError("the batch's full histories no longer fit the reconstruction window")
        self.used += prefix_len + extend_len

    def reset(self):
        self.used = 0


def prefill_request_groups(request_lengths, capacity: int):
    """(offset, count) runs over the flattened rows of consecutive requests: whole requests are merged while
    they fit ``capacity``; a request longer than the window is cut into window-sized pieces of its own."""
    if type(capacity) is not int or capacity < 1:
        raise ValueError("prefill window capacity must be a positive integer")
    offset = start = count = 0
    for length in request_lengths:
        if type(length) is not int or length < 0:
            raise ValueError("request lengths must be non-negative integers")
        if length > capacity:
            if count:
                yield start, count
            for at in range(offset, offset + length, capacity):
                yield at, min(capacity, offset + length - at)
            offset += length
            start, count = offset, 0
            continue
        if count + length > capacity:
            yield start, count
            start, count = offset, 0
        count += length
        offset += length
    if count:
        yield start, count


class PrefillReadPlans:
    """Per forward: ONE plan for the dense read of the admitted histories and ONE for the sparse read of the current
    shared-selection group.  Layers of the forward reuse them (index tensors only; every layer gathers its own
    payload through ``reader``, a :class:`~ulacache_b200.cache.prefill.window.WindowedPrefillReader`).  The source
    tensors stay referenced so that their identity (the cache key) cannot be recycled while a plan is live."""

    def __init__(self, reader, layer_groups, capacity: int):
        if type(capacity) is not int or capacity < 1:
            raise ValueError("prefill window capacity must be a positive integer")
        self.reader, self.layer_groups, self.capacity = reader, layer_groups, capacity
        self.plans_built = 0
        self.reset()

    def reset(self):
        self.dense = self.sparse = None

    def _validate(self, rows, request_lengths):
        if rows.numel() > self.capacity:
            raise ValueError("the full histories exceed the fixed window capacity")
        lengths = (int(rows.numel()),) if request_lengths is None else tuple(request_lengths)
        if any(type(n) is not int or n < 0 for n in lengths):
            raise ValueError("request lengths must be non-negative integers")
        if sum(lengths) != rows.numel():
            raise ValueError("request lengths disagree with the flattened rows")
        return lengths

    def read(self, layer: int, rows, consume, *, request_lengths=None):
        """Dense read of complete histories (``rows``: flattened logical ids in request order)."""
        import torch

        lengths = self._validate(rows, request_lengths)
        key = (id(rows), lengths)
        if self.dense is None or self.dense[0] != key:
            flat = rows.reshape(-1).to(torch.int32).contiguous()
            parts = []
            for offset, count in prefill_request_groups(lengths, min(self.capacity, self.reader.bound)):
                part = flat.narrow(0, offset, count)
                parts.append((part, self.reader.prepare_read_plan(part)))
                self.plans_built += 1
            self.dense = (key, rows, parts)
        outs = [self.reader.read_records(layer, part, consume, read_plan=plan) for part, plan in self.dense[2]]
        if not outs:
            raise ValueError("a dense prefill read needs a non-empty history")
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)

    def read_selected(self, layer: int, rows, indices, consume, *, request_lengths=None):
        """Sparse read: ``indices`` int32 [Q, K] point into ``rows`` (-1 = masked).  The union of what they name is
        read once per shared-selection group; returns (records of the union, indices re-based onto it).  When
        the selection is wider than the history the dense read is returned with the indices unchanged."""
        import torch
        from .window import PrefillReadPlan, PrefillRecordWindow, compact_selection

        self._validate(rows, request_lengths)
        if indices.numel() > rows.numel():
            return self.read(layer, rows, consume, request_lengths=request_lengths), indices
        group = self.layer_groups.group(layer)
        key = (group, id(rows), id(indices))
        if self.sparse is None or self.sparse[0] != key:
            flat = rows.reshape(-1)
            named = torch.where(indices >= 0, flat[indices.clamp(min=0).long()].to(torch.int32),
                                torch.full_like(indices, -1, dtype=torch.int32))
            ids, remap, staging = compact_selection(named, None, self.reader._current_ids, id_space=self.reader.id_space)
            if ids.numel() > self.reader.bound:
                raise ValueError("the selection's union exceeds the window bound")
            plan = PrefillReadPlan((PrefillRecordWindow(ids, torch.arange(ids.numel(), dtype=torch.int32, device=ids.device),
                                                        staging),))
            self.sparse = (key, rows, indices, ids, remap, plan)
            self.plans_built += 1
        _, _, _, ids, remap, plan = self.sparse
        if not ids.numel():
            return self.read(layer, rows, consume, request_lengths=request_lengths), indices
        return self.reader.read_records(layer, ids, consume, read_plan=plan), remap
