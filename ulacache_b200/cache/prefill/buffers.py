"""Windows of encoded records that prefill attention reads instead of the pool.

A window holds up to ``capacity`` records (1,048,576 by default in the reference's setup) of one
layer, each distinct record once.  Two of them alternate per layer so that the window of layer
l + 1 fills on a side stream while layer l computes.

Reference: ulacache/cache/prefill/buffers.py:1-413 (two 1,048,576-record encoded windows,
cross-rank agreement on the union size :155-168).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

DEFAULT_WINDOW_RECORDS = 1 << 20


class PrefillWindow:
    def __init__(self, capacity: int, record_bytes: int, device):
        import torch

        self.capacity, self.record_bytes = int(capacity), int(record_bytes)
        self.data = torch.zeros((self.capacity, self.record_bytes), dtype=torch.uint8, device=device)
        self.ids = torch.full((self.capacity,), -1, dtype=torch.int32, device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)     # on the device: graph friendly
        self.layer = -1
        self.ready = None          # CUDA event recorded when the fill finished

    @property
    def nbytes(self) -> int:
        return self.data.numel()

    def rows(self) -> int:
        return int(self.count)


class PrefillWindowPair:
    """Double buffer: ``current`` is read by attention, ``next`` is being filled."""

    def __init__(self, capacity: int, record_bytes: int, device):
        self.windows = [PrefillWindow(capacity, record_bytes, device) for _ in range(2)]
        self._turn = 0

    @property
    def current(self) -> PrefillWindow:
        return self.windows[self._turn]

    @property
    def next(self) -> PrefillWindow:
        return self.windows[self._turn ^ 1]

    def swap(self):
        self._turn ^= 1

    @property
    def nbytes(self) -> int:
        return sum(w.nbytes for w in self.windows)


def agree_on_union_size(count, group=None, world: int = 1) -> int:
    """Every rank must size its window for the largest union among the ranks."""
    import torch
    import torch.distributed as dist

    if world == 1 or group is None:
        return int(count)
    t = torch.tensor([int(count)], dtype=torch.int64)
    if hasattr(count, "is_cuda") and count.is_cuda:
        t = t.to(count.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t)


# ----------------------------------------------------------------------------------------------
# Request-group prefill: the queries of a forward are cut into groups (whole requests, at most
# `query_chunk` queries, bisected while the union of a group's complete selections exceeds the
# window), and the two windows alternate between GROUPS: the copy of group g + 1 runs on the
# side stream while attention reads group g.
#
# Reference: ulacache/cache/prefill/buffers.py:13-81 (PrefillQueryGroup, request_query_ranges,
# prepare_query_groups), :239-413 (RequestPrefillBuffers.begin_forward / select / run /
# read_records / inventory).
# ----------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class PrefillQueryGroup:
    request: int
    start: int
    stop: int
    records: Any          # int32 [n] ascending distinct logical ids of the group
    indices: Any          # int32 [stop - start, K] window rows of the group's selection (-1 masked)


def request_query_ranges(query_counts, query_count: int):
    """((request, first query, last query + 1), ...) in the model's request order; empty requests are skipped."""
    if query_counts is None:
        raise ValueError("request-group prefill needs the per-request query counts")
    counts = tuple(query_counts)
    if any(type(c) is not int or c < 0 for c in counts) or sum(counts) != query_count:
        raise ValueError("the request query counts must partition the query tensor")
    out, start = [], 0
    for request, count in enumerate(counts):
        if count:
            out.append((request, start, start + count))
        start += count
    return tuple(out)


def prepare_query_groups(selected, query_counts, capacity: int, *, query_chunk: int = 256, union=None):
    """Groups whose complete selections fit ``capacity`` distinct records.  ``union``: optional callable that maps a
    group's ids to the ids all tensor-parallel readers agree on (it may only add ids)."""
    import torch
    from .window import compact_selection

    if type(capacity) is not int or capacity < 1 or type(query_chunk) is not int or query_chunk < 1:
        raise ValueError("record and query bounds must be positive integers")
    if selected.ndim != 2 or selected.dtype not in (torch.int32, torch.int64):
        raise ValueError("selections are a two-dimensional integer tensor")

    def split(request, start, stop):
        ids, rows, _ = compact_selection(torch.where(selected[start:stop] > 0, selected[start:stop],
                                                     torch.full_like(selected[start:stop], -1)))
        if union is not None:
            joint = union(ids)
            if joint.numel() != ids.numel():
                to_joint = torch.searchsorted(joint, ids, out_int32=True)
                rows = torch.where(rows >= 0, to_joint[rows.clamp(min=0).long()], torch.full_like(rows, -1))
                ids = joint
        if ids.numel() > capacity:
            if stop - start == 1:
                raise ValueError("one query's complete selection exceeds the prefill window")
            mid = (start + stop) // 2
            yield from split(request, start, mid)
            yield from split(request, mid, stop)
            return
        yield PrefillQueryGroup(request, start, stop, ids, rows.contiguous())

    out = []
    for request, first, last in request_query_ranges(query_counts, selected.shape[0]):
        for start in range(first, last, query_chunk):
            out.extend(split(request, start, min(last, start + query_chunk)))
    return tuple(out)


class RequestPrefillBuffers:
    """Two reusable windows shared by every layer and request group of a forward.

    ``reader``: a :class:`~ulacache_b200.cache.prefill.reader.ReadOnlyPrefillReader` (copies never promote,
    evict or touch recency).  ``attend(query_slice, window_records, rows)`` gets the group's queries, the window
    (uint8 [capacity, record_bytes]) and the selection as window rows, and returns one output row per query."""

    def __init__(self, reader, record_bytes: int, record_capacity: int, device, *, query_chunk: int = 256,
                 prefetch: bool = True, union=None):
        import torch

        if type(record_capacity) is not int or record_capacity < 1:
            raise ValueError("the window's record capacity must be positive")
        self.reader, self.record_capacity, self.query_chunk, self.union = reader, record_capacity, query_chunk, union
        self.pair = PrefillWindowPair(record_capacity, record_bytes, device)
        self.cuda = torch.device(device).type == "cuda"
        self.prefetch = prefetch and self.cuda
        self.stream = torch.cuda.Stream(device=device) if self.prefetch else None
        self.retired = [None, None]                  # event after the last attention that read the window
        self.pending_layer = None
        self.query_counts = None
        self.copy_count = self.group_count = self.maximum_union = 0

    def begin_forward(self, query_counts):
        if self.pending_layer is not None:
            raise RuntimeError("consume the pending prefill selection before starting another forward")
        self.query_counts = None if query_counts is None else tuple(int(c) for c in query_counts)

    def select(self, layer: int, ids):
        if self.pending_layer is not None:
            raise RuntimeError("consume the previous prefill selection before replacing it")
        self.pending_layer = layer
        return ids

    def _copy(self, layer, group, slot):
        import torch

        window = self.pair.windows[slot]
        if self.prefetch:
            main = torch.cuda.current_stream()
            self.stream.wait_stream(main)
            with torch.cuda.stream(self.stream):
                group.records.record_stream(self.stream)
                if self.retired[slot] is not None:
                    self.stream.wait_event(self.retired[slot])      # the window's previous readers are done
                self.reader.fill(window, layer, group.records, int(group.records.numel()))
        else:
            self.reader.fill(window, layer, group.records, int(group.records.numel()))
        self.copy_count += int(group.records.numel())
        self.maximum_union = max(self.maximum_union, int(group.records.numel()))

    def run(self, queries, selected, attend):
        import torch

        if self.cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("request prefill buffers run eagerly")
        if self.pending_layer is None:
            raise RuntimeError("select() the layer's ids before its attention")
        layer = self.pending_layer
        groups = prepare_query_groups(selected, self.query_counts, self.record_capacity, query_chunk=self.query_chunk,
                                      union=self.union)
        outputs = []
        if groups:
            self._copy(layer, groups[0], 0)
        for i, g in enumerate(groups):
            slot = i % 2
            window = self.pair.windows[slot]
            if self.cuda and window.ready is not None:
                torch.cuda.current_stream().wait_event(window.ready)
            if i + 1 < len(groups):
                self._copy(layer, groups[i + 1], (i + 1) % 2)
            out = attend(queries[g.start:g.stop], window.data, g.indices)
            if out.shape[0] != g.stop - g.start:
                raise ValueError("the attention callback must return one row per query, in query order")
            outputs.append(out)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record()
                self.retired[slot] = ev
            self.group_count += 1
        self.pending_layer = None
        return torch.cat(outputs, dim=0) if outputs else queries.new_empty(queries.shape)

    def read_records(self, layer: int, records, read_native):
        """A complete prefix as ONE selection (no query splitting): ``read_native(window_records, rows)`` returns
        independent rows before the window retires.  The forward's request partition is kept for later layers."""
        if records.ndim != 1:
            raise ValueError("a prefix read takes one-dimensional logical ids")
        counts = self.query_counts
        sel = records.reshape(1, -1)
        self.select(layer, sel)
        self.query_counts = (1,)
        try:
            return self.run(sel, sel, lambda q, data, rows: read_native(data, rows.reshape(-1)).unsqueeze(0))[0]
        finally:
            self.query_counts = counts

    def inventory(self) -> dict:
        return {w.data.untyped_storage().data_ptr(): w.data.untyped_storage().nbytes() for w in self.pair.windows}

    def close(self):
        if self.stream is not None:
            self.stream.synchronize()
        for ev in self.retired:
            if ev is not None:
                ev.synchronize()
