"""Bounded record windows for prefill: union, remap, fresh-row overlay, cross-rank agreement, grouped attention.

Prefill attention does not read the pool.  The distinct records a group of queries selected are gathered ONCE
into a window of bounded size (read-only: no promotion, no recency update), the selection is rewritten as rows
of that window, and attention runs on the window.  This module holds the index side of that:

* :func:`compact_selection` - the ascending union of a [Q, K] selection, the selection as window rows, and for
  every union id the row of the CURRENT chunk's staging buffer when the chunk has just produced that record
  (the fresh copy wins over whatever the cache still holds under the id);
* :func:`shared_union` - all tensor-parallel readers agree on one union (so one residency decision and one
  split decision serve every rank), or report that it exceeds the bound;
* :class:`PrefillReadPlan` - windows computed once per chunk and replayed for every layer of a shared-selection
  group (index tensors only; every layer still gathers its own payload);
* :class:`WindowedPrefillReader` - ``read_records`` (an ordered dense-prefix read through windows of at most
  ``bound`` records, handed window by window to a consumer) and ``attend`` (query groups sized so that
  ``8 * bound / topk`` queries share a window; a group whose union overflows the bound is bisected until it
  fits, a single query that overflows is an error of the startup budget).

Reference: ulacache/cache/prefill/window.py:15-341 (``CompactPrefillRecordWindow``, ``compact_topk_rows``,
``_shared_cpu_union``, ``run_compact_prefill_records``, ``run_compact_prefill_attention``),
cache/kernels/prefix_selection.py:8 (``_union``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Iterator, Optional, Tuple


class SelectionWindowMap:
    def __init__(self, id_space: int, capacity: int):
        self.id_space, self.capacity = int(id_space), int(capacity)
        self._ws = {}

    def build(self, selection, *, status=None):
        """Returns (union_ids int32 [capacity] ascending then -1, count int32 [1], rows like selection)."""
        from ...ops import prefill as P

        return P.selection_union(selection, self.id_space, capacity=self.capacity, workspace=self._ws, status=status)


@dataclass(frozen=True)
class PrefillRecordWindow:
    record_ids: Any        # int32 [n] distinct logical ids, ascending
    output_rows: Any       # int32, shape of the request: window row of every requested id, -1 = masked
    staging_rows: Any      # int32 [n] row of the current chunk's staging buffer, -1 = read from the cache


@dataclass(frozen=True)
class PrefillReadPlan:
    """Windows of one ordered read; valid while the history order and the chunk's write ids stay unchanged."""

    windows: Tuple[PrefillRecordWindow, ...]

    @property
    def records(self) -> int:
        return sum(int(w.output_rows.numel()) for w in self.windows)


def _staging_rows(union_ids, current_ids):
    """For every id of ``union_ids`` (ascending): its position in ``current_ids`` (the LAST one when the chunk
    wrote an id twice), or -1."""
    import torch

    if current_ids is None or current_ids.numel() == 0 or union_ids.numel() == 0:
        return torch.full_like(union_ids, -1)
    cur = current_ids.reshape(-1).to(union_ids.dtype)
    order = torch.argsort(cur, stable=True)
    sorted_cur = cur[order]
    at = torch.searchsorted(sorted_cur, union_ids, right=True) - 1          # last equal element
    safe = at.clamp(min=0)
    hit = (at >= 0) & (sorted_cur[safe] == union_ids)
    return torch.where(hit, order[safe].to(torch.int32), torch.full_like(union_ids, -1)).to(torch.int32).contiguous()


def compact_selection(selection, lengths=None, current_ids=None, *, id_space: int = 0, workspace=None):
    """``selection`` int32 [Q, K] of logical ids (negative = masked; columns at or beyond ``lengths[q]`` are
    masked too).  Returns (ids int32 [n] ascending, rows int32 [Q, K], staging int32 [n]).

    On CUDA with a known ``id_space`` the union runs in the flag / scan / scatter kernel of
    ``ops.prefill.selection_union``; otherwise (CPU, tests) it is ``torch.unique`` + ``searchsorted``."""
    import torch

    sel = selection.to(torch.int32)
    if sel.ndim != 2:
        raise ValueError("a selection is [queries, width]")
    if lengths is not None:
        cols = torch.arange(sel.shape[1], device=sel.device)[None, :]
        sel = torch.where(cols < lengths.reshape(-1, 1).to(sel.device), sel, torch.full_like(sel, -1))
    live = sel >= 0
    if sel.is_cuda and id_space > 0:
        from ...ops import prefill as P

        cap = min(int(sel.numel()), id_space)
        ids_full, count, rows = P.selection_union(sel.contiguous(), id_space, capacity=cap, workspace=workspace)
        ids = ids_full[: int(count)].contiguous()
    else:
        ids = torch.unique(sel[live], sorted=True).to(torch.int32)
        rows = torch.searchsorted(ids, sel.contiguous().clamp(min=0), out_int32=True) if ids.numel() else \
            torch.zeros_like(sel)
        rows = torch.where(live, rows, torch.full_like(rows, -1)).to(torch.int32).contiguous()
    return ids, rows, _staging_rows(ids, current_ids)


def shared_union(ids, rows, staging, current_ids, *, group=None, world: int = 1, bound: int):
    """One union for all ``world`` readers: every rank contributes its ids, all end with the same ascending
    list, ``rows`` is re-based onto it and ``staging`` recomputed.  Returns None when the joint union exceeds
    ``bound`` (the caller bisects its query group; all ranks take the same branch because the sizes agree)."""
    import torch
    import torch.distributed as dist

    if world == 1 or group is None:
        return (ids, rows, staging) if ids.numel() <= bound else None
    largest = torch.tensor([ids.numel()], dtype=torch.int64, device=ids.device)
    dist.all_reduce(largest, op=dist.ReduceOp.MAX, group=group)
    width = int(largest.item())
    if width > bound:
        return None
    if width == 0:
        return ids, rows, staging
    send = torch.full((width,), -1, dtype=torch.int32, device=ids.device)
    send[: ids.numel()] = ids
    if ids.is_cuda:
        recv = torch.empty(world * width, dtype=torch.int32, device=ids.device)
        dist.all_gather_into_tensor(recv, send, group=group)
    else:
        parts = [torch.empty_like(send) for _ in range(world)]
        dist.all_gather(parts, send, group=group)
        recv = torch.cat(parts)
    joint = torch.unique(recv[recv >= 0], sorted=True).to(torch.int32)
    if joint.numel() > bound:
        return None
    if ids.numel():
        to_joint = torch.searchsorted(joint, ids, out_int32=True)
        rows = torch.where(rows >= 0, to_joint[rows.clamp(min=0).long()], torch.full_like(rows, -1)).contiguous()
    return joint, rows, _staging_rows(joint, current_ids)


class WindowedPrefillReader:
    """Reads cached history (and the chunk's own fresh records) through one bounded window.

    ``reader``: a :class:`~ulacache_b200.cache.prefill.reader.ReadOnlyPrefillReader`; ``window``: a
    :class:`~ulacache_b200.cache.prefill.buffers.PrefillWindow` of at least ``bound`` rows.  ``group`` /
    ``world``: the tensor-parallel readers that must agree on every union.  ``id_space``: logical id space
    (enables the union kernel on CUDA)."""

    def __init__(self, reader, window, *, bound: Optional[int] = None, group=None, world: int = 1, id_space: int = 0,
                 leases=None):
        self.reader, self.window = reader, window
        self.bound = int(bound if bound is not None else window.capacity)
        if not 0 < self.bound <= window.capacity:
            raise ValueError("the window bound must be positive and fit the window")
        self.group, self.world, self.id_space = group, world, id_space
        self.leases = leases
        self._ws = {}
        self._current_ids = None
        self._staging = None
        self.fills = 0
        self.missing = 0

    # ------------------------------------------------------------ current chunk --
    def set_current_chunk(self, ids, staging_records):
        """The chunk being prefilled has produced ``staging_records`` uint8 [n, record_bytes] for logical
        ``ids`` [n]; reads of those ids take the staging row, not the cache."""
        if ids is not None and ids.numel() != (0 if staging_records is None else staging_records.shape[0]):
            raise ValueError("one staging row per current id")
        self._current_ids, self._staging = ids, staging_records

    def clear_current_chunk(self):
        self._current_ids = self._staging = None

    # ------------------------------------------------------------------- windows --
    def _window_for(self, ids_2d, lengths=None):
        ids, rows, staging = compact_selection(ids_2d, lengths, self._current_ids, id_space=self.id_space,
                                               workspace=self._ws)
        joined = shared_union(ids, rows, staging, self._current_ids, group=self.group, world=self.world,
                              bound=self.bound)
        if joined is None:
            return None
        return PrefillRecordWindow(*joined)

    def prepare_read_plan(self, ids) -> PrefillReadPlan:
        """Windows for an ordered read of ``ids`` (any shape, flattened), computed once and reused for every
        layer that reads the same history."""
        import torch

        flat = ids.reshape(-1).to(torch.int32)
        if not flat.numel():
            raise ValueError("an ordered prefix read needs at least one id")
        if bool((flat < 0).any()):
            raise ValueError("an ordered prefix read takes valid ids only")
        windows = []
        for part in flat.split(self.bound):
            w = self._window_for(part.reshape(1, -1))
            if w is None:
                raise ValueError("the joint union of an ordered read exceeds the window bound")
            # own compact copies: nothing may alias a sort or collective workspace larger than its view
            windows.append(PrefillRecordWindow(w.record_ids.clone(), w.output_rows.reshape(-1).clone(),
                                               w.staging_rows.clone()))
        return PrefillReadPlan(tuple(windows))

    def _fill(self, layer: int, w: PrefillRecordWindow):
        import torch

        win = self.window
        if self.leases is not None:
            self.leases.check_refill(win)
        n = int(w.record_ids.numel())
        if n:
            miss = self.reader.fill(win, layer, w.record_ids, n)
            fresh = w.staging_rows >= 0
            if self._staging is not None and bool(fresh.any()):
                dst = torch.nonzero(fresh).reshape(-1)
                if win.data.is_cuda:
                    # the overlay must follow the gather on the stream that the consumer will wait on
                    if win.ready is not None:
                        torch.cuda.current_stream().wait_event(win.ready)
                    win.data.index_copy_(0, dst, self._staging.index_select(0, w.staging_rows[fresh].long()))
                    win.ready = torch.cuda.Event()
                    win.ready.record()
                else:
                    win.data[dst] = self._staging[w.staging_rows[fresh].long()]
            self.missing = miss
        else:
            win.count.fill_(0)
        self.fills += 1
        return win

    # --------------------------------------------------------------------- reads --
    def read_records(self, layer: int, ids, consume: Callable, *, output_buffer=None,
                     read_plan: Optional[PrefillReadPlan] = None):
        """Materialise the records of ``ids`` IN ORDER through windows of at most ``bound`` records.
        ``consume(window_records uint8 [capacity, record_bytes], rows int32 [m])`` returns a tensor with one
        leading row per requested id (e.g. dequantised latents); the results are concatenated.  With
        ``output_buffer`` it is called as ``consume(window_records, rows, destination_slice)`` and writes in
        place."""
        import torch

        plan = read_plan if read_plan is not None else self.prepare_read_plan(ids)
        if plan.records != int(ids.numel()):
            raise ValueError("the read plan was prepared for a different number of ids")
        outputs, at = [], 0
        for w in plan.windows:
            win = self._fill(layer, w)
            if win.data.is_cuda and win.ready is not None:
                torch.cuda.current_stream().wait_event(win.ready)
            m = int(w.output_rows.numel())
            if output_buffer is None:
                outputs.append(consume(win.data, w.output_rows))
            else:
                consume(win.data, w.output_rows, output_buffer.narrow(0, at, m))
            at += m
        if output_buffer is not None:
            return output_buffer
        return torch.cat(outputs, dim=0) if len(outputs) > 1 else outputs[0]

    def _groups(self, selection, lengths, start: int, stop: int) -> Iterator:
        w = self._window_for(selection[start:stop], None if lengths is None else lengths[start:stop])
        if w is None:
            if stop - start == 1:
                raise RuntimeError("one query's complete selection exceeds the reserved window")
            mid = (start + stop) // 2
            yield from self._groups(selection, lengths, start, mid)
            yield from self._groups(selection, lengths, mid, stop)
        else:
            yield start, stop, w

    def attend(self, layer: int, query, selection, lengths, attend_fn: Callable, *, topk: Optional[int] = None,
               max_queries: Optional[int] = None):
        """Attention over complete query groups that share one window.
        ``attend_fn(query_slice, rows int32 [q, K], window_records, lengths_slice)`` returns a tensor whose
        leading dimension is its query count.  Groups hold up to ``8 * bound / topk`` queries (at most
        ``max_queries``); a group whose union overflows the bound is bisected."""
        import torch

        if selection.ndim != 2 or selection.dtype != torch.int32 or selection.device != query.device:
            raise ValueError("queries and their int32 [Q, K] selection must sit on one device")
        if query.shape[0] != selection.shape[0] or (lengths is not None and lengths.numel() != selection.shape[0]):
            raise ValueError("query, selection and lengths disagree on the number of queries")
        k = int(topk if topk is not None else selection.shape[1])
        if selection.shape[1] != k:
            raise ValueError("the selection width disagrees with the budgeted top-k")
        if self.bound < k:
            raise ValueError("the window cannot hold one complete selection")
        if not query.shape[0]:
            return query
        if max_queries is not None and query.shape[0] > max_queries:
            raise ValueError("more prefill queries than the startup bound")
        group_queries = max(1, 8 * self.bound // k)
        if max_queries is not None:
            group_queries = min(group_queries, max_queries)
        lens = None if lengths is None else lengths.reshape(-1)
        outputs = []
        for g0 in range(0, query.shape[0], group_queries):
            g1 = min(g0 + group_queries, query.shape[0])
            for first, last, w in self._groups(selection, lens, g0, g1):
                win = self._fill(layer, w)
                if win.data.is_cuda and win.ready is not None:
                    torch.cuda.current_stream().wait_event(win.ready)
                outputs.append(attend_fn(query[first:last], w.output_rows, win.data,
                                         None if lens is None else lens[first:last].contiguous()))
        return torch.cat(outputs, dim=0) if len(outputs) > 1 else outputs[0]
