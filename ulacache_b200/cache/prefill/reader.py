"""Read-only access to cached history during prefill: records are gathered through the directories
into a window without touching residency state (no promotion, no recency update), so a long prefill
cannot evict what decode requests are using.

Reference: ulacache/cache/prefill/reader.py:1-138, cache/kernels/read_only_prefill.py:1-260.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


class ReadOnlyPrefillReader:
    def __init__(self, engine):
        """``engine``: a cache engine exposing ``_pool_view(layer)`` (GPU) or ``read_records`` (CPU)."""
        self.engine = engine

    def fill(self, window, layer: int, union_ids, count):
        """Window rows [0, count) := records of ``union_ids`` for ``layer``.  Returns the number of ids
        that were not readable from this rank (unallocated, or on another rank's host tier)."""
        import torch

        n = int(count)
        if n > window.capacity:
            raise MemoryError("union larger than the window")
        window.layer = layer
        window.ids[:n] = union_ids[:n]
        window.count.fill_(n)
        if window.data.is_cuda:
            from ...ops import prefill as P

            missing = torch.zeros(1, dtype=torch.int32, device=window.data.device)
            P.gather_by_directory(self.engine._pool_view(layer), union_ids[:n].contiguous(), window.data,
                                  missing=missing, status=getattr(self.engine, "status", None))
            window.ready = torch.cuda.Event()
            window.ready.record()
            return missing
        recs, ok = self.engine.read_records(layer, union_ids[:n])
        window.data[:n] = recs
        return int((~ok).sum())


# ----------------------------------------------------------------------------------------------
# Full-history read plan and the two callbacks of the layer pipeline.
#
# A prefill forward reconstructs the complete history of the admitted sequences once per layer:
# cached records are GATHERED read-only into the layer's window, the records the chunk has just
# produced are INSTALLED from the writer's tensors (they win over anything cached under the same
# id).  The plan - distinct ids, where each comes from, and the model's rows rewritten as window
# rows - is computed once per forward and shared by all layers.
#
# Reference: ulacache/cache/prefill/reader.py:12-138 (UnifiedPrefillReadPlan, prepare_read_plan,
# UnifiedPrefillMaterializer.begin / record_current / gather_history / install_current / finish).
# ----------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class HistoryReadPlan:
    record_ids: Any              # int32 [n] ascending distinct ids: row i of the window holds record_ids[i]
    fresh_positions: Any         # int32 [n] index into the chunk's current rows, -1 = read from the cache
    input_record_rows: Any       # int32, shape of the history: its ids as window rows
    current_ids: Any             # int32 [m] ids written by the current chunk

    @property
    def record_count(self) -> int:
        return int(self.record_ids.numel())

    @property
    def keepalive_tensors(self):
        return (self.record_ids, self.fresh_positions, self.input_record_rows, self.current_ids)

    def map_rows(self, ids):
        """Window rows of arbitrary logical ``ids`` (-1 where an id is padding or not part of the plan)."""
        import torch

        ids32 = ids.contiguous().to(torch.int32)
        at = torch.searchsorted(self.record_ids, ids32, out_int32=True)
        safe = at.clamp(max=max(0, self.record_count - 1))
        ok = (ids32 > 0) & (at < self.record_count)
        if self.record_count:
            ok &= self.record_ids[safe.long()] == ids32
        return torch.where(ok, at, torch.full_like(at, -1)).to(torch.int32).contiguous()


def prepare_history_read_plan(full_history_ids, current_ids, *, capacity_records: int = 1 << 20) -> HistoryReadPlan:
    """Compact the COMPLETE history (never a top-k union) plus the chunk's own ids; overlap is removed."""
    import torch
    from .window import compact_selection

    if full_history_ids is None:
        full_history_ids = current_ids.new_empty((0,))
    if full_history_ids.device != current_ids.device or current_ids.ndim != 1 or type(capacity_records) is not int \
            or capacity_records < 1:
        raise ValueError("history and current ids must share a device; the record bound must be positive")
    hist = full_history_ids.reshape(-1).to(torch.int32)
    cur = current_ids.to(torch.int32)
    both = torch.cat((hist, cur)).reshape(1, -1)
    ids, rows, fresh = compact_selection(torch.where(both > 0, both, torch.full_like(both, -1)), None, cur)
    if ids.numel() > capacity_records:
        raise ValueError("the full history exceeds the prefill admission window")
    return HistoryReadPlan(ids, fresh, rows.reshape(-1)[: hist.numel()].reshape(full_history_ids.shape).contiguous(), cur)


class PrefillMaterializer:
    """The two callbacks a layer pipeline needs, over a cache engine.  Ownership of the records stays with the
    cache: nothing here promotes, evicts or changes a directory."""

    def __init__(self, engine):
        self.engine = engine
        self._current = {}
        self.gathered = 0
        self.installed = 0

    def begin(self):
        # copies of an earlier decode step that still run on the side stream must land before records are read
        ev = getattr(self.engine, "_layer_events", None)
        if ev and getattr(self.engine, "is_cuda", False):
            import torch

            for e in set(ev.values()):
                torch.cuda.current_stream().wait_event(e)
        self._current.clear()

    def record_current(self, layer: int, ids, encoded_records):
        """Borrow what the layer's writer has just produced: ``encoded_records`` uint8 [m, record_bytes] for
        ``ids`` [m] (only the most recent layer is kept: a layer that never reads must not pin its payload)."""
        self._current.clear()
        self._current[layer] = (ids, encoded_records)

    def gather_history(self, layer: int, plan: HistoryReadPlan, window):
        """Window rows of every cached record of the plan (rows of fresh records are left for ``install_current``)."""
        import torch

        n = plan.record_count
        if n > window.capacity:
            raise MemoryError("history larger than the window")
        cached = plan.fresh_positions < 0
        window.layer = layer
        window.ids[:n] = plan.record_ids
        window.count.fill_(n)
        if window.data.is_cuda:
            from ...ops import prefill as P

            # one gather over all ids (fresh ones read whatever the cache holds; install_current overwrites them)
            P.gather_by_directory(self.engine._pool_view(layer), plan.record_ids.contiguous(), window.data,
                                  missing=None, status=getattr(self.engine, "status", None))
            window.ready = torch.cuda.Event()
            window.ready.record()
        else:
            ids = plan.record_ids[cached]
            recs, _ = self.engine.read_records(layer, ids)
            window.data[torch.nonzero(cached).reshape(-1)] = recs
        self.gathered += int(cached.sum())

    def install_current(self, layer: int, plan: HistoryReadPlan, window):
        if layer not in self._current:
            raise RuntimeError("the layer's current records must be written before its prefill read")
        import torch

        ids, encoded = self._current.pop(layer)
        fresh = plan.fresh_positions >= 0
        rows = torch.nonzero(fresh).reshape(-1)
        if rows.numel():
            src = plan.fresh_positions[fresh].long()
            if int(src.max()) >= encoded.shape[0]:
                raise ValueError("the plan names more current rows than the writer produced")
            window.data.index_copy_(0, rows, encoded.index_select(0, src))
        self.installed += int(rows.numel())

    def finish(self):
        self._current.clear()
