"""Byte budget of a tensor-parallel pool: what is charged against the GPU budget besides the
striped record shards (pulled-record cache, prefill windows, staging, lookup metadata), and the
lifetime colouring that lets attention workspaces of different layer groups share memory.

Reference: FlowKVLayout (ulacache/storage/workspace.py:28, report :243), PlainPrefillLayout
:307, AttentionWorkspaceLifetime :387 and its colouring at :399.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

from .capacity import request_history_capacity
from .layout import PAGE_TOKENS


@dataclass(frozen=True)
class PoolLayout:
    layers: int
    groups: int                     # shared-selection layer groups
    record_bytes: int
    slots_per_rank: int             # striped shard rows per layer on this rank
    max_queries: int
    topk: int
    cache_multiplier: float = 3.0   # pulled-record cache rows = queries * topk * multiplier (0 = none)
    prefill_window_rows: int = 0
    prefill_windows: int = 2
    staging_rows: int = 8192
    pulled_record_cache: bool = False

    def __post_init__(self):
        if min(self.layers, self.groups, self.record_bytes, self.slots_per_rank, self.max_queries, self.topk) < 1:
            raise ValueError("Pool geometry must be positive")
        if self.slots_per_rank % PAGE_TOKENS:
            raise ValueError("slots_per_rank must be a whole number of pages")
        w = self.prefill_window_rows
        if w and (w < 2048 or w % PAGE_TOKENS):
            raise ValueError("prefill_window_rows must be 0 or a page multiple of at least 2048")

    @property
    def shard_bytes(self) -> int:
        return self.layers * self.slots_per_rank * self.record_bytes

    @property
    def cache_rows(self) -> int:
        if not self.pulled_record_cache:
            return 0
        return request_history_capacity(self.max_queries, self.topk, self.cache_multiplier)

    @property
    def cache_bytes(self) -> int:
        return self.groups * self.cache_rows * self.record_bytes

    @property
    def prefill_buffer_bytes(self) -> int:
        return self.prefill_windows * self.prefill_window_rows * self.record_bytes

    @property
    def staging_bytes(self) -> int:
        return self.staging_rows * self.record_bytes

    @property
    def selected_bytes(self) -> int:
        return self.groups * self.max_queries * self.topk * 4 * 2      # selection + resolved locations

    @property
    def metadata_bytes(self) -> int:
        per_slot = 5 * 4
        return self.groups * (self.slots_per_rank * per_slot + self.cache_rows * 3 * 4)

    def report(self) -> Dict[str, int]:
        parts = {"record_shards": self.shard_bytes, "pulled_record_cache": self.cache_bytes,
                 "prefill_windows": self.prefill_buffer_bytes, "write_staging": self.staging_bytes,
                 "selections": self.selected_bytes, "metadata": self.metadata_bytes}
        parts["total"] = sum(parts.values())
        return parts


@dataclass(frozen=True)
class AttentionWorkspaceLifetime:
    """Interval [first_layer, last_layer] during which a group's attention workspace is live."""

    group: int
    first_layer: int
    last_layer: int


def colour_workspaces(lifetimes: Sequence[AttentionWorkspaceLifetime]) -> Tuple[List[int], int]:
    """Greedy interval colouring: groups whose lifetimes do not overlap share a workspace.
    Returns (colour per lifetime in input order, number of colours)."""
    order = sorted(range(len(lifetimes)), key=lambda i: (lifetimes[i].first_layer, lifetimes[i].last_layer))
    free_at: List[int] = []          # colour -> layer after which it is free
    colours = [0] * len(lifetimes)
    for i in order:
        lt = lifetimes[i]
        for c, end in enumerate(free_at):
            if end < lt.first_layer:
                colours[i] = c
                free_at[c] = lt.last_layer
                break
        else:
            colours[i] = len(free_at)
            free_at.append(lt.last_layer)
    return colours, len(free_at)


CacheLayout = PoolLayout                     # the name the reference exports for a pool's byte layout


@dataclass(frozen=True)
class ResidentQueryLayout(PoolLayout):
    """A pool whose big buffers are sized from the number of REAL queries that can be resident, not from the
    power-of-two bound that per-query metadata is padded to.  ``max_queries`` stays that padded bound (a power of
    two, at most 2048); ``max_resident_queries`` (0 = the padded bound) is what the pulled-record cache and the
    selections are sized for.

    Reference: ulacache/storage/workspace.py:263-305."""

    max_resident_queries: int = 0

    def __post_init__(self):
        super().__post_init__()
        q = self.max_queries
        if not 0 < q <= 2048 or q & (q - 1):
            raise ValueError("Per-query metadata is padded to a power of two of at most 2048")
        if not 0 <= self.max_resident_queries <= q:
            raise ValueError("Resident queries cannot exceed the metadata bound")

    @property
    def resident_query_capacity(self) -> int:
        return self.max_resident_queries or self.max_queries

    @property
    def cache_rows(self) -> int:
        if not self.pulled_record_cache:
            return 0
        return request_history_capacity(self.resident_query_capacity, self.topk, self.cache_multiplier)

    @property
    def selected_bytes(self) -> int:
        return self.groups * self.resident_query_capacity * self.topk * 4 * 2

    @property
    def rows_per_layer(self) -> int:
        """Pulled-record rows plus one current record per resident query, whole pages."""
        rows = self.cache_rows + self.resident_query_capacity
        return (rows + PAGE_TOKENS - 1) // PAGE_TOKENS * PAGE_TOKENS
