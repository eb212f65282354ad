"""Tensor-parallel attention engine: queries and selections are replicated on every
rank, KV is stored ONCE, striped over the ranks by 64-token page.

Each rank runs the residency transaction for the records it owns (it sees the
same selection as everybody else, so no miss lists travel), a cross-rank barrier
follows, and every rank then resolves the full selection by reading the owners'
directories.  The attention kernel reads selected records straight from the
owners' HBM pools: there is no local copy of remote KV.

The reference instead keeps a per-rank *attention buffer* that caches pulled
records (ulacache/cache/tp_cache.py:389-519, ulacache/csrc/cache/common.cuh:1037);
`PulledRecordCache` below offers the same behaviour as an option for links slower
than NVLink 5.

Reference: NativeTensorParallelExecution (ulacache/cache/tensor_parallel.py:13),
configure_pool (ulacache/cache/tp_cache.py:30).
"""
from __future__ import annotations

from .engine import CacheEngine, CollectiveTransport, P2PTransport


class TensorParallelResidency(CacheEngine):
    def __init__(self, spec, bindings):
        import torch

        device = torch.device(bindings.device)
        world, rank = bindings.world_size, bindings.rank
        transport = heap = None
        want = bindings.transport
        if want == "auto":
            want = "p2p" if device.type == "cuda" and world > 1 else "collective"
        if world > 1 and want == "p2p":
            from ..parallel.symmetric import SymmetricHeap

            heap = bindings.pool if bindings.pool is not None else SymmetricHeap(
                cpu_group=bindings.process_group, rank=rank, world_size=world,
                nbytes=self.required_heap_bytes(spec), device=device)
            transport = P2PTransport(heap)
        elif world > 1:
            transport = CollectiveTransport(bindings.process_group, rank, world)
        self._owns_heap = heap is not None and bindings.pool is None
        opts = bindings.execution_options
        super().__init__(spec, device=device, owners=bindings.owners, my_rank=rank, transport=transport,
                         heap=heap, options=opts, host_pool_factory=bindings.allocate_host_record_storage,
                         replicated_selections=True)
        self.cache_options = bindings.options

    @staticmethod
    def required_heap_bytes(spec) -> int:
        cap = spec.capacity_plan
        layers = spec.layer_reuse.unique_key_value_storage_count
        planes = sum(p.bytes_per_record for p in spec.storage_layout.record_planes)
        groups = spec.layer_reuse.residency_groups().group_count
        directory = (cap.logical_record_capacity + 8 * 64 + 64) * 4 * groups * 2
        return layers * planes * cap.device_record_capacity + directory + (1 << 20)

    def close(self):
        super().close()
        if self._owns_heap and self.heap is not None:
            self.heap.close()
            self.heap = None


class PulledRecordCache:
    """Optional per-rank cache of records pulled from peers, keyed by global ID, with
    step-age replacement (the reference's attention buffer, ulacache/cache/attention_buffers.py:30).
    Capacity is ``max_queries * topk * multiplier`` rows (multiplier >= 3).

    State is three tensors on ``device`` (``tags``: id held by each row or -1, ``pins``: step of last use,
    ``storage``: the rows); lookup is a sort + binary search over the tags and victim selection a masked sort, so a
    step costs a handful of tensor operations whatever the number of ids."""

    def __init__(self, *, record_bytes: int, max_queries: int, topk: int, multiplier: float = 3.0,
                 policy: str = "age_lru", device="cpu"):
        import torch

        if multiplier < 3:
            raise ValueError("The pulled-record cache needs a capacity multiplier of at least 3")
        if policy not in ("age_lru", "circular"):
            raise ValueError("policy must be age_lru or circular")
        self.capacity = (int(max_queries * topk * multiplier) + 63) // 64 * 64
        self.policy = policy
        self.device = torch.device(device)
        self.storage = torch.zeros((self.capacity, record_bytes), dtype=torch.uint8, device=device)
        self.tags = torch.full((self.capacity,), -1, dtype=torch.int64, device=device)
        self.pins = torch.zeros(self.capacity, dtype=torch.int64, device=device)
        self.step = 0
        self.hand = 0
        self.hits = self.misses = 0

    def begin_step(self):
        self.step += 1

    def _find(self, ids):
        """Row of each id, -1 where the id is not cached."""
        import torch

        order = torch.argsort(self.tags)
        ordered = self.tags[order]
        at = torch.searchsorted(ordered, ids).clamp(max=self.capacity - 1)
        return torch.where(ordered[at] == ids, order[at], torch.full_like(at, -1))

    def lookup(self, ids):
        """Return (slots, miss_mask) for a flat list (or tensor) of global IDs; hits are pinned."""
        import torch

        ids = torch.as_tensor(ids, dtype=torch.int64, device=self.device).reshape(-1)
        slots = self._find(ids)
        hit = slots >= 0
        self.pins[slots[hit]] = self.step
        self.hits += int(hit.sum())
        return slots, ~hit

    def _victims(self, n: int):
        """``n`` replaceable rows: free rows first, then unpinned rows oldest first (age policy) or in ring order
        behind the hand (circular policy).  Rows used in the current step are never taken."""
        import torch

        free = (self.tags < 0).nonzero().flatten()[:n]
        need = n - free.numel()
        if need == 0:
            return free
        usable = (self.tags >= 0) & (self.pins != self.step)
        if int(usable.sum()) < need:
            raise MemoryError("every cached row is pinned by the current step")
        if self.policy == "circular":
            ring = (torch.arange(self.capacity, device=self.device) + self.hand) % self.capacity
            taken = ring[usable[ring]][:need]
            self.hand = (int(taken[-1]) + 1) % self.capacity
        else:
            age_key = torch.where(usable, self.pins, torch.full_like(self.pins, torch.iinfo(torch.int64).max))
            taken = torch.argsort(age_key, stable=True)[:need]
        return torch.cat([free, taken])

    def allocate(self, miss_ids):
        """Assign a row to every missed ID (each distinct id once) and return the rows in the order given."""
        import torch

        ids = torch.as_tensor(miss_ids, dtype=torch.int64, device=self.device).reshape(-1)
        if ids.numel() == 0:
            return []
        have = self._find(ids)
        fresh = torch.unique(ids[have < 0])
        if fresh.numel():
            rows = self._victims(int(fresh.numel()))
            self.tags[rows] = fresh
            self.misses += int(fresh.numel())
            have = self._find(ids)
        self.pins[have] = self.step
        return have.tolist()

    def fill(self, rows, records):
        """Store pulled records in their assigned rows."""
        import torch

        self.storage[torch.as_tensor(rows, dtype=torch.int64, device=self.device)] = records.to(self.device)

    def read(self, rows):
        import torch

        return self.storage[torch.as_tensor(rows, dtype=torch.int64, device=self.device)]
