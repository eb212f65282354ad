"""Capacity planning: how many KV records fit a GPU + host memory budget.

``plan_cache_capacity`` answers the headline "KV tokens admitted at a fixed budget": given
byte budgets for HBM and pinned host memory and a callback that prices a (device tokens, host
tokens) pair completely (payload, directories, recency metadata, index pages, workspaces), it
first maximises the TOTAL number of tokens and then, at that total, the share held in HBM.

Reference: ulacache/storage/capacity.py (request_history_capacity :13,
flowkv_cpu_pool_geometry :67, CacheMemoryUsage/Budget/Plan :90-157, plan_cache_capacity :205,
RecordOwnerCapacity :303, RequiredCachePartitionCapacity :322, RequestNamespaceCapacityBounds :339,
calculate_addressable_history_capacity :403, plan_position_capacity :531).
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Callable

from .layout import INDEX_PAGE_BYTES, PAGE_TOKENS


def request_history_capacity(max_requests: int, topk: int, multiplier: float, page_size: int = PAGE_TOKENS) -> int:
    """Rows of a per-rank pulled-record cache: every query's top-k, times a reuse multiplier
    (at least 3), rounded up to whole pages."""
    if max_requests < 1 or topk < 1 or multiplier < 3:
        raise ValueError("Need positive requests and top-k and a multiplier of at least 3")
    rows = int(max_requests * topk * multiplier)
    return (rows + page_size - 1) // page_size * page_size


def host_pool_geometry(*, device_slots: int, cpu_slots: int = 0, cpu_ratio: float = 2.0,
                       page_size: int = PAGE_TOKENS) -> int:
    """Host slots per owner: explicit ``cpu_slots`` or ``cpu_ratio`` times the device slots, page aligned."""
    slots = cpu_slots if cpu_slots > 0 else int(device_slots * cpu_ratio)
    return slots // page_size * page_size


@dataclass(frozen=True)
class CacheMemoryUsage:
    device_bytes: int
    host_bytes: int


@dataclass(frozen=True)
class CacheMemoryBudget:
    device_bytes: int
    host_bytes: int

    def contains(self, usage: CacheMemoryUsage) -> bool:
        return usage.device_bytes <= self.device_bytes and usage.host_bytes <= self.host_bytes


@dataclass(frozen=True)
class CacheCapacityPlan:
    device_token_capacity_per_owner: int
    host_token_capacity_per_owner: int
    storage_owner_count: int
    usage: CacheMemoryUsage
    budget: CacheMemoryBudget

    def __post_init__(self):
        if self.device_token_capacity_per_owner < 1 or self.host_token_capacity_per_owner < 0 or self.storage_owner_count < 1:
            raise ValueError("A capacity plan needs a positive device capacity and owner count")
        if not self.budget.contains(self.usage):
            raise ValueError("The planned usage exceeds its budget")

    @property
    def token_capacity_per_owner(self) -> int:
        return self.device_token_capacity_per_owner + self.host_token_capacity_per_owner

    @property
    def unique_token_capacity(self) -> int:
        """Tokens the whole group can hold: every record is stored exactly once."""
        return self.token_capacity_per_owner * self.storage_owner_count

    def usable_history_token_capacity(self, page_size: int = PAGE_TOKENS) -> int:
        """One allocation page stays reserved (logical ID 0 is the padding value)."""
        return self.unique_token_capacity - page_size * self.storage_owner_count


def _largest(lo: int, hi: int, ok: Callable[[int], bool]) -> int:
    """Largest v in [lo, hi] with ok(v), given ok is monotone (true then false) and ok(lo)."""
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if ok(mid):
            lo = mid
        else:
            hi = mid - 1
    return lo


def plan_cache_capacity(*, memory_budget: CacheMemoryBudget, measure_memory_usage: Callable[[int, int], CacheMemoryUsage],
                        minimum_device_token_capacity: int, maximum_token_capacity_per_owner: int,
                        page_size: int = PAGE_TOKENS, storage_owner_count: int = 1,
                        minimum_host_token_capacity: int = 0) -> CacheCapacityPlan:
    """Maximise total tokens per owner, then the HBM share at that total.

    ``measure_memory_usage(device_tokens, host_tokens)`` must be monotone: more tokens never cost
    fewer bytes, and moving a page from host to HBM never lowers device bytes nor raises host bytes."""
    if (page_size < 1 or storage_owner_count < 1 or minimum_device_token_capacity < page_size
            or minimum_device_token_capacity % page_size or minimum_host_token_capacity < 0
            or minimum_host_token_capacity % page_size
            or maximum_token_capacity_per_owner < minimum_device_token_capacity + minimum_host_token_capacity):
        raise ValueError("Capacity bounds must be page aligned and leave room for the minimum working set")
    dmin, hmin = minimum_device_token_capacity // page_size, minimum_host_token_capacity // page_size
    tmax = maximum_token_capacity_per_owner // page_size

    @lru_cache(maxsize=None)
    def cost(dev_pages: int, host_pages: int) -> CacheMemoryUsage:
        return measure_memory_usage(dev_pages * page_size, host_pages * page_size)

    def least_device_pages(total: int):
        """Fewest HBM pages such that the rest fits the host budget (None if even all-HBM does not)."""
        hi = total - hmin
        if cost(hi, total - hi).host_bytes > memory_budget.host_bytes:
            return None
        lo = dmin
        while lo < hi:
            mid = (lo + hi) // 2
            if cost(mid, total - mid).host_bytes <= memory_budget.host_bytes:
                hi = mid
            else:
                lo = mid + 1
        return lo

    def total_fits(total: int) -> bool:
        d = least_device_pages(total)
        return d is not None and memory_budget.contains(cost(d, total - d))

    if not total_fits(dmin + hmin):
        raise ValueError("The minimum working set does not fit the memory budget")
    total = _largest(dmin + hmin, tmax, total_fits)
    d_lo = least_device_pages(total)
    dev = _largest(d_lo, total - hmin, lambda d: memory_budget.contains(cost(d, total - d)))
    return CacheCapacityPlan(dev * page_size, (total - dev) * page_size, storage_owner_count,
                             cost(dev, total - dev), memory_budget)


def price_payload_replacement(*, native_device_bytes: int, native_payload_bytes: int, replacement_device_bytes: int,
                              replacement_host_bytes: int, native_host_bytes: int = 0,
                              allocation_plan: CacheCapacityPlan) -> CacheMemoryUsage:
    """What a deployment costs when the pooled cache REPLACES a framework's own KV payload: everything else the
    framework charged on the device (index, request tables, sliding state, allocator headroom) stays, only the
    payload named here is subtracted, and the pool's device and host bytes are added.  The result must fit the usage
    that ``allocation_plan`` was admitted under, or the plan was made with numbers that do not describe this process.

    Reference: ulacache/storage/capacity.py:160-202."""
    values = (native_device_bytes, native_payload_bytes, replacement_device_bytes, replacement_host_bytes, native_host_bytes)
    if any(type(v) is not int or v < 0 for v in values):
        raise ValueError("Byte charges are non-negative integers")
    if native_payload_bytes > native_device_bytes:
        raise ValueError("The replaced payload is part of the native device charge")
    usage = CacheMemoryUsage(native_device_bytes - native_payload_bytes + replacement_device_bytes,
                             native_host_bytes + replacement_host_bytes)
    if usage.device_bytes > allocation_plan.usage.device_bytes or usage.host_bytes > allocation_plan.usage.host_bytes:
        raise ValueError("Native plus replacement charges exceed the usage the allocation plan declared")
    if not allocation_plan.budget.contains(allocation_plan.usage):
        raise ValueError("The allocation plan no longer fits its budget")
    return usage


def residency_workspace_bytes(plan_capacity: int, groups: int, device_slots: int) -> dict:
    """Host-tier transaction workspace of ``groups`` residency groups: the shared plan arrays (five int32 words per
    plan item plus the new / promote / candidate lists: 32 bytes per item), and per group its expiry list (bounded by
    the device slots) and counters."""
    if min(plan_capacity, groups, device_slots) < 1:
        raise ValueError("Workspace dimensions are positive")
    fixed = 32 * plan_capacity + 56 * groups
    expiry = 4 * groups * min(plan_capacity, device_slots)
    return dict(fixed_bytes=fixed, expiry_bytes=expiry, total_bytes=fixed + expiry)


def kv_token_bytes(*, record_bytes: int, layers: int, index_layers: int = 0, metadata_groups: int = 0) -> int:
    """Bytes one resident token costs in a tier: its records in every layer, its share of the
    index pages, and the per-slot metadata of every residency group."""
    index = index_layers * (INDEX_PAGE_BYTES // PAGE_TOKENS)
    metadata = metadata_groups * 5 * 4        # stamp, tag, free-stack entry, directory, promotion time
    return record_bytes * layers + index + metadata


def simple_usage_model(*, record_bytes: int, layers: int, index_layers: int = 0, metadata_groups: int = 0,
                       fixed_device_bytes: int = 0, fixed_host_bytes: int = 0):
    """A linear ``measure_memory_usage`` callback: the index lives in HBM for every token
    (device and host resident alike), payload follows the tier."""
    per_dev = kv_token_bytes(record_bytes=record_bytes, layers=layers, metadata_groups=metadata_groups)
    index = index_layers * (INDEX_PAGE_BYTES // PAGE_TOKENS)
    dir_bytes = metadata_groups * 8

    def measure(device_tokens: int, host_tokens: int) -> CacheMemoryUsage:
        dev = fixed_device_bytes + device_tokens * per_dev + (device_tokens + host_tokens) * (index + dir_bytes)
        host = fixed_host_bytes + host_tokens * record_bytes * layers
        return CacheMemoryUsage(dev, host)

    return measure


def addressable_tokens_per_owner(*, maximum_requests: int, maximum_context_tokens: int, owners: int = 1,
                                 page_size: int = PAGE_TOKENS) -> int:
    """The addressing limit, not a memory limit: int32 logical ids striped over ``owners``, and no more than
    every request at its longest context; whole pages."""
    if min(maximum_requests, maximum_context_tokens, owners, page_size) < 1:
        raise ValueError("Namespace bounds must be positive")
    id_limit = (2 ** 31 - 1) // owners
    need = maximum_requests * maximum_context_tokens // owners
    return min(id_limit, need) // page_size * page_size


@dataclass(frozen=True)
class RecordOwnerCapacity:
    """Cold-record slots of one owner of a partition.  Owners hold disjoint records; ``physical_replica_count``
    copies of an owner hold the same records (they cost memory, they add no capacity)."""

    owner_rank: int
    device_record_capacity: int
    host_record_capacity: int
    physical_replica_count: int = 1

    def __post_init__(self):
        if min(self.device_record_capacity, self.host_record_capacity) < 0 or self.physical_replica_count < 1:
            raise ValueError("Capacities are non-negative and an owner exists at least once")


@dataclass(frozen=True)
class RequiredCachePartitionCapacity:
    """One storage partition that every token of a request namespace needs (the KV tier, a compressed tier, an
    Index tier ...).  The record counts cover all payload banks of the partition: layers and storage aliases do not
    multiply history capacity."""

    request_namespace_id: int
    partition_name: str
    storage_layout: object                       # StorageLayout (name, tokens_per_record)
    record_owners: tuple
    reserved_logical_record_count: int = 0


@dataclass(frozen=True)
class RequestNamespaceCapacityBounds:
    """Token limits of one independent allocation domain that are not storage: what its allocator can hand out,
    and what its request addressing (page tables, int32 ids) can name.  Ranks that share one allocator are ONE
    namespace."""

    request_namespace_id: int
    native_allocator_usable_token_slots: int
    request_address_token_slots: int

    def __post_init__(self):
        if min(self.native_allocator_usable_token_slots, self.request_address_token_slots) < 0:
            raise ValueError("Allocator and address limits are non-negative")


def _partition_account(part: RequiredCachePartitionCapacity) -> dict:
    owners = tuple(part.record_owners)
    if len({o.owner_rank for o in owners}) != len(owners):
        raise ValueError("An owner appears once per partition")
    device = sum(o.device_record_capacity for o in owners)
    host = sum(o.host_record_capacity for o in owners)
    if not 0 <= part.reserved_logical_record_count <= device + host:
        raise ValueError("The reserved records must fit inside the partition")
    per_record = getattr(part.storage_layout, "tokens_per_record", 1)
    return dict(
        request_namespace_id=part.request_namespace_id, partition_name=part.partition_name,
        storage_layout_name=getattr(part.storage_layout, "name", str(part.storage_layout)),
        tokens_per_record=per_record, record_owner_count=len(owners),
        record_owners=[dict(owner_rank=o.owner_rank, device_record_capacity=o.device_record_capacity,
                            host_record_capacity=o.host_record_capacity,
                            physical_replica_count=o.physical_replica_count) for o in owners],
        unique_device_cold_record_slots=device, unique_host_cold_record_slots=host,
        physical_device_cold_record_slots=sum(o.device_record_capacity * o.physical_replica_count for o in owners),
        physical_host_cold_record_slots=sum(o.host_record_capacity * o.physical_replica_count for o in owners),
        reserved_logical_record_count=part.reserved_logical_record_count,
        usable_history_token_slots=(device + host - part.reserved_logical_record_count) * per_record)


def calculate_addressable_history_capacity(required_partitions, namespace_bounds) -> dict:
    """History tokens a deployment can hold, as an audit: per partition the disjoint owners are summed (replicas
    are not); a namespace holds what its SMALLEST required partition holds, capped by its allocator and by its
    addressing; namespaces add up.  This is accounting of allocations: it says nothing about the working set,
    running concurrency or memory peaks."""
    parts = [_partition_account(p) for p in required_partitions]
    bounds = tuple(namespace_bounds)
    ids = {b.request_namespace_id for b in bounds}
    if len(ids) != len(bounds):
        raise ValueError("One bound per request namespace")
    if {p["request_namespace_id"] for p in parts} != ids:
        raise ValueError("Every namespace needs both its partitions and its bounds")
    namespaces = []
    for b in bounds:
        mine = [p for p in parts if p["request_namespace_id"] == b.request_namespace_id]
        cold = min(p["usable_history_token_slots"] for p in mine)
        namespaces.append(dict(
            request_namespace_id=b.request_namespace_id, required_partition_names=[p["partition_name"] for p in mine],
            cold_storage_history_token_slots=cold,
            native_allocator_usable_token_slots=b.native_allocator_usable_token_slots,
            request_address_token_slots=b.request_address_token_slots,
            usable_history_token_slots=min(cold, b.native_allocator_usable_token_slots, b.request_address_token_slots)))
    return dict(required_partitions=parts, request_namespaces=namespaces,
                total_usable_history_token_slots=sum(n["usable_history_token_slots"] for n in namespaces))


def position_residency_bytes(*, tokens: int, record_bytes: int, layers: int, degree: int) -> int:
    """Payload bytes one context-parallel rank holds for ``tokens`` global positions."""
    local = (tokens + degree - 1) // degree
    return local * record_bytes * layers


def plan_position_capacity(*, memory_budget: CacheMemoryBudget, record_bytes: int, layers: int, degree: int,
                           minimum_device_token_capacity: int, maximum_global_tokens: int,
                           index_layers: int = 0, page_size: int = PAGE_TOKENS) -> CacheCapacityPlan:
    """Capacity of a position-sharded (context-parallel) group: each of ``degree`` ranks keeps its
    own HBM + host tier for positions ``p % degree == rank``; the plan is per rank."""
    measure = simple_usage_model(record_bytes=record_bytes, layers=layers, index_layers=index_layers)
    per_rank_max = (maximum_global_tokens + degree - 1) // degree // page_size * page_size
    return plan_cache_capacity(memory_budget=memory_budget, measure_memory_usage=measure,
                               minimum_device_token_capacity=minimum_device_token_capacity,
                               maximum_token_capacity_per_owner=max(per_rank_max, minimum_device_token_capacity),
                               page_size=page_size, storage_owner_count=degree)
