"""Choose and build the execution engine for a specification + bindings pair.

Reference: ulacache/cache/create.py:10-45 (prefetch policy checks), :47-87 (one of four engines plus the
context-parallel wrapper), :90-116 (position-owner geometry checks).
"""
from __future__ import annotations

from ..bindings import (LocalCacheBindings, PositionShardBindings, RecordOwnerBindings,
                        TensorParallelCacheBindings)


def validate_prefetch_configuration(spec, bindings):
    """Refuse start-up policies that cannot do what they say, before any device memory is allocated.
    Asynchronous follower copies move the records of a selection group's follower layers on a side stream while
    the anchor layer computes: without a shared selection group there is no follower, and a prefetch policy on
    top of that would silently do nothing.  Per-layer completion needs every layer to own its KV storage (aliased
    storage completes with its owner)."""
    options = getattr(bindings, "execution_options", None)
    if options is None or not options.copy_follower_records_asynchronously:
        return
    sharing = spec.layer_reuse
    owners = tuple(sharing.sparse_selection_owners)
    if all(layer == owner for layer, owner in enumerate(owners)):
        raise ValueError("asynchronous follower copies need at least one shared selection group: "
                         "every layer here selects for itself, so there is nothing to copy ahead")
    if options.follower_copy_mode == "layer":
        if tuple(sharing.key_value_storage_owners) != tuple(range(sharing.layer_count)):
            raise NotImplementedError("per-layer follower completion needs every layer to own its KV storage")


def validate_position_configuration(spec, bindings):
    """Geometry a position-sharded (context-parallel) cache supports: one record plane in 64-record pages, more
    than one rank, and a selection bound that fits the rank's device tier (each rank makes its share of every
    selection resident at once)."""
    storage = spec.storage_layout
    if len(storage.record_planes) != 1 or storage.records_per_page != 64:
        raise NotImplementedError("position sharding binds one record plane in 64-record pages")
    if bindings.position_layout.ranks < 2:
        raise ValueError("position sharding over one rank is the rank-local cache: bind LocalCacheBindings")
    access, capacity = spec.sparse_access, spec.capacity_plan
    share = -(-access.maximum_selected_record_count // bindings.position_layout.ranks)
    if access.maximum_padded_query_count * share > capacity.device_record_capacity:
        raise ValueError("a rank's share of one step's selections does not fit its device tier")


def create_execution_engine(spec, bindings):
    from .local_cache import UnifiedLocalResidency
    from .local_paged_cache import NativePagedResidency
    from .owner_cache import RecordOwnerPagedResidency
    from .position_residency import PositionShardedResidency
    from .tensor_parallel import TensorParallelResidency

    validate_prefetch_configuration(spec, bindings)
    if isinstance(bindings, PositionShardBindings):
        validate_position_configuration(spec, bindings)
        inner = _local(spec, bindings, UnifiedLocalResidency, NativePagedResidency)
        return PositionShardedResidency(inner, bindings.position_layout, bindings.rank)
    if isinstance(bindings, LocalCacheBindings):
        return _local(spec, bindings, UnifiedLocalResidency, NativePagedResidency)
    if isinstance(bindings, RecordOwnerBindings):
        return RecordOwnerPagedResidency(spec, bindings)
    if isinstance(bindings, TensorParallelCacheBindings):
        return TensorParallelResidency(spec, bindings)
    raise TypeError(f"Unsupported cache bindings {type(bindings).__name__}")


def _local(spec, bindings, contiguous_cls, paged_cls):
    backend = bindings.execution_options.record_storage_backend
    if backend == "native_paged":
        return paged_cls(spec, bindings)
    if backend == "contiguous_records":
        if len(spec.storage_layout.record_planes) != 1:
            raise ValueError("Contiguous record storage holds exactly one plane; use native_paged")
        return contiguous_cls(spec, bindings)
    raise ValueError(f"A rank-local cache cannot use the {backend!r} storage backend")
