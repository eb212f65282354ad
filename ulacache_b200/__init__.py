"""ulacache_b200 — pooled sparse-KV cache framework for B200 (sm_100a).

One logical address space for KV records and index pages across every GPU's HBM
and pinned host memory, with the cache verbs ``init / alloc / write / access /
free``.  Importing this package (or any sub-package) does not import torch or
CUDA; heavy modules load on first attribute access.

Reference: ulacache/__init__.py:51-108 (lazy exports).
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_EXPORTS = {
    "init": "ulacache_b200.client",
    "UlaCache": "ulacache_b200.client",
    "UnifiedMemoryCache": "ulacache_b200.client",
    "ResidentView": "ulacache_b200.cache.access",
    "SparseAttentionAccessPlan": "ulacache_b200.cache.access",
    "ForwardExecutionContext": "ulacache_b200.cache.access",
    "UnifiedCacheSpecification": "ulacache_b200.cache.specification",
    "MemoryTierCapacity": "ulacache_b200.cache.specification",
    "SparseAccessSpecification": "ulacache_b200.cache.specification",
    "LayerReuseSpecification": "ulacache_b200.cache.layers",
    "CacheOptions": "ulacache_b200.cache_config",
    "CacheExecutionOptions": "ulacache_b200.cache_config",
    "PrefetchPolicy": "ulacache_b200.cache_config",
    "LocalCacheBindings": "ulacache_b200.bindings",
    "RecordOwnerBindings": "ulacache_b200.bindings",
    "TensorParallelCacheBindings": "ulacache_b200.bindings",
    "PositionShardBindings": "ulacache_b200.bindings",
    "BackendServices": "ulacache_b200.bindings",
    "load_model_configuration": "ulacache_b200.config.model_configuration",
    "FileRecordSource": "ulacache_b200.transfer.file_io",
    "ResidentAttentionInputs": "ulacache_b200.cache.access",
    "LayerGroupPlan": "ulacache_b200.cache.layers",
    "RequestPagePool": "ulacache_b200.cache.request_pages",
    "LogicalSlotAllocator": "ulacache_b200.bindings",
    "KeyValueRecordPlane": "ulacache_b200.storage.layout",
    "KeyValueStorageLayout": "ulacache_b200.storage.layout",
    "StorageLayout": "ulacache_b200.storage.layout",
    "NativePageLayout": "ulacache_b200.storage.layout",
    "InterleavedRecordLayout": "ulacache_b200.storage.layout",
    "PositionShardLayout": "ulacache_b200.storage.layout",
    "history_capacity": "ulacache_b200.storage.layout",
    "CacheLayout": "ulacache_b200.storage.workspace",
    "ResidentQueryLayout": "ulacache_b200.storage.workspace",
    "RecordSpec": "ulacache_b200.storage.layout",
    "CacheMemoryUsage": "ulacache_b200.storage.capacity",
    "CacheMemoryBudget": "ulacache_b200.storage.capacity",
    "CacheCapacityPlan": "ulacache_b200.storage.capacity",
    "plan_cache_capacity": "ulacache_b200.storage.capacity",
    "RecordOwnerCapacity": "ulacache_b200.storage.capacity",
    "RequiredCachePartitionCapacity": "ulacache_b200.storage.capacity",
    "RequestNamespaceCapacityBounds": "ulacache_b200.storage.capacity",
    "calculate_addressable_history_capacity": "ulacache_b200.storage.capacity",
}

__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name):
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module 'ulacache_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(target), name)
    globals()[name] = value
    return value
