"""Pool adapters: from a decoded model configuration (one of the adapter families) to the cache
specification, the bindings and the sizes of everything a rank keeps for the cache, charged against a
GPU byte budget BEFORE anything is allocated.

    plan = plan_pool(cfg, layers=61, world=8, rank=0, gpu_budget_bytes=72 << 30)
    cache = plan.build(device, process_group)            # client.init(spec, bindings)

Families (``cfg.adapter``):

* ``native_tp`` / ``native_dpa``  the tensor-parallel pool (records striped over the ranks) and the rank-local
  pool of data-parallel attention, MLA latent records in the configured native format;
* ``dsa`` / ``dsa_optimized``     the record-owner engine: independent requests per rank over one namespace
  of owners, a distributed Index with a choice of score transport;
* ``glm_flash``                   as ``dsa`` with an Index compressed 4:1 (one key per four tokens), a shared
  tensor-parallel attention buffer and a prefill buffer of ``prefill_buffer_records``;
* ``paged``                       K and V as a pair of record planes in native pages, one storage bank per
  managed compression ratio (ratio 2 keeps one record per two tokens);
* ``qsa``                         ``paged`` with a single owner, selections given as regions.

What a plan charges to the GPU: device records (all planes, all layers), index pages, residency metadata
(4 words per device slot, 2 per logical id), the attention workspace and the prefill window.

Reference: patches/sglang.patch files native_dsa_pool.py, native_dsa_optimized_pool.py, native_paged_pool.py,
native_paired_pool.py, native_glm_flash_pool.py, native_qsa_pool.py, native_tensor_parallel_pool.py,
unified_local_adapter.py, flowkv_pool_configurator.py (pool sizing against the GPU budget),
native_cache_geometry / capacity_inventory.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

PAGE = 64
INDEX_RECORD_BYTES = 132


@dataclass(frozen=True)
class PoolPlan:
    adapter: str
    engine: str                       # tensor_parallel | local | record_owner
    planes: Tuple[str, ...]           # record plane names (aliases of storage.layout)
    compression_ratios: Tuple[int, ...]
    owners: int
    layers: int
    device_records: int               # per owner
    host_records: int
    index_pages: int
    index_compression_ratio: int
    index_transport: str
    prefill_window_records: int
    max_queries: int
    topk: int
    write_max: int
    bytes: dict = field(default_factory=dict)

    @property
    def gpu_bytes(self) -> int:
        return sum(v for k, v in self.bytes.items() if k != "host_records")

    def specification(self):
        from ..cache.access import SparseAccessSpecification
        from ..cache.layers import LayerReuseSpecification
        from ..cache.specification import MemoryTierCapacity, UnifiedCacheSpecification
        from ..storage.layout import StorageLayout, record_plane

        planes = tuple(record_plane(p) for p in self.planes)
        return UnifiedCacheSpecification(
            storage_layout=StorageLayout(record_planes=planes),
            layer_reuse=LayerReuseSpecification.independent(self.layers),
            sparse_access=SparseAccessSpecification(self.max_queries, self.topk),
            capacity_plan=MemoryTierCapacity(
                device_record_capacity=self.device_records, host_record_capacity=self.host_records,
                maximum_write_record_count=self.write_max,
                maximum_residency_input_record_count=min(self.device_records, self.max_queries * (self.topk + 1))))

    def bindings(self, device, *, process_group=None, rank: int = 0):
        from ..bindings import LocalCacheBindings, RecordOwnerBindings, TensorParallelCacheBindings
        from ..cache_config import CacheExecutionOptions

        if self.engine == "tensor_parallel" and self.owners > 1:
            return TensorParallelCacheBindings(device=device, process_group=process_group, rank=rank, world_size=self.owners)
        if self.engine == "record_owner" and self.owners > 1:
            return RecordOwnerBindings(device=device, owner_process_group=process_group, rank=rank, world_size=self.owners,
                                       maximum_prefill_record_count=self.prefill_window_records)
        backend = "native_paged" if len(self.planes) > 1 else "contiguous_records"
        return LocalCacheBindings(device=device, execution_options=CacheExecutionOptions(record_storage_backend=backend))

    def build(self, device, *, process_group=None, rank: int = 0):
        from .. import client

        return client.init(self.specification(), self.bindings(device, process_group=process_group, rank=rank))


def _record_bytes(planes) -> int:
    from ..storage.layout import record_plane

    return sum(record_plane(p).bytes_per_record for p in planes)


def plan_pool(cfg, *, layers: int, world: int = 1, rank: int = 0, gpu_budget_bytes: Optional[int] = None,
              max_queries: int = 64, topk: int = 2048, kv_format: str = "scaled656") -> PoolPlan:
    """Size the pool of ``cfg`` for one rank.  Capacities come from the configuration (per owner); when a GPU
    budget is given the device tier is cut down to what fits after index pages, metadata, workspace and prefill
    window are charged (never below one page per query), and the records cut move to the host tier."""
    if not cfg.enabled:
        raise ValueError("the native control arm has no pooled cache")
    o = cfg.options
    adapter = cfg.adapter
    fmt = getattr(o, "native_kv_format", kv_format)
    ratios: Tuple[int, ...] = (1,)
    index_ratio = int(getattr(o, "index_compression_ratio", 1) or 1)
    transport = getattr(o, "index_score_transport", "peer_topk")
    prefill = int(getattr(o, "prefill_window_rows", 0) or getattr(o, "maximum_prefill_record_count", 0)
                  or getattr(o, "prefill_buffer_records", 0) or 0)
    if adapter == "native_tp":
        engine, planes, owners = "tensor_parallel", (fmt,), world
    elif adapter == "native_dpa":
        engine, planes, owners = "local", (fmt,), 1
    elif adapter in ("dsa", "dsa_optimized", "glm_flash"):
        owners = int(getattr(o, "storage_owner_count", None) or world)
        engine, planes = ("record_owner" if owners > 1 else "local"), (fmt,)
    elif adapter in ("paged", "qsa"):
        owners = int(getattr(o, "storage_owner_count", None) or (1 if adapter == "qsa" else world))
        engine = "record_owner" if owners > 1 else "local"
        planes = ("bf16", "bf16")                      # K and V planes of a paired layout
        ratios = tuple(getattr(o, "managed_compression_ratios", (1,)))
        topk = int(getattr(o, "maximum_selected_records", None) or topk)
    else:
        raise ValueError(f"no pool adapter for {adapter!r}")
    if getattr(o, "maximum_padded_query_count", None):
        max_queries = int(o.maximum_padded_query_count)
    dev = cfg.device_token_capacity_per_owner or getattr(o, "device_record_capacity", 0) or 0
    host = cfg.host_token_capacity_per_owner or getattr(o, "host_record_capacity", 0) or 0
    if dev <= 0:
        raise ValueError(f"adapter {adapter} carries no capacity: set capacity.device_token_capacity_per_owner")
    dev, host = dev // PAGE * PAGE, host // PAGE * PAGE
    rb = _record_bytes(planes)
    # a bank of ratio r keeps one record per r tokens: records per token summed over the banks
    per_token = sum(1.0 / r for r in ratios)
    write_max = int(getattr(o, "maximum_write_record_count", 8192))

    logical_total = dev + host                  # a budget moves records between the tiers, it drops none

    def charge(dev_records: int) -> dict:
        logical = logical_total
        index_pages = (logical // index_ratio + PAGE - 1) // PAGE + 2
        return dict(device_records=int(dev_records * rb * layers * per_token),
                    host_records=int((logical_total - dev_records) * rb * layers * per_token),
                    index_pages=index_pages * PAGE * INDEX_RECORD_BYTES * layers,
                    metadata=4 * (4 * dev_records + 2 * logical),
                    attention_workspace=max_queries * topk * (4 + 4) + max_queries * 128 * 513 * 4,
                    prefill_window=prefill * rb)

    b = charge(dev)
    budget = gpu_budget_bytes if gpu_budget_bytes is not None else getattr(o, "device_cache_budget_bytes", None)
    if budget is not None:
        fixed = lambda d: sum(v for k, v in charge(d).items() if k not in ("host_records", "device_records"))
        floor = max(PAGE, (max_queries * topk + PAGE - 1) // PAGE * PAGE)
        lo, hi = 0, dev // PAGE
        while lo < hi:                                   # largest device tier (in pages) that fits
            mid = (lo + hi + 1) // 2
            c = charge(mid * PAGE)
            if c["device_records"] + fixed(mid * PAGE) <= budget:
                lo = mid
            else:
                hi = mid - 1
        fit = lo * PAGE
        if fit < floor:
            raise MemoryError(f"a GPU budget of {budget} bytes cannot hold the working set of {floor} records")
        if fit < dev:
            host += dev - fit
            dev = fit
        b = charge(dev)
    logical = dev + host
    return PoolPlan(adapter=adapter, engine=engine, planes=planes, compression_ratios=ratios, owners=owners, layers=layers,
                    device_records=dev, host_records=host, index_pages=(logical // index_ratio + PAGE - 1) // PAGE + 2,
                    index_compression_ratio=index_ratio, index_transport=transport, prefill_window_records=prefill,
                    max_queries=max_queries, topk=topk, write_max=write_max, bytes=b)
