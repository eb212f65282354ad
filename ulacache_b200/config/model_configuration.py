"""The configuration JSON pointed to by ``ULACACHE_CONFIGURATION``: parsing and validation.

Top level: ``{"schema_version": 1, "adapter": <name>, "framework_release": "v0.5.22" | absent,
"cpu_ngram_embedding": bool, "capacity": {"device_token_capacity_per_owner": int,
"host_token_capacity_per_owner": int}, "options": {...}}``.  Unknown keys and duplicate keys are
errors; ``native`` / ``native_tp`` take no ``capacity`` (they are sized by the serving
arguments) and ``native`` takes no options; every other adapter needs exactly the two capacity
fields and may not repeat them inside ``options``.

Reference: decode_model_configuration (patches/sglang.patch:8414-8473) and the per-adapter
option classes (patches/sglang.patch:15750-15800, 15243-15275, 9362-9400, 10060-10075,
10612-10635, 8265-8281); example files under scripts/configs/models/.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Optional

from ..cache_config import PrefetchPolicy

ADAPTERS = ("native", "native_tp", "native_dpa", "dsa_optimized", "dsa", "paged", "glm_flash", "qsa")
RELEASES = ("v0.5.22",)
_TOP_KEYS = {"schema_version", "adapter", "framework_release", "cpu_ngram_embedding", "capacity", "options"}
_CAP_KEYS = ("device_token_capacity_per_owner", "host_token_capacity_per_owner")


class ConfigurationError(ValueError):
    pass


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise ConfigurationError(f"Duplicate configuration key {k!r}")
        seen[k] = v
    return seen


def _check_fields(cls, options: dict, what: str):
    known = {f.name for f in fields(cls)}
    unknown = sorted(set(options) - known)
    if unknown:
        raise ConfigurationError(f"Unknown {what} option(s): {', '.join(unknown)}")


def _page_aligned(v, name):
    if type(v) is not int or v < 0 or v % 64:
        raise ConfigurationError(f"{name} must be a non-negative multiple of 64")


@dataclass(frozen=True)
class OwnerTPConfiguration:
    """``native_tp`` with a framework release: owner-striped pool with optional host tier."""

    enabled: bool = True
    cpu_offload: bool = False
    cpu_slots: int = 0
    cpu_ratio: float = 2.0
    prefetch: Any = True
    local_eviction_policy: str = "age_lru"
    host_exchange_blocks: int = 64
    host_exchange_threads: int = 256
    low_query_pull_blocks: Optional[int] = None
    cache_capacity_multiplier: float = 3.0
    device_cache_budget_bytes: Optional[int] = None
    native_kv_format: str = "raw576"
    prefill_window_rows: int = 0
    index_sharding: bool = True
    owner_index_draft: bool = False

    def __post_init__(self):
        if isinstance(self.prefetch, dict):
            object.__setattr__(self, "prefetch", PrefetchPolicy(**self.prefetch))
        elif type(self.prefetch) is bool:
            object.__setattr__(self, "prefetch", PrefetchPolicy(enabled=self.prefetch))
        elif not isinstance(self.prefetch, PrefetchPolicy):
            raise ConfigurationError("prefetch must be a bool or {enabled, completion}")
        _page_aligned(self.cpu_slots, "cpu_slots")
        if not self.cpu_ratio > 0:
            raise ConfigurationError("cpu_ratio must be positive")
        if self.local_eviction_policy not in ("age_lru", "circular"):
            raise ConfigurationError("local_eviction_policy must be age_lru or circular")
        if self.cache_capacity_multiplier < 3:
            raise ConfigurationError("cache_capacity_multiplier must be at least 3")
        if self.native_kv_format not in ("raw576", "scaled656"):
            raise ConfigurationError("native_kv_format must be raw576 or scaled656")
        w = self.prefill_window_rows
        if type(w) is not int or not (w == 0 or (w >= 2048 and w % 64 == 0)):
            raise ConfigurationError("prefill_window_rows must be 0 or a multiple of 64 that is at least 2048")
        if self.host_exchange_threads % 32 or not 0 < self.host_exchange_threads <= 1024 or self.host_exchange_blocks < 1:
            raise ConfigurationError("host exchange needs positive blocks and warp-aligned threads up to 1024")


@dataclass(frozen=True)
class NativeTensorParallelConfiguration:
    prefill_window_rows: int = 512
    low_query_pull_blocks: int = 0
    reuse_prefill_metadata: bool = False


@dataclass(frozen=True)
class DPAConfiguration:
    """``native_dpa`` with a framework release: rank-local unified cache."""

    device_record_capacity: int = 0
    host_record_capacity: int = 0
    device_cache_budget_bytes: Optional[int] = None
    maximum_running_requests: int = 128
    maximum_write_record_count: int = 8192
    exchange_blocks: int = 64
    exchange_threads: int = 256
    local_current_publication: bool = False
    maximum_padded_query_count: Optional[int] = None
    host_cache_budget_bytes: Optional[int] = None

    def __post_init__(self):
        _page_aligned(self.device_record_capacity, "device_record_capacity")
        _page_aligned(self.host_record_capacity, "host_record_capacity")
        if self.device_record_capacity + self.host_record_capacity >= 2 ** 31:
            raise ConfigurationError("device + host record capacity must stay below 2^31")
        if self.exchange_threads % 32 or not 0 < self.exchange_threads <= 1024 or self.exchange_blocks < 1:
            raise ConfigurationError("exchange launch needs positive blocks and warp-aligned threads up to 1024")


@dataclass(frozen=True)
class NativeDataParallelConfiguration:
    device_cache_budget_bytes: Optional[int] = None
    host_cache_budget_bytes: int = 128_000_000_000
    cpu_prefill: bool = False
    parallel_prepare: bool = False
    parallel_victims: bool = False
    asynchronous_followers: bool = False


@dataclass(frozen=True)
class NativeSparseLatentPoolConfiguration:
    """``dsa`` / ``dsa_optimized``: record-owner engine for DSA latent KV."""

    maximum_write_record_count: int = 8192
    device_cache_budget_bytes: Optional[int] = None
    index_compression_ratio: int = 1
    native_attention_backend: str = "sparse_mla_tcgen05"
    maximum_padded_query_count: Optional[int] = None
    prepare_in_parallel: bool = True
    independent_tensor_parallel_caches: bool = False
    storage_owner_count: Optional[int] = None
    maximum_prefill_record_count: Optional[int] = None
    native_record_writes_replicated: bool = True
    native_selections_replicated: bool = False
    distributed_indexer: bool = True
    maximum_index_prefill_query_count: int = 256
    index_prefill_score_mode: str = "native"
    index_score_transport: str = "flash_ag"
    reuse_attention_workspaces: bool = False
    prefill_buffer_records: int = 0
    prefill_query_chunk: int = 256
    prefill_buffer_prefetch: bool = True
    use_shared_tensor_parallel_cache: bool = False
    low_query_pull_blocks: int = 0
    device_record_capacity: int = 0
    host_record_capacity: int = 0

    def __post_init__(self):
        if self.index_prefill_score_mode not in ("native", "distributed"):
            raise ConfigurationError("index_prefill_score_mode must be native or distributed")
        if self.index_score_transport not in ("flash_ag", "nccl", "peer_topk"):
            raise ConfigurationError("index_score_transport must be flash_ag, nccl or peer_topk")


@dataclass(frozen=True)
class NativeGlmFlashPoolConfiguration(NativeSparseLatentPoolConfiguration):
    index_compression_ratio: int = 4
    distributed_indexer: bool = False
    use_shared_tensor_parallel_cache: bool = True
    low_query_pull_blocks: int = 16
    prefill_buffer_records: int = 1048576
    allocation_plan: Optional[dict] = None
    minimum_native_profile_available_bytes: Optional[int] = None


@dataclass(frozen=True)
class NativePagedPoolConfiguration:
    maximum_padded_query_count: Optional[int] = None
    maximum_write_record_count: int = 8192
    maximum_selected_records: Optional[int] = None
    managed_compression_ratios: tuple = (1, 2)
    storage_owner_count: Optional[int] = None
    maximum_prefill_record_count: Optional[int] = None
    native_record_writes_replicated: bool = True
    allocation_plan: Optional[dict] = None
    native_selections_replicated: bool = False
    distributed_indexer: bool = True
    prepare_in_parallel: bool = False
    reuse_attention_workspaces: bool = False
    device_record_capacity: int = 0
    host_record_capacity: int = 0

    def __post_init__(self):
        object.__setattr__(self, "managed_compression_ratios", tuple(self.managed_compression_ratios))


@dataclass(frozen=True)
class NativeQsaPoolConfiguration(NativePagedPoolConfiguration):
    def __post_init__(self):
        super().__post_init__()
        if self.storage_owner_count not in (None, 1):
            raise ConfigurationError("qsa requires storage_owner_count == 1")


@dataclass(frozen=True)
class ModelConfiguration:
    schema_version: int
    adapter: str
    framework_release: Optional[str]
    cpu_ngram_embedding: bool
    device_token_capacity_per_owner: Optional[int]
    host_token_capacity_per_owner: Optional[int]
    options: Any
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @property
    def enabled(self) -> bool:
        """``native`` is the control arm: the pooled cache is off."""
        return self.adapter != "native"


def _options_class(adapter: str, release: Optional[str]):
    if adapter == "native_tp":
        return OwnerTPConfiguration if release else NativeTensorParallelConfiguration
    if adapter == "native_dpa":
        return DPAConfiguration if release else NativeDataParallelConfiguration
    if adapter in ("dsa", "dsa_optimized"):
        return NativeSparseLatentPoolConfiguration
    if adapter == "glm_flash":
        return NativeGlmFlashPoolConfiguration
    if adapter == "paged":
        return NativePagedPoolConfiguration
    if adapter == "qsa":
        return NativeQsaPoolConfiguration
    return None


def decode_model_configuration(text: str) -> ModelConfiguration:
    try:
        doc = json.loads(text, object_pairs_hook=_no_duplicates)
    except json.JSONDecodeError as exc:
        raise ConfigurationError(f"Configuration is not valid JSON: {exc}") from exc
    if not isinstance(doc, dict):
        raise ConfigurationError("Configuration must be a JSON object")
    unknown = sorted(set(doc) - _TOP_KEYS)
    if unknown:
        raise ConfigurationError(f"Unknown configuration field(s): {', '.join(unknown)}")
    if doc.get("schema_version") != 1 or type(doc.get("schema_version")) is not int:
        raise ConfigurationError("schema_version must be exactly 1")
    adapter = doc.get("adapter")
    if adapter not in ADAPTERS:
        raise ConfigurationError(f"adapter must be one of {ADAPTERS}")
    release = doc.get("framework_release")
    if release is not None and release not in RELEASES:
        raise ConfigurationError(f"framework_release must be one of {RELEASES} or absent")
    ngram = doc.get("cpu_ngram_embedding", False)
    if type(ngram) is not bool:
        raise ConfigurationError("cpu_ngram_embedding must be a bool")
    if ngram and adapter != "qsa":
        raise ConfigurationError("cpu_ngram_embedding is only valid with the qsa adapter")
    options = doc.get("options", {})
    if not isinstance(options, dict):
        raise ConfigurationError("options must be an object")
    capacity = doc.get("capacity")
    dev = host = None
    if adapter in ("native", "native_tp"):
        if capacity is not None:
            raise ConfigurationError(f"{adapter} is sized by the serving arguments and takes no capacity")
        if adapter == "native" and options:
            raise ConfigurationError("native takes no options")
    else:
        if not isinstance(capacity, dict) or set(capacity) != set(_CAP_KEYS):
            raise ConfigurationError(f"{adapter} requires capacity with exactly {_CAP_KEYS}")
        dev, host = (capacity[k] for k in _CAP_KEYS)
        for k, v in zip(_CAP_KEYS, (dev, host)):
            if type(v) is not int or v < 0:
                raise ConfigurationError(f"{k} must be a non-negative int")
        for k in ("device_record_capacity", "host_record_capacity", *_CAP_KEYS):
            if k in options:
                raise ConfigurationError(f"{k} belongs in capacity, not in options")
    cls = _options_class(adapter, release)
    parsed = None
    if cls is not None:
        _check_fields(cls, options, adapter)
        kw = dict(options)
        if dev is not None and "device_record_capacity" in {f.name for f in fields(cls)}:
            kw.update(device_record_capacity=dev, host_record_capacity=host)
        try:
            parsed = cls(**kw)
        except (TypeError, ValueError) as exc:
            raise ConfigurationError(f"Invalid {adapter} options: {exc}") from exc
    return ModelConfiguration(1, adapter, release, ngram, dev, host, parsed, raw=doc)


# One configuration file replaced a family of per-adapter variables; a process that still exports one of them next
# to the file would be configured twice, so it is refused.  Reference: patches/sglang.patch:8286-8291, :8548-8550.
LEGACY_CONFIGURATION_VARIABLES = (
    "ULACACHE_NATIVE_DSA_CONFIGURATION", "ULACACHE_NATIVE_PAGED_CONFIGURATION", "ULACACHE_GLM_FLASH_CONFIGURATION",
    "ULACACHE_QSA_CONFIGURATION", "ULACACHE_NATIVE_OWNER_INDEX_CONFIGURATION", "ULACACHE_V0522_CONFIGURATION",
)


def launch_environment(configuration: ModelConfiguration, environ=None) -> dict:
    """The launch variables that scripts and workers of a deployment read (slot counts, byte budgets, launch
    shapes), derived from the one configuration so that every worker sees the same values.  A variable that is
    already exported with a DIFFERENT value is a conflict, not an override.  Returns the variables to export
    (the given environment is not changed).

    Reference: patches/sglang.patch:8495-8530 (``configure_launch``), scripts/7_2_throughput/start_ulacache.sh:121-165."""
    env = os.environ if environ is None else environ
    legacy = [name for name in LEGACY_CONFIGURATION_VARIABLES if env.get(name)]
    if legacy:
        raise ConfigurationError(f"use ULACACHE_CONFIGURATION without the legacy configuration variables {legacy}")
    o, out = configuration.options, {}
    if configuration.adapter == "native_tp":
        out = {"UDCACHE_PLAIN_PREFILL_WINDOW_ROWS": getattr(o, "prefill_window_rows", 0),
               "ULACACHE_TP_LOW_QUERY_PULL_BLOCKS": getattr(o, "low_query_pull_blocks", 0),
               "ULACACHE_REUSE_PREFILL_METADATA": int(bool(getattr(o, "reuse_prefill_metadata", False)))}
    elif configuration.adapter == "native_dpa":
        dev = configuration.device_token_capacity_per_owner or getattr(o, "device_record_capacity", 0)
        host = configuration.host_token_capacity_per_owner or getattr(o, "host_record_capacity", 0)
        out = {"UDCACHE_DPA_GPU_SLOTS": dev, "UDCACHE_DPA_CPU_SLOTS": host}
        for name, field in (("UDCACHE_DPA_CACHE_BUDGET_BYTES", "device_cache_budget_bytes"),
                            ("UDCACHE_CPU_CACHE_CAP_BYTES", "host_cache_budget_bytes"),
                            ("UDCACHE_DPA_EXCHANGE_BLOCKS", "exchange_blocks"),
                            ("UDCACHE_DPA_EXCHANGE_THREADS", "exchange_threads")):
            value = getattr(o, field, None)
            if value is not None:
                out[name] = value
        for name, field in (("UDCACHE_DPA_CPU_PREFILL", "cpu_prefill"), ("UDCACHE_DPA_PARALLEL_PREPARE", "parallel_prepare"),
                            ("UDCACHE_DPA_PARALLEL_VICTIMS", "parallel_victims"),
                            ("UDCACHE_DPA_ASYNC_FOLLOWERS", "asynchronous_followers")):
            if hasattr(o, field):
                out[name] = int(bool(getattr(o, field)))
    out = {k: str(v) for k, v in out.items()}
    for name, value in out.items():
        if name in env and env[name] != value:
            raise ConfigurationError(f"{name}={env[name]} in the environment conflicts with the configuration ({value})")
    return out


def load_model_configuration(path: Optional[str] = None, environ=None) -> Optional[ModelConfiguration]:
    """Read the file named by ``path`` or by ``ULACACHE_CONFIGURATION``; None when neither is set."""
    env = os.environ if environ is None else environ
    path = path or env.get("ULACACHE_CONFIGURATION")
    if not path:
        return None
    legacy = [name for name in LEGACY_CONFIGURATION_VARIABLES if env.get(name)]
    if legacy:
        raise ConfigurationError(f"use ULACACHE_CONFIGURATION without the legacy configuration variables {legacy}")
    with open(path) as f:
        return decode_model_configuration(f.read())
