"""The names a user of the reference imports from the package root, and the accounting behind them."""
import pytest


REFERENCE_ROOT_NAMES = """CacheLayout ResidentQueryLayout InterleavedRecordLayout NativePageLayout LayerGroupPlan
RequestPagePool RecordSpec history_capacity KeyValueRecordPlane KeyValueStorageLayout LayerReuseSpecification
SparseAccessSpecification SparseAttentionAccessPlan ResidentAttentionInputs ResidentView MemoryTierCapacity
UnifiedCacheSpecification UlaCache UnifiedMemoryCache LocalCacheBindings CacheExecutionOptions ForwardExecutionContext
RecordOwnerBindings TensorParallelCacheBindings PositionShardBindings PositionShardLayout LogicalSlotAllocator
FileRecordSource PrefetchPolicy init RecordOwnerCapacity RequiredCachePartitionCapacity RequestNamespaceCapacityBounds
calculate_addressable_history_capacity CacheMemoryUsage CacheMemoryBudget CacheCapacityPlan plan_cache_capacity""".split()


def test_every_root_name_of_the_reference_resolves():
    import ulacache_b200 as ula

    for name in REFERENCE_ROOT_NAMES:
        assert getattr(ula, name) is not None, name
        assert name in ula.__all__
    with pytest.raises(AttributeError):
        ula.no_such_name


def test_history_capacity_and_native_page_layout():
    from ulacache_b200 import NativePageLayout, history_capacity
    from ulacache_b200.storage.layout import INDEX_FP8, MLA_SCALED656

    assert history_capacity(64, 2048, 1.0, 64) == 131072
    assert history_capacity(3, 100, 1.01, 64) == 320                 # ceil(303) -> 5 pages, not 6
    for bad in (dict(max_queries=0, topk=1, multiplier=1, page_size=1), dict(max_queries=1, topk=1, multiplier=0.5, page_size=1),
                dict(max_queries=1 << 20, topk=2048, multiplier=1.0, page_size=64)):
        with pytest.raises(ValueError):
            history_capacity(**bad)
    page = NativePageLayout(64, (128, 8), 16)                        # keys then scales, segment after segment
    assert page.row_bytes == 136 and page.bytes_per_page == 64 * 136
    assert page.byte_offset(0, 0) == 0 and page.byte_offset(1, 0) == 128
    assert page.byte_offset(1, 130) == 64 * 128 + 8 + 2              # second segment of row 1
    assert page.byte_offset(64, 5) == page.bytes_per_page + 5        # next page
    with pytest.raises(IndexError):
        page.byte_offset(0, 136)
    with pytest.raises(ValueError):
        NativePageLayout(64, (128, 4), 16)                           # 4-byte segment: not a transport unit
    whole = NativePageLayout.of_plane(MLA_SCALED656)
    assert whole.segment_bytes == (656,) and whole.byte_offset(3, 10) == MLA_SCALED656.record_offset(3) + 10
    with pytest.raises(ValueError):
        NativePageLayout.of_plane(INDEX_FP8)


def test_storage_tier_fields_and_packed_record_spec():
    from ulacache_b200 import KeyValueStorageLayout, RecordSpec
    from ulacache_b200.storage.layout import MLA_SCALED656, KeyValueRecordPlane

    tier = KeyValueStorageLayout(record_planes=(MLA_SCALED656,))
    assert (tier.name, tier.tokens_per_record, tier.records_per_page, tier.bytes_per_record) == ("kv", 1, 64, 656)
    assert tier.calculate_storage_bytes(0) == 0 and tier.calculate_storage_bytes(65) == 2 * 64 * 656
    with pytest.raises(ValueError):
        KeyValueStorageLayout(record_planes=(MLA_SCALED656,), tokens_per_record=4)       # token records stand for one token
    with pytest.raises(ValueError):
        KeyValueStorageLayout(record_planes=(MLA_SCALED656, KeyValueRecordPlane("x", (64,), "x", page_tokens=32)))
    spec = RecordSpec(compression_ratio=4, indexed_layer_ids=(2, 3, 4, 7, 8), topk=2304, row_bytes=584,
                      native_segment_bytes=(576, 8), index_layer_anchors=(2, 2, 4, 7, 7), page_storage_alignment=576)
    assert spec.local_layer_count(0, 5) == 3 and spec.local_layer_count(5, 9) == 2
    assert spec.local_layer_anchors(0, 5) == (0, 0, 2) and spec.local_layer_anchors(5, 9) == (0, 0)
    with pytest.raises(ValueError):
        spec.local_layer_anchors(3, 9)                                # layer 3's anchor (2) is in another stage
    plane = spec.plane()
    assert plane.segment_major and plane.bytes_per_record == 584 and plane.bytes_per_page % 576 == 0
    packed = spec.storage_layout()
    assert packed.record_kind == "compressed" and packed.tokens_per_record == 4
    with pytest.raises(NotImplementedError):
        RecordSpec(1, (0,), 2000, 584, (576, 8), (0,))
    with pytest.raises(ValueError):
        RecordSpec(1, (0, 1), 2048, 584, (576, 8), (0, 5))           # anchor is not an indexed layer


def test_addressable_history_audit():
    from ulacache_b200 import (RecordOwnerCapacity, RequestNamespaceCapacityBounds, RequiredCachePartitionCapacity,
                               calculate_addressable_history_capacity)
    from ulacache_b200.storage.capacity import addressable_tokens_per_owner
    from ulacache_b200.storage.layout import MLA_SCALED656, StorageLayout

    kv = StorageLayout(record_planes=(MLA_SCALED656,), name="kv")
    c4 = StorageLayout(record_planes=(MLA_SCALED656,), name="c4", record_kind="compressed", tokens_per_record=4)
    owners = tuple(RecordOwnerCapacity(r, 1000, 3000) for r in range(4))
    parts = [
        RequiredCachePartitionCapacity(0, "kv", kv, owners, reserved_logical_record_count=64),
        # the compressed tier keeps a quarter of the records, twice replicated: replicas add bytes, not capacity
        RequiredCachePartitionCapacity(0, "c4", c4, tuple(RecordOwnerCapacity(r, 500, 400, 2) for r in range(4)), 0),
        RequiredCachePartitionCapacity(1, "kv", kv, owners[:1], 0),
    ]
    bounds = [RequestNamespaceCapacityBounds(0, 20000, 1 << 30), RequestNamespaceCapacityBounds(1, 1 << 30, 2500)]
    audit = calculate_addressable_history_capacity(parts, bounds)
    p = {(x["request_namespace_id"], x["partition_name"]): x for x in audit["required_partitions"]}
    assert p[(0, "kv")]["usable_history_token_slots"] == 16000 - 64
    assert p[(0, "c4")]["usable_history_token_slots"] == 3600 * 4
    assert p[(0, "c4")]["physical_device_cold_record_slots"] == 4000 and p[(0, "c4")]["unique_device_cold_record_slots"] == 2000
    n = {x["request_namespace_id"]: x for x in audit["request_namespaces"]}
    assert n[0]["cold_storage_history_token_slots"] == 14400 and n[0]["usable_history_token_slots"] == 14400
    assert n[1]["usable_history_token_slots"] == 2500                 # the address limit binds
    assert audit["total_usable_history_token_slots"] == 16900
    with pytest.raises(ValueError):
        calculate_addressable_history_capacity(parts, bounds[:1])     # namespace 1 has partitions but no bounds
    with pytest.raises(ValueError):
        calculate_addressable_history_capacity([RequiredCachePartitionCapacity(0, "kv", kv, owners + owners[:1], 0)], bounds[:1])
    with pytest.raises(ValueError):
        calculate_addressable_history_capacity([RequiredCachePartitionCapacity(0, "kv", kv, owners, 10 ** 6)], bounds[:1])
    assert addressable_tokens_per_owner(maximum_requests=256, maximum_context_tokens=131072, owners=8) == 256 * 131072 // 8
    assert addressable_tokens_per_owner(maximum_requests=1 << 20, maximum_context_tokens=1 << 20, owners=8) == (2 ** 31 - 1) // 8 // 64 * 64


def test_resident_query_layout_sizes_from_real_queries():
    from ulacache_b200 import CacheLayout, ResidentQueryLayout

    base = dict(layers=4, groups=2, record_bytes=656, slots_per_rank=64 * 100, topk=2048, pulled_record_cache=True)
    padded = CacheLayout(max_queries=256, **base)
    real = ResidentQueryLayout(max_queries=256, max_resident_queries=80, **base)
    assert real.resident_query_capacity == 80 and ResidentQueryLayout(max_queries=256, **base).resident_query_capacity == 256
    assert real.cache_rows * 256 == padded.cache_rows * 80 and real.selected_bytes < padded.selected_bytes
    assert real.rows_per_layer % 64 == 0 and real.rows_per_layer >= real.cache_rows + 80
    assert real.report()["total"] < padded.report()["total"]
    for bad in (dict(max_queries=100), dict(max_queries=4096), dict(max_queries=64, max_resident_queries=65)):
        with pytest.raises(ValueError):
            ResidentQueryLayout(**{**base, **bad})


def _client(backend=None, **kw):
    import dataclasses

    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings

    from helpers import make_spec

    b = LocalCacheBindings(device="cpu")
    if backend:
        b = dataclasses.replace(b, execution_options=dataclasses.replace(b.execution_options, record_storage_backend=backend))
    return ula.init(make_spec(**kw), b)


def test_client_forwards_engine_capabilities_of_the_native_paged_backend():
    import torch

    from ulacache_b200.ops import records

    from helpers import random_kv

    cache = _client("native_paged", layers=2, device_pages=4, host_pages=16, queries=8, topk=64)
    assert cache.supports_local_native_current_publication is False      # true on a GPU only
    ids = cache.alloc(320)
    latent, rope = random_kv(320, 4)
    enc = records.encode_scaled656(latent, rope)
    # native segments (latent + scales | rope) concatenate to records; a wrong width is refused
    cache.write_native_record_segments(0, ids, (enc[:, :528], enc[:, 528:]))
    with pytest.raises(ValueError):
        cache.write_native_record_segments(0, ids, (enc[:, :528],))
    assert torch.equal(cache.engine.read_records(0, ids)[0], enc)
    # native pages + source rows
    pages = enc.flip(0).contiguous().view(5, 64, 656)
    cache.write_native_paged_records(1, ids[:100], pages, torch.arange(319, 219, -1))
    assert torch.equal(cache.engine.read_records(1, ids[:100])[0], enc[:100])
    # prefill: eager union, then a borrowed chunk
    sel = ids[torch.randperm(320, generator=torch.Generator().manual_seed(0))[:128]].view(2, 64)
    cache.begin_model_forward()
    view = cache.prepare_prefill_attention_inputs(0, sel)
    assert view.records_per_page == 64 and view.device_record_indices.shape == sel.shape
    assert torch.equal(view.gpu_buffer[view.device_record_indices[0].long()], enc[(sel[0] - ids[0]).long()])
    cache.finish_layer_attention(0)
    cache.finish_model_forward()
    chunk = cache.prepare_prefill_record_chunk(1, ids[:64])
    assert bool((chunk.device_record_indices >= 0).all())
    with pytest.raises(RuntimeError):
        cache.prepare_prefill_record_chunk(1, ids[64:128])            # the domain's chunk is still borrowed
    cache.finish_prefill_record_chunk(1)
    # hints that this engine does not implement are harmless; receive rows and inventories are forwarded
    assert cache.prepare_forward_current_records(ids[:4]) is False
    cache.prepare_next_residency_epochs()
    cache.prepare_layer_execution(0)
    fresh = torch.arange(1024, 1088, dtype=torch.int32)              # ids the framework's own allocator handed out
    rows = cache.register_receive_records(fresh)
    assert rows.numel() == 64 and bool((rows >= 0).all()) and rows.unique().numel() == 64
    cache.release_logical_records(fresh)
    assert cache.get_device_storage_inventory() and cache.get_host_storage_inventory()
    assert cache.get_memory_inventory() == cache.memory_inventory()
    assert len(cache.get_device_record_planes(0)) == 1 and cache.device_record_storage.shape[0] == 2
    with pytest.raises(NotImplementedError):
        cache.prepare_native_prefill_read_plan(sel)                   # no windowed reader bound
    cache.close()


def test_client_refuses_capabilities_the_backend_lacks_and_serves_a_bound_reader():
    import torch

    cache = _client(None, layers=1, device_pages=4, host_pages=4)
    assert not cache.supports_local_native_current_publication
    ids = cache.alloc(64)
    for call in (lambda: cache.register_receive_records(ids), lambda: cache.prepare_prefill_record_chunk(0, ids),
                 lambda: cache.write_native_paged_records(0, ids, torch.zeros(64, 656, dtype=torch.uint8), torch.arange(64))):
        with pytest.raises(NotImplementedError):
            call()
    with pytest.raises(ValueError):
        cache.write_native_paged_records(0, ids, None, None, local_device_after_commit=True)
    inv = cache.get_device_storage_inventory()
    assert sum(inv.values()) >= 4 * 64 * 656 and sum(cache.get_host_storage_inventory().values()) >= 4 * 64 * 656

    class Reader:
        def prepare_read_plan(self, ids):
            return ("plan", int(ids.numel()))

        def read_records(self, layer, ids, consume, *, output_buffer=None, read_plan=None):
            return (layer, read_plan, output_buffer)

        def attend(self, layer, query, selection, lengths, fn):
            return fn(query)

    cache.bind_prefill_reader(Reader())
    assert cache.prepare_native_prefill_read_plan(ids) == ("plan", 64)
    assert cache.read_native_prefill_records(0, ids, None, output="buf", read_plan="p") == (0, "p", "buf")
    assert cache.attend_native_prefill_records(0, 3, ids, None, lambda q: q + 1) == 4
    cache.close()


def test_factory_refuses_policies_that_cannot_do_what_they_say():
    import dataclasses

    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings, PositionShardBindings
    from ulacache_b200.storage.layout import PositionShardLayout

    from helpers import make_spec

    b = LocalCacheBindings(device="cpu")
    ahead = dataclasses.replace(b, execution_options=dataclasses.replace(b.execution_options,
                                                                        copy_follower_records_asynchronously=True))
    with pytest.raises(ValueError):
        ula.init(make_spec(layers=4), ahead)                           # no shared selection group: nothing to copy ahead
    cache = ula.init(make_spec(layers=4, shared_groups=((0, 1), (2, 3))), ahead)
    cache.close()
    with pytest.raises(ValueError):
        ula.init(make_spec(), PositionShardBindings(device="cpu", position_layout=PositionShardLayout(1), rank=0))
    with pytest.raises(ValueError):                                    # 16 queries x 64 records per rank > 2 pages
        ula.init(make_spec(device_pages=2, queries=16, topk=128),
                 PositionShardBindings(device="cpu", position_layout=PositionShardLayout(2), rank=0))


def test_canary_build_catches_a_write_outside_a_plane(monkeypatch):
    import torch

    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.ops import records
    from ulacache_b200.storage.buffers import GUARD_BYTE, GUARD_ROWS

    from helpers import make_spec, random_kv

    monkeypatch.setenv("ULC_CANARY", "1")
    cache = ula.init(make_spec(layers=2, device_pages=2, host_pages=4), LocalCacheBindings(device="cpu"))
    st = cache.engine.storages[0]
    assert st.guard == GUARD_ROWS and st.gpu.shape[1] == 128 and st.host.shape[1] == 256
    assert st.device_bytes() == 2 * (128 + 2 * GUARD_ROWS) * 656
    ids = cache.alloc(300)                                           # fills the device tier and spills to the host
    latent, rope = random_kv(300, 1)
    for layer in range(2):
        cache.write(ids, layer, (latent, rope))
    cache.begin_model_forward()
    cache.access(ids[200:264].view(1, 64), 1)                        # promotions and evictions through both tiers
    got = records.decode_scaled656(cache.gather_selected_records(1))
    assert torch.equal(got, records.decode_scaled656(records.encode_scaled656(latent, rope))[200:264])
    cache.finish_layer_attention(1)
    cache.finish_model_forward()
    cache.check()                                                    # every guard record is intact
    st._device_block[1, GUARD_ROWS + 128, 5] = 0                     # one byte past layer 1's last device slot
    with pytest.raises(RuntimeError, match="after the device slots of storage layer"):
        cache.check()
    st._device_block[1, GUARD_ROWS + 128, 5] = GUARD_BYTE
    st.host_pool.storage[0, GUARD_ROWS - 1, 0] = 1                   # and one before layer 0's first host slot
    with pytest.raises(RuntimeError, match="before the host slots"):
        cache.check()
    cache.close()
    monkeypatch.setenv("ULC_CANARY", "0")
    plain = ula.init(make_spec(layers=1), LocalCacheBindings(device="cpu"))
    assert plain.engine.storages[0].guard == 0 and plain.engine.storages[0].gpu.is_contiguous()
    plain.check()
    plain.close()


def test_heap_carved_planes_keep_the_storage_interface():
    """Planes that live in the symmetric heap skip the base constructor; they must still answer everything the
    engine asks of a plane storage (host view, guard check, byte counts)."""
    import torch

    from ulacache_b200.cache.engine import _HeapPlaneStorage
    from ulacache_b200.storage.buffers import PinnedHostRecordPool
    from ulacache_b200.storage.layout import MLA_SCALED656

    class Heap:
        device = torch.device("cpu")

        def alloc(self, name, shape, dtype):
            return torch.zeros(shape, dtype=dtype)

    st = _HeapPlaneStorage(MLA_SCALED656, heap=Heap(), layers=2, hbm_slots=64, host_slots=128,
                           host_pool_factory=lambda **kw: PinnedHostRecordPool(pin=False, **{k: v for k, v in kw.items() if k != "device"}))
    assert st.guard == 0 and st.host.shape == (2, 128, 656) and st.device_bytes() == 2 * 64 * 656
    st.check_canaries()
    assert st.host_bytes() == 2 * 128 * 656
    st.close()


def test_launch_environment_is_derived_once_and_conflicts_are_refused():
    import os

    from ulacache_b200.config.model_configuration import (ConfigurationError, launch_environment,
                                                          load_model_configuration)

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ulacache_b200", "config", "models")
    dpa = load_model_configuration(os.path.join(root, "b200-native-dpa.json"), environ={})
    env = launch_environment(dpa, environ={})
    assert int(env["UDCACHE_DPA_GPU_SLOTS"]) > 0 and int(env["UDCACHE_DPA_GPU_SLOTS"]) % 64 == 0
    assert "UDCACHE_DPA_CPU_SLOTS" in env and all(isinstance(v, str) for v in env.values())
    assert launch_environment(dpa, environ=dict(env)) == env                       # the same values are no conflict
    with pytest.raises(ConfigurationError, match="conflicts"):
        launch_environment(dpa, environ={"UDCACHE_DPA_GPU_SLOTS": "64"})
    with pytest.raises(ConfigurationError, match="legacy"):
        launch_environment(dpa, environ={"ULACACHE_QSA_CONFIGURATION": "x.json"})
    with pytest.raises(ConfigurationError, match="legacy"):
        load_model_configuration(os.path.join(root, "b200-native-dpa.json"), environ={"ULACACHE_V0522_CONFIGURATION": "y"})
    tp = load_model_configuration(os.path.join(root, "native-tp-arena.json"), environ={})
    assert set(launch_environment(tp, environ={})) == {"UDCACHE_PLAIN_PREFILL_WINDOW_ROWS", "ULACACHE_TP_LOW_QUERY_PULL_BLOCKS",
                                                       "ULACACHE_REUSE_PREFILL_METADATA"}
    dsa = load_model_configuration(os.path.join(root, "dsa-peer-topk.json"), environ={})
    assert launch_environment(dsa, environ={}) == {}


def test_quickstart_example_runs_on_cpu():
    from ulacache_b200.examples.quickstart import run

    out = run("cpu", tokens=600, steps=2)
    assert out["reads_exact"] == out["reads"] and out["promotions"] > 0 and out["unserved"] == 0


def test_payload_replacement_pricing_and_workspace_bytes():
    from ulacache_b200.storage.capacity import (CacheCapacityPlan, CacheMemoryBudget, CacheMemoryUsage,
                                                price_payload_replacement, residency_workspace_bytes)

    plan = CacheCapacityPlan(64 * 100, 64 * 300, 8, CacheMemoryUsage(80 << 30, 120 << 30), CacheMemoryBudget(90 << 30, 128 << 30))
    usage = price_payload_replacement(native_device_bytes=70 << 30, native_payload_bytes=60 << 30,
                                      replacement_device_bytes=64 << 30, replacement_host_bytes=100 << 30,
                                      native_host_bytes=4 << 30, allocation_plan=plan)
    assert usage == CacheMemoryUsage(74 << 30, 104 << 30)
    with pytest.raises(ValueError, match="exceed"):
        price_payload_replacement(native_device_bytes=70 << 30, native_payload_bytes=10 << 30,
                                  replacement_device_bytes=64 << 30, replacement_host_bytes=0, allocation_plan=plan)
    with pytest.raises(ValueError, match="part of"):
        price_payload_replacement(native_device_bytes=1, native_payload_bytes=2, replacement_device_bytes=0,
                                  replacement_host_bytes=0, allocation_plan=plan)
    w = residency_workspace_bytes(4096, 61, 1 << 20)
    assert w["fixed_bytes"] == 32 * 4096 + 56 * 61 and w["expiry_bytes"] == 4 * 61 * 4096
    assert residency_workspace_bytes(4096, 2, 100)["expiry_bytes"] == 800
    with pytest.raises(ValueError):
        residency_workspace_bytes(0, 1, 1)


def test_capacity_experiment_prints_the_history_audit():
    from ulacache_b200.experiments.capacity import history_audit

    audit = history_audit(device_gb=72.0, host_gb=128.0, ranks=8, layers=61, requests=512, max_context=131072)
    part, space = audit["required_partitions"][0], audit["request_namespaces"][0]
    assert part["record_owner_count"] == 8 and part["reserved_logical_record_count"] == 512
    assert space["usable_history_token_slots"] == min(space["cold_storage_history_token_slots"],
                                                      space["native_allocator_usable_token_slots"],
                                                      space["request_address_token_slots"])
    assert audit["total_usable_history_token_slots"] > 30_000_000
    tight = history_audit(device_gb=72.0, host_gb=128.0, ranks=8, layers=61, requests=8, max_context=4096)
    assert tight["total_usable_history_token_slots"] == 8 * 4096          # addressing binds, not memory
