"""CPU tests: configuration JSON, capacity planner, speculative contracts, snapshot round trip."""
import json
import os

import pytest
import torch

import ulacache_b200 as ula
from ulacache_b200.bindings import LocalCacheBindings
from ulacache_b200.config.model_configuration import ConfigurationError, decode_model_configuration
from ulacache_b200.speculative.linear import LinearVerifyConfig, expand_verify_rows, index_query_metadata
from ulacache_b200.storage.capacity import (CacheMemoryBudget, plan_cache_capacity, request_history_capacity,
                                            simple_usage_model)
from ulacache_b200.storage.workspace import AttentionWorkspaceLifetime, PoolLayout, colour_workspaces
from ulacache_b200.tools import cli
from ulacache_b200.tools.snapshot import cache_io
from ulacache_b200.tools.snapshot.format import SnapshotLayout, SnapshotReader, SnapshotRequest, finalize_snapshot

from helpers import make_spec, random_kv

CONFIG_DIR = os.path.join(os.path.dirname(ula.__file__), "config", "models")


def test_example_configurations_parse():
    for name in os.listdir(CONFIG_DIR):
        cfg = decode_model_configuration(open(os.path.join(CONFIG_DIR, name)).read())
        assert cfg.schema_version == 1
    tp = decode_model_configuration(open(os.path.join(CONFIG_DIR, "owner-tp-scaled656.json")).read())
    assert tp.options.native_kv_format == "scaled656" and tp.options.prefetch.completion == "layer"
    dpa = decode_model_configuration(open(os.path.join(CONFIG_DIR, "b200-native-dpa.json")).read())
    assert dpa.options.device_record_capacity == 1048576


@pytest.mark.parametrize("doc", [
    {"schema_version": 2, "adapter": "native"},
    {"schema_version": 1, "adapter": "nope"},
    {"schema_version": 1, "adapter": "native", "options": {"x": 1}},
    {"schema_version": 1, "adapter": "native_tp", "capacity": {"device_token_capacity_per_owner": 64, "host_token_capacity_per_owner": 0}},
    {"schema_version": 1, "adapter": "dsa"},
    {"schema_version": 1, "adapter": "dsa", "capacity": {"device_token_capacity_per_owner": 64}},
    {"schema_version": 1, "adapter": "native_tp", "framework_release": "v0.5.22", "options": {"cache_capacity_multiplier": 2}},
    {"schema_version": 1, "adapter": "native_tp", "framework_release": "v0.5.22", "options": {"unknown": 1}},
    {"schema_version": 1, "adapter": "native", "surprise": True},
])
def test_bad_configurations_are_rejected(doc):
    with pytest.raises(ConfigurationError):
        decode_model_configuration(json.dumps(doc))


def test_duplicate_keys_are_rejected():
    with pytest.raises(ConfigurationError):
        decode_model_configuration('{"schema_version": 1, "adapter": "native", "adapter": "native"}')


def test_capacity_planner_maximises_total_then_device_share():
    measure = simple_usage_model(record_bytes=656, layers=4, index_layers=4, metadata_groups=4)
    budget = CacheMemoryBudget(device_bytes=2_000_000_000, host_bytes=1_000_000_000)
    plan = plan_cache_capacity(memory_budget=budget, measure_memory_usage=measure, minimum_device_token_capacity=64,
                               maximum_token_capacity_per_owner=1 << 26, storage_owner_count=8)
    assert budget.contains(plan.usage)
    d, h = plan.device_token_capacity_per_owner, plan.host_token_capacity_per_owner
    assert d % 64 == 0 and h % 64 == 0
    # one more page anywhere breaks the budget
    assert not budget.contains(measure(d + 64, h)) and not budget.contains(measure(d, h + 64))
    assert plan.unique_token_capacity == 8 * (d + h)
    assert request_history_capacity(64, 2048, 3.0) == 64 * 2048 * 3


def test_workspace_colouring_and_pool_report():
    lifetimes = [AttentionWorkspaceLifetime(0, 0, 2), AttentionWorkspaceLifetime(1, 3, 5), AttentionWorkspaceLifetime(2, 2, 3)]
    colours, n = colour_workspaces(lifetimes)
    assert n == 2 and colours[0] == colours[1] != colours[2]
    rep = PoolLayout(layers=4, groups=2, record_bytes=656, slots_per_rank=1024, max_queries=8, topk=128).report()
    assert rep["total"] == sum(v for k, v in rep.items() if k != "total")


def test_speculative_contracts():
    LinearVerifyConfig("EAGLE", 2, 1, 3).validate()
    for bad in (LinearVerifyConfig("EAGLE", 2, 2, 3), LinearVerifyConfig("EAGLE", 2, 1, 4), LinearVerifyConfig("tree", 2, 1, 1)):
        with pytest.raises(NotImplementedError):
            bad.validate()
    table = torch.arange(6).view(2, 3)
    rows, lengths = expand_verify_rows(table, torch.tensor([100, 7]), 3)
    assert rows.shape == (6, 3) and lengths.tolist() == [101, 102, 103, 8, 9, 10]
    t, l = index_query_metadata("verify", rows, torch.tensor([100, 7]).repeat_interleave(3), lengths)
    assert l is lengths


def test_snapshot_round_trip(tmp_path):
    spec = make_spec(layers=2, device_pages=2, host_pages=8, queries=4, topk=64)
    cache = ula.init(spec, LocalCacheBindings(device="cpu"))
    ids = cache.alloc(300)
    lat, rope = random_kv(300, 5)
    for l in range(2):
        cache.write(ids, l, (lat + l, rope))
    layout = SnapshotLayout("test-model", owners=2, layers=2, mla_row_bytes=656)
    reqs = [SnapshotRequest("a", tuple(range(100)), (1, 2)), SnapshotRequest("b", tuple(range(150)), (3,))]
    req_ids = {"a": ids[:101], "b": ids[101:251]}
    path = str(tmp_path / "bank")
    for owner in range(2):
        cache_io.save_shard(cache, path, layout, reqs, req_ids, owner)
    with pytest.raises(ValueError):
        SnapshotReader(path)                       # not committed yet
    finalize_snapshot(path)
    assert cli.main(["verify", path]) == 0 and cli.main(["inspect", path]) == 0
    fresh = ula.init(spec, LocalCacheBindings(device="cpu"))
    new_ids = fresh.alloc(300)
    new_req = {"a": new_ids[:101], "b": new_ids[101:251]}
    assert cache_io.restore(fresh, path, new_req, verify_payload=True) == 2 * (101 + 150)
    for l in range(2):
        for c, idmap in ((cache, req_ids), (fresh, new_req)):
            c.begin_model_forward()
            c.access(idmap["b"][:64].view(1, 64), l)
            rows = c.gather_selected_records(l).clone()
            c.finish_layer_attention(l)
            c.finish_model_forward()
            if c is cache:
                want = rows
        assert torch.equal(rows, want)
    # a part of the bank, read back through the cache after every chunk; the page tail of the allocation is released
    part = ula.init(spec, LocalCacheBindings(device="cpu"))
    part_ids = part.alloc(192)                                   # three pages for a history of 150 + 1 tokens
    assert cache_io.restore(part, path, {"b": part_ids}, verify_restored=True) == 2 * 150
    before = part.counters()["registered"]
    assert cache_io.release_unwritten_padding(part, part_ids, 150) == 42
    assert part.counters()["registered"] == before - 2 * 42     # (counted once per residency group)
    with pytest.raises(ValueError):
        cache_io.restore(part, path, {"c": part_ids})            # not a request of this bank
    with pytest.raises(ValueError):
        cache_io.release_unwritten_padding(part, part_ids, 0)
    # corrupt one byte: verification must fail
    f = os.path.join(path, "owner_000", "request_00000.mla_000.bin")
    raw = bytearray(open(f, "rb").read())
    raw[10] ^= 0xFF
    open(f, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        SnapshotReader(path).verify()
    with pytest.raises(ValueError):            # payload verification is the default of a restore
        cache_io.restore(ula.init(spec, LocalCacheBindings(device="cpu")), path, new_req)
    # a committed directory is never written into again, and cannot be committed twice
    with pytest.raises(FileExistsError):
        cache_io.save_shard(cache, path, layout, reqs, req_ids, 0)
    with pytest.raises(FileExistsError):
        finalize_snapshot(path)


def _write_owner_shard(args):
    path, owner, keys = args
    from ulacache_b200.tools.snapshot.format import SnapshotLayout, SnapshotRequest, SnapshotWriter

    layout = SnapshotLayout("m", owners=4, layers=3, mla_row_bytes=16, index_anchors=(0,), index_segment_bytes=(8, 4))
    reqs = [SnapshotRequest(k, tuple(range(37 + i)), (5,)) for i, k in enumerate(keys)]
    w = SnapshotWriter(path, layout, reqs, owner)
    for req in reqs:
        for plane, width in layout.planes().items():
            rows = req.owned_rows(owner, layout.owners)
            w.write_plane(req.key, plane, [bytes([owner]) * (rows * width)])
    return w.finish()["metadata_sha256"]


def test_snapshot_owners_write_in_parallel_processes_and_disagreement_is_refused(tmp_path):
    import multiprocessing as mp

    from ulacache_b200.tools.snapshot.format import SnapshotWriter

    path = str(tmp_path / "par")
    ctx = mp.get_context("spawn")
    with ctx.Pool(4) as pool:
        hashes = pool.map(_write_owner_shard, [(path, o, ("a", "b", "c")) for o in range(4)])
    assert len(set(hashes)) == 1
    commit = finalize_snapshot(path)
    assert commit["request_count"] == 3 and sorted(commit["owners"]) == ["0", "1", "2", "3"]
    r = SnapshotReader(path)
    assert r.verify()["verified_bytes"] == sum(os.path.getsize(os.path.join(path, f"owner_{o:03d}", n))
                                               for o in range(4) for n in os.listdir(os.path.join(path, f"owner_{o:03d}"))
                                               if n.endswith(".bin"))
    assert b"".join(r.iter_plane(2, "b", "index_000")) == bytes([2]) * (r.plane_rows(2, "b") * 12)
    # an owner that saved the requests under other keys (same sizes, other metadata) is refused at commit
    bad = str(tmp_path / "bad")
    for o in (0, 1, 2):
        _write_owner_shard((bad, o, ("a", "b", "c")))
    _write_owner_shard((bad, 3, ("a", "c", "b")))
    with pytest.raises(ValueError):
        finalize_snapshot(bad)
    # the same owner cannot write twice into one snapshot directory
    with pytest.raises(FileExistsError):
        _write_owner_shard((bad, 0, ("a", "b", "c")))


def test_every_shipped_model_configuration_loads():
    import glob
    import os

    from ulacache_b200.config.model_configuration import decode_model_configuration

    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ulacache_b200", "config", "models")
    files = sorted(glob.glob(os.path.join(here, "*.json")))
    assert len(files) >= 11
    adapters = set()
    for f in files:
        with open(f) as fh:
            cfg = decode_model_configuration(fh.read())
        adapters.add(cfg.adapter)
    assert {"native", "native_tp", "native_dpa", "dsa", "glm_flash", "paged", "qsa"} <= adapters


def test_restore_routing_per_layout():
    from ulacache_b200.tools.snapshot.bank import restore_routing, shard_positions

    keys = ["a", "b", "c"]
    dpa = restore_routing(2, keys, world=2, mode="dpa")
    assert [(s.owner, s.request) for s in dpa[0]] == [(0, "a"), (1, "a"), (0, "c"), (1, "c")]
    assert [(s.owner, s.request) for s in dpa[1]] == [(0, "b"), (1, "b")] and dpa[1][0].keep == "all"
    placed = restore_routing(1, keys, world=4, mode="dpa", placement={"a": 3, "b": 3, "c": 0})
    assert [len(p) for p in placed] == [1, 0, 0, 2]
    tp = restore_routing(4, keys, world=8, mode="tp")
    assert all(len(p) == 12 and p[0].keep == "owned" for p in tp)
    assert restore_routing(4, keys, world=8, mode="tp", kv_layout="replicated")[5][0].keep == "all"
    assert list(shard_positions(1, 4, 11)) == [1, 5, 9]
    with pytest.raises(ValueError):
        restore_routing(1, keys, world=2, mode="dpa", placement={"a": 0, "b": 2, "c": 0})


def test_prefix_tree_rebuilt_from_snapshot_requests():
    from ulacache_b200.serving.radix_tree import RadixPrefixTree
    from ulacache_b200.tools.snapshot.bank import rebuild_prefix_tree
    from ulacache_b200.tools.snapshot.format import SnapshotRequest

    shared = list(range(100, 228))                          # two pages of 64 tokens
    r1 = SnapshotRequest("one", shared + list(range(500, 570)), [7, 8])
    r2 = SnapshotRequest("two", shared + list(range(900, 964)), [9])
    tree = RadixPrefixTree()
    dup = rebuild_prefix_tree(tree, [r1, r2], {"one": [10, 11, 12, 13], "two": [20, 21, 22]})
    assert dup == {"one": 0, "two": 2}                      # request two's copies of the shared pages are duplicates
    hit = tree.match(shared + list(range(900, 964)) + [1, 2, 3])
    assert [n.page for n in hit] == [10, 11, 22]
    with pytest.raises(ValueError):
        rebuild_prefix_tree(RadixPrefixTree(), [r1], {"one": [10]})


def test_speculative_continuation_round_trip(tmp_path):
    import torch
    from ulacache_b200.tools.snapshot.bank import load_continuation, save_continuation

    saved_ids = torch.tensor([640, 641, 642, 643, 704, 705], dtype=torch.int32)      # logical ids of positions 0..5
    sel = torch.tensor([[705, 640, -1, 642]], dtype=torch.int32)
    path = tmp_path / "cont.pt"
    sha = save_continuation(path, hidden_state=torch.randn(1, 16), draft_tokens=torch.tensor([[5, 6, 7]]),
                            selection_ids=sel, request_ids=saved_ids)
    restored_ids = torch.tensor([64, 65, 66, 67, 128, 129], dtype=torch.int32)       # the restored run's ids differ
    out = load_continuation(path, sha, request_ids=restored_ids)
    assert out["selection_ids"].tolist() == [[129, 64, -1, 66]] and out["draft_tokens"].tolist() == [[5, 6, 7]]
    assert out["draft_probs"] is None and out["hidden_state"].shape == (1, 16)
    with pytest.raises(ValueError):
        load_continuation(path, "0" * 64, request_ids=restored_ids)
    with pytest.raises(FileExistsError):
        save_continuation(path, hidden_state=torch.zeros(1, 4))
    with pytest.raises(ValueError):
        save_continuation(tmp_path / "bad.pt", hidden_state=torch.zeros(1, 4), selection_ids=torch.tensor([[999]]),
                          request_ids=saved_ids)


def test_pool_adapters_plan_and_build_every_family():
    """Every shipped configuration that enables the cache becomes a pool plan; a GPU budget cuts the device
    tier and moves the difference to the host tier; single-owner plans build a working cache on CPU."""
    import glob
    import os

    import torch
    from ulacache_b200.config.model_configuration import load_model_configuration
    from ulacache_b200.serving.pools import plan_pool

    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ulacache_b200", "config", "models")
    seen = set()
    for path in sorted(glob.glob(os.path.join(here, "*.json"))):
        cfg = load_model_configuration(path)
        if not cfg.enabled or cfg.device_token_capacity_per_owner is None:
            continue
        plan = plan_pool(cfg, layers=4, world=8, max_queries=8)
        seen.add(plan.adapter)
        assert plan.device_records % 64 == 0 and plan.gpu_bytes > 0 and plan.bytes["device_records"] > 0
        tight = plan_pool(cfg, layers=4, world=8, max_queries=8, gpu_budget_bytes=plan.gpu_bytes * 2 // 3)
        assert tight.device_records < plan.device_records and tight.gpu_bytes <= plan.gpu_bytes * 2 // 3
        assert tight.device_records + tight.host_records == plan.device_records + plan.host_records
        if plan.adapter == "glm_flash":
            assert plan.index_compression_ratio == 4 and plan.index_pages < (plan.device_records + plan.host_records) // 64
        if plan.adapter == "paged":
            assert plan.compression_ratios == (1, 2) and len(plan.planes) == 2
            one = plan_pool(cfg, layers=4, world=8, max_queries=8).bytes["device_records"]
            assert one == int(plan.device_records * 2 * 1152 * 4 * 1.5)
    assert {"glm_flash", "paged", "qsa"} <= seen
    # a budget too small for the fixed charges is refused before anything is allocated
    cfg = load_model_configuration(os.path.join(here, "qsa-regions-cpu-ngram.json"))
    with pytest.raises(MemoryError):
        plan_pool(cfg, layers=2, world=1, gpu_budget_bytes=1 << 16)
    # single-owner plans of every family build a cache that allocates on CPU
    import json

    from ulacache_b200.config.model_configuration import decode_model_configuration

    for adapter, opts, engine in (("qsa", {"maximum_write_record_count": 512}, "NativePagedResidency"),
                                  ("glm_flash", {"prefill_buffer_records": 0}, "UnifiedLocalResidency"),
                                  ("paged", {"storage_owner_count": 1}, "NativePagedResidency")):
        small = decode_model_configuration(json.dumps({
            "schema_version": 1, "adapter": adapter,
            "capacity": {"device_token_capacity_per_owner": 4096, "host_token_capacity_per_owner": 8192}, "options": opts}))
        plan = plan_pool(small, layers=2, world=1, max_queries=2, topk=64)
        assert plan.engine == "local" and plan.owners == 1
        cache = plan.build("cpu")
        assert type(cache.engine).__name__ == engine
        ids = cache.alloc(128)
        assert ids is not None and ids.numel() == 128
        cache.free(ids)
