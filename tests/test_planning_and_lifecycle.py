import pytest

from ulacache_b200.cache.attention_access import LifecycleError, NativeSparseCacheExecution
from ulacache_b200.cache.layers import LayerReuseSpecification
from ulacache_b200.cache.planning import lower_layer_reuse
from ulacache_b200.cache.pool_lifecycle import PoolLifecycle
from ulacache_b200.cache.prefetch import FollowerPrefetcher
from ulacache_b200.cache_config import PrefetchPolicy


def test_lowering_groups_banks_domains_and_workspaces():
    # 6 layers: selection shared in groups {0,1,2} and {3,4}; layer 5 alone; KV of 4 aliases 3
    spec = LayerReuseSpecification.from_layer_groups(6, key_value_groups=[(3, 4)], selection_groups=[(0, 1, 2), (3, 4)])
    plan = lower_layer_reuse(spec)
    assert plan.describe() == {"layers": 6, "storage_banks": 5, "index_banks": 6, "residency_domains": 3,
                               "attention_workspaces": 1}
    assert plan.is_anchor(0) and not plan.is_anchor(2) and plan.followers(1) == (1, 2)
    assert plan.bank_of_layer[3] == plan.bank_of_layer[4] and plan.domains[1].banks == (plan.bank_of_layer[3],)
    assert plan.selection_producer == (0, 0, 0, 3, 3, 5)
    # interleaved domains cannot share a workspace
    inter = LayerReuseSpecification.from_layer_groups(4, selection_groups=[(0, 2), (1, 3)])
    assert lower_layer_reuse(inter).workspace_count == 2


def test_domain_with_mixed_selection_is_rejected():
    bad = LayerReuseSpecification((0, 1), (0, 1), (0, 1), (0, 0))
    with pytest.raises(ValueError):
        lower_layer_reuse(bad)


def test_prefetcher_and_lifecycle_order():
    done = []
    pf = FollowerPrefetcher(PrefetchPolicy(enabled=True), "native_paged")
    pf.launch([1, 2], done.append)
    pf.wait(1)
    assert done == [1, 2] and pf.completion == "layer" and pf.pending() == 0
    order = []
    with PoolLifecycle() as life:
        life.on_quiesce(lambda: order.append("quiesce"))
        life.on_close(lambda: order.append("free pool"))
        life.on_close(lambda: order.append("unmap peers"))
    assert order == ["quiesce", "unmap peers", "free pool"] and life.closed


class _Client:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        return lambda *a, **k: self.calls.append(name) or "view"


def test_execution_lifecycle_enforces_order():
    c = _Client()
    ex = NativeSparseCacheExecution(c, 2)
    with pytest.raises(LifecycleError):
        ex.prepare(0, None)
    ex.begin()
    with pytest.raises(LifecycleError):
        ex.view(0)
    ex.prepare(0, "sel", "cur")
    ex.publish(0, "ids", "vals")
    assert ex.view(0) == "view"
    with pytest.raises(LifecycleError):
        ex.finish()
    ex.finish_layer(0)
    ex.finish()
    assert c.calls == ["begin_model_forward", "prepare_sparse_attention", "write", "get_resident_attention_inputs",
                       "finish_layer_attention", "finish_model_forward"]
    ex.begin(); ex.abort()
    assert c.calls[-1] == "abort_model_forward"


def test_shared_selection_lifecycle_orders_plans_pulls_and_joins():
    import pytest
    from ulacache_b200.cache.layers import LayerReuseSpecification
    from ulacache_b200.cache.prefetch import SharedSelectionLifecycle
    from ulacache_b200.cache_config import PrefetchPolicy
    from ulacache_b200.transfer.prefill_pipeline import HostStreamRuntime

    groups = LayerReuseSpecification.from_layer_groups(5, selection_groups=((0, 1, 2), (3, 4))).residency_groups()
    calls = []
    published = []

    def make(prefetch, rt=None):
        calls.clear()
        return SharedSelectionLifecycle(groups, plan_selection=lambda l, s: calls.append(("plan", l)),
                                        pull_history=lambda l, a: calls.append(("pull", l, a)),
                                        publish_step=lambda: published.append(1), prefetch=prefetch, runtime=rt)

    def forward(life):
        life.begin_forward()
        for layer in range(5):
            life.before_layer_prepare(layer)
            if layer in groups.anchors:
                life.on_selection_ready(layer, object())
            life.before_history_consume(layer)
            life.after_attention(layer)
        life.finish_forward()

    # without prefetch: plan at the anchor, every layer pulls just before it reads
    life = make(False)
    forward(life)
    assert calls == [("plan", 0), ("pull", 0, True), ("pull", 1, False), ("pull", 2, False), ("plan", 3),
                     ("pull", 3, True), ("pull", 4, False)]
    assert published == [1] and life.plans == 2 and life.pulls == 5 and not life.in_forward

    # with prefetch, one event per follower layer: the anchor's pull follows its plan at once, the followers'
    # pulls are queued when the anchor's attention has been launched, every follower joins its own event
    rt = HostStreamRuntime()
    life = make(PrefetchPolicy(enabled=True, completion="layer"), rt)
    forward(life)
    assert calls == [("plan", 0), ("pull", 0, True), ("pull", 1, False), ("pull", 2, False), ("plan", 3),
                     ("pull", 3, True), ("pull", 4, False)]
    ev1 = life._layer_ready[1]
    rec = [i for i, e in enumerate(rt.log) if e[:2] == ("record", ev1)]
    wait = [i for i, e in enumerate(rt.log) if e[:1] == ("wait_event",) and e[2] == ev1]
    assert rec and wait and rec[0] < wait[0]
    assert sum(1 for e in rt.log if e[0] == "wait_event") == 2 + 3     # two anchors, three followers

    # one event per group: only the first follower joins
    rt = HostStreamRuntime()
    life = make(PrefetchPolicy(enabled=True, completion="group"), rt)
    forward(life)
    assert sum(1 for e in rt.log if e[0] == "wait_event") == 2 + 2

    # misuse is refused
    life = make(True, HostStreamRuntime())
    life.begin_forward()
    with pytest.raises(RuntimeError):
        life.begin_forward()
    with pytest.raises(RuntimeError):
        life.join_idle_prefetch()
    with pytest.raises(RuntimeError):
        life.before_history_consume(0)                     # no plan yet
    with pytest.raises(RuntimeError):
        life.on_selection_ready(1, object())               # not an anchor
    life.on_selection_ready(0, object())
    with pytest.raises(RuntimeError):
        life.on_selection_ready(0, object())               # planned twice
    with pytest.raises(RuntimeError):
        life.before_layer_prepare(1)                       # follower not scheduled: the anchor has not attended
    with pytest.raises(RuntimeError):
        life.finish_forward()                              # unconsumed layers
    life.abort_forward()
    assert not life.in_forward
    life.join_idle_prefetch()
    with pytest.raises(TypeError):
        SharedSelectionLifecycle(groups, plan_selection=print, pull_history=print, prefetch="yes")


def test_framework_adapter_decode_prefill_reconstruction_and_pages():
    import pytest
    import torch
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.cache.attention_access import FrameworkCacheExecution, LifecycleError, WriterStaging
    from ulacache_b200.ops import records
    from helpers import make_spec, random_kv

    spec = make_spec(layers=3, device_pages=4, host_pages=16, queries=8, topk=32, shared_groups=((0, 1),))
    import dataclasses

    b = LocalCacheBindings(device="cpu")
    b = dataclasses.replace(b, execution_options=dataclasses.replace(b.execution_options, record_storage_backend="native_paged"))
    cache = ula.init(spec, b)
    ids = cache.alloc(600)
    latent, rope = random_kv(600, 4)
    enc = records.encode_scaled656(latent, rope)
    for layer in range(3):
        cache.write(ids, layer, enc)
    pos = {int(i): n for n, i in enumerate(ids.tolist())}
    staging = WriterStaging()
    fx = FrameworkCacheExecution(cache, 3, device="cpu", query_capacity=8, writer_staging=staging,
                                 prefill_chunk_capacity=100)
    with pytest.raises(LifecycleError):
        fx.prepare_attention(0, ids[:8].reshape(2, 4))                 # no forward open

    # ---- a decode-like forward: 3 real queries padded to 4, the writer staged 3 new records per layer ----
    new = cache.alloc(3)
    sel = torch.stack([ids[torch.randperm(600, generator=torch.Generator().manual_seed(q))[:32]] for q in range(4)]).to(torch.int32)
    fx.begin_forward(decode_like=True, query_count=4)
    for layer in range(3):
        fresh = torch.full((3, 656), 50 + layer, dtype=torch.uint8)
        staging.stage(layer, new, fresh)
        rows = fx.prepare_attention(layer, sel.reshape(4, 1, 32))
        assert rows.shape == (4, 1, 32) and bool((rows >= 0).all())
        got = cache.gather_selected_records(layer).view(4, 32, 656)
        assert torch.equal(got[0], enc[[pos[int(i)] for i in sel[0].tolist()]])
        back = cache.engine.read_records(layer, new)[0]
        assert bool((back == 50 + layer).all())                        # published after the transaction
        fx.finish_attention(layer)
    fx.finish()
    assert staging.published_records == 9 and staging.pending_logical_record_ids(0) is None

    # ---- an eager prefill forward through the engine's union ----
    fx.begin_forward(decode_like=False, query_count=4)
    staging.stage(2, new, torch.full((3, 656), 77, dtype=torch.uint8))
    fx.publish_after_native_write(2)
    assert bool((cache.engine.read_records(2, new)[0] == 77).all())
    for layer in (0, 1, 2):
        rows = fx.prepare_attention(layer, sel)
        got = cache.engine.layer_plane(layer)[rows[1].long()]
        assert torch.equal(got, enc[[pos[int(i)] for i in sel[1].tolist()]])
        fx.finish_attention(layer)
    fx.finish()

    # ---- prefix reconstruction in chunks of 100 records ----
    prefix = ids[100:350].to(torch.int32)
    out = torch.zeros(250, 656, dtype=torch.uint8)
    chunks = []

    def read_native(planes, rows, dst):
        chunks.append(int(rows.numel()))
        dst.copy_(planes[0][rows.long()])

    fx.reconstruct_prefill_records(1, prefix, out, read_native)
    assert chunks == [100, 100, 50] and torch.equal(out, enc[100:350])

    # ---- page-granular registration, clear, inventory ----
    page = torch.tensor([int(ids.max()) // 64 + 2])
    fx.register_full_pages(page, prefer_device=False)
    assert cache.counters()["registered"] == 2 * (603 + 64)             # (counted once per residency group: two groups)
    fx.release_full_pages(page)
    assert cache.counters()["registered"] == 2 * 603
    assert len(fx.get_device_storage_inventory()) >= 3
    fx.clear_records()
    assert cache.counters()["registered"] == 2 * 63                    # only the reserved records of the first page
    with pytest.raises(ValueError):
        fx.begin_forward(decode_like=True, query_count=9)
    cache.close()


def test_plan_details_owner_lowering_and_specification_checks():
    import dataclasses
    from ulacache_b200.cache.planning import lower_for_record_owners, validate_rank_local_specification
    from ulacache_b200.cache.access import SparseAccessSpecification
    from ulacache_b200.cache.specification import MemoryTierCapacity
    from helpers import make_spec

    spec = LayerReuseSpecification.from_layer_groups(6, key_value_groups=[(3, 4)], selection_groups=[(0, 1, 2), (3, 4)])
    plan = lower_layer_reuse(spec)
    assert plan.selection_producers == (0, 3, 5) and plan.selection_index_of_layer == (0, 0, 0, 1, 1, 2)
    assert plan.last_consumer_of_selection == (2, 4, 5) and plan.step_reader_retirement_layer == 5
    assert plan.bank_ranges_of_domain == (((0, 3),), ((3, 4),), ((4, 5),))
    # record owners: one directory per KV bank; a selection shared by several banks is planned per bank
    shared = LayerReuseSpecification.from_layer_groups(4, key_value_groups=[(2, 3)], selection_groups=[(0, 1, 2, 3)])
    owner_plan = lower_for_record_owners(shared)
    assert owner_plan.describe()["residency_domains"] == 3 and owner_plan.selection_producer == (0, 1, 2, 2)
    assert owner_plan.step_reader_retirement_layer == 3

    good = make_spec(layers=4, shared_groups=((0, 1),))
    validate_rank_local_specification(good)
    with pytest.raises(ValueError):
        validate_rank_local_specification(dataclasses.replace(
            good, capacity_plan=MemoryTierCapacity(device_record_capacity=100, host_record_capacity=64,
                                                   maximum_write_record_count=64)))
    with pytest.raises(NotImplementedError):
        validate_rank_local_specification(dataclasses.replace(
            good, sparse_access=SparseAccessSpecification(16, 8, selection_unit="block", records_per_selected_unit=16)))
    with pytest.raises(NotImplementedError):                      # a selection shared across two directories
        validate_rank_local_specification(dataclasses.replace(
            good, layer_reuse=LayerReuseSpecification((0, 1, 2, 3), (0, 1, 2, 3), (0, 0, 2, 3), (0, 1, 2, 3))))


def _position_sharded_scenario(device):
    import torch
    import ulacache_b200 as ula
    from ulacache_b200.bindings import PositionShardBindings
    from ulacache_b200.cache.access import SparseAttentionAccessPlan
    from ulacache_b200.storage.layout import PositionShardLayout
    from helpers import make_spec

    spec = make_spec(layers=2, device_pages=4, host_pages=16, queries=4, topk=32)
    cache = ula.init(spec, PositionShardBindings(device=device, position_layout=PositionShardLayout(2), rank=1))
    eng = cache.engine
    ids = cache.alloc(400)
    sel = ids[torch.arange(4 * 32).reshape(4, 32)].to(torch.int32).to(device)
    cur = ids[300:304].to(torch.int32).to(device)
    cache.begin_model_forward()
    buf = eng.selected.data_ptr()
    eng.plan(0, SparseAttentionAccessPlan(sel, cur))
    counts = eng.selected_counts(0)
    assert counts.tolist() == [int(((sel[q] % 2) == 1).sum()) for q in range(4)]
    assert eng.selected.data_ptr() == buf and eng.selected_counts(0).data_ptr() == eng.selected_count[0].data_ptr()
    mapped = eng._map_current(cur)                                # cached by the identity of the tensor
    assert mapped.tolist() == [int(i) // 2 if int(i) % 2 == 1 else -1 for i in cur.tolist()]
    eng.current[:4] = 123
    assert eng._map_current(cur).tolist() == [123] * 4           # same tensor: not recomputed
    eng.after_attention(0)
    cache.finish_model_forward()
    assert eng._current_signature is None
    cache.begin_model_forward()
    with pytest.raises(ValueError):
        eng.plan(0, SparseAttentionAccessPlan(torch.ones(5, 32, dtype=torch.int32, device=device), None))   # too many queries
    with pytest.raises(ValueError):
        eng.plan(0, SparseAttentionAccessPlan(sel, cur[:3]))                                  # current per query
    cache.abort_model_forward()
    with pytest.raises(NotImplementedError):
        eng.allocate_receive_rows(ids[:4])
    with pytest.raises(NotImplementedError):
        eng.plan_prefill(0, sel)
    inv = eng.memory_inventory()
    assert inv["record_distribution"] == "position_modulo_cp" and inv["storage_owner_count"] == 2
    assert inv["additional_mapping_bytes"] == (2 * 4 * 32 + 2 * 4 + 4) * 4 and len(eng.device_storage_inventory()) >= 3
    # a full step through the public API: this rank's share of every selection resolves to its local rows
    lat, rope = torch.randn(400, 512, device=device), torch.randn(400, 64, device=device)
    cache.write(ids.to(device), 0, (lat, rope))
    cache.begin_model_forward()
    view = cache.access(sel, 0)
    counts = eng.selected_counts(0)
    loc = view.device_record_indices
    for q in range(4):
        c = int(counts[q])
        assert bool((loc[q, :c] >= 0).all())
    cache.finish_layer_attention(0)
    cache.finish_model_forward()
    cache.check("position-sharded step")
    cache.close()


def test_position_sharded_engine_bounds_buffers_and_inventory():
    _position_sharded_scenario("cpu")


@pytest.mark.gpu
def test_position_sharded_engine_on_the_gpu(native):
    _position_sharded_scenario("cuda")
