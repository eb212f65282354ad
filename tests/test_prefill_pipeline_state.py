"""Prefill subsystem beyond the windows: admission budget, request groups, reusable read plans, request-group
buffers, prefix page leases, full-history plans with fresh-row installation, and the layer pipeline's ordering."""
import pytest
import torch

from ulacache_b200.cache.layers import LayerReuseSpecification
from ulacache_b200.cache.prefill import (PrefillMaterializer, PrefillReadPlans, PrefillSequenceBudget, PrefillWindow,
                                         PrefixPageLeases, ReadOnlyPrefillReader, RequestPrefillBuffers,
                                         WindowedPrefillReader, prefill_physical_tokens, prefill_request_groups,
                                         prepare_history_read_plan, prepare_query_groups, request_query_ranges)
from ulacache_b200.transfer.prefill_pipeline import HistoryPrefillPipeline, HostStreamRuntime, allocate_prefill_windows


class _Engine:
    """Records 1..n of 16 bytes per layer; record i of layer l is filled with (i + 7 * l) % 251."""

    def __init__(self, n=200, rb=16, layers=3):
        self.n, self.rb = n, rb
        self.store = {l: ((torch.arange(n + 1)[:, None] + 7 * l) % 251).to(torch.uint8).repeat(1, rb) for l in range(layers)}
        self.reads = []

    def read_records(self, layer, ids):
        self.reads.append((layer, int(ids.numel())))
        return self.store[layer][ids.long()], torch.ones(ids.numel(), dtype=torch.bool)


def test_sequence_budget_and_request_groups():
    b = PrefillSequenceBudget(100)
    assert b.can_reserve(30, 20)
    b.reserve(30, 20)
    assert not b.can_reserve(40, 20)
    with pytest.raises(RuntimeError):
        b.reserve(40, 20)
    with pytest.raises(ValueError):
        b.can_reserve(90, 20)                                   # one sequence larger than the window
    with pytest.raises(ValueError):
        b.can_reserve(-1, 2)
    b.reset()
    assert b.can_reserve(60, 40)
    # whole requests merge while they fit; a long one is cut into window-sized pieces of its own
    assert list(prefill_request_groups([30, 30, 50, 0, 10], 64)) == [(0, 60), (60, 60)]
    assert list(prefill_request_groups([10, 150, 20], 64)) == [(0, 10), (10, 64), (74, 64), (138, 22), (160, 20)]
    assert list(prefill_request_groups([], 8)) == []
    with pytest.raises(ValueError):
        list(prefill_request_groups([3, -1], 8))


def test_query_groups_respect_requests_chunks_and_the_window():
    assert request_query_ranges([2, 0, 3], 5) == ((0, 0, 2), (2, 2, 5))
    with pytest.raises(ValueError):
        request_query_ranges([2, 2], 5)
    sel = torch.tensor([[1, 2, 3, 0], [2, 3, 4, -1], [10, 11, 12, 13], [20, 21, 22, 23], [30, 31, 32, 33]], dtype=torch.int32)
    groups = prepare_query_groups(sel, [2, 3], capacity=8, query_chunk=2)
    assert [(g.request, g.start, g.stop) for g in groups] == [(0, 0, 2), (1, 2, 4), (1, 4, 5)]
    assert groups[0].records.tolist() == [1, 2, 3, 4] and groups[0].indices.tolist() == [[0, 1, 2, -1], [1, 2, 3, -1]]
    tight = prepare_query_groups(sel, [2, 3], capacity=4, query_chunk=4)      # request 1's union (12) must split
    assert [(g.start, g.stop) for g in tight] == [(0, 2), (2, 3), (3, 4), (4, 5)]
    with pytest.raises(ValueError):
        prepare_query_groups(sel, [2, 3], capacity=3)                         # a single selection does not fit
    joint = prepare_query_groups(sel[:2], [2], capacity=8, union=lambda ids: torch.unique(torch.cat([ids, torch.tensor([7, 9], dtype=torch.int32)])))
    assert joint[0].records.tolist() == [1, 2, 3, 4, 7, 9] and joint[0].indices.tolist() == [[0, 1, 2, -1], [1, 2, 3, -1]]


def test_request_prefill_buffers_alternate_windows_between_groups():
    eng = _Engine()
    buf = RequestPrefillBuffers(ReadOnlyPrefillReader(eng), 16, 8, "cpu", query_chunk=2)
    sel = torch.tensor([[1, 2, 3, 4], [2, 3, 4, 5], [10, 11, 12, 13], [20, 21, 22, -1], [30, 31, 32, 33]], dtype=torch.int32)
    q = torch.arange(5).float()[:, None]
    seen = []

    def attend(qs, data, rows):
        seen.append(data.data_ptr())
        vals = data[rows.clamp(min=0).long(), 0].float() * (rows >= 0)
        return vals.sum(1, keepdim=True) + qs

    buf.begin_forward([2, 3])
    with pytest.raises(RuntimeError):
        buf.run(q, sel, attend)                                   # nothing selected yet
    buf.select(1, sel)
    with pytest.raises(RuntimeError):
        buf.select(1, sel)
    out = buf.run(q, sel, attend)
    want = torch.stack([((sel[i][sel[i] > 0] + 7) % 251).float().sum() + i for i in range(5)])[:, None]
    assert torch.equal(out, want)
    assert buf.group_count == 3 and buf.maximum_union == 7 and buf.copy_count == 5 + 7 + 4
    assert seen[0] != seen[1] and seen[0] == seen[2]              # the two windows alternate
    prefix = torch.tensor([5, 6, 7, 8, 9], dtype=torch.int32)
    rows = buf.read_records(2, prefix, lambda data, r: data[r.long(), :2].float())
    assert rows[:, 0].tolist() == [((i + 14) % 251) for i in range(5, 10)] and buf.query_counts == (2, 3)
    assert len(buf.inventory()) == 2
    buf.close()


def test_prefix_page_leases_and_physical_demand():
    pl = PrefixPageLeases()
    assert pl.acquire("a", {1: 11, 2: 12}) == [1, 2]
    assert pl.acquire("b", {2: 12, 3: 13}) == [2, 3]
    assert pl.acquire("a", {2: 12}) == [] and pl.readers(2) == 2
    with pytest.raises(ValueError):
        pl.acquire("c", {5: 15, 2: 99})                           # page 2 moved under its readers: nothing is acquired
    assert pl.readers(5) == 0
    with pytest.raises(ValueError):
        pl.acquire("c", {0: 3})
    with pytest.raises(ValueError):
        pl.assert_reclaimable([3])
    assert pl.release("a") == {1: 11}                              # page 2 still has reader b
    with pytest.raises(ValueError):
        pl.release("b", [1])
    assert pl.release("b", [2]) == {2: 12} and pl.release("b") == {3: 13} and pl.release("b") == {}
    pl.assert_reclaimable([1, 2, 3])
    assert prefill_physical_tokens(prefix_tokens=1000, held_prefix_tokens=300, extend_tokens=130, hot_tokens=256,
                                   scratch_tokens=64, page_size=64) == 704 + 192 + 256 + 64 + 64
    with pytest.raises(ValueError):
        prefill_physical_tokens(prefix_tokens=1, held_prefix_tokens=0, extend_tokens=-1, hot_tokens=0, scratch_tokens=0,
                                page_size=64)


def test_read_plans_are_built_once_per_forward_and_group():
    eng = _Engine()
    reader = WindowedPrefillReader(ReadOnlyPrefillReader(eng), PrefillWindow(64, 16, "cpu"), bound=64)
    groups = LayerReuseSpecification.from_layer_groups(3, selection_groups=((0, 1),)).residency_groups()
    plans = PrefillReadPlans(reader, groups, capacity=128)
    rows = torch.arange(1, 101, dtype=torch.int32)                # two requests of 60 and 40 rows
    take = lambda data, r: data[r.long(), :1].float()
    for layer in range(3):
        out = plans.read(layer, rows, take, request_lengths=(60, 40))
        assert out.reshape(-1).tolist() == [float((i + 7 * layer) % 251) for i in range(1, 101)]
    assert plans.plans_built == 2                                  # (60) and (40): the windows hold 64
    idx = torch.tensor([[0, 5, 99, -1], [5, 6, 7, 8]], dtype=torch.int32)
    recs0, remap0 = plans.read_selected(0, rows, idx, take, request_lengths=(60, 40))
    recs1, remap1 = plans.read_selected(1, rows, idx, take, request_lengths=(60, 40))   # same group: same plan
    assert plans.plans_built == 3 and torch.equal(remap0, remap1)
    assert recs0.reshape(-1).tolist() == [float(i % 251) for i in (1, 6, 7, 8, 9, 100)]
    assert remap0.tolist() == [[0, 1, 5, -1], [1, 2, 3, 4]]
    plans.read_selected(2, rows, idx, take, request_lengths=(60, 40))                   # another group: a new plan
    assert plans.plans_built == 4
    plans.reset()
    with pytest.raises(ValueError):
        plans.read(0, rows, take, request_lengths=(60, 41))
    with pytest.raises(ValueError):
        plans.read(0, torch.arange(1, 201, dtype=torch.int32), take)


def test_history_plan_installs_the_chunks_own_records_and_the_pipeline_keeps_order():
    eng = _Engine()
    history = torch.tensor([[3, 4, 5, 6], [4, 9, 0, 0]], dtype=torch.int32)          # 0 = padding
    current = torch.tensor([9, 50], dtype=torch.int32)
    plan = prepare_history_read_plan(history, current, capacity_records=16)
    assert plan.record_ids.tolist() == [3, 4, 5, 6, 9, 50] and plan.fresh_positions.tolist() == [-1, -1, -1, -1, 0, 1]
    assert plan.input_record_rows.tolist() == [[0, 1, 2, 3], [1, 4, -1, -1]]
    assert plan.map_rows(torch.tensor([50, 7, 0, 3])).tolist() == [5, -1, -1, 0]
    with pytest.raises(ValueError):
        prepare_history_read_plan(history, current, capacity_records=4)

    mat = PrefillMaterializer(eng)
    rt = HostStreamRuntime()
    windows = allocate_prefill_windows("cpu", capacity_records=16, record_bytes=16)
    pipe = HistoryPrefillPipeline(windows, gather_history=mat.gather_history, install_current=mat.install_current, runtime=rt)
    with pytest.raises(ValueError):
        HistoryPrefillPipeline((windows[0], windows[0]), gather_history=mat.gather_history, install_current=mat.install_current)
    with pytest.raises(ValueError):
        pipe.begin(plan, layer_count=3, record_count=17)
    mat.begin()
    pipe.begin(plan, layer_count=3, record_count=plan.record_count, keepalive_tensors=plan.keepalive_tensors)
    with pytest.raises(RuntimeError):
        pipe.begin(plan, layer_count=3, record_count=6)
    with pytest.raises(RuntimeError):
        pipe.prepare(1)                                          # layers are consumed in order
    for layer in range(3):
        w = pipe.prepare(layer)
        assert w is windows[layer % 2]
        if layer == 1:                                           # a layer that never reads its window
            pipe.skip_unused(layer)
            continue
        with pytest.raises(RuntimeError):
            pipe.after_attention(layer)                          # not read yet
        fresh = torch.full((2, 16), 200 + layer, dtype=torch.uint8)
        mat.record_current(layer, current, fresh)
        w = pipe.read(layer)
        got = w.data[plan.input_record_rows.clamp(min=0).long(), 0]
        want = (history + 7 * layer) % 251
        want[1, 1] = 200 + layer                                 # id 9 was written by this chunk
        assert torch.equal(got[history > 0], want[history > 0].to(torch.uint8))
        assert int(w.data[5, 0]) == 200 + layer                  # id 50 exists only in the chunk
        pipe.after_attention(layer)
        with pytest.raises(RuntimeError):
            pipe.after_attention(layer)
    pipe.finish()
    mat.finish()
    assert pipe.forwards == 1 and mat.installed == 4 and pipe.memory_inventory()["encoded_window_bytes"] == 2 * 16 * 16
    # ordering the CUDA runtime would enforce: layer 2 reuses window 0 only after layer 0's retired event
    retired0 = pipe.retired[0]
    waits = [i for i, e in enumerate(rt.log) if e[:1] == ("wait_event",) and e[2] == retired0]
    records = [i for i, e in enumerate(rt.log) if e[:2] == ("record", retired0)]
    assert waits and records and records[0] < waits[0]
    # an unfinished forward must be aborted, not finished
    pipe.begin(plan, layer_count=2, record_count=6)
    pipe.prepare(0)
    with pytest.raises(RuntimeError):
        pipe.finish()
    pipe.abort()
    pipe.begin(plan, layer_count=1, record_count=6)
    pipe.prepare(0)
    mat.record_current(0, current, torch.zeros(2, 16, dtype=torch.uint8))
    pipe.read(0)
    pipe.after_attention(0)
    pipe.finish()
    pipe.close()


def _real_cache_pipeline(device):
    """The layer pipeline over a real cache: history gathered read-only (device and host tier), the chunk's records
    installed from the writer's bytes, residency counters untouched."""
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from helpers import make_spec, random_kv

    cache = ula.init(make_spec(layers=3, device_pages=4, host_pages=16), LocalCacheBindings(device=device))
    engine = cache.engine if hasattr(cache, "engine") else cache
    ids = cache.alloc(700)
    latent, rope = random_kv(700, 9)
    for layer in range(3):
        cache.write(ids, layer, (latent.to(device) * (layer + 1), rope.to(device)))
    before = dict(cache.counters())
    rb = engine.layer_plane(0).shape[-1]
    hist = ids[torch.randperm(700, generator=torch.Generator().manual_seed(2))[:400]].to(device).reshape(4, 100)
    current = torch.cat([hist[0, :3].reshape(-1), ids[690:695].to(device)]).to(torch.int32)
    plan = prepare_history_read_plan(hist, current, capacity_records=512)
    mat = PrefillMaterializer(engine)
    windows = allocate_prefill_windows(device, capacity_records=512, record_bytes=rb)
    pipe = HistoryPrefillPipeline(windows, gather_history=mat.gather_history, install_current=mat.install_current)
    mat.begin()
    pipe.begin(plan, layer_count=3, record_count=plan.record_count, keepalive_tensors=plan.keepalive_tensors)
    for layer in range(3):
        pipe.prepare(layer)
        fresh = torch.full((current.numel(), rb), 100 + layer, dtype=torch.uint8, device=device)
        mat.record_current(layer, current, fresh)
        w = pipe.read(layer)
        got = w.data[plan.input_record_rows.reshape(-1).long()]
        want = engine.read_records(layer, hist.reshape(-1))[0].clone()
        want[torch.isin(hist.reshape(-1), current)] = 100 + layer     # whatever the chunk wrote wins over the cache
        assert torch.equal(got, want)
        assert bool((w.data[plan.map_rows(ids[690:695].to(device)).long()] == 100 + layer).all())
        pipe.after_attention(layer)
    pipe.finish()
    after = dict(cache.counters())
    assert after["promotions"] == before["promotions"] and after["evictions"] == before["evictions"]
    cache.close()


def test_layer_pipeline_over_a_real_cache_cpu():
    _real_cache_pipeline("cpu")


@pytest.mark.gpu
def test_layer_pipeline_over_a_real_cache_gpu(native):
    _real_cache_pipeline("cuda")
