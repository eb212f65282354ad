"""Two gloo ranks drive the engines that the tensor-parallel oracle test does not: the record-owner
engine with INDEPENDENT selections per consumer, and the position-sharded (context-parallel) wrapper
whose partial attention results merge to the dense answer."""
import os
import socket

import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _owner_rank(rank, world, port, out):
    import torch.distributed as dist

    import ulacache_b200 as ula
    from ulacache_b200.bindings import RecordOwnerBindings
    from ulacache_b200.cache.owner_cache import RecordOwnerPagedResidency
    from ulacache_b200.ops import records
    from ulacache_b200.storage.layout import MLA_BF16

    from helpers import make_spec

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layers, queries, topk = 2, 4, 64
    spec = make_spec(layers=layers, device_pages=6, host_pages=40, queries=queries, topk=topk, plane=MLA_BF16)
    cache = ula.init(spec, RecordOwnerBindings(device="cpu", owner_process_group=dist.group.WORLD, rank=rank,
                                               world_size=world, native_selections_replicated=False))
    assert isinstance(cache.engine, RecordOwnerPagedResidency)
    torch.manual_seed(0)                                   # the namespace and the records are common
    n = 1500
    ids = cache.alloc(n)
    kv = []
    for layer in range(layers):
        latent = torch.randn(n, 512).to(torch.bfloat16).float()
        rope = torch.randn(n, 64).to(torch.bfloat16).float()
        cache.write(ids, layer, (latent, rope))
        kv.append(torch.cat([latent, rope], dim=1))
    g = torch.Generator().manual_seed(100 + rank)          # every consumer asks for something else
    checked = 0
    for step in range(4):
        cache.begin_model_forward()
        for layer in range(layers):
            pos = torch.stack([torch.randperm(n, generator=g)[:topk] for _ in range(queries)])
            sel = ids[pos].to(torch.int32)
            view = cache.access(sel, layer)
            assert bool((view.device_record_indices >= 0).all())
            window = records.decode_bf16(cache.gather_selected_records(layer)).view(queries, topk, 576)
            assert torch.equal(window, kv[layer][pos]), (rank, step, layer)
            checked += queries
            cache.finish_layer_attention(layer)
        cache.finish_model_forward()
    c = cache.counters()
    assert c["unserved"] == 0 and c["promotions"] > 0, c   # owners promoted records other ranks asked for
    cache.free(ids)
    cache.close()
    out[rank] = checked
    dist.destroy_process_group()


def test_record_owner_engine_serves_independent_selections():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_owner_rank, args=(2, _free_port(), out), nprocs=2, join=True)
    assert dict(out) == {0: 4 * 2 * 4, 1: 4 * 2 * 4}


def _cp_rank(rank, world, port, out):
    import torch.distributed as dist

    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings, PositionShardBindings
    from ulacache_b200.cache.position_residency import PositionShardedResidency, merge_partial_attention
    from ulacache_b200.ops import records
    from ulacache_b200.storage.layout import MLA_BF16, PositionShardLayout

    from helpers import make_spec

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layers, queries, topk, heads = 1, 3, 96, 2
    spec = make_spec(layers=layers, device_pages=4, host_pages=30, queries=queries, topk=topk, plane=MLA_BF16)
    cache = ula.init(spec, PositionShardBindings(device="cpu",
                                                 position_layout=PositionShardLayout(world), rank=rank))
    assert isinstance(cache.engine, PositionShardedResidency)
    torch.manual_seed(1)
    n = 1200
    ids = cache.alloc(n)                                   # global slots; rank r keeps slot % world == r
    latent = torch.randn(n, 512).to(torch.bfloat16).float()
    rope = torch.randn(n, 64).to(torch.bfloat16).float()
    cache.write(ids, 0, (latent, rope))
    full = torch.cat([latent, rope], dim=1)
    row_of = {int(i): k for k, i in enumerate(ids.tolist())}
    for step in range(3):
        q = torch.randn(queries, heads, 576) * 0.2
        pos = torch.stack([torch.randperm(n)[:topk] for _ in range(queries)])
        sel = ids[pos].to(torch.int32)
        cache.begin_model_forward()
        cache.access(sel, 0)
        counts = cache.engine.selected_counts(0)
        window = records.decode_bf16(cache.gather_selected_records(0)).view(queries, topk, 576)
        o = torch.zeros(queries, heads, 512)
        lse = torch.full((queries, heads), float("-inf"))
        for r in range(queries):
            c = int(counts[r])
            mine = [p for p in sel[r].tolist() if p % world == rank]
            assert c == len(mine)
            if c == 0:
                continue
            rows = window[r, :c]
            # the local window holds exactly this rank's share of the selection (order free)
            want = full[[row_of[p] for p in mine]]
            assert torch.equal(rows.sort(dim=0).values, want.sort(dim=0).values)
            sc = torch.einsum("hd,td->ht", q[r], rows) * 576 ** -0.5
            lse[r] = torch.logsumexp(sc, dim=-1)
            o[r] = torch.softmax(sc, dim=-1) @ rows[:, :512]
        cache.finish_layer_attention(0)
        cache.finish_model_forward()
        outs = [torch.empty_like(o) for _ in range(world)]
        lses = [torch.empty_like(lse) for _ in range(world)]
        dist.all_gather(outs, o)
        dist.all_gather(lses, lse)
        merged, _ = merge_partial_attention(torch.stack(outs), torch.stack(lses))
        for r in range(queries):
            rows = full[pos[r]]
            sc = torch.einsum("hd,td->ht", q[r], rows) * 576 ** -0.5
            dense = torch.softmax(sc, dim=-1) @ rows[:, :512]
            assert torch.allclose(merged[r], dense, rtol=1e-4, atol=1e-5), (rank, step, r)
    cache.free(ids)
    cache.close()
    out[rank] = True
    dist.destroy_process_group()


def test_position_sharded_engine_merges_to_the_dense_answer():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_cp_rank, args=(2, _free_port(), out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}


def test_pulled_record_cache_policies_against_a_plain_model():
    """The optional per-rank cache of pulled records: hits pin, misses take free rows first, then
    the oldest unpinned row (age policy) or the next unpinned row behind the hand (circular policy);
    rows used in the current step are never replaced."""
    import pytest
    from ulacache_b200.cache.tensor_parallel import PulledRecordCache

    for policy in ("age_lru", "circular"):
        cache = PulledRecordCache(record_bytes=16, max_queries=2, topk=32, multiplier=3.0, policy=policy)
        assert cache.capacity == 192
        last_used = {}                                    # plain model: id -> step of last use
        g = torch.Generator().manual_seed(3)
        for step in range(1, 40):
            cache.begin_step()
            ids = torch.randperm(400, generator=g)[:64].tolist()
            slots, miss = cache.lookup(ids)
            want_hits = [i for i in ids if i in last_used]
            assert int((~miss).sum()) == len(want_hits)
            got = cache.allocate([i for i, m in zip(ids, miss.tolist()) if m])
            assert len(set(got)) == len(got) and all(0 <= s < cache.capacity for s in got)
            for i in ids:
                last_used[i] = step
            resident = {int(t) for t in cache.tags.tolist() if t >= 0}
            assert set(ids) <= resident and len(resident) <= cache.capacity
            evicted = set(last_used) - resident
            if policy == "age_lru" and evicted:
                # nothing evicted was used more recently than something still resident
                assert max(last_used[i] for i in evicted) <= min(last_used[i] for i in resident)
            for i in evicted:
                del last_used[i]
        assert cache.hits > 0 and cache.misses > 0
    small = PulledRecordCache(record_bytes=16, max_queries=1, topk=8, multiplier=3.0)
    small.begin_step()
    rows = small.allocate([7, 9, 7])                      # a repeated id gets one row
    assert rows[0] == rows[2] != rows[1]
    small.fill(rows[:2], torch.arange(32, dtype=torch.uint8).view(2, 16))
    assert small.read([rows[1]]).tolist() == [list(range(16, 32))]
    slots, miss = small.lookup(torch.tensor([9, 8]))
    assert slots.tolist() == [rows[1], -1] and miss.tolist() == [False, True]
    small = PulledRecordCache(record_bytes=16, max_queries=1, topk=8, multiplier=3.0)
    small.begin_step()
    small.allocate(list(range(small.capacity)))
    with pytest.raises(MemoryError):
        small.allocate([10_000])                          # every row is pinned by this step
