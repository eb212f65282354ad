"""Bounded prefill windows: union / remap / fresh overlay, plans reused across layers, grouped attention with
bisection, and the cross-rank union (two gloo ranks)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from ulacache_b200.cache.prefill import (PrefillWindow, ReadOnlyPrefillReader, WindowedPrefillReader, WindowLeases,
                                         compact_selection, shared_union)


class _Engine:
    """Three layers of 64 records of 16 bytes; record i of layer l is filled with (l * 64 + i) % 251."""

    def __init__(self, n=64, rb=16, layers=3):
        self.store = {l: ((torch.arange(n)[:, None] + l * n) % 251).to(torch.uint8).repeat(1, rb) for l in range(layers)}
        self.reads = 0

    def read_records(self, layer, ids):
        self.reads += int(ids.numel())
        return self.store[layer][ids.long()], torch.ones(ids.numel(), dtype=torch.bool)


def test_compact_selection_union_rows_and_fresh_overlay():
    sel = torch.tensor([[9, 3, 9, -1, 40], [7, 3, 0, 12, 41]], dtype=torch.int32)
    lengths = torch.tensor([4, 5])                             # query 0 sees its first four columns only
    current = torch.tensor([12, 50, 9, 12], dtype=torch.int32)  # the chunk wrote 12 twice: the later row wins
    ids, rows, staging = compact_selection(sel, lengths, current)
    assert ids.tolist() == [0, 3, 7, 9, 12, 41]
    assert rows.tolist() == [[3, 1, 3, -1, -1], [2, 1, 0, 4, 5]]
    assert staging.tolist() == [-1, -1, -1, 2, 3, -1]
    ids2, rows2, staging2 = compact_selection(sel, None, None)
    assert ids2.tolist() == [0, 3, 7, 9, 12, 40, 41] and (staging2 == -1).all()
    empty = compact_selection(torch.full((2, 3), -1, dtype=torch.int32))
    assert empty[0].numel() == 0 and (empty[1] == -1).all()


def test_ordered_read_through_bounded_windows_with_plan_reuse():
    eng = _Engine()
    win = PrefillWindow(8, 16, "cpu")
    rd = WindowedPrefillReader(ReadOnlyPrefillReader(eng), win, bound=8, leases=WindowLeases())
    ids = torch.tensor([5, 5, 9, 1, 33, 60, 2, 2, 2, 7, 8, 10, 11, 12, 13, 14, 15, 16, 17], dtype=torch.int32)
    staging = torch.full((2, 16), 200, dtype=torch.uint8)
    staging[1] = 201
    rd.set_current_chunk(torch.tensor([33, 17], dtype=torch.int32), staging)
    plan = rd.prepare_read_plan(ids)
    assert len(plan.windows) == 3 and plan.records == ids.numel()
    assert plan.windows[0].record_ids.tolist() == [1, 2, 5, 9, 33, 60]     # 8 requested, 6 distinct
    for layer in range(3):
        out = rd.read_records(layer, ids, lambda data, rows: data[rows.long(), :1].float(), read_plan=plan)
        want = ((ids + layer * 64) % 251).float()
        want[ids == 33], want[ids == 17] = 200.0, 201.0                    # the chunk's own records win
        assert torch.equal(out.reshape(-1), want)
    assert rd.fills == 9
    buf = torch.zeros(ids.numel(), 2)
    got = rd.read_records(0, ids, lambda data, rows, dst: dst.copy_(data[rows.long(), :2].float()), output_buffer=buf)
    assert got is buf and torch.equal(buf[:, 0], torch.where(ids == 33, 200, torch.where(ids == 17, 201, ids % 251)).float())
    with pytest.raises(ValueError):
        rd.read_records(0, ids[:5], lambda d, r: d, read_plan=plan)
    with pytest.raises(ValueError):
        rd.prepare_read_plan(torch.tensor([3, -1], dtype=torch.int32))


def test_grouped_attention_bisects_groups_that_overflow_the_window():
    eng = _Engine()
    win = PrefillWindow(8, 16, "cpu")
    rd = WindowedPrefillReader(ReadOnlyPrefillReader(eng), win, bound=8)
    # 6 queries x top-4: queries 0-1 share ids, 2-5 are disjoint, so a group of 6 (union 20) must split
    sel = torch.tensor([[1, 2, 3, 4], [2, 3, 4, 5], [10, 11, 12, 13], [20, 21, 22, 23], [30, 31, 32, -1],
                        [40, 41, 42, 43]], dtype=torch.int32)
    lengths = torch.tensor([4, 4, 4, 4, 3, 2])
    q = torch.arange(6).float()[:, None]
    calls = []

    def attend(qs, rows, data, lens):
        calls.append((qs.shape[0], int((rows >= 0).sum())))
        vals = data[rows.clamp(min=0).long(), 0].float() * (rows >= 0)
        return vals.sum(1, keepdim=True) + qs

    out = rd.attend(1, q, sel, lengths, attend, topk=4)
    want = torch.stack([((sel[i, :lengths[i]] + 64) % 251).float().sum() + i for i in range(6)])[:, None]
    assert torch.equal(out, want)
    assert sum(c[0] for c in calls) == 6 and len(calls) >= 3 and all(c[1] <= 8 for c in calls)
    with pytest.raises(ValueError):
        rd.attend(1, q, sel, lengths, attend, topk=8)
    with pytest.raises(ValueError):
        rd.attend(1, q, sel, lengths, attend, topk=4, max_queries=4)
    tiny = WindowedPrefillReader(ReadOnlyPrefillReader(eng), PrefillWindow(4, 16, "cpu"), bound=3)
    with pytest.raises(ValueError):                                        # cannot hold one complete selection
        tiny.attend(1, q, sel, lengths, attend, topk=4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _union_main(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sel = torch.tensor([[3, 9, 5, -1]] if rank == 0 else [[9, 20, 1, 2]], dtype=torch.int32)
    current = torch.tensor([20, 3], dtype=torch.int32)
    ids, rows, staging = compact_selection(sel, None, current)
    joint = shared_union(ids, rows, staging, current, group=dist.group.WORLD, world=world, bound=8)
    j_ids, j_rows, j_staging = joint
    ok = j_ids.tolist() == [1, 2, 3, 5, 9, 20] and j_staging.tolist() == [-1, -1, 1, -1, -1, 0]
    ok = ok and j_rows.tolist() == ([[2, 4, 3, -1]] if rank == 0 else [[4, 5, 0, 1]])
    # the same branch on every rank when the joint union is too large, although each local one fits
    ok = ok and shared_union(ids, rows, staging, current, group=dist.group.WORLD, world=world, bound=5) is None
    out[rank] = ok
    dist.destroy_process_group()


def test_two_ranks_agree_on_one_union():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_union_main, args=(2, _free_port(), out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}


def _engine_scenario(device):
    """A real cache with records in HBM and in the host tier: a windowed read of a shuffled id list returns the
    stored bytes in request order, the chunk's fresh records win, residency state does not move."""
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from helpers import make_spec, random_kv

    cache = ula.init(make_spec(layers=2, device_pages=4, host_pages=16), LocalCacheBindings(device=device))
    ids = cache.alloc(600)                                   # 256 fit in HBM, the rest is in the host tier
    latent, rope = random_kv(600, 3)
    for layer in range(2):
        cache.write(ids, layer, (latent.to(device) * (layer + 1), rope.to(device)))
    before = dict(cache.counters())
    engine = cache.engine if hasattr(cache, "engine") else cache
    rb = engine.layer_plane(0).shape[-1]
    g = torch.Generator().manual_seed(5)
    order = ids[torch.randperm(600, generator=g)[:500]].to(device)
    win = PrefillWindow(128, rb, device)
    rd = WindowedPrefillReader(ReadOnlyPrefillReader(engine), win, bound=128, id_space=int(ids.max()) + 1)
    fresh_ids = order[[7, 300]].clone()
    fresh = torch.full((2, rb), 9, dtype=torch.uint8, device=device)
    rd.set_current_chunk(fresh_ids, fresh)
    plan = rd.prepare_read_plan(order)
    assert len(plan.windows) == 4
    for layer in range(2):
        got = rd.read_records(layer, order, lambda data, rows: data[rows.long()].clone(), read_plan=plan)
        want = engine.read_records(layer, order)[0].clone()
        want[7], want[300] = 9, 9
        assert torch.equal(got, want)
    after = dict(cache.counters())
    assert after["promotions"] == before["promotions"] and after["evictions"] == before["evictions"]
    cache.close()


def test_windowed_read_of_a_real_cache_cpu():
    _engine_scenario("cpu")


@pytest.mark.gpu
def test_windowed_read_of_a_real_cache_gpu(native):
    _engine_scenario("cuda")
