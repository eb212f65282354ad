import pytest
import torch

from ulacache_b200.cache.prefill import (PrefillWindowPair, ReadOnlyPrefillReader, SelectionWindowMap, WindowLeases,
                                         plan_prefill_chunks)
from ulacache_b200.cache.prefill.leases import WindowLeaseError
from ulacache_b200.ops import prefill as P
from ulacache_b200.transfer.prefill_pipeline import LayerPrefillPipeline


def test_selection_union_cpu():
    sel = torch.tensor([[5, 3, 5, -1], [9, 3, 0, 7]], dtype=torch.int32)
    ids, count, rows = P.selection_union(sel, 16, capacity=8)
    assert int(count) == 5 and ids[:5].tolist() == [0, 3, 5, 7, 9] and ids[5:].tolist() == [-1] * 3
    assert rows.tolist() == [[2, 1, 2, -1], [4, 1, 0, 3]]
    with pytest.raises(MemoryError):
        P.selection_union(sel, 16, capacity=3)


def test_chunk_plans_respect_the_window():
    plans = plan_prefill_chunks(100_000, cached_prefix=4096, chunk_tokens=8192, topk=2048, window_capacity=65536)
    assert plans[0].start == 4096 and sum(p.tokens for p in plans) == 100_000 - 4096
    assert all(p.window_records <= 65536 for p in plans)
    assert all(a.start + a.tokens == b.start for a, b in zip(plans, plans[1:]))


class _FakeEngine:
    def __init__(self, n, rb):
        self.store = {l: torch.randint(0, 255, (n, rb), dtype=torch.uint8) for l in range(3)}

    def read_records(self, layer, ids):
        ok = ids < self.store[layer].shape[0] - 2          # the last two ids are "not readable here"
        out = torch.zeros((ids.numel(), self.store[layer].shape[1]), dtype=torch.uint8)
        out[ok] = self.store[layer][ids[ok].long()]
        return out, ok


def test_pipeline_double_buffers_and_leases():
    eng = _FakeEngine(32, 16)
    pair = PrefillWindowPair(16, 16, "cpu")
    leases = WindowLeases()
    pipe = LayerPrefillPipeline(ReadOnlyPrefillReader(eng), SelectionWindowMap(32, 16), pair, leases)
    sel = torch.tensor([[1, 4, 4, 30], [2, 1, -1, 31]], dtype=torch.int32)
    pipe.prime(0, sel)
    for layer in range(3):
        window, rows = pipe.acquire(layer)
        if layer + 1 < 3:
            pipe.prefetch(layer + 1, sel)
        got = window.data[rows.clamp(min=0).long()]
        want = eng.store[layer][sel.clamp(min=0).long()]
        keep = (sel >= 0) & (sel < 30)
        assert torch.equal(got[keep], want[keep]) and int(got[sel >= 30].sum()) == 0
        assert window.rows() == 5 and leases.readers(window) == 1
        with pytest.raises(WindowLeaseError):
            leases.check_refill(window)
        pipe.release(layer)
    assert leases.readers(pair.current) == 0


@pytest.mark.gpu
def test_union_localize_merge_on_gpu(native):
    torch.manual_seed(0)
    sel = torch.randint(-1, 5000, (7, 300), dtype=torch.int32, device="cuda")
    ids, count, rows = P.selection_union(sel, 5000, capacity=2100)
    rids, rcount, rrows = P.selection_union(sel.cpu(), 5000, capacity=2100)
    assert int(count) == int(rcount) and torch.equal(ids.cpu(), rids) and torch.equal(rows.cpu(), rrows)
    ids2, count2, _ = P.selection_union(sel[:2], 5000, capacity=2100)        # workspace flags were left clean
    assert int(count2) == int(torch.unique(sel[:2][sel[:2] >= 0]).numel())
    loc, cnt = P.cp_localize(sel, 4, 1)
    rloc, rcnt = P.cp_localize(sel.cpu(), 4, 1)
    assert torch.equal(cnt.cpu(), rcnt)
    for q in range(7):
        n = int(rcnt[q])
        assert torch.equal(loc[q, :n].cpu(), rloc[q, :n]) and int(loc[q, n:].abs().sum()) == 0
    po = torch.randn(3, 11, 512, device="cuda")
    pl = torch.randn(3, 11, device="cuda")
    pl[1, 4] = float("-inf")
    o, lse = P.merge_partial_attention(po, pl)
    ro, rl = P.merge_partial_attention(po.cpu(), pl.cpu())
    assert (o.float().cpu() - ro.float()).abs().max() < 0.03 and (lse.cpu() - rl).abs().max() < 1e-4


def test_packed_regions_expand_and_remap_cpu():
    from ulacache_b200.cache.sparse_regions import PackedRegionLayout, expand_packed_regions, remap_packed_regions

    lay = PackedRegionLayout(tokens_per_region=4, region_slots_per_query=3)
    packed = torch.tensor([[(5 << 32) | 17, (2 << 32) | 3, -1], [(9 << 32) | 1, (7 << 32) | 2, (1 << 32) | 9]])
    toks = expand_packed_regions(packed, torch.tensor([2, 2]), lay, active_rows=2)
    assert toks[0].tolist() == [20, 21, 22, 23, 8, 9, 10, 11, -4, -3, -2, -1]
    assert toks[1].tolist()[8:] == [-4, -3, -2, -1]                     # beyond the row's count
    out = remap_packed_regions(packed, torch.tensor([[40, -1, 0], [36, 28, 4]]), lay)
    assert out[0].tolist() == [(10 << 32) | 17, -1, -1] and out[1].tolist() == [(9 << 32) | 1, (7 << 32) | 2, (1 << 32) | 9]


def _offload_scenario(device):
    """Write 256 records into a cache whose HBM tier holds them all, offload half to the host tier, and
    read everything back through the access path (which promotes what the selection needs)."""
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.ops import records
    from helpers import make_spec, random_kv

    cache = ula.init(make_spec(layers=2, device_pages=6, host_pages=8, queries=2, topk=128), LocalCacheBindings(device=device))
    ids = cache.alloc(256)
    latent, rope = random_kv(256, 3)
    latent, rope = latent.to(device), rope.to(device)
    for layer in range(2):
        cache.write(ids, layer, (latent * (layer + 1), rope))
    res = cache.engine.residency[0]
    assert bool((res.directory[ids.long()] >= 0).all())                   # everything starts in HBM
    moved = ids[64:192]
    cache.engine.offload_prefill(moved)
    entry = res.directory[ids.long()].cpu()
    out = {"on_host": int((entry[64:192] <= -2).sum()), "still_device": int((entry >= 0).sum())}
    got = {}
    for k, part in enumerate((ids[:128], ids[128:])):            # one access per layer and forward
        cache.begin_model_forward()
        for layer in range(2):
            cache.access(part.view(1, -1).to(torch.int32), layer)
            got[(layer, k)] = cache.gather_selected_records(layer).clone().cpu().view(-1, 656)
            cache.finish_layer_attention(layer)
        cache.finish_model_forward()
    cache.check()
    # the byte-exact reference is what the cache held before the offload: re-encode on the same device path
    fresh = ula.init(make_spec(layers=2, device_pages=6, host_pages=8, queries=2, topk=128), LocalCacheBindings(device=device))
    ids2 = fresh.alloc(256)
    for layer in range(2):
        fresh.write(ids2, layer, (latent * (layer + 1), rope))
    want = {}
    for k, part in enumerate((ids2[:128], ids2[128:])):
        fresh.begin_model_forward()
        for layer in range(2):
            fresh.access(part.view(1, -1).to(torch.int32), layer)
            want[(layer, k)] = fresh.gather_selected_records(layer).clone().cpu().view(-1, 656)
            fresh.finish_layer_attention(layer)
        fresh.finish_model_forward()
    out["bytes_equal"] = all(torch.equal(got[key], want[key]) for key in want)
    return out


def test_offload_prefill_rows_cpu():
    out = _offload_scenario("cpu")
    assert out == {"on_host": 128, "still_device": 128, "bytes_equal": True}


@pytest.mark.gpu
def test_offload_prefill_rows_with_the_copy_kernel(native):
    out = _offload_scenario("cuda")
    assert out == {"on_host": 128, "still_device": 128, "bytes_equal": True}
