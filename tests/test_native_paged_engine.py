"""The rank-local engine over native pages: caller-supplied unions, eager prefill unions, receive rows, native-page
publication and inventories (CPU; the same scenario runs on a GPU under -m gpu)."""
import dataclasses

import pytest
import torch

import ulacache_b200 as ula
from ulacache_b200.bindings import LocalCacheBindings
from ulacache_b200.cache.local_paged_cache import NativePagedResidency
from ulacache_b200.ops import records

from helpers import make_spec, random_kv


def _paged(device, **kw):
    b = LocalCacheBindings(device=device)
    b = dataclasses.replace(b, execution_options=dataclasses.replace(b.execution_options,
                                                                    record_storage_backend="native_paged"))
    cache = ula.init(make_spec(**kw), b)
    eng = cache.engine if hasattr(cache, "engine") else cache
    assert isinstance(eng, NativePagedResidency)
    return cache, eng


def _scenario(device):
    cache, eng = _paged(device, layers=2, device_pages=4, host_pages=16, queries=8, topk=64)
    ids = cache.alloc(700)                                   # 256 device rows, the rest in the host tier
    latent, rope = random_kv(700, 1)
    enc = records.encode_scaled656(latent, rope)
    for layer in range(2):
        cache.write(ids, layer, (latent.to(device), rope.to(device)))
    pos = {int(i): n for n, i in enumerate(ids.tolist())}

    # --- a caller-supplied union with repeats and padding ---
    want = ids[torch.tensor([500, 3, 3, 650, 10, 500])].to(device)
    padded = torch.cat([want, torch.tensor([-1, 0], dtype=want.dtype, device=device)])
    uni, rows = eng.prepare_record_residency(0, padded)
    assert uni.tolist() == sorted(set(want.tolist())) and bool((rows >= 0).all())
    got = eng.layer_plane(0)[rows.long()].cpu()
    assert torch.equal(got, enc[[pos[int(i)] for i in uni.tolist()]])
    with pytest.raises(RuntimeError):                         # the domain is leased
        eng.prepare_record_residency(0, want)
    with pytest.raises(RuntimeError):                         # lifetime changes need retired readers
        eng.release(ids[:4])
    eng.finish_record_residency(0)
    with pytest.raises(RuntimeError):
        eng.finish_record_residency(0)

    # --- eager prefill: one union per selection producer and forward ---
    sel = torch.stack([ids[torch.randperm(700, generator=torch.Generator().manual_seed(q))[:64]] for q in range(3)]).to(device)
    sel[1, 60:] = -1
    eng.begin_forward()
    promos = cache.counters()["promotions"]
    rows = eng.plan_prefill(0, sel)
    assert rows.shape == sel.shape and bool((rows[sel > 0] >= 0).all()) and bool((rows[sel <= 0] == -1).all())
    got = eng.layer_plane(0)[rows[0].long()].cpu()
    assert torch.equal(got, enc[[pos[int(i)] for i in sel[0].tolist()]])
    again = eng.plan_prefill(0, sel)                          # same producer, same forward: no second transaction
    assert torch.equal(again, rows) and cache.counters()["promotions"] >= promos
    eng.after_attention(0)
    eng.finish_forward()
    assert eng.memory_inventory()["live_residency_domains"] == []
    with pytest.raises(ValueError):                           # a union larger than the device tier
        eng.begin_forward()
        eng.plan_prefill(1, ids[:300].reshape(1, -1).to(device))
    eng.abort_forward()

    # --- one borrowed chunk ---
    chunk = ids[100:164].to(device)
    r = eng.prepare_prefill_record_chunk(1, chunk)
    assert torch.equal(eng.layer_plane(1)[r.long()].cpu(), enc[100:164])
    with pytest.raises(RuntimeError):
        eng.prepare_prefill_record_chunk(1, chunk)
    eng.finish_prefill_record_chunk(1)

    # --- inventories ---
    inv = eng.memory_inventory()
    assert inv["residency_directory_count"] == 2 and inv["record_planes"] == 1 and inv["host_bytes"] > 0
    assert sum(eng.host_storage_inventory().values()) == inv["host_bytes"]
    if device == "cuda":
        assert inv["gpu_bytes"] >= inv["gpu_kv_bytes"] > 0 and inv["gpu_metadata_bytes"] > 0
        assert eng.supports_local_native_current_publication

    # --- publication from native pages ---
    pages = torch.zeros(2 * 64, 656, dtype=torch.uint8, device=device)
    src = torch.tensor([5, 70, 127], device=device)
    pages[src] = torch.arange(3, dtype=torch.uint8, device=device)[:, None] + 40
    tgt = ids[:3].to(device)
    eng.write_native_paged_records(0, tgt, pages, src)
    back = eng.read_records(0, tgt)[0].cpu()
    assert back[:, 0].tolist() == [40, 41, 42]
    assert len(eng.get_device_record_planes(0)) == 1 and len(eng.device_record_banks_by_layer) == 2
    cache.close()


def test_native_paged_engine_cpu():
    _scenario("cpu")


@pytest.mark.gpu
def test_native_paged_engine_gpu(native):
    _scenario("cuda")


def test_receive_rows_land_in_the_host_tier():
    cache, eng = _paged("cpu", layers=1, device_pages=2, host_pages=4)
    base = cache.alloc(64)                                    # keeps the id allocator honest
    fresh = torch.arange(int(base.max()) + 1, int(base.max()) + 33, dtype=torch.int32)
    rows = eng.allocate_receive_rows(fresh)
    assert rows.numel() == 32 and rows.unique().numel() == 32 and int(rows.min()) >= 0
    payload = torch.randint(0, 255, (32, 656), dtype=torch.uint8)
    eng.layer_host_plane(0)[rows] = payload
    got, found = eng.read_records(0, fresh)
    assert bool(found.all()) and torch.equal(got, payload)
    uni, dev_rows = eng.prepare_record_residency(0, fresh)    # and they promote like any other record
    assert torch.equal(eng.layer_plane(0)[dev_rows.long()], payload)
    eng.finish_record_residency(0)
    cache.close()
