"""GPU residency kernels against the PyTorch reference transaction, and the cache API on CUDA."""
import pytest
import torch

import ulacache_b200 as ula
from ulacache_b200.bindings import LocalCacheBindings
from ulacache_b200.cache.residency import (CNT_EPOCH, ResidencyGeometry, TorchResidency, make_residency)
from ulacache_b200.ops import records
from ulacache_b200.storage.layout import OwnerMap

from helpers import make_spec, random_kv

pytestmark = pytest.mark.gpu


def _age_multiset(res, slots):
    epoch = int(res.counters[CNT_EPOCH])
    return sorted((epoch - res.stamps[slots.long()]).clamp(max=255).tolist())


@pytest.mark.parametrize("index", ["stamps", "bitmap"])
def test_transaction_matches_reference(native, index):
    geom = ResidencyGeometry(dir_len=4096, hbm_slots=256, host_slots=1024, plan_capacity=512)
    owners = OwnerMap(1, 6)
    ref = TorchResidency(geom, owners, 0, "cpu")
    gpu = make_residency(geom, owners, 0, "cuda", victim_index=index)
    ids = torch.arange(1, 1201, dtype=torch.int32)
    ref.register(ids)
    gpu.register(ids.cuda())
    torch.cuda.synchronize()
    assert gpu.stats() == ref.stats()
    ref.load_state(gpu.state_dict())      # which IDs won the HBM slots is a race on the GPU
    g = torch.Generator().manual_seed(0)
    for step in range(12):
        sel = ids[torch.randperm(1200, generator=g)[:180]].view(3, 60)
        for r, s in ((ref, sel), (gpu, sel.cuda())):
            r.begin_step()
            r.pin(s)
            r.plan_step()
        torch.cuda.synchronize()
        gpu.check_status()
        pr, pg = ref.plan_items(), gpu.plan_items().cpu()
        assert pr.shape == pg.shape
        # same rows promoted (order may differ), same number of evictions, victims equally old
        assert sorted(pr[0].tolist()) == sorted(pg[0].tolist())
        assert int((pr[4] >= 0).sum()) == int((pg[4] >= 0).sum())
        ev_r, ev_g = pr[1][pr[4] >= 0], pg[1][pg[4] >= 0]
        if ev_r.numel():
            assert _age_multiset(ref, ev_r) == _age_multiset(gpu, ev_g.cuda())
        ref.commit()
        gpu.commit()
        torch.cuda.synchronize()
        sr, sg = ref.stats(), gpu.stats()
        assert sr == sg, (sr, sg)
        assert torch.equal(ref.ring, gpu.ring.cpu())
        # every selected row is now in HBM on both sides
        assert (gpu.directory[sel.reshape(-1).long().cuda()] >= 0).all()
        assert (ref.directory[sel.reshape(-1).long()] >= 0).all()
        # equally old victims may be different slots: continue from one common state
        ref.load_state(gpu.state_dict())
    if index == "bitmap":
        # the bitmaps say what the stamps say: one bit per attached slot, in the bucket of its stamp
        kept_bits, kept_summary = gpu.bits.clone(), gpu.summary.clone()
        gpu.rebuild_victim_index()
        assert torch.equal(kept_bits, gpu.bits)
        assert bool(((kept_summary & gpu.summary) == gpu.summary).all())      # summaries may keep stale bits, never miss one
    gpu.release(ids.cuda())
    ref.release(ids)
    torch.cuda.synchronize()
    assert gpu.stats() == ref.stats()
    assert int(gpu.ring.sum()) == 0
    if index == "bitmap":
        assert int(gpu.bits.abs().sum()) == 0


def test_bitmap_index_through_a_full_ring_rotation(native):
    """More than 255 steps: slots expire into the cold bucket (drain launch) and cold victims are taken first."""
    geom = ResidencyGeometry(dir_len=2048, hbm_slots=128, host_slots=512, plan_capacity=128)
    owners = OwnerMap(1, 6)
    gpus = [make_residency(geom, owners, 0, "cuda", victim_index=i) for i in ("stamps", "bitmap")]
    ids = torch.arange(1, 201, dtype=torch.int32).cuda()          # 128 land in HBM, 72 on the host
    for r in gpus:
        r.register(ids)
    gpus[1].load_state(gpus[0].state_dict())
    g = torch.Generator().manual_seed(3)
    saw_cold = 0
    for step in range(300):
        # a few warm rows every step; two host rows every 20 steps, so most slots stay untouched long
        # enough to expire into the cold bucket and the rare victims come out of it
        warm = ids[torch.randperm(20, generator=g)[:4].cuda()]
        extra = ids[:0]
        if step % 20 == 19:
            # which ids sit in the host tier is decided by the order registration's threads ran in: ask the directory
            on_host = ids[gpus[1].directory[gpus[1]._owned_locals(ids)[1].long()] <= -2]
            extra = on_host[torch.randperm(on_host.numel(), generator=g)[:2].cuda()]
        sel = torch.cat([warm, extra]).view(1, -1)
        for r in gpus:
            r.begin_step()
            r.pin(sel)
            r.plan_step()
        torch.cuda.synchronize()
        a, b = gpus[0].plan_items().cpu(), gpus[1].plan_items().cpu()
        assert sorted(a[0].tolist()) == sorted(b[0].tolist()), step
        ev_a, ev_b = a[1][a[4] >= 0], b[1][b[4] >= 0]
        assert _age_multiset(gpus[0], ev_a.cuda()) == _age_multiset(gpus[1], ev_b.cuda()), step
        for r in gpus:
            r.commit()
        torch.cuda.synchronize()
        assert gpus[0].stats() == gpus[1].stats(), step
        assert torch.equal(gpus[0].ring, gpus[1].ring)
        gpus[1].check_status()
        saw_cold = max(saw_cold, int(gpus[1].ring[255]))
        gpus[0].load_state(gpus[1].state_dict())                                   # equally old victims may differ
    assert saw_cold > 50 and gpus[1].stats()["evictions"] >= 10, gpus[1].stats()
    kept = gpus[1].bits.clone()
    gpus[1].rebuild_victim_index()
    assert torch.equal(kept, gpus[1].bits)


def test_cache_api_on_cuda_with_host_tier(native):
    cache = ula.init(make_spec(device_pages=4, host_pages=16), LocalCacheBindings(device="cuda"))
    ids = cache.alloc(1000)
    latent, rope = random_kv(1000, 0)
    latent, rope = latent.cuda(), rope.cuda()
    for layer in range(2):
        cache.write(ids, layer, (latent * (layer + 1), rope))
    truth = [records.decode_scaled656(records.encode_scaled656(latent * (l + 1), rope)) for l in range(2)]
    g = torch.Generator().manual_seed(1)
    pos = {int(i): n for n, i in enumerate(ids.tolist())}
    for step in range(6):
        pick = torch.stack([ids[torch.randperm(1000, generator=g)[:128].cuda()] for _ in range(2)])
        cache.begin_model_forward()
        for layer in range(2):
            view = cache.access(pick, layer)
            assert (view.device_record_indices >= 0).all()
            got = records.decode_scaled656(cache.gather_selected_records(layer)).view(2, 128, 576)
            want = truth[layer][torch.tensor([[pos[int(i)] for i in row] for row in pick.tolist()]).cuda()]
            err = (got - want).abs().max().item()
            assert err < 0.13 * want.abs().max().item()      # writer rounding ties only
            assert (got == want).float().mean() > 0.99
            cache.finish_layer_attention(layer)
        cache.finish_model_forward()
    cache.check()
    c = cache.counters()
    assert c["promotions"] > 0 and c["evictions"] > 0 and c["unserved"] == 0
    cache.free(ids)
    cache.close()


def test_receive_leases_and_publication_on_the_device(native):
    """Lease kernels == the CPU path (leased slots are never victims, last release re-attaches), and the
    publication kernel copies every layer of every record to its tier."""
    import torch
    from test_receive_and_tools import _lease_scenario, _leased_residency

    cpu = _lease_scenario("cpu")
    for index in ("stamps", "bitmap"):
        gpu = _lease_scenario("cuda", victim_index=index)
        for key in ("loc", "ring_leased", "still_leased", "stamps", "ring_after", "leases"):
            assert cpu[key] == gpu[key], (index, key)
        assert len(gpu["victims"]) == 3 and not set(gpu["victims"]) & {gpu["loc"][0], gpu["loc"][1]}
    res, ids, leases = _leased_residency("cuda")
    loc = leases.acquire(ids[[2, 10, 5, 11]])
    staging = torch.randint(0, 255, (5, 6, 656), dtype=torch.uint8, device="cuda")
    dev_plane = torch.zeros(5, 8, 656, dtype=torch.uint8, device="cuda")
    host_plane = torch.zeros(5, 16, 656, dtype=torch.uint8).pin_memory()
    rows = torch.tensor([3, 0, 1, 5])
    leases.publish(staging, rows, loc, dev_plane, host_plane)
    torch.cuda.synchronize()
    res.check_status("publish")
    for i, r in enumerate(rows.tolist()):
        e = int(loc[i])
        got = dev_plane[:, e].cpu() if e >= 0 else host_plane[:, -e - 2]
        assert torch.equal(got, staging[:, r].cpu()), i
    leases.release(ids[[2, 10, 5, 11]], loc)
    torch.cuda.synchronize()
    res.check_status("release")
    assert int(leases.leases.sum()) == 0


def test_staged_receive_window_publishes_from_pinned_memory(native):
    """The window's pinned pages are read by the publication kernel through their mapped address; records land in
    whichever tier holds them now, sidecar banks (kernel path at 128-byte rows, index copy at 132) by record id."""
    from ulacache_b200.transfer.receive_window import StagedReceiveWindow

    cache = ula.init(make_spec(device_pages=2, host_pages=8), LocalCacheBindings(device="cuda"))
    window = StagedReceiveWindow(cache, record_capacity=512, copy_chunk_records=200)
    assert window.pinned and window.staging.is_pinned()
    wide = torch.zeros(4096, 128, dtype=torch.uint8, device="cuda")
    odd = torch.zeros(4096, 132, dtype=torch.uint8, device="cuda")
    window.add_sidecar("wide", [wide])
    window.add_sidecar("odd", [odd])
    n = 300
    ids = cache.alloc(320)
    window.reserve("room", ids, record_count=n)
    latent, rope = random_kv(n, 3)
    payload = [records.encode_scaled656(latent * (l + 1), rope) for l in range(2)]
    src = window.staging_rows("room")
    for l in range(2):
        window.staging[l, src] = payload[l]
    side = {k: torch.randint(0, 255, (n, w), dtype=torch.uint8) for k, w in (("wide", 128), ("odd", 132))}
    for k, v in side.items():
        window._sidecars[k]["storage"][0, src] = v
    assert window.publish("room") == n
    assert torch.equal(wide[ids[:n].long()].cpu(), side["wide"]) and torch.equal(odd[ids[:n].long()].cpu(), side["odd"])
    truth = records.decode_scaled656(payload[1])
    pick_pos = torch.randperm(n, generator=torch.Generator().manual_seed(0))[:64]
    cache.begin_model_forward()
    cache.access(ids[pick_pos.cuda()].view(1, 64), 1)
    got = records.decode_scaled656(cache.gather_selected_records(1)).view(64, 576)
    assert torch.equal(got.cpu(), truth[pick_pos])
    cache.finish_layer_attention(1)
    cache.finish_model_forward()
    cache.check()
    assert int(window.leases[0].leases.sum()) == 0
    cache.close()


def test_file_restore_alternates_two_pinned_buffers(native, tmp_path):
    """A hashed file source streams into a CUDA cache through two pinned buffers; every record reads back equal."""
    import hashlib

    from ulacache_b200.transfer.file_io import FileRecordSource, restore_file_records

    cache = ula.init(make_spec(layers=1, device_pages=2, host_pages=8), LocalCacheBindings(device="cuda"))
    n = 300
    latent, rope = random_kv(n, 1)
    payload = records.encode_scaled656(latent, rope)
    raw = payload.numpy().tobytes()
    path = tmp_path / "kv.bin"
    path.write_bytes(raw)
    ids = cache.alloc(320)[:n]
    stats = {}
    src = FileRecordSource(str(path), 0, n, 656, "mla_scaled656", sha256=hashlib.sha256(raw).hexdigest(), file_bytes=len(raw))
    assert restore_file_records(cache.engine, 0, ids, src, chunk_bytes=656 * 64, statistics=stats) == n
    assert stats["chunks_read"] == 5 and stats["payload_sha256_verified"] and stats["leased_buffers"] == 0
    assert torch.equal(cache.engine.read_records(0, ids)[0].cpu(), payload)
    cache.check()
    cache.close()


def test_canary_build_of_the_storage_on_cuda(native, monkeypatch):
    """ULC_CANARY=1: guard records around every layer's device and pinned host plane survive writes, promotions
    and evictions through the kernels (planes become strided views), and a byte written past a plane is reported."""
    from ulacache_b200.storage.buffers import GUARD_ROWS

    monkeypatch.setenv("ULC_CANARY", "1")
    cache = ula.init(make_spec(device_pages=4, host_pages=16), LocalCacheBindings(device="cuda"))
    st = cache.engine.storages[0]
    assert st.guard == GUARD_ROWS and not st.gpu.is_contiguous()
    ids = cache.alloc(1000)
    latent, rope = random_kv(1000, 0)
    latent, rope = latent.cuda(), rope.cuda()
    for layer in range(2):
        cache.write(ids, layer, (latent * (layer + 1), rope))
    truth = records.decode_scaled656(records.encode_scaled656(latent * 2, rope))
    g = torch.Generator().manual_seed(1)
    for step in range(4):
        pick = torch.stack([torch.randperm(1000, generator=g)[:128] for _ in range(2)]).cuda()
        cache.begin_model_forward()
        cache.access(ids[pick], 1)
        got = records.decode_scaled656(cache.gather_selected_records(1)).view(2, 128, 576)
        assert (got == truth[pick]).float().mean() > 0.99
        cache.finish_layer_attention(1)
        cache.finish_model_forward()
    cache.check()
    assert cache.counters()["promotions"] > 0 and cache.counters()["evictions"] > 0
    st._device_block[0, 0, 3] = 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="before the device slots"):
        cache.check()
    cache.close()
