"""Single-request prefix snapshots over byte banks, and their off-line striping."""
import pytest
import torch

from ulacache_b200.tools.snapshot.format import SnapshotReader, SnapshotRequest
from ulacache_b200.tools.snapshot.prefix import (ByteBanks, iter_prefix_records, restore_prefix_to_banks,
                                                 save_prefix_from_banks, stripe_prefix)


def _banks(seed, slots=256, pages=8):
    g = torch.Generator().manual_seed(seed)
    records = torch.randint(0, 255, (2, slots, 656), dtype=torch.uint8, generator=g)
    index = {0: torch.randint(0, 255, (pages, 64 * 132), dtype=torch.uint8, generator=g)}
    return ByteBanks(records, index)


def test_prefix_round_trip_through_banks_and_stripes(tmp_path):
    src = _banks(0)
    n = 150
    rows = torch.randperm(256, generator=torch.Generator().manual_seed(1))[:n]
    request = SnapshotRequest("r", tuple(range(100)), tuple(range(51)))
    assert request.next_position == n
    calls = []
    path = str(tmp_path / "prefix")
    save_prefix_from_banks(path, request, src, rows, "model-x", quiesce=lambda: calls.append("q"))
    assert calls == ["q"]
    with pytest.raises(ValueError):
        save_prefix_from_banks(str(tmp_path / "bad"), request, src, rows[:-1], "model-x", quiesce=lambda: None)
    got = b"".join(raw for _, raw in iter_prefix_records(path, "r", "mla_001", chunk_rows=37))
    assert got == src.records[1][rows].numpy().tobytes()

    dst = _banks(5)
    new_rows = torch.randperm(256, generator=torch.Generator().manual_seed(2))[:n]
    out = restore_prefix_to_banks(path, "r", dst, new_rows, "model-x", quiesce=lambda: calls.append("q"), verify=True,
                                  chunk_rows=64)
    assert out["next_position"] == n and out["next_token_id"] == 50 and out["restored_bytes"] == n * (2 * 656 + 132)
    assert calls == ["q", "q", "q"]
    for plane in ("mla_000", "mla_001", "index_000"):
        assert dst.read(plane, new_rows) == src.read(plane, rows)
    for bad in (dict(fingerprint="other"), dict(key="zz"), dict(rows=new_rows[:10])):
        kw = dict(key="r", rows=new_rows, fingerprint="model-x")
        kw.update(bad)
        with pytest.raises(ValueError):
            restore_prefix_to_banks(path, kw["key"], dst, kw["rows"], kw["fingerprint"], quiesce=lambda: None)
    with pytest.raises(ValueError):                                   # other geometry: no Index bank bound
        restore_prefix_to_banks(path, "r", ByteBanks(dst.records), new_rows, "model-x", quiesce=lambda: None)

    striped = str(tmp_path / "striped")
    stripe_prefix(path, striped, 4, chunk_rows=30)                   # 30 -> chunks of 28 rows, split evenly
    reader = SnapshotReader(striped, verify_payload=True)
    assert reader.layout.owners == 4 and reader.verify()["owners"] == 4
    for owner in range(4):
        for plane in ("mla_000", "index_000"):
            raw = b"".join(reader.iter_plane(owner, "r", plane))
            width = reader.layout.planes()[plane]
            want = torch.frombuffer(bytearray(src.read(plane, rows)), dtype=torch.uint8).view(n, width)[owner::4]
            assert raw == want.numpy().tobytes(), (owner, plane)
    with pytest.raises(ValueError):
        stripe_prefix(striped, str(tmp_path / "again"), 2)            # already striped
    from ulacache_b200.tools import cli

    assert cli.main(["stripe", path, "--to", str(tmp_path / "by_cli"), "--owners", "3", "--chunk-rows", "64"]) == 0
    assert SnapshotReader(str(tmp_path / "by_cli")).layout.owners == 3 and cli.main(["verify", str(tmp_path / "by_cli")]) == 0
    with pytest.raises(FileExistsError):
        stripe_prefix(path, striped, 4)


def test_byte_banks_validate_their_bindings():
    with pytest.raises(ValueError):
        ByteBanks(torch.zeros(4, 656, dtype=torch.uint8))
    with pytest.raises(ValueError):
        ByteBanks(torch.zeros(2, 8, 656, dtype=torch.uint8), {5: torch.zeros(2, 8448, dtype=torch.uint8)})
    with pytest.raises(ValueError):
        ByteBanks(torch.zeros(2, 8, 656, dtype=torch.uint8), {0: torch.zeros(2, 100, dtype=torch.uint8)})
    banks = ByteBanks(torch.zeros(2, 8, 656, dtype=torch.uint8))
    with pytest.raises(ValueError):
        banks.write("mla_000", torch.arange(3), bytes(656 * 2))
    lay = banks.layout("f")
    assert lay.owners == 1 and lay.layers == 2 and lay.index_anchors == ()


def test_a_striped_snapshot_restores_into_a_single_owner_cache_with_one_lookup(tmp_path):
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.ops import records
    from ulacache_b200.tools.snapshot import cache_io
    from ulacache_b200.tools.snapshot.format import SnapshotLayout, finalize_snapshot
    from ulacache_b200.tools.snapshot.restore import PreparedSequenceRestore, iter_sequence_plane, restore_request

    from helpers import make_spec, random_kv

    spec = make_spec(layers=2, device_pages=2, host_pages=8)
    cache = ula.init(spec, LocalCacheBindings(device="cpu"))
    ids = cache.alloc(320)
    lat, rope = random_kv(320, 9)
    for l in range(2):
        cache.write(ids, l, (lat + l, rope))
    layout = SnapshotLayout("m", owners=4, layers=2, mla_row_bytes=656)
    request = SnapshotRequest("a", tuple(range(250)), (1, 2, 3))      # 252 positions: an uneven last stripe
    path = str(tmp_path / "bank")
    for owner in range(4):
        cache_io.save_shard(cache, path, layout, [request], {"a": ids[:253]}, owner)
    finalize_snapshot(path)
    reader = SnapshotReader(path, verify_payload=True)
    seq = torch.cat([d for _, d in iter_sequence_plane(reader, "a", "mla_001", chunk_rows=40)])
    assert torch.equal(seq, cache.engine.read_records(1, ids[:252])[0])
    with pytest.raises(ValueError):
        list(iter_sequence_plane(reader, "a", "mla_001", chunk_rows=42))     # not whole stripes

    fresh = ula.init(spec, LocalCacheBindings(device="cpu"))
    new = fresh.alloc(256)[:252]
    out = restore_request(fresh, reader, "a", new, verify=True, chunk_rows=50)
    assert out["source_owners"] == 4 and out["restored_bytes"] == 2 * 252 * 656 and out["next_token_id"] == 3
    for l in range(2):
        assert torch.equal(fresh.engine.read_records(l, new)[0], cache.engine.read_records(l, ids[:252])[0])
    # the restored records are served like any other (host-resident ones get promoted)
    fresh.begin_model_forward()
    fresh.access(new[200:232].view(1, 32), 1)
    got = records.decode_scaled656(fresh.gather_selected_records(1))
    want = records.decode_scaled656(cache.engine.read_records(1, ids[200:232])[0])
    assert torch.equal(got, want)
    fresh.finish_layer_attention(1)
    fresh.finish_model_forward()
    with pytest.raises(ValueError):
        restore_request(fresh, reader, "a", new[:10])
    freed = fresh.alloc(64)
    fresh.free(freed)
    with pytest.raises(ValueError):
        PreparedSequenceRestore(fresh, freed)                        # no storage behind these ids
    with PreparedSequenceRestore(fresh, new) as prepared:
        with pytest.raises(ValueError):
            prepared.write(0, 250, torch.zeros(8, 656, dtype=torch.uint8))
    with pytest.raises(RuntimeError):
        prepared.write(0, 0, torch.zeros(8, 656, dtype=torch.uint8))
    cache.close()
    fresh.close()
