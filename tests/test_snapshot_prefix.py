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
