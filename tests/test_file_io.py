"""File record sources: ranges, stripes, hashes, leased buffers, double-buffered restore."""
import hashlib
import os

import pytest
import torch

from ulacache_b200.transfer.file_io import FileRecordReader, FileRecordSource, restore_file_records


def _file(tmp_path, rows=100, width=48, header=32, trailer=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    data = torch.randint(0, 255, (rows, width), dtype=torch.uint8, generator=g)
    path = tmp_path / "plane.bin"
    path.write_bytes(b"H" * header + data.numpy().tobytes() + b"T" * trailer)
    return str(path), data


def test_source_validation_and_views(tmp_path):
    path, data = _file(tmp_path)
    digest = hashlib.sha256(data.numpy().tobytes()).hexdigest()
    src = FileRecordSource(path, 32, 100, 48, "raw", sha256=digest.upper())
    assert src.verify_payload and src.sha256 == digest and src.range_end == 32 + 4800 and src.nbytes == 4800
    for bad in (dict(sha256="abc"), dict(verify_payload=True), dict(file_bytes=100), dict(record_stride=0)):
        with pytest.raises(ValueError):
            FileRecordSource(path, 32, 100, 48, "raw", **bad)
    part = src.slice(10, 5)
    assert (part.offset, part.record_count, part.sha256, part.verify_payload) == (32 + 480, 5, "", False)
    with pytest.raises(ValueError):
        src.select_owner(1, 4)                                       # a hashed source cannot be striped
    plain = FileRecordSource(path, 32, 100, 48, "raw")
    stripe = plain.select_owner(1, 4)
    assert (stripe.record_count, stripe.record_stride, stripe.offset) == (25, 4, 32 + 48)
    assert stripe.select_owner(1, 2).record_stride == 8 and stripe.select_owner(1, 2).record_count == 12
    assert plain.select_owner(3, 4).range_end <= 32 + 4800
    got = torch.cat([rows for _, rows in FileRecordReader(stripe, chunk_bytes=48 * 7)])
    assert torch.equal(got, data[1::4])
    got = torch.cat([rows for _, rows in stripe.slice(3, 9).open(48 * 4)])
    assert torch.equal(got, data[1::4][3:12])
    assert list(FileRecordReader(FileRecordSource(path, 32, 0, 48, "raw"))) == []


def test_reader_leases_buffers_and_verifies_before_the_last_chunk(tmp_path):
    path, data = _file(tmp_path, trailer=8)
    digest = hashlib.sha256(data.numpy().tobytes()).hexdigest()
    size = os.path.getsize(path)
    src = FileRecordSource(path, 32, 100, 48, "raw", sha256=digest, file_bytes=size)
    buf = torch.empty(64, 48, dtype=torch.uint8)
    with src.open() as reader:
        first = reader.readinto(buf)
        assert first.first == 0 and torch.equal(first.data, data[:64])
        with pytest.raises(RuntimeError):
            reader.readinto(buf[10:20])                              # overlaps the live lease
        with pytest.raises(ZeroDivisionError):
            first.release(after=lambda: 1 / 0)                       # a failed wait keeps the lease
        assert not first.released and reader.statistics()["leased_buffers"] == 1
        first.release()
        with pytest.raises(ValueError):
            reader.readinto(torch.empty(4, 47, dtype=torch.uint8))   # wrong row width
        last = reader.readinto(buf)
        assert last.first == 64 and last.data.shape[0] == 36 and torch.equal(last.data, data[64:])
        last.release()
        assert reader.readinto(buf) is None
        st = reader.statistics()
        assert st["payload_sha256_verified"] and st["bytes_read"] == 4800 and st["chunks_read"] == 2
    assert reader.statistics()["closed"] and reader.statistics()["wall_seconds"] is not None
    # a wrong hash: the last chunk is never handed out
    wrong = FileRecordSource(path, 32, 100, 48, "raw", sha256="0" * 64)
    reader = wrong.open()
    assert reader.readinto(buf) is not None
    with pytest.raises(ValueError):
        reader.readinto(torch.empty(64, 48, dtype=torch.uint8))
    assert reader.statistics()["closed"]
    with pytest.raises(ValueError):
        list(FileRecordReader(wrong, chunk_bytes=48 * 10))
    # the file's size is bound too
    with pytest.raises(ValueError):
        FileRecordSource(path, 32, 100, 48, "raw", file_bytes=size + 1).open()
    with pytest.raises(ValueError):
        FileRecordSource(path, 32, 101, 48, "raw").open()


def test_restore_streams_through_the_cache_and_reports_statistics(tmp_path):
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.ops import records

    from helpers import make_spec, random_kv

    cache = ula.init(make_spec(layers=1, device_pages=2, host_pages=8), LocalCacheBindings(device="cpu"))
    n = 300
    latent, rope = random_kv(n, 1)
    payload = records.encode_scaled656(latent, rope)
    path = tmp_path / "kv.bin"
    path.write_bytes(payload.numpy().tobytes())
    digest = hashlib.sha256(payload.numpy().tobytes()).hexdigest()
    ids = cache.alloc(320)[:n]
    stats = {}
    src = FileRecordSource(str(path), 0, n, 656, "mla_scaled656", sha256=digest, file_bytes=n * 656)
    assert restore_file_records(cache.engine, 0, ids, src, chunk_bytes=656 * 70, statistics=stats) == n
    assert stats["chunks_read"] == 5 and stats["payload_sha256_verified"] and stats["leased_buffers"] == 0
    assert torch.equal(cache.engine.read_records(0, ids)[0], payload)
    bad = FileRecordSource(str(path), 0, n, 656, "mla_scaled656", sha256="1" * 64)
    with pytest.raises(ValueError):
        cache.write(ids, 0, bad)
    cache.close()


def test_source_from_a_committed_snapshot(tmp_path):
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.tools.snapshot import cache_io
    from ulacache_b200.tools.snapshot.format import SnapshotLayout, SnapshotReader, SnapshotRequest, finalize_snapshot

    from helpers import make_spec, random_kv

    spec = make_spec(layers=1, device_pages=4, host_pages=4)
    cache = ula.init(spec, LocalCacheBindings(device="cpu"))
    ids = cache.alloc(128)
    lat, rope = random_kv(128, 2)
    cache.write(ids, 0, (lat, rope))
    layout = SnapshotLayout("m", owners=2, layers=1, mla_row_bytes=656)
    reqs = [SnapshotRequest("a", tuple(range(99)), (7,))]
    path = str(tmp_path / "bank")
    for owner in range(2):
        cache_io.save_shard(cache, path, layout, reqs, {"a": ids[:100]}, owner)
    finalize_snapshot(path)
    reader = SnapshotReader(path, verify_payload=True)
    with pytest.raises(ValueError):
        FileRecordSource.from_snapshot(reader, "a", "mla_000")        # two owners: name one
    src = FileRecordSource.from_snapshot(reader, "a", "mla_000", owner=1)
    assert src.verify_payload and src.record_count == reader.plane_rows(1, "a") and src.file_bytes == src.nbytes
    got = torch.cat([rows for _, rows in src.open(656 * 16)])
    want = cache.engine.read_records(0, ids[:100][1::2][:src.record_count])[0]
    assert torch.equal(got, want)
    loose = FileRecordSource.from_snapshot(reader, "a", "mla_000", owner=0, verify_payload=False)
    assert not loose.verify_payload and loose.sha256 == ""
    with pytest.raises(ValueError):
        FileRecordSource.from_snapshot(reader, "zz", "mla_000", owner=0)
    cache.close()
