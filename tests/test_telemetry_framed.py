"""Framed sparse trace: frames, events, drains and the lookup oracle (CPU)."""
import pytest
import torch

from ulacache_b200.telemetry.sparse_trace import (EVENT_ALLOCATE, EVENT_RELEASE, FramedSparseTrace, SparseTraceGeometry,
                                                  frames_to_lookups, historical_lookups)


def test_lookup_oracle_drops_padding_and_current_records():
    sel = [[5, 6, 0, 9], [6, 7, -1, 9], [5, 5, 5, 5], [1, 2, 3, 4]]
    reqs = [0, 0, 1, -1]
    cur = [9, 10, 11, 1]
    got = historical_lookups(sel, reqs, cur)
    assert got == {(0, 5), (0, 6), (0, 7), (1, 5)}                  # 9 is written by request 0; row 3 has no request
    with pytest.raises(ValueError):
        historical_lookups(sel, reqs[:2], cur)


def test_geometry_is_checked_and_priced():
    g = SparseTraceGeometry(groups=2, query_rows=4, topk=8, frames=8, chunk_frames=4, event_capacity=16)
    assert g.payload_bytes == 8 * 4 * 9 * 4 + 8 * 12 + 16 * 24 + 40
    with pytest.raises(ValueError):
        SparseTraceGeometry(groups=2, query_rows=4, topk=8, frames=10, chunk_frames=4)
    with pytest.raises(ValueError):
        SparseTraceGeometry(groups=0, query_rows=4, topk=8)
    with pytest.raises(ValueError):
        FramedSparseTrace(g, device="cpu", max_gpu_bytes=100)


def test_frames_events_and_drains():
    g = SparseTraceGeometry(groups=2, query_rows=4, topk=8, frames=8, chunk_frames=2, event_capacity=6)
    tr = FramedSparseTrace(g, device="cpu")
    sel = torch.arange(1, 25, dtype=torch.int32).view(3, 8)
    cur = torch.tensor([100, 101, 17], dtype=torch.int32)
    tr.begin_frame(3)
    tr.observe(0, sel, cur, 7)                                        # not armed yet: lands in the spare slot
    assert int(tr.seen[:-1].max()) == -1
    tr.start()
    tr.observe_event(torch.tensor([64, 65]), release=False)
    for frame in range(2):
        tr.begin_frame(3)
        for group in range(2):
            tr.observe(group, sel + frame, cur, torch.tensor(40 + frame))
    with pytest.raises(RuntimeError):
        tr.begin_frame(3)                                             # the chunk is full and not drained
    chunk = tr.drain_chunk()
    assert chunk["first_frame"] == 0 and chunk["selected"].shape == (2, 2, 4, 8)
    assert torch.equal(chunk["selected"][1, 1, :3], sel + 1) and chunk["epochs"].tolist() == [[40, 40], [41, 41]]
    assert chunk["current"][0, 0].tolist() == [100, 101, 17, -1]
    ids, reqs = frames_to_lookups(chunk, [0, 0, 1, -1])[0]
    assert 17 not in ids and 8 in [i for i, r in zip(ids, reqs) if r == 0]       # request 1 is writing 17
    assert len(ids) == 23 and reqs.count(1) == 7
    # a frame that misses a group is refused at the drain
    tr.begin_frame(2)
    tr.observe(0, sel[:2], cur[:2], 42)
    tr.begin_frame(2)
    tr.observe(0, sel[:2], cur[:2], 43)
    tr.observe(1, sel[:2], cur[:2], 43)
    with pytest.raises(RuntimeError):
        tr.drain_chunk()
    # events: allocation and release are logged with their frame; overflow sets an error bit instead of writing
    tr.observe_event(torch.tensor([64]), release=True)
    ev = tr.event_snapshot()
    assert ev.tolist() == [[0, EVENT_ALLOCATE, 64], [0, EVENT_ALLOCATE, 65], [3, EVENT_RELEASE, 64]]
    tr.observe_event(torch.arange(10), release=False)
    with pytest.raises(RuntimeError):
        tr.event_snapshot()
    with pytest.raises(ValueError):
        tr.observe(2, sel, cur, 0)
    with pytest.raises(ValueError):
        tr.observe(0, torch.zeros(5, 8, dtype=torch.int32), torch.zeros(5, dtype=torch.int32), 0)
    tr.stop()
    assert tr.gpu_bytes > 0


def test_framed_capture_file_feeds_the_policy_replay(tmp_path):
    import numpy as np

    from ulacache_b200.experiments.scheduler_study import _load, run

    steps, layers, batch, topk = 6, 2, 3, 16
    g = torch.Generator().manual_seed(0)
    selected = torch.randint(1, 400, (steps, layers, batch, topk), generator=g, dtype=torch.int32)
    current = torch.arange(1000, 1000 + steps * batch, dtype=torch.int32).view(steps, 1, batch).expand(steps, layers, batch).contiguous()
    selected[:, :, :, 0] = current                                    # every row also selects the record it writes
    path = str(tmp_path / "frames.npz")
    np.savez(path, selected=selected.numpy(), current=current.numpy(), seen=np.full((steps, layers), batch, dtype=np.int32),
             epochs=np.zeros((steps, layers), dtype=np.int64), events=np.zeros((0, 3), dtype=np.int64),
             query_requests=np.arange(batch, dtype=np.int64))
    frames = list(_load(path))
    assert len(frames) == steps
    ids, reqs = frames[2]
    assert len(ids) == len(reqs) and set(reqs) == {0, 1, 2} and not set(ids) & set(current[2, 0].tolist())
    rows = list(run(frames, 64, per_request=32, record_bytes=656, layers=1))
    assert rows and all(0.0 <= r["hit_rate"] <= 1.0 for r in rows)
