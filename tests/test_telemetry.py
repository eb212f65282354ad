import os
import pytest

import torch

from ulacache_b200.telemetry import (CacheHitSampler, GpuSparseTraceRecorder, ReplayMetrics, load_trace,
                                     validate_bucket_rotation, validate_trace_coverage)


def test_hit_sampler_classifies_all_entries_at_shift_zero():
    d = torch.tensor([5, -1, -7, 2], dtype=torch.int32)
    s = CacheHitSampler("cpu", sample_shift=0)
    s.observe(d, torch.tensor([[0, 1, 2, 3], [3, 9, -1, 0]], dtype=torch.int32))
    snap = s.snapshot()
    assert snap["sampled"] == 7 and snap["device_hits"] == 4 and snap["host_hits"] == 1
    assert snap["unallocated"] == 1 and snap["out_of_range"] == 1 and abs(snap["device_hit_rate"] - 0.8) < 1e-9
    s2 = CacheHitSampler("cpu", sample_shift=3)
    big = torch.zeros(100000, dtype=torch.int32)
    s2.observe(torch.zeros(4, dtype=torch.int32), big)
    assert 0.09 < s2.snapshot()["sampled"] / 100000 < 0.16


def test_trace_recorder_round_trip(tmp_path):
    rec = GpuSparseTraceRecorder("cpu", capacity_triples=40)
    rec.record(0, 0, torch.tensor([1, 2, 3]))
    rec.record(0, 1, torch.tensor([4, 5]))
    rec.record(1, 0, torch.arange(50))            # does not fit: dropped whole
    assert rec.dropped == 50 and rec.drain() == 5
    rec.record(1, 0, torch.tensor([7]))
    path = os.path.join(tmp_path, "t.npy")
    assert rec.save(path) == 6
    tr = load_trace(path)
    assert tr[(0, 0)].tolist() == [1, 2, 3] and tr[(0, 1)].tolist() == [4, 5] and tr[(1, 0)].tolist() == [7]
    assert validate_trace_coverage(tr, 2, 2) == [(1, 1)]


def test_replay_metrics_and_rotation():
    m = ReplayMetrics(record_bytes=656, layers_per_group=3)
    m.add_counters({"promotes": 2, "swaps": 1}, {"promotes": 12, "swaps": 5})
    assert m.h2d_bytes == 10 * 656 * 3 and m.d2h_bytes == 4 * 656 * 3 and m.summary()["steps"] == 1
    labels = [-1] * 255
    for e in range(1, 300):
        labels[e % 255] = e
    assert validate_bucket_rotation(labels, 299) == []
    labels[7] = 7                                  # a stale bucket (should be 262)
    assert validate_bucket_rotation(labels, 299) == [7]


def test_device_replay_probes_cpu_path():
    """Unique historical lookups per request, split by tier; plan bytes by direction; host-written rows."""
    from ulacache_b200.telemetry import DeviceReplayProbes

    directory = torch.tensor([5, -2, -1, 7, -3, 9, -4, 2], dtype=torch.int32)
    # two requests x two queries each (width 2), top-4
    selected = torch.tensor([[0, 1, 3, -1], [1, 3, 4, 6], [0, 1, 5, 5], [7, 6, -1, -1]], dtype=torch.int32)
    current = torch.tensor([3, 6, 5, 7], dtype=torch.int32)        # rows written this step: not lookups
    requests = torch.tensor([10, 11], dtype=torch.int32)
    probes = DeviceReplayProbes(1, 4, 4, device="cpu")
    probes.before_plan(0, selected, current, requests, directory, width=2)
    # request 10: {0, 1, 4} (3 and 6 are its own rows) -> device 1, host 2; request 11: {0, 1, 6} -> device 1, host 2
    assert probes.counts[0, :5].tolist() == [6, 2, 4, 0, 0]
    plan = torch.full((5, 8), -1, dtype=torch.int32)
    plan[2, :3] = torch.tensor([4, 5, 6])          # three promotions from the host
    plan[3, :2] = torch.tensor([4, 5])             # two of them swap a victim out
    probes.after_group(0, plan, torch.tensor([3], dtype=torch.int32), current, directory, layers=2, row_bytes=656)
    snap = probes.snapshot()
    assert snap["totals"]["history_h2d_bytes"] == 3 * 2 * 656 and snap["totals"]["victim_d2h_bytes"] == 2 * 2 * 656
    assert snap["totals"]["new_cpu_backup_bytes"] == 1 * 2 * 656          # row 6 lives on the host
    # an unallocated lookup makes the snapshot fail loudly
    probes.before_plan(0, torch.tensor([[2, -1, -1, -1]] * 4, dtype=torch.int32), current, requests, directory, width=2)
    with pytest.raises(RuntimeError):
        probes.snapshot()


def test_tp_miss_trace_cpu_path_and_begin_rotation():
    from ulacache_b200.telemetry import GpuTpMissTrace, validate_fused_begin_rotation

    tr = GpuTpMissTrace(groups=2, query_rows=3, topk=4, frames=10, chunk_frames=2, device="cpu")
    rows = torch.tensor([[4, 5, 0, 0], [9, 0, 0, 0], [1, 2, 3, 0]], dtype=torch.int32)
    counts = torch.tensor([2, 1, 3], dtype=torch.int32)
    tr.begin_frame(3, 2)
    tr.observe(1, rows, counts)
    snap = tr.snapshot_chunk()
    slot = (3 % 2) * 2 + 1
    assert snap["local_miss_rows"][slot].tolist() == [[4, 5, -1, -1], [9, -1, -1, -1], [-1, -1, -1, -1]]
    assert snap["local_miss_counts"][slot].tolist() == [2, 1, -1] and int(snap["source_bucket_rows"][slot]) == 3
    tr.begin_frame(4, 5)                        # more valid rows than the source holds: flagged, not written
    tr.observe(0, rows, counts)
    with pytest.raises(RuntimeError):
        tr.snapshot_chunk()
    # a full rotation of a 4-bucket ring, two rows pinned per step
    obs, cold = [], 0
    for epoch in range(1, 9):
        bucket = epoch % 4
        age = epoch - 4 if epoch > 4 else -1
        old = 2 if age >= 0 else 0
        obs.append((epoch, bucket, age, old, epoch, 2, cold, cold + old))
        cold += old
    out = validate_fused_begin_rotation(obs, 4, [2] * 8)
    assert out["full_rotation"] and out["expired_members"] == 8 and out["expired_headers"] == 4
    bad = list(obs)
    bad[5] = (6, 2, 5, 2, 6, 2, bad[5][6], bad[5][7])          # a one-step-old bucket cannot expire
    with pytest.raises(ValueError):
        validate_fused_begin_rotation(bad, 4, [2] * 8)
