"""Ablation policies and telemetry kernels on the GPU against the CPU oracle / CPU tensor paths."""
import random

import pytest
import torch

from ulacache_b200.eviction import (ExactLruPolicy, HotBufferPolicy, LinkedListLruPolicy, PolicyOracle, PresenceRingPolicy,
                                    trace_hits)
from ulacache_b200.telemetry import CacheHitSampler, GpuSparseTraceRecorder

pytestmark = pytest.mark.gpu


def _trace(seed, steps=30, ids=3000, per_step=400):
    rng = random.Random(seed)
    hot = list(range(300))
    return [sorted(set(rng.sample(hot, 150)) | set(rng.sample(range(ids), per_step - 150))) for _ in range(steps)]


def test_exact_lru_victims_match_oracle(native):
    pol = ExactLruPolicy(1024, 3000, "cuda")
    ora = PolicyOracle("exact_lru", 1024)
    for ids in _trace(1):
        resident = [i for i in ids if int(pol.dir[i]) >= 0]
        ordered = resident + [i for i in ids if int(pol.dir[i]) < 0]
        h, m, ev = pol.step(torch.tensor(ids))
        oh, om, oev, _ = ora.step(ordered)
        assert (h, m) == (oh, om) and sorted(ev.tolist()) == sorted(oev)
    assert pol.totals["evictions"] > 0


def test_linked_list_lru_matches_oracle(native):
    pol = LinkedListLruPolicy(512, 3000, "cuda")
    ora = PolicyOracle("linked_list", 512)
    for ids in _trace(2, per_step=200):
        h, m, ev = pol.step(torch.tensor(ids))
        oh, om, oev, over = ora.step(ids)
        assert (h, m) == (oh, om) and ev.tolist() == oev and over == 0


def test_presence_ring_on_the_device_matches_the_oracle(native):
    """The presence-bitmap ring header runs unchanged in a device kernel: same hits, misses and
    evicted records, in order, as the stamp-scanning bucket ring of the CPU oracle."""
    pol = PresenceRingPolicy(512, 3000, "cuda")
    ora = PolicyOracle("bucket_ring", 512)
    for ids in _trace(5, per_step=200):
        h, m, ev = pol.step(torch.tensor(ids))
        oh, om, oev, over = ora.step(ids)
        assert (h, m) == (oh, om) and ev.tolist() == oev and over == 0
    assert pol.totals["evictions"] > 0


def test_hot_buffer_matches_cpu_path(native):
    g, c = HotBufferPolicy(3, 64, "cuda"), HotBufferPolicy(3, 64, "cpu")
    rng = random.Random(3)
    for _ in range(10):
        rows = [[rng.randrange(200) for _ in range(rng.randrange(1, 90))] for _ in range(3)]
        ids = torch.tensor([x for r in rows for x in r], dtype=torch.int32)
        offs = torch.tensor([0, len(rows[0]), len(rows[0]) + len(rows[1]), ids.numel()], dtype=torch.int32)
        assert g.step(ids.cuda(), offs.cuda()) == c.step(ids, offs)
    assert torch.equal(g.tags.cpu().sort(dim=1).values, c.tags.sort(dim=1).values)


def test_observers(native):
    d = torch.randint(-3, 50, (4000,), dtype=torch.int32)
    sel = torch.randint(-1, 4100, (64, 512), dtype=torch.int32)
    assert trace_hits(d.cuda(), sel.cuda()) == trace_hits(d, sel)
    a, b = CacheHitSampler("cuda", sample_shift=2), CacheHitSampler("cpu", sample_shift=2)
    for _ in range(3):
        a.observe(d.cuda(), sel.cuda())
        b.observe(d, sel)
    assert a.snapshot() == b.snapshot()
    rec = GpuSparseTraceRecorder("cuda", capacity_triples=5000)
    rec.record(3, 1, sel[0].cuda())
    rec.record(3, 2, sel[:20].cuda())              # 10240 triples: dropped whole
    assert rec.dropped == 20 * 512 and rec.drain() == 512
    assert rec.chunks[0][:, 2].tolist() == sel[0].tolist() and set(rec.chunks[0][:, 0]) == {3}


def test_replay_probes_and_miss_trace_match_the_host_path(native):
    """Device counters of the replay probes and the local-miss trace == their CPU twins on random inputs."""
    from ulacache_b200.telemetry import DeviceReplayProbes, GpuTpMissTrace

    g = torch.Generator().manual_seed(11)
    dir_len, queries, width, topk = 4096, 24, 2, 64
    directory = torch.randint(-40, 400, (dir_len,), generator=g, dtype=torch.int32)
    directory[directory == -1] = -2                     # no unallocated rows: the snapshot must pass
    selected = torch.randint(-1, dir_len, (queries, topk), generator=g, dtype=torch.int32)
    selected[:, 5] = selected[:, 4]                     # duplicates inside a query
    selected[1] = selected[0]                           # and across the two queries of a request
    current = torch.randint(0, dir_len, (queries,), generator=g, dtype=torch.int32)
    requests = torch.arange(queries // width, dtype=torch.int32) + 3
    plan = torch.randint(-1, 50, (5, 128), generator=g, dtype=torch.int32)
    count = torch.tensor([77], dtype=torch.int32)
    outs = []
    for dev in ("cpu", "cuda"):
        p = DeviceReplayProbes(2, queries, topk, device=dev)
        p.before_plan(1, selected.to(dev), current.to(dev), requests.to(dev), directory.to(dev), width=width)
        p.after_group(1, plan.to(dev), count.to(dev), current.to(dev), directory.to(dev), layers=3, row_bytes=656)
        outs.append(p.snapshot())
    assert outs[0] == outs[1] and outs[0]["totals"]["lookup_tokens"] > 0
    rows = torch.randint(0, 1000, (6, 16), generator=g, dtype=torch.int32)
    counts = torch.randint(0, 17, (6,), generator=g, dtype=torch.int32)
    snaps = []
    for dev in ("cpu", "cuda"):
        tr = GpuTpMissTrace(groups=3, query_rows=8, topk=16, frames=100, chunk_frames=4, device=dev)
        for frame, valid in ((5, 6), (6, 3)):
            tr.begin_frame(frame, valid)
            tr.observe(frame % 3, rows.to(dev), counts.to(dev))
        snaps.append(tr.snapshot_chunk())
    for key in snaps[0]:
        assert torch.equal(snaps[0][key], snaps[1][key]), key


def test_parallel_presence_ring_matches_its_cpu_twin_step_by_step(native):
    """Parallel bitmap ring on the device == the transaction-semantics oracle, eviction by eviction, over
    more than two rotations of the 255-bucket ring (cold bucket, drains and stale summaries included)."""
    from ulacache_b200.eviction import ParallelPresenceRingPolicy

    rng = random.Random(4)
    capacity, id_space = 700, 5000
    cpu = ParallelPresenceRingPolicy(capacity, id_space, "cpu")
    gpu = ParallelPresenceRingPolicy(capacity, id_space, "cuda")
    hot = list(range(200))
    for step in range(600):
        n_cold = 3 if step % 50 else 400                   # bursts force evictions deep into old buckets
        ids = sorted(set(rng.sample(hot, 60)) | set(rng.sample(range(id_space), n_cold)))
        rng.shuffle(ids)
        t = torch.tensor(ids, dtype=torch.int32)
        a, b = cpu.step(t), gpu.step(t)
        assert a[:2] == b[:2], step
        assert a[2].tolist() == b[2].cpu().tolist(), step
    assert cpu.totals == gpu.totals and gpu.totals["evictions"] > 1000
    # the device directory and the twin's agree
    assert torch.equal(cpu.dir, gpu.dir.cpu()) and torch.equal(cpu.id_of, gpu.id_of.cpu())
    ring = gpu.ring
    assert int(ring.count.sum()) == capacity - gpu.nfree
    pop = sum(bin(int(w) & 0xffffffff).count("1") for w in ring.bits.cpu().flatten().tolist())
    assert pop == capacity - gpu.nfree


def test_captured_decode_trace_replays_through_the_device_policies(native, tmp_path):
    """Selections of a running engine -> device trace ring -> file -> replay through every device policy."""
    from ulacache_b200.experiments import scheduler_study as S
    from ulacache_b200.telemetry import load_trace, validate_trace_coverage

    path = str(tmp_path / "trace.npy")
    n = S.capture_decode_trace(path, steps=5, batch=3, prompt_len=600, layers=2, tiny=True)
    assert n == 5 * 2 * 3 * 128                                   # steps x layers x requests x top-k
    trace = load_trace(path)
    assert validate_trace_coverage(trace, 5, 2) == []
    steps = [ids for ids, _ in S.trace_from_file(path)]
    rows = S.gpu_policy_timing(steps, 256, max(max(s) for s in steps) + 1)
    by = {r["policy"]: r for r in rows}
    assert set(by) == {"exact_lru", "linked_list", "presence_ring_one_thread", "presence_ring_parallel"}
    assert all(r["median_us_per_step"] > 0 and 0.0 <= r["hit_rate"] <= 1.0 for r in rows)
    # pinning every hit before choosing victims can only help: no more misses than the in-order ring
    assert by["presence_ring_parallel"]["hit_rate"] >= by["presence_ring_one_thread"]["hit_rate"] - 1e-9
