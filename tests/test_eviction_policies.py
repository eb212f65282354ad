"""Replacement-policy oracle (C++ and Python twins) and the ablation policies on CPU tensors."""
import random

import pytest
import torch

from ulacache_b200.eviction import (ExactLruPolicy, HotBufferPolicy, LinkedListLruPolicy, PolicyOracle, replay_trace,
                                    trace_hits, victim_launch_config)


def _trace(seed, steps=40, ids=200, per_step=24):
    rng = random.Random(seed)
    hot = list(range(30))
    out = []
    for _ in range(steps):
        s = set(rng.sample(hot, 10)) | set(rng.sample(range(ids), per_step - 10))
        out.append(sorted(s))
    return out


@pytest.mark.parametrize("kind", ["bucket_ring", "exact_lru", "linked_list", "clock", "per_request"])
def test_cpp_oracle_matches_python_twin(kind):
    trace = _trace(1)
    reqs = [[i % 4 for i in range(len(s))] for s in trace]
    a = PolicyOracle(kind, 64, per_request=16, native=True)
    b = PolicyOracle(kind, 64, per_request=16, native=False)
    assert a.is_native and not b.is_native
    for ids, rq in zip(trace, reqs):
        ra = a.step(ids, rq if kind == "per_request" else None)
        rb = b.step(ids, rq if kind == "per_request" else None)
        assert ra == rb
    assert a.totals == b.totals and a.resident() == b.resident() <= 64
    a.release(trace[-1]); b.release(trace[-1])
    assert a.resident() == b.resident()


def test_recency_policies_beat_clock_on_a_hot_set():
    trace = _trace(2, steps=80)
    lru = replay_trace("exact_lru", 48, trace)
    ring = replay_trace("bucket_ring", 48, trace)
    assert lru["hit_rate"] > 0.2 and abs(ring["hit_rate"] - lru["hit_rate"]) < 0.02   # ring == LRU within 255 steps
    assert lru["overflow"] == 0 and lru["resident"] == 48


def test_exact_lru_tensor_policy_matches_oracle():
    trace = _trace(3)
    pol = ExactLruPolicy(64, 200, "cpu")
    ora = PolicyOracle("exact_lru", 64)
    for ids in trace:
        # the tensor policy pins the whole step's hits before it picks victims (as the residency
        # transaction does); the oracle sees the same order when the resident ids come first
        resident = [i for i in ids if int(pol.dir[i]) >= 0]
        ordered = resident + [i for i in ids if int(pol.dir[i]) < 0]
        h, m, ev = pol.step(torch.tensor(ids))
        oh, om, oev, _ = ora.step(ordered)
        assert (h, m) == (oh, om) and sorted(ev.tolist()) == sorted(oev)


def test_linked_list_and_hot_buffer_cpu_paths():
    trace = _trace(4)
    ll = LinkedListLruPolicy(64, 200, "cpu")
    ora = PolicyOracle("linked_list", 64)
    for ids in trace:
        assert ll.step(torch.tensor(ids))[:2] == ora.step(ids)[:2]
    hb = HotBufferPolicy(2, 8, "cpu")
    ids = torch.tensor([1, 2, 3, 1, 9, 9], dtype=torch.int32)
    assert hb.step(ids, torch.tensor([0, 4, 6])) == (2, 4)
    assert hb.step(ids, torch.tensor([0, 4, 6])) == (6, 0)


def test_presence_ring_policy_cpu_path():
    from ulacache_b200.eviction import PresenceRingPolicy

    pol = PresenceRingPolicy(64, 200, "cpu")
    ora = PolicyOracle("bucket_ring", 64)
    for ids in _trace(6):
        h, m, ev = pol.step(torch.tensor(ids))
        oh, om, oev, _ = ora.step(ids)
        assert (h, m) == (oh, om) and ev.tolist() == oev


def test_trace_hits_and_launch_config():
    d = torch.tensor([3, -1, -5, 0, 7], dtype=torch.int32)
    assert trace_hits(d, torch.tensor([[0, 1, 2], [4, -1, 9]])) == (2, 4)
    cfg = victim_launch_config(1 << 20)
    assert cfg.blocks <= 148 and cfg.threads == 256


def test_presence_bitmap_tree_against_a_python_set():
    """The 32-ary presence bitmap (set / clear / lowest set slot at or after a position / count)
    against a plain set, on a size that needs three tree levels."""
    import ctypes as C
    import random

    from ulacache_b200.ops import _native as N

    lib = N.host()
    lib.ulc_presence_create.restype = C.c_void_p
    lib.ulc_presence_create.argtypes = [C.c_longlong]
    lib.ulc_presence_op.restype = C.c_longlong
    lib.ulc_presence_op.argtypes = [C.c_void_p, C.c_int, C.c_longlong]
    lib.ulc_presence_destroy.argtypes = [C.c_void_p]
    slots = 40000                                   # 1250 + 40 + 2 + 1 words
    h = lib.ulc_presence_create(slots)
    rng = random.Random(3)
    ref = set()
    try:
        for step in range(6000):
            s = rng.randrange(slots) if rng.random() < 0.7 else rng.choice([0, 31, 32, 1023, 1024, 32767, 32768, slots - 1])
            if rng.random() < 0.6:
                assert lib.ulc_presence_op(h, 0, s) == (0 if s in ref else 1)
                ref.add(s)
            else:
                assert lib.ulc_presence_op(h, 1, s) == (1 if s in ref else 0)
                ref.discard(s)
            if step % 50 == 0:
                assert lib.ulc_presence_op(h, 4, 0) == len(ref)
                for start in (0, rng.randrange(slots), slots - 1):
                    want = min((x for x in ref if x >= start), default=-1)
                    assert lib.ulc_presence_op(h, 3, start) == want
                probe = rng.randrange(slots)
                assert lib.ulc_presence_op(h, 2, probe) == (1 if probe in ref else 0)
        for s in sorted(ref):                       # drain in order through find-first
            assert lib.ulc_presence_op(h, 3, 0) == s
            assert lib.ulc_presence_op(h, 1, s) == 1
        assert lib.ulc_presence_op(h, 4, 0) == 0 and lib.ulc_presence_op(h, 3, 0) == -1
    finally:
        lib.ulc_presence_destroy(h)


def test_bitmap_ring_takes_the_bucket_ring_decisions():
    """Policy 5 (hierarchical presence bitmaps) evicts exactly what policy 0 (scan over the stamps)
    evicts, step by step, including records that stay untouched for more than 255 steps."""
    import random

    from ulacache_b200.eviction.oracle import PolicyOracle

    rng = random.Random(11)
    a = PolicyOracle("bucket_ring", 96, native=True)
    b = PolicyOracle("bitmap_ring", 96, native=True)
    assert a.is_native and b.is_native
    hot = list(range(1, 40))
    for step in range(700):
        ids = [rng.choice(hot) for _ in range(rng.randrange(1, 12))]
        if step % 3 == 0:
            ids += [1000 + step * 7 + j for j in range(rng.randrange(0, 9))]     # a stream of new records
        if step % 97 == 0:
            gone = [1000 + (step - 50) * 7 + j for j in range(4)]
            a.release(gone)
            b.release(gone)
        ra, rb = a.step(ids), b.step(ids)
        assert ra == rb, (step, ra, rb)
    assert a.resident() == b.resident()
    # records that age past 255 epochs before there is any pressure: victims come from the cold bucket
    a = PolicyOracle("bucket_ring", 400, native=True)
    b = PolicyOracle("bitmap_ring", 400, native=True)
    first = list(range(5000, 5300))
    assert a.step(first) == b.step(first)
    for step in range(300):
        ids = [5000 + rng.randrange(20) for _ in range(4)]
        assert a.step(ids) == b.step(ids)
    evicted = []
    for step in range(40):
        ids = [9000 + step * 10 + j for j in range(10)]
        ra, rb = a.step(ids), b.step(ids)
        assert ra == rb, (step, ra, rb)
        evicted += ra[2]
    assert evicted and all(5020 <= e < 5300 for e in evicted[:100])       # old, untouched records go first
    # the Python twin takes the same decisions too
    c = PolicyOracle("bitmap_ring", 8, native=False)
    d = PolicyOracle("bucket_ring", 8, native=False)
    for step in range(50):
        ids = [rng.randrange(1, 30) for _ in range(5)]
        assert c.step(ids) == d.step(ids)


def test_parallel_ring_policy_cpu_semantics():
    """Transaction semantics of the parallel ring's CPU twin: hits are pinned before victims are chosen,
    victims are the oldest (cold first), lowest slot first; epochs before the first advance count."""
    import torch
    from ulacache_b200.eviction import ParallelPresenceRingPolicy

    pol = ParallelPresenceRingPolicy(4, 32, "cpu")
    assert pol.step(torch.tensor([1, 2, 3, 4]))[:2] == (0, 4)          # fills slots 0..3
    h, m, ev = pol.step(torch.tensor([9, 1]))                          # 1 is hit AFTER 9 in the list, yet pinned first
    assert (h, m) == (1, 1) and ev.tolist() == [2]                     # victim: lowest untouched slot (slot 1 = id 2)
    h, m, ev = pol.step(torch.tensor([3, 10, 11]))
    assert (h, m) == (1, 2) and ev.tolist() == [4, 1]                  # id 4 (epoch 1) is the oldest; then epoch 2's lowest slot (slot 0 = id 1)
    assert pol.totals == dict(hits=2, misses=7, evictions=3, overflow=0)
    h, m, ev = pol.step(torch.tensor([20, 21, 22, 23, 24]))            # more misses than evictable slots
    assert m == 5 and len(ev) == 4 and pol.totals["overflow"] == 1


def test_sequential_ring_handles_touches_before_the_first_advance():
    """Slots touched at epoch 0 are victims while recent, turn cold when their bucket is reused at epoch 255 and
    are evicted first afterwards (host build of the presence-bitmap header)."""
    import ctypes as C

    from ulacache_b200.ops import _native as N

    lib = N.host()
    for epochs in (1, 3, 254, 255, 256, 300, 520):
        assert lib.ulc_presence_ring_epoch0_check(C.c_int(2048), C.c_int(5), C.c_int(epochs)) == 0, epochs
