import os

import pytest
import torch

from ulacache_b200.tools.benchmark_budget import hot_buffer_records, pooled_records
from ulacache_b200.tools.fixed_output import FixedMTPReplay, FixedTokenReplay, ReplayExhausted
from ulacache_b200.tools.fp8_loading import dequantize_block_scaled
from ulacache_b200.transfer.direct_receive import (OrderedReceiveWindow, ReceiveNotComplete, coalesce_slots,
                                                   plan_direct_receive, publish_received)
from ulacache_b200.transfer.index_pages import PAGE_BYTES, plan_index_page_receive


def test_extents_coalesce_and_cover_every_record_once():
    slots = [10, 11, 12, 40, 41, 7, 100, 101, 102, 103]
    assert coalesce_slots(slots) == [(0, 10, 3), (3, 40, 2), (5, 7, 1), (6, 100, 4)]
    assert coalesce_slots(slots, 2)[0] == (0, 10, 2)
    plan = plan_direct_receive(slots, record_bytes=656, layers=3, layer_stride=1 << 20, base_address=1 << 30,
                               pool_slots=1024)
    assert plan.chunk_count == 12 and plan.total_bytes == 3 * len(slots) * 656
    e = plan.extents[2][3]
    assert e.address == (1 << 30) + 2 * (1 << 20) + 100 * 656 and e.records == 4 and e.first_record == 6
    # the planned bytes, copied by a stand-in transport, reproduce the records at their slots
    src = torch.randint(0, 255, (len(slots), 656), dtype=torch.uint8)
    pool = torch.zeros(1024 * 656, dtype=torch.uint8)
    for ext in plan.extents[0]:
        off = ext.address - (1 << 30)
        pool[off:off + ext.nbytes] = src[ext.first_record:ext.first_record + ext.records].reshape(-1)
    assert torch.equal(pool.view(1024, 656)[torch.tensor(slots)], src)
    with pytest.raises(ValueError):
        plan_direct_receive([1, 1], record_bytes=656, layers=1, layer_stride=0, base_address=0)


def test_ordered_window_and_publication_gate():
    w = OrderedReceiveWindow(4)
    w.accept(2); w.accept(0)
    assert w.ready_prefix == 1 and not w.complete and w.missing() == [1, 3]
    with pytest.raises(ReceiveNotComplete):
        publish_received(lambda ids: ids, [1, 2], w)
    with pytest.raises(ValueError):
        w.accept(2)
    w.accept(1); w.accept(3)
    assert w.ready_prefix == 4 and publish_received(lambda ids: len(ids), [1, 2], w) == 2


def test_index_page_plan_partial_last_page():
    ext = plan_index_page_receive([5, 9], tokens=64 * 2 + 10, base_address=0, layer_stride=1 << 20, layers=1,
                                  ranks=2, rank=1)
    # rank 1 owns tokens [64,128) fully and [192,256) not at all (138 tokens only)
    assert ext == [[(5 * PAGE_BYTES, PAGE_BYTES)]]
    ext0 = plan_index_page_receive([5, 9], tokens=138, base_address=0, layer_stride=0, layers=1, ranks=2, rank=0)
    assert ext0[0][0] == (5 * PAGE_BYTES, PAGE_BYTES) and ext0[0][1:] == [(9 * PAGE_BYTES, 10 * 128),
                                                                          (9 * PAGE_BYTES + 8192, 40)]


def test_replays_budgets_and_fp8(tmp_path):
    rep = FixedTokenReplay.record([7, 9], [[1, 2], [3, 4], [5, 6]])
    assert rep.next_tokens([7, 9]) == [1, 2] and rep.next_tokens([9]) == [4] and rep.remaining(9) == 1
    p = os.path.join(tmp_path, "r.json")
    rep.save(p)
    assert FixedTokenReplay.load(p).next_tokens([7]) == [1]
    mtp = FixedMTPReplay({1: [10, 11, 12, 13]}, {1: [2, 0]}, draft_steps=2)
    assert mtp.next_verify(1) == [10, 11, 12] and mtp.next_verify(1) == [13]
    with pytest.raises(ReplayExhausted):
        mtp.next_verify(1)
    assert hot_buffer_records(61 * 656 * 64 * 100, requests=64, record_bytes=656, layers=61) == 100
    dev, host = pooled_records(10**9, 10**9, record_bytes=656, layers=61)
    assert host == 10**9 // (656 * 61) and 0 < dev < host
    q = torch.randn(256, 128).to(torch.float8_e4m3fn)
    s = torch.tensor([[2.0], [0.5]])
    d = dequantize_block_scaled(q, s)
    assert torch.equal(d[:128], q[:128].float() * 2) and torch.equal(d[128:], q[128:].float() * 0.5)


def test_direct_receiver_places_bytes_into_canonical_records():
    import ctypes

    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from ulacache_b200.ops import records
    from ulacache_b200.transfer.direct_receiver import DirectReceiver

    from helpers import make_spec, random_kv

    cache = ula.init(make_spec(layers=2, device_pages=2, host_pages=8), LocalCacheBindings(device="cpu"))
    rx = DirectReceiver(cache, layers=2, chunk_records=32)
    n = 300                                            # 128 records fit the device tier, the rest go to host slots
    ticket = rx.prepare(n)
    assert set(ticket.plans) == {"device", "host"}
    latent, rope = random_kv(n, 5)
    payload = [records.encode_scaled656(latent * (l + 1), rope) for l in range(2)]
    with pytest.raises(ReceiveNotComplete):
        rx.publish(ticket)
    for tier, plan in ticket.plans.items():
        pos = ticket.positions[tier]
        seq = 0
        for layer, extents in enumerate(plan.extents):
            src = payload[layer][pos]                 # this tier's records of the layer, in plan order
            for e in extents:                          # the "transport": a raw byte copy to the planned address
                buf = src[e.first_record:e.first_record + e.records].contiguous()
                ctypes.memmove(e.address, buf.data_ptr(), e.nbytes)
                ticket.windows[tier].accept(seq)
                seq += 1
    ids = rx.publish(ticket)[:n]
    # the cache now serves those records like any it wrote itself (host-resident ones get promoted)
    truth = records.decode_scaled656(payload[1])
    g = torch.Generator().manual_seed(0)
    pick = ids[torch.randperm(n, generator=g)[:64]].view(1, 64)
    cache.begin_model_forward()
    cache.access(pick, 1)
    got = records.decode_scaled656(cache.gather_selected_records(1)).view(64, 576)
    where = {int(i): k for k, i in enumerate(ids.tolist())}
    assert torch.equal(got, truth[torch.tensor([where[int(i)] for i in pick[0]])])
    cache.finish_layer_attention(1)
    cache.finish_model_forward()
    cache.close()


def _leased_residency(device, **kw):
    import torch
    from ulacache_b200.cache.residency import ResidencyGeometry, make_residency
    from ulacache_b200.storage.layout import OwnerMap
    from ulacache_b200.transfer.receive_lease import ReceiveLeases

    res = make_residency(ResidencyGeometry(dir_len=512, hbm_slots=8, host_slots=16, plan_capacity=16), OwnerMap(1, 6), 0, device, **kw)
    ids = torch.arange(1, 13, dtype=torch.int32, device=device)          # 8 land in HBM, 4 on the host
    res.begin_step()
    res.register(ids)
    return res, ids, ReceiveLeases(res)


def _lease_scenario(device, **kw):
    """Leased device slots cannot be victims; the last release re-attaches them as touched now."""
    import torch
    from ulacache_b200.cache.residency import CNT_PLAN

    res, ids, leases = _leased_residency(device, **kw)
    incoming = ids[[0, 1, 9]]                                            # two device rows and a host row
    loc = leases.acquire(incoming)
    loc2 = leases.acquire(incoming[:1])                                  # a second writer on the first row
    ring_leased = int(res.ring.sum())
    # a later step wants three promotions: with slots 0 and 1 leased, victims must come from the other six
    for _ in range(2):
        res.begin_step()
    res.pin(ids[8:11])                                                   # three host rows -> three promotions
    res.plan_step()
    n = int(res.counters[CNT_PLAN])
    victims = res.plan[1, :n].cpu().tolist()
    leases.release(incoming[:1], loc2)
    still = int(res.stamps[int(loc[0])])
    leases.release(incoming, loc)
    out = dict(loc=loc.cpu().tolist(), ring_leased=ring_leased, victims=sorted(victims), still_leased=still,
               stamps=[int(res.stamps[int(loc[0])]), int(res.stamps[int(loc[1])])], ring_after=int(res.ring.sum()),
               leases=int(leases.leases.sum()))
    if hasattr(res, "check_status"):
        res.check_status("receive leases")
    return out


def test_receive_leases_cpu():
    out = _lease_scenario("cpu")
    assert out["loc"][0] >= 0 and out["loc"][1] >= 0 and out["loc"][2] <= -2
    assert out["ring_leased"] == 6 and out["still_leased"] == -2 and out["leases"] == 0
    assert len(out["victims"]) == 3 and not set(out["victims"]) & {out["loc"][0], out["loc"][1]}
    assert out["stamps"] == [3, 3] and out["ring_after"] == 8


def test_publish_copies_to_both_tiers_cpu():
    import torch
    from ulacache_b200.transfer.receive_lease import ReceiveLeases

    res, ids, leases = _leased_residency("cpu")
    loc = leases.acquire(ids[[2, 10, 5]])
    staging = torch.randint(0, 255, (3, 4, 656), dtype=torch.uint8)
    dev_plane, host_plane = torch.zeros(3, 8, 656, dtype=torch.uint8), torch.zeros(3, 16, 656, dtype=torch.uint8)
    leases.publish(staging, torch.tensor([3, 0, 1]), loc, dev_plane, host_plane)
    assert torch.equal(dev_plane[:, int(loc[0])], staging[:, 3]) and torch.equal(dev_plane[:, int(loc[2])], staging[:, 1])
    assert torch.equal(host_plane[:, -int(loc[1]) - 2], staging[:, 0])
    assert int(dev_plane.sum()) == int(staging[:, 3].sum()) + int(staging[:, 1].sum())


def test_recorded_cohort_replays_check_order_positions_and_hash(tmp_path):
    import torch
    from ulacache_b200.tools.fixed_output import (MTP_SCHEMA, ReplayMismatch, ReplayTrace, TraceMTPReplay,
                                                  TraceTokenReplay, force_logits)

    outputs = {"a": [5, 6, 7, 8], "b": [9, 10, 11, 12]}
    trace = ReplayTrace.from_token_run(attention_dp=2, repeat=0, rank=1, keys=["a", "b"], input_tokens=[100, 40],
                                       outputs=outputs)
    sha = trace.save(str(tmp_path / "t.json.gz"))
    again = ReplayTrace.load(str(tmp_path / "t.json.gz"))
    assert again.sha256 == sha and not again.speculative
    rp = TraceTokenReplay(again, attention_dp=2, rank=1)
    for step in range(4):
        rp.begin("c0", repeat=0, keys=["a", "b"], seq_lens=[100 + step, 40 + step], trace_sha256=sha)
        got = rp.sample(torch.zeros(2, dtype=torch.int64))
        assert got.tolist() == [outputs["a"][step], outputs["b"][step]]
        with pytest.raises(ReplayMismatch):
            rp.sample(torch.zeros(2, dtype=torch.int64))            # one sampler call per step
        rp.end()
    r = rp.receipt("c0")
    assert r["complete"] and r["frames"] == r["expected_frames"] == 4 and not r["natural_accuracy_claimed"]
    with pytest.raises(ReplayMismatch):                              # past the recorded budget
        rp.begin("c0", repeat=0, keys=["a", "b"], seq_lens=[104, 44])
    other = TraceTokenReplay(again, attention_dp=2, rank=1)
    with pytest.raises(ReplayMismatch):                              # a different request order is a different workload
        other.begin("c1", repeat=0, keys=["b", "a"], seq_lens=[40, 100])
    with pytest.raises(ReplayMismatch):
        other.begin("c1", repeat=0, keys=["a", "b"], seq_lens=[100, 40], trace_sha256="0" * 64)
    with pytest.raises(ReplayMismatch):
        again.episode(4, 0, 2, 1)
    with pytest.raises(ValueError):
        ReplayTrace(dict(schema="ulc-fixed-output-replay-v1", speculative=False, output_tokens=3, cases={},
                         episodes={"e": dict(keys=["a"], input_tokens=[1], saved_bootstrap_tokens=0,
                                             expected_output_ids={"a": [1, 2]})}))

    frames = [dict(keys=["a", "b"], seq_lens=[10, 20], draft_tokens=[[1, 2, 3], [4, 5, 6]], accept_lens=[3, 1],
                   emitted=[[1, 2, 3], [4]]),
              dict(keys=["a"], seq_lens=[13], draft_tokens=[[7, 8, 9]], accept_lens=[2], emitted=[[7, 8]])]
    mtp = ReplayTrace(dict(schema=MTP_SCHEMA, forced_acceptance=True, output_tokens=8, cases={"1:0:2:0": "e"},
                           episodes={"e": dict(steps=2, verify_width=3, batch=2, frames=frames)}))
    mr = TraceMTPReplay(mtp, attention_dp=1, rank=0)
    d = mr.draft("c", repeat=0, keys=["a", "b"], seq_lens=[10, 20], steps=2)
    assert d.tolist() == [[1, 2, 3], [4, 5, 6]]
    with pytest.raises(ReplayMismatch):
        mr.draft("c", repeat=0, keys=["a", "b"], seq_lens=[10, 20], steps=2)      # overlapping step
    tok, ln = mr.sample(torch.zeros(2, 3, dtype=torch.int32), torch.zeros(2, dtype=torch.int32))
    assert tok.tolist() == [[1, 2, 3], [4, -1, -1]] and ln.tolist() == [3, 1]
    d = mr.draft("c", repeat=0, keys=["a"], seq_lens=[13], steps=2)
    tok, ln = mr.sample(torch.zeros(1, 3, dtype=torch.int32), torch.zeros(1, dtype=torch.int32))
    assert tok.tolist() == [[7, 8, -1]] and mr.completed("c") and mr.receipt("c")["forced_acceptance"]
    with pytest.raises(ValueError):
        ReplayTrace(dict(schema=MTP_SCHEMA, forced_acceptance=True, output_tokens=8, cases={},
                         episodes={"e": dict(steps=2, verify_width=4, batch=1, frames=[])}))

    logits = torch.randn(2, 16)
    force_logits(logits, [[3, 4], [9]], [1, 0])
    assert logits.argmax(1).tolist() == [4, 9] and int(torch.isinf(logits).sum()) == 30
    with pytest.raises(ReplayMismatch):
        force_logits(torch.randn(1, 4), [[7]], [0])


def test_received_index_records_are_published_to_their_owners_pages():
    import numpy as np
    import torch
    from ulacache_b200.transfer.index_pages import (PAGE_BYTES, IndexRecordCopy, plan_index_record_copies,
                                                    publish_index_record_bytes, publish_index_records, record_offsets,
                                                    validate_index_record_plan)

    ranks = 2
    # logical records of pages 2..5 (pages 0-1 are the owners' padding pages); rank 1 owns pages 3 and 5
    logical = [2 * 64 + 5, 3 * 64 + 0, 3 * 64 + 63, 5 * 64 + 7, 4 * 64 + 1]
    received = [0, 1, 64, 65, 2]
    plan = plan_index_record_copies(logical, received, ranks=ranks, rank=1)
    assert [p.logical_record for p in plan] == [3 * 64, 3 * 64 + 63, 5 * 64 + 7]
    assert [p.destination_record for p in plan] == [64, 127, 2 * 64 + 7]
    assert record_offsets(65) == (PAGE_BYTES + 128, PAGE_BYTES + 8192 + 4)
    rng = np.random.default_rng(0)
    staging = rng.integers(0, 255, 2 * PAGE_BYTES, dtype=np.uint8)
    canon = np.zeros(3 * PAGE_BYTES, dtype=np.uint8)
    assert publish_index_record_bytes(staging, canon, plan, transport_quiesced=True) == 3
    for p in plan:
        assert np.array_equal(canon[p.destination_key_byte:p.destination_key_byte + 128], staging[p.source_key_byte:p.source_key_byte + 128])
        assert np.array_equal(canon[p.destination_scale_byte:p.destination_scale_byte + 4], staging[p.source_scale_byte:p.source_scale_byte + 4])
    assert int((canon != 0).sum()) <= 3 * 132
    # the tensor form writes the same bytes
    canon_t = torch.zeros(3, PAGE_BYTES, dtype=torch.uint8)
    assert publish_index_records(torch.from_numpy(staging).view(2, PAGE_BYTES), canon_t, plan, transport_quiesced=True) == 3
    assert np.array_equal(canon_t.numpy().reshape(-1), canon)
    with pytest.raises(RuntimeError):
        publish_index_record_bytes(staging, canon, plan, transport_quiesced=False)
    with pytest.raises(ValueError):
        publish_index_record_bytes(canon, canon, plan, transport_quiesced=True)            # aliasing
    with pytest.raises(ValueError):
        publish_index_record_bytes(staging, canon[: 2 * PAGE_BYTES].copy(), plan, transport_quiesced=True)   # beyond storage
    with pytest.raises(ValueError):
        plan_index_record_copies([5], [0], ranks=2, rank=0)                                 # padding page
    with pytest.raises(ValueError):
        plan_index_record_copies([200, 200], [0, 1], ranks=2, rank=0)                       # duplicates
    with pytest.raises(ValueError):
        IndexRecordCopy(2, 0, 3 * 64, 0, 64, 0, 0, 8192, 8192)                              # page 3 belongs to rank 1
    dup = plan + (plan[0],)
    with pytest.raises(ValueError):
        validate_index_record_plan(dup, 2 * PAGE_BYTES, 3 * PAGE_BYTES)


def test_budget_and_fp8_loading_helpers():
    import torch
    from ulacache_b200.ops import fp8
    from ulacache_b200.tools import benchmark_budget as B, fp8_loading as F

    assert B.restored_cohort_metadata_tokens(requests=32, page_size=64) == 33 * 64
    # 1M physical rows, 32 requests, a 32K prefill reserve: (1048576 - 32768) / (32 * 64) pages, minus one page, capped at 2^15
    assert B.hot_buffer_rows(physical_rows=1 << 20, requests=32, prefill_rows=32768) == min((1015808 // 2048) * 64 - 64, 32768)
    assert B.hot_buffer_rows(physical_rows=1 << 22, requests=8, prefill_rows=1000) == 32768          # rank limit
    with pytest.raises(ValueError):
        B.hot_buffer_rows(physical_rows=100000, requests=64, prefill_rows=32768)                     # below one selection
    with pytest.raises(ValueError):
        B.restored_cohort_metadata_tokens(requests=0)
    x = torch.randn(5, 512)
    q, s = fp8.act_quant_reference(x.to(torch.bfloat16))
    back = F.dequantize_aligned_rows(q, s, (1, 128))
    assert back.shape == (5, 512) and (back - x).abs().max() < 0.3
    assert F.aligned_row_block_scales(q.view(torch.float8_e4m3fn), s, (1, 128))
    assert not F.aligned_row_block_scales(q, s, (128, 128)) and not F.aligned_row_block_scales(q, s[:, :3], (1, 128))
    with pytest.raises(ValueError):
        F.dequantize_aligned_rows(q, s.double(), (1, 128))
