"""Staged receive window: page leases, page arithmetic, publication to current locations, sidecars."""
import pytest
import torch


def test_staging_pages_lease_lifecycle():
    from ulacache_b200.transfer.receive_window import StagingPages

    pages = StagingPages(4)
    a = pages.reserve("a", 3)
    assert a.pages == (0, 1, 2) and pages.available_pages == 1
    with pytest.raises(ValueError):
        pages.reserve("a", 1)
    with pytest.raises(BufferError):
        pages.reserve("b", 2)
    with pytest.raises(RuntimeError):
        pages.release(a, transport_quiesced=False)
    pages.release(a, transport_quiesced=True)
    with pytest.raises(ValueError):
        pages.release(a, transport_quiesced=True)                # stale
    b = pages.reserve("a", 2)
    assert b.generation == a.generation + 1 and b.pages == (0, 1)


def test_page_arithmetic():
    from ulacache_b200.transfer import receive_window as W

    assert W.received_record_count(3, 64) == 192 and W.received_record_count(3, 64, 130) == 130
    assert W.received_record_count(0, 64, 0) == 0
    for bad in (128, 193):
        with pytest.raises(ValueError):
            W.received_record_count(3, 64, bad)
    assert W.drop_committed_prefix([5, 6, 7], [9, 8, 4], 128, 64) == ([7], [4])
    with pytest.raises(ValueError):
        W.drop_committed_prefix([5, 6], [9, 8], 100, 64)
    assert W.staged_state_pages([11, 12, 13, 14], [0, 3], prefix_tokens=128, page_size=64) == (11, 12, 0, 3)
    with pytest.raises(ValueError):
        W.staged_state_pages([11, 12, 13], [0, 3], prefix_tokens=128, page_size=64)
    with pytest.raises(ValueError):
        W.staged_state_pages([0, 12], [1, 3], prefix_tokens=0, page_size=64)      # canonical page 0 is padding
    assert W.transfer_pages_of_allocation_pages([2, 5], allocation_page_size=256, transfer_page_size=64) == (
        8, 9, 10, 11, 20, 21, 22, 23)
    with pytest.raises(ValueError):
        W.transfer_pages_of_allocation_pages([2, 2], allocation_page_size=256, transfer_page_size=64)
    with pytest.raises(ValueError):
        W.transfer_pages_of_allocation_pages([2], allocation_page_size=96, transfer_page_size=64)


def _cache(layers=2, device_pages=2, host_pages=8, **kw):
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings

    from helpers import make_spec

    return ula.init(make_spec(layers=layers, device_pages=device_pages, host_pages=host_pages, **kw),
                    LocalCacheBindings(device="cpu"))


def test_window_publishes_to_current_locations_with_a_sidecar():
    from ulacache_b200.ops import records
    from ulacache_b200.transfer.receive_window import StagedReceiveWindow

    from helpers import random_kv

    cache = _cache()
    window = StagedReceiveWindow(cache, record_capacity=512, copy_chunk_records=96)
    draft = torch.zeros(4096, 132, dtype=torch.uint8)               # a bank addressed by record id, odd row width
    draft_registration = window.add_sidecar("draft", [draft])
    banks = window.registration()
    assert len(banks) == 2 and banks[0][1] == 512 * 656 and banks[0][2] == 64 * 656
    assert draft_registration()[0][2] == 64 * 132
    with pytest.raises(RuntimeError):
        window.add_sidecar("late", [draft])                          # addresses are already out

    n = 300
    ids = cache.alloc(320)                                           # 128 land in HBM, the rest in host slots
    lease = window.reserve("room", ids, record_count=n)
    assert len(lease.pages) == 5 and window.available_records == 512 - 320
    with pytest.raises(ValueError):
        window.reserve("room", ids)
    latent, rope = random_kv(n, 3)
    payload = [records.encode_scaled656(latent * (l + 1), rope) for l in range(2)]
    src = window.staging_rows("room")
    for l in range(2):
        window.staging[l, src] = payload[l]                          # the "transport"
    side = torch.randint(0, 255, (n, 132), dtype=torch.uint8)
    window._sidecars["draft"]["storage"][0, src] = side
    assert window.publish("room") == n
    assert window.available_records == 512 and window.memory_inventory()["pending_publications"] == 0
    assert torch.equal(draft[ids[:n].long()], side)
    # the cache serves the published records like any it wrote itself
    truth = records.decode_scaled656(payload[1])
    g = torch.Generator().manual_seed(0)
    pick_pos = torch.randperm(n, generator=g)[:64]
    cache.begin_model_forward()
    cache.access(ids[pick_pos].view(1, 64), 1)
    got = records.decode_scaled656(cache.gather_selected_records(1)).view(64, 576)
    assert torch.equal(got, truth[pick_pos])
    cache.finish_layer_attention(1)
    cache.finish_model_forward()
    # leases are gone: every device slot is back in the recency ring
    res = cache.engine.residency[0]
    assert int(window.leases[0].leases.sum()) == 0 and int((res.stamps == -2).sum()) == 0
    cache.close()


def test_window_refuses_bad_pages_and_drops_aborted_transfers():
    from ulacache_b200.transfer.receive_window import StagedReceiveWindow

    cache = _cache()
    window = StagedReceiveWindow(cache, record_capacity=128)
    ids = cache.alloc(128)
    with pytest.raises(ValueError):
        window.reserve("x", ids[:100])                               # not whole pages
    with pytest.raises(ValueError):
        window.reserve("x", torch.cat([ids[:64], ids[:64]]))         # a page twice
    with pytest.raises(ValueError):
        window.reserve("x", ids.roll(1))                             # not page-ordered
    window.reserve("x", ids)
    with pytest.raises(BufferError):
        window.reserve("y", cache.alloc(64))
    pages = sorted({int(i) // 64 for i in ids})
    window.logical_pages_freed(pages[:1])
    assert window.available_records == 0                             # one page of the transfer is still live
    window.logical_pages_freed(pages[1:])
    assert window.available_records == 128 and not window._pending
    # a published-after-free transfer is refused, and its leases do not leak
    ids2 = cache.alloc(64)
    window.reserve("z", ids2)
    cache.free(ids2)
    with pytest.raises(RuntimeError):
        window.publish("z")
    assert int(window.leases[0].leases.sum()) == 0
    cache.close()


def test_window_handles_layer_groups_that_share_a_placement():
    from ulacache_b200.transfer.receive_window import StagedReceiveWindow, _layer_runs

    assert _layer_runs([0, 1, 2, 5, 6], {0: 0, 1: 1, 2: 2, 5: 3, 6: 4}) == [(0, 0, 3), (5, 3, 2)]
    assert _layer_runs([0, 2], (0, 1, 1)) == [(0, 0, 1), (2, 1, 1)]
    cache = _cache(layers=4, device_pages=4, host_pages=4)
    window = StagedReceiveWindow(cache, record_capacity=64)
    ids = cache.alloc(64)
    window.reserve(1, ids)
    window.staging.copy_(torch.randint(0, 255, window.staging.shape, dtype=torch.uint8))
    window.publish(1)
    eng = cache.engine
    for layer in range(4):
        res = eng.residency[eng.groups.group(layer)]
        loc = res.directory[res._owned_locals(ids.to(torch.int32))[1].long()]
        assert bool((loc >= 0).all())
        assert torch.equal(eng.layer_plane(layer)[loc.long()], window.staging[layer, :64])
    cache.close()


def test_plan_travels_as_bytes_and_is_checked_on_arrival():
    import struct

    from ulacache_b200.transfer.direct_receive import decode_plan, encode_plan, plan_direct_receive

    slots = [5, 6, 7, 20, 21, 3]
    plan = plan_direct_receive(slots, record_bytes=656, layers=3, layer_stride=1 << 20, base_address=1 << 30,
                               tier="host", chunk_records=2)
    wire = encode_plan(plan)
    assert decode_plan(wire, record_limit=6) == plan
    with pytest.raises(ValueError):
        decode_plan(wire, record_limit=5)                            # more records than the request may carry
    with pytest.raises(ValueError):
        decode_plan(b"XXXXXXXX" + wire[8:], record_limit=6)
    with pytest.raises(ValueError):
        decode_plan(wire[:-8], record_limit=6)                       # cut short
    # a run that overlaps another in the destination is refused
    (size,) = struct.unpack_from("<I", wire, 8)
    body = bytearray(wire)
    struct.pack_into("<q", body, 12 + size + 24 * 1 + 8, 0)          # second run starts on the first run's slot
    with pytest.raises(ValueError):
        decode_plan(bytes(body), record_limit=6)
    struct.pack_into("<q", body, 12 + size + 24 * 1, 5)              # and a gap in the request
    with pytest.raises(ValueError):
        decode_plan(bytes(body), record_limit=6)


def test_sender_batches_move_every_byte_once_also_from_paged_sources():
    import ctypes
    from concurrent.futures import ThreadPoolExecutor

    from ulacache_b200.transfer.direct_receive import encode_plan, iter_segments, plan_direct_receive, send_chunk

    rb, layers, n = 32, 2, 200
    dest = torch.zeros(layers, 512, rb, dtype=torch.uint8)
    g = torch.Generator().manual_seed(0)
    slots = torch.randperm(512, generator=g)[:n].sort().values.tolist()           # fragmented destination
    plan = plan_direct_receive(slots, record_bytes=rb, layers=layers, layer_stride=dest.stride(0),
                               base_address=dest.data_ptr(), chunk_records=16)
    source = torch.randint(0, 255, (layers, 256, rb), dtype=torch.uint8, generator=g)
    rows = torch.randperm(256, generator=g)[:n].tolist()                          # paged source
    bases = [source[l].data_ptr() for l in range(layers)]
    segs = [s for b in iter_segments(plan, bases, source_rows=rows, max_segments=7) for s in b]
    assert sum(s[2] for s in segs) == layers * n * rb
    assert all(len(b) <= 7 for b in iter_segments(plan, bases, source_rows=rows, max_segments=7))

    def write(batch):
        for src, dst, nbytes in batch:
            ctypes.memmove(dst, src, nbytes)
        return 0

    seen = []
    with ThreadPoolExecutor(2) as pool:
        # two chunks, the plan decoded from its wire form on the way
        assert send_chunk(write, encode_plan(plan), bases, source_rows=rows, record_count=120, record_limit=n,
                          executors=(pool,), max_inflight=3, max_segments=5, audit=seen.append) == 0
        assert send_chunk(write, plan, bases, source_rows=rows, first_record=120, executors=(pool,), audit=seen.append) == 0
    assert torch.equal(dest[:, slots], source[:, rows])
    assert int((dest.sum(-1) != 0).sum()) <= layers * n
    assert seen[0]["bytes"] + seen[1]["bytes"] == layers * n * rb and seen[0]["peak_inflight"] <= 3
    # a consecutive source coalesces to one segment per destination run
    runs = sum(1 for a, b in zip(slots, slots[1:]) if b != a + 1) + 1
    dense = [s for b in iter_segments(plan_direct_receive(slots, record_bytes=rb, layers=1, layer_stride=0,
                                                          base_address=dest.data_ptr(), chunk_records=0),
                                      bases[:1]) for s in b]
    assert len(dense) == runs
    # a failing write stops new batches, joins the rest and reports the status; an exception is re-raised
    calls = []

    def failing(batch):
        calls.append(len(batch))
        return 7 if len(calls) == 2 else 0

    assert send_chunk(failing, plan, bases, max_segments=4) == 7 and len(calls) == 2

    def raising(batch):
        raise OSError("link down")

    with pytest.raises(OSError):
        send_chunk(raising, plan, bases, max_segments=4)
    with pytest.raises(ValueError):
        list(iter_segments(plan, bases, first_record=150, record_count=100))


def test_receiver_rooms_lease_destinations_until_completion():
    from ulacache_b200.transfer.direct_receiver import DirectReceiver

    cache = _cache(device_pages=4, host_pages=8, queries=1, topk=63)          # working set: 65 device records
    audits = []
    rx = DirectReceiver(cache, layers=2, chunk_records=64, audit=audits.append)
    assert rx.working_records == 65
    assert rx.available_records == 8 * 64 + (4 * 64 - 65)
    rx.note_waiting("a")
    assert rx.can_accept(320) and not rx.can_accept(10_000)
    ids = cache.alloc(320)                                                     # 256 device + 64 host
    plans, positions = rx.reserve("a", ids, request_id=17)
    assert set(plans) == {"device", "host"} and positions["device"].numel() == 256
    res = cache.engine.residency[0]
    assert int((res.stamps == -2).sum()) == 256                                # out of the eviction ring
    assert rx.available_records == 7 * 64                                      # device side is exhausted by the room
    with pytest.raises(ValueError):
        rx.reserve("a", ids)
    with pytest.raises(ValueError):
        rx.reserve("b", ids[:64])                                              # page already has a writer
    with pytest.raises(ValueError):
        rx.reserve("b", ids[1:65])
    rx.metadata_sent("a", encoding_seconds=0.001, metadata_bytes=99)
    inv = rx.metadata_inventory()
    assert inv["pending_rooms"] == 1 and inv["leased_device_records"] == 256 and inv["payload_staging_bytes"] == 0
    assert rx.complete("a") == 320
    assert int((res.stamps == -2).sum()) == 0 and rx.metadata_inventory()["leased_device_records"] == 0
    assert audits[0]["request_id"] == 17 and audits[0]["metadata_bytes"] == 99 and audits[0]["transport_quiesced"]
    # abort: pages retire only together and only after the transport drained
    cache.free(ids)
    ids2 = cache.alloc(128)
    rx.reserve("c", ids2)
    pages = sorted({int(i) // 64 for i in ids2})
    with pytest.raises(RuntimeError):
        rx.logical_pages_freed(pages[:1], transport_quiesced=True)
    with pytest.raises(RuntimeError):
        rx.logical_pages_freed(pages, transport_quiesced=False)
    rx.logical_pages_freed(pages + [9999], transport_quiesced=True)
    assert rx.metadata_inventory()["pending_rooms"] == 0 and len(audits) == 2
    cache.close()


def test_index_records_ride_under_the_same_lease():
    from ulacache_b200.tools.snapshot.cache_io import read_index_records
    from ulacache_b200.transfer.index_pages import PAGE_BYTES
    from ulacache_b200.transfer.receive_window import IndexStagedReceiveWindow

    cache = _cache(device_pages=4, host_pages=8)
    window = IndexStagedReceiveWindow(cache, record_capacity=256, ranks=2, rank=1)
    target = torch.zeros(16, PAGE_BYTES, dtype=torch.uint8)          # this rank's Index pages of one layer
    draft = torch.zeros(32, PAGE_BYTES, dtype=torch.uint8)           # a replicated draft Index
    reg = window.add_index_page_banks("target", [target])
    window.add_index_page_banks("draft", [draft], replicated=True)
    with pytest.raises(ValueError):
        window.add_index_page_banks("target", [target])
    with pytest.raises(ValueError):
        window.add_index_page_banks("odd", [torch.zeros(100, dtype=torch.uint8)])
    assert reg()[0][2] == PAGE_BYTES
    ids = cache.alloc(256)                                           # four pages: logical pages 1..4
    window.reserve("room", ids[:192], record_count=150)
    src = window.staging_rows("room")
    g = torch.Generator().manual_seed(0)
    for name in ("target", "draft"):
        st = window._index_banks[name]["staging"]
        st.copy_(torch.randint(0, 255, st.shape, dtype=torch.uint8, generator=g))
    staged = {n: read_index_records(window._index_banks[n]["staging"][0], src) for n in ("target", "draft")}
    assert window.publish("room") == 150
    rows = ids[:150].long()
    page = rows // 64
    mine = (page % 2 == 1) & (rows >= 2 * 64)                        # this rank's stripe, padding page excluded
    local = (page // 2) * 64 + rows % 64
    assert torch.equal(read_index_records(target, local[mine]), staged["target"][mine])
    assert int(mine.sum()) > 0 and window.memory_inventory()["published_index_records"] == int(mine.sum()) + int((rows >= 64).sum())
    everyone = rows >= 64
    assert torch.equal(read_index_records(draft, rows[everyone]), staged["draft"][everyone])
    untouched = torch.ones(16 * 64, dtype=torch.bool)
    untouched[local[mine]] = False
    assert int(read_index_records(target, untouched.nonzero().flatten()).sum()) == 0
    cache.close()
