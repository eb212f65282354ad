import pytest
import torch

from ulacache_b200.cache.request_access import request_physical_rows
from ulacache_b200.cache.request_pages import PageBudgetError, RequestPagePool
from ulacache_b200.cache.request_storage import RequestPageStorage
from ulacache_b200.transfer.page_exchange import PageExchangeExecutor


def _admit(pool, ex, req, tokens):
    txn = pool.reserve_request(req, tokens)
    moved = ex.execute(pool, txn)
    return txn, moved


def test_offload_onload_waves_preserve_bytes():
    pool = RequestPagePool(device_pages=7, host_pages=8, logical_pages=32)
    st = RequestPageStorage(layers=2, device_pages=7, host_pages=8, record_bytes=16, device="cpu", pin_host=False)
    ex = PageExchangeExecutor(st)
    _admit(pool, ex, 1, 4 * 64)                       # 4 pages
    for lp in pool.pages_of[1]:
        st.device_pool[:, pool.where[lp][1]] = lp + 10
    _admit(pool, ex, 2, 2 * 64)                       # one device page left
    assert pool.is_resident(1) and pool.is_resident(2) and len(pool.free_device) == 1
    txn, moved = _admit(pool, ex, 3, 3 * 64)          # must push 2 pages of the LRU request (1) out
    assert moved == 2 and pool.resident_pages(1) == 2 and pool.is_resident(3)
    assert pool.stats["offloaded"] == 2
    # request 1 comes back: its parked pages return with their bytes; the pages of idle request 2 leave
    pool.attach(3)
    txn, moved = _admit(pool, ex, 1, 4 * 64)
    assert pool.is_resident(1) and pool.is_resident(3)          # attached requests are never victims
    for lp in pool.pages_of[1]:
        tier, dp = pool.where[lp]
        assert tier == "d" and int(st.device_pool[0, dp, 0]) == lp + 10 and int(st.device_pool[1, dp, 5]) == lp + 10
    m = pool.page_map()
    assert sorted(int(x) for x in m[m >= 0]) == sorted(dp for t, dp in pool.where.values() if t == "d")
    pool.retire(3)
    pool.free_request(3)
    assert pool.resident_pages(2) == 0
    assert len(pool.free_device) + sum(1 for t, _ in pool.where.values() if t == "d") == 7


def test_budget_errors_and_cancel():
    pool = RequestPagePool(device_pages=2, host_pages=1, logical_pages=8)
    with pytest.raises(PageBudgetError):
        pool.reserve_request(1, 5 * 64)
    txn = pool.reserve_request(1, 2 * 64)
    with pytest.raises(RuntimeError):
        pool.reserve_request(2, 64)
    pool.cancel(txn)
    assert 1 not in pool.pages_of and len(pool.free_device) == 2


def test_physical_rows():
    page_map = torch.tensor([3, -1, 0, 5], dtype=torch.int32)
    req_pages = torch.tensor([[0, 2, -1], [3, 1, -1]], dtype=torch.int32)
    pos = torch.tensor([[0, 65, 130, -1], [63, 64, 1, 200]], dtype=torch.int32)
    rows = request_physical_rows(page_map, req_pages, pos)
    assert rows.tolist() == [[3 * 64, 1, -1, -1], [5 * 64 + 63, -1, 5 * 64 + 1, -1]]


class _Runtime:
    def __init__(self):
        self.retired = True
        self.validated = 0

    def validate(self, tier):
        assert tier.storage.plane_shapes()["record_gpu"][1] == tier.pool.device_pages
        self.validated += 1

    def readers_retired(self, tier):
        return self.retired


def test_request_tier_moves_records_and_index_pages_and_publishes_at_boundaries():
    from ulacache_b200.cache.request_storage import INDEX_PAGE_BYTES, RequestTier, request_workspace_rows

    assert request_workspace_rows(64, 4, 2, 16) == 4 * 33 and request_workspace_rows(64, 1, 1, 8) == 64
    with pytest.raises(ValueError):                            # the host side is sized before anything is allocated
        RequestTier(layers=4, device_pages=8, host_pages=64, logical_pages=64, record_bytes=656, device="cpu",
                    host_memory_budget_bytes=1 << 20, pin_host=False)
    tier = RequestTier(layers=2, device_pages=8, host_pages=8, logical_pages=32, record_bytes=16, device="cpu",
                       index_anchor_layers=(0,), pin_host=False, topk=16)
    assert tier.pool.usable_device_pages == 7 and tier.check_gpu_capacity(7 * 64) and not tier.check_gpu_capacity(8 * 64)
    with pytest.raises(NotImplementedError):
        tier.attach_native_pages(1)
    rt = _Runtime()
    with pytest.raises(ValueError):
        tier.bind_runtime(None)
    tier.bind_runtime(rt)
    assert rt.validated == 1 and tier.capacity_audit()["runtime_connected"]

    tier.admit(1, 4 * 64)
    for lp in tier.pool.pages_of[1]:
        dp = tier.pool.where[lp][1]
        assert dp != 0                                          # the sentinel page is never handed out
        tier.storage.device_pool[:, dp] = lp + 10
        tier.storage.index_view(0)[dp] = lp + 50
    assert tier.page_map[tier.pool.pages_of[1]].tolist() == [tier.pool.where[lp][1] for lp in tier.pool.pages_of[1]]
    tier.admit(2, 2 * 64)
    pubs = tier.publisher.publications
    # request 3 needs 3 pages, one is free: two pages of the idle LRU request (1) are parked with their Index pages
    rt.retired = False
    with pytest.raises(RuntimeError):                          # pages cannot move under live readers
        tier.admit(3, 3 * 64)
    assert 3 not in tier.pool.pages_of and tier.publisher.publications == pubs
    rt.retired = True
    assert tier.admit(3, 3 * 64) == 2 and tier.pool.resident_pages(1) == 2
    parked = [lp for lp in tier.pool.pages_of[1] if tier.pool.where[lp][0] == "h"]
    assert all(int(tier.page_map[lp]) == -1 for lp in parked)
    for lp in parked:
        hp = tier.pool.where[lp][1]
        assert int(tier.storage.host_pool[1, hp, 3]) == lp + 10 and int(tier.storage.index.host_pool[0, hp, 100]) == lp + 50
    pages3 = tier.attach_native_pages(3)
    assert len(pages3) == 3 and 0 not in pages3
    tier.admit(1, 4 * 64)                                       # request 1 returns; request 2 (idle) makes room
    for lp in tier.pool.pages_of[1]:
        dp = int(tier.page_map[lp])
        assert dp > 0 and int(tier.storage.device_pool[0, dp, 0]) == lp + 10 and int(tier.storage.index_view(0)[dp, 7]) == lp + 50
    with pytest.raises(RuntimeError):
        tier.retire_native_pages(3, readers_retired=False)
    tier.retire_native_pages(3, readers_retired=True)
    tier.free_request(3)
    audit = tier.capacity_audit()
    assert audit["plane_shapes"]["index_gpu"] == (1, 8, INDEX_PAGE_BYTES) and audit["moved_bytes"]["d2h"] > 0
    assert audit["gpu_free_pages"] == tier.gpu_free_pages and audit["transactions"]["transactions"] == 4
    tier.clear()
    assert bool((tier.page_map == -1).all()) and tier.gpu_free_pages == 7
    tier.close()


def test_fresh_bindings_are_settled_before_a_boundary_publication():
    from ulacache_b200.cache.request_storage import PageMapPublisher

    pool = RequestPagePool(device_pages=4, host_pages=2, logical_pages=8)
    pub = PageMapPublisher(pool, "cpu")
    pub.begin_binding(2)
    with pytest.raises(RuntimeError):
        pub.publish([(0, 1)])
    pub.device_map[3], pub.device_map[4] = 2, 3                 # the allocator's own scatter on the device map
    pub.record_completed_bindings([(3, 2), (4, 3)])
    pub.publish([(0, 1)])                                       # keeps the fresh bindings
    assert pub.device_map.tolist() == [1, -1, -1, 2, 3, -1, -1, -1]


def test_request_address_runtime_brackets_forwards_and_guards_page_moves():
    from ulacache_b200.cache.request_access import RequestAddressRuntime
    from ulacache_b200.cache.request_storage import RequestTier

    tier = RequestTier(layers=2, device_pages=8, host_pages=8, logical_pages=32, record_bytes=16, device="cpu",
                       pin_host=False, topk=16)
    rt = RequestAddressRuntime(device="cpu")
    tier.bind_runtime(rt)
    tier.admit(1, 3 * 64)
    tier.admit(2, 4 * 64)
    rt.begin_forward()
    with pytest.raises(RuntimeError):
        rt.begin_forward()
    with pytest.raises(RuntimeError):                          # request 3 needs request 1's pages: readers are in flight
        tier.admit(3, 3 * 64)
    assert 3 not in tier.pool.pages_of or not tier.pool.pages_of[3]
    rt.finish_forward()
    with pytest.raises(RuntimeError):
        rt.finish_forward()
    assert tier.admit(3, 3 * 64) > 0 and rt.boundary_waits >= 1 and rt.forwards == 1
    rt.begin_prefill()
    rt.finish_prefill()
    assert rt.forwards == 2

    class Publication:                                         # peers that have not published their phase yet
        def __init__(self):
            self.published, self.free = [], False

        def publish(self, domain, phase):
            self.published.append((domain, phase))

        def may_move_records(self, domain):
            return self.free

    pub = Publication()
    grouped = RequestAddressRuntime(device="cpu", publication=pub, domain=2)
    other = RequestTier(layers=1, device_pages=4, host_pages=4, logical_pages=16, record_bytes=16, device="cpu", pin_host=False)
    other.bind_runtime(grouped)
    grouped.begin_forward()
    grouped.finish_forward()
    assert pub.published == [(2, 1)] and grouped.readers_retired(other) is False
    pub.free = True
    assert grouped.readers_retired(other) is True
    wrong = RequestTier(layers=1, device_pages=4, host_pages=4, logical_pages=16, record_bytes=16, device="cpu", pin_host=False)
    wrong.page_map = wrong.page_map.to(torch.int64)
    with pytest.raises(ValueError):
        RequestAddressRuntime(device="cpu").validate(wrong)
