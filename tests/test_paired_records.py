"""Paired record planes (K / V), request-table composition and receive-side slot ordering: references on the CPU,
kernels against them on the GPU."""
import pytest
import torch

from ulacache_b200.ops import paired


def _inputs(device, seed=0):
    g = torch.Generator().manual_seed(seed)
    requests_total, context, rows, width = 5, 300, 7, 40
    table = torch.randint(0, 5000, (requests_total, context), generator=g, dtype=torch.int32)
    requests = torch.randint(0, requests_total, (rows,), generator=g, dtype=torch.int32)
    lengths = torch.randint(1, context + 50, (rows,), generator=g, dtype=torch.int32)
    positions = torch.randint(-1, context + 20, (rows, width + 8), generator=g, dtype=torch.int32)[:, :width]   # row stride 48
    return [t.to(device) for t in (table, requests, positions, lengths)]


def _compose_want(table, requests, positions, lengths):
    rows, width = positions.shape
    want = torch.full((rows, width), -1, dtype=torch.int32)
    for r in range(rows):
        for c in range(width):
            p = int(positions[r, c])
            if 0 <= p < min(int(lengths[r]), table.shape[1]):
                want[r, c] = table[int(requests[r]), p]
    return want


def _pairs_case(device, dtype, heads, dim, seed=1):
    g = torch.Generator().manual_seed(seed)
    slots, rows, selected = 200, 5, 24
    key = torch.randn(slots, heads * dim, generator=g).to(dtype)
    value = torch.randn(slots, heads * dim + 8, generator=g).to(dtype)[:, : heads * dim]       # another record stride
    records = torch.randint(-1, slots, (rows, selected), generator=g, dtype=torch.int32)
    positions = torch.randint(-1, 60, (rows, selected), generator=g, dtype=torch.int32)
    lengths = torch.randint(20, 70, (rows,), generator=g, dtype=torch.int32)
    spans = torch.randint(0, selected + 1, (rows,), generator=g)
    offsets = torch.zeros(rows + 1, dtype=torch.int32)
    offsets[1:] = spans.cumsum(0)
    total = int(offsets[-1]) + selected                      # room for the padded form's tail
    return [t.to(device) for t in (key, value, records, positions, lengths, offsets)], total


def test_compose_and_pairs_references():
    table, requests, positions, lengths = _inputs("cpu")
    assert torch.equal(paired.compose_record_ids(table, requests, positions, lengths),
                       _compose_want(table, requests, positions, lengths))
    (key, value, records, positions, lengths, offsets), total = _pairs_case("cpu", torch.float32, 2, 8)
    ok, ov = paired.gather_pairs(key, value, records, positions, lengths, offsets, heads=2, total=total)
    r, c = 1, 0
    start, span = int(offsets[r]), int(offsets[r + 1] - offsets[r])
    for c in range(24):
        p, slot = int(positions[r, c]), int(records[r, c])
        if c < span and 0 <= p < int(lengths[r]) and slot >= 0:
            assert torch.equal(ok[start + c].reshape(-1), key[slot]) and torch.equal(ov[start + c].reshape(-1), value[slot])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,heads,dim", [(torch.bfloat16, 8, 128), (torch.float32, 3, 20), (torch.uint8, 2, 7)])
def test_compose_and_pairs_kernels_match_the_references(native, dtype, heads, dim):
    table, requests, positions, lengths = _inputs("cuda")
    got = paired.compose_record_ids(table, requests, positions, lengths)
    assert torch.equal(got.cpu(), _compose_want(table.cpu(), requests.cpu(), positions.cpu(), lengths.cpu()))
    for padded in (False, True):
        (key, value, records, pos, lens, offsets), total = _pairs_case("cuda", dtype if dtype != torch.uint8 else torch.float32,
                                                                       heads, dim)
        if dtype == torch.uint8:
            key, value = (key * 20).to(torch.uint8), (value * 20).to(torch.uint8)
        if padded:          # the padded form writes `columns` rows per query: the output rows of two queries must not overlap
            offsets = (torch.arange(records.shape[0] + 1, dtype=torch.int32) * 20).to("cuda")
            total = int(offsets[-1]) + 24
        gk, gv = paired.gather_pairs(key, value, records, pos, lens, offsets, heads=heads, total=total, padded=padded, columns=20)
        rk, rv = paired.gather_pairs(key.cpu(), value.cpu(), records.cpu(), pos.cpu(), lens.cpu(), offsets.cpu(), heads=heads,
                                     total=total, padded=padded, columns=20)
        assert torch.equal(gk.cpu(), rk) and torch.equal(gv.cpu(), rv)


def _tail_case(device):
    g = torch.Generator().manual_seed(3)
    stack = torch.randperm(40000, generator=g).to(torch.int32).to(device)
    count = torch.tensor([30000], dtype=torch.int32, device=device)
    return stack, count


def _check_tail(stack, count, before, window):
    n = int(count)
    start = n - window
    assert torch.equal(stack[:start].cpu(), before[:start]) and torch.equal(stack[n:].cpu(), before[n:])
    tail = stack[start:n].cpu()
    assert torch.equal(tail, torch.sort(before[start:n], descending=True).values)      # same set, descending: pops ascend


def test_sort_free_tail_reference_and_residency_hook():
    stack, count = _tail_case("cpu")
    before = stack.clone()
    assert paired.sort_free_tail(stack, count, 1000) is True
    _check_tail(stack, count, before, 16384)
    assert paired.sort_free_tail(stack, count, 20000) is False and paired.sort_free_tail(stack, count, 0) is False
    # through the engine: after churn, receive rows come out as few contiguous extents
    import dataclasses
    import ulacache_b200 as ula
    from ulacache_b200.bindings import LocalCacheBindings
    from helpers import make_spec

    def extents(order):
        b = LocalCacheBindings(device="cpu")
        b = dataclasses.replace(b, execution_options=dataclasses.replace(b.execution_options, record_storage_backend="native_paged"))
        cache = ula.init(make_spec(layers=1, device_pages=2, host_pages=32), b)
        ids = cache.alloc(128 + 1500)                              # fills the device tier and most of the host tier
        gen = torch.Generator().manual_seed(7)
        gone = ids[128:][torch.randperm(1500, generator=gen)[:900]]
        cache.free(gone)                                           # scattered holes on the host free stack
        fresh = torch.arange(int(ids.max()) + 1, int(ids.max()) + 401, dtype=torch.int32)
        rows = cache.engine.allocate_receive_rows(fresh, order_free_tail=order)
        runs = 1 + int((rows[1:] != rows[:-1] + 1).sum())
        cache.close()
        return runs

    assert extents(True) < extents(False) / 2       # 60 % of the slots were freed at random: runs of 2 to 3 adjacent rows


@pytest.mark.gpu
def test_sort_free_tail_kernel(native):
    for records, window in ((1000, 16384), (9000, 32768)):
        stack, count = _tail_case("cuda")
        before = stack.cpu().clone()
        assert paired.sort_free_tail(stack, count, records)
        torch.cuda.synchronize()
        if int(count) >= window:
            _check_tail(stack, count, before, window)
        else:                                                     # the window reaches below the stack: everything is sorted
            assert torch.equal(stack[: int(count)].cpu(), torch.sort(before[: int(count)], descending=True).values)
    small = torch.tensor([5, 9, 1, 7, 3, 100, 200], dtype=torch.int32, device="cuda")
    cnt = torch.tensor([5], dtype=torch.int32, device="cuda")
    paired.sort_free_tail(small, cnt, 4)
    assert small.tolist() == [9, 7, 5, 3, 1, 100, 200]
