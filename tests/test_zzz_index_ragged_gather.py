"""Ragged gather of Index keys for prefill scoring over an owner-striped Index."""
import pytest
import torch

from ulacache_b200.ops import indexer


def _case(device, ranks, queries=5, pages_per_owner=12, width=9, seed=0):
    g = torch.Generator().manual_seed(seed)
    pools = [torch.randint(0, 255, (pages_per_owner, 8448), dtype=torch.uint8, generator=g).to(device) for _ in range(ranks)]
    table = torch.randint(1, pages_per_owner * ranks, (queries, width), generator=g, dtype=torch.int32)
    table[1, 2] = 0                                                   # a padding page in the middle of a prefix
    lengths = torch.tensor([width * 64, 130, 1, 0, 333][:queries], dtype=torch.int32)
    return pools, table.to(device), lengths.to(device)


def test_reference_layout_on_cpu():
    pools, table, lengths = _case("cpu", 2)
    keys, scales = indexer.index_ragged_gather_reference(pools, table, lengths)
    assert keys.shape == (int(lengths.sum()), 128) and scales.shape == (int(lengths.sum()),)
    # token 70 of query 0 is record 6 of logical page table[0, 1]: owner = page % 2, local page = page // 2
    page = int(table[0, 1])
    row = pools[page % 2][page // 2]
    assert torch.equal(keys[70], row[6 * 128:7 * 128])
    assert scales[70].item() == row[8192 + 24:8192 + 28].view(torch.float32).item() or scales[70].isnan()
    start = int(lengths[0])                                           # query 1: its third page is padding -> zeros
    assert int(keys[start + 128:start + 130].sum()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("ranks", [1, 2, 8])
def test_kernel_matches_reference(ranks):
    from ulacache_b200.ops import _native as N

    pools, table, lengths = _case("cuda", ranks)
    status = N.new_status(torch.device("cuda"))
    keys, scales = indexer.index_ragged_gather(pools, table, lengths, pool_pages=pools[0].shape[0], status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "index_ragged_gather")
    want_k, want_s = indexer.index_ragged_gather_reference(pools, table, lengths)
    assert torch.equal(keys, want_k)
    assert torch.equal(scales.view(torch.int32), want_s.view(torch.int32))           # bit-equal, NaN payloads included
    # a strided page table (a slice of a wider one) and an empty batch
    wide = torch.zeros((table.shape[0], table.shape[1] + 3), dtype=torch.int32, device="cuda")
    wide[:, :table.shape[1]] = table
    k2, _ = indexer.index_ragged_gather(pools, wide[:, :table.shape[1]], lengths, pool_pages=pools[0].shape[0], status=status)
    assert torch.equal(k2, want_k)
    k0, s0 = indexer.index_ragged_gather(pools, table, torch.zeros_like(lengths), pool_pages=pools[0].shape[0])
    assert k0.shape == (0, 128) and s0.numel() == 0
