"""Selection forms over Index scores: rank-major gathered, compact (ragged) gathered, paged transform."""
import pytest
import torch

from ulacache_b200.indexer.ownership import IndexOwnership
from ulacache_b200.indexer.topk import merge_candidates, paged_record_ids, topk_compact, topk_local, topk_rank_major


def _case(device, ranks=4, rows=5, cols=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    own = IndexOwnership(ranks, 64)
    width = ranks * cols
    logical = torch.randn(rows, width, generator=g)
    logical[:, 100] = logical[:, 300]                          # a tie: the lower token must win
    lengths = torch.tensor([width, 700, 65, 64, 3][:rows])
    gathered = torch.stack([logical[:, own.logical_token(r, torch.arange(cols))] for r in range(ranks)])
    return own, logical, lengths, gathered.to(device)


def _want(logical, lengths, k):
    out = []
    for r in range(logical.shape[0]):
        n = int(lengths[r])
        out.append(sorted(torch.sort(logical[r, :n], descending=True, stable=True).indices[:k].tolist()))
    return out


def _sets(ids):
    return [sorted(i for i in row.tolist() if i >= 0) for row in ids]


def _check_forms(device):
    own, logical, lengths, gathered = _case(device)
    k = 48
    assert _sets(topk_rank_major(gathered, lengths, k, own)) == _want(logical, lengths, k)
    # paged transform: token t of row r lives in record page_table[r, t // 64] * 64 + t % 64
    pages = torch.stack([torch.randperm(64, generator=torch.Generator().manual_seed(r))[:16] for r in range(5)]).to(torch.int32)
    rec = topk_rank_major(gathered, lengths, k, own, page_table=pages.to(device))
    tok = topk_rank_major(gathered, lengths, k, own)
    assert _sets(rec) == _sets(paged_record_ids(tok.cpu(), pages))
    # forced windows
    forced = topk_rank_major(gathered, lengths, k, own, always_first=4, always_recent=8)
    for r, row in enumerate(_sets(forced)):
        n = int(lengths[r])
        must = set(range(min(4, n))) | set(range(max(0, n - 8), n))
        assert must <= set(row) and len(row) == min(k, n)
    # compact input: ranks sent only a prefix of each row; the fill value must never win
    sent = torch.stack([own.local_length(lengths, r) for r in range(own.ranks)]).to(torch.int32)
    ragged = gathered.clone()
    col = torch.arange(gathered.shape[2], device=device)[None, None, :]
    ragged[col >= sent.to(device)[:, :, None]] = 1e9
    assert _sets(topk_compact(ragged, sent, lengths, k, own)) == _want(logical, lengths, k)


def test_rank_major_compact_and_paged_forms_cpu():
    _check_forms("cpu")


@pytest.mark.gpu
def test_rank_major_compact_and_paged_forms_gpu(native):
    _check_forms("cuda")


def test_local_and_merge_forms_cpu():
    torch.manual_seed(1)
    s = torch.randn(3, 200)
    ids = topk_local(s, 16, lengths=torch.tensor([200, 10, 0], dtype=torch.int32))
    assert _sets(ids)[1] == list(range(10)) and _sets(ids)[2] == []
    vals = torch.tensor([[0.5, 2.0, float("-inf"), 1.0]])
    cid = torch.tensor([[7, 9, 11, 3]], dtype=torch.int32)
    assert merge_candidates(vals, cid, 3).tolist() == [[9, 3, 7]]
    assert merge_candidates(vals, cid, 4).tolist() == [[9, 3, 7, -1]]
