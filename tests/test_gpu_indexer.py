"""Indexer score kernel (fp8 tcgen05) against the fp32 PyTorch reference."""
import pytest
import torch

from ulacache_b200.ops import _native as N
from ulacache_b200.ops import indexer, records
from ulacache_b200.storage import layout as L

pytestmark = pytest.mark.gpu


def _index_pool(pages, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pool = torch.zeros(pages, L.INDEX_PAGE_BYTES, dtype=torch.uint8, device="cuda")
    k = torch.randn(pages * 64, 128, device="cuda", generator=g)
    q, sc = records.encode_index_key(k)
    pool[:, :8192] = q.view(pages, 8192)
    pool[:, 8192:] = sc.view(pages, 64).contiguous().view(torch.uint8).view(pages, 256)
    return pool


@pytest.mark.parametrize("R,n_q,max_pages,ranks,rank", [(1, 1, 4, 1, 0), (3, 1, 37, 1, 0), (2, 2, 16, 2, 1),
                                                       (2, 4, 9, 4, 3), (5, 1, 200, 8, 5)])
def test_index_score_matches_reference(native, R, n_q, max_pages, ranks, rank):
    torch.manual_seed(R * 100 + max_pages)
    pages = 512
    pool = _index_pool(pages)
    q = torch.randn(R, n_q, 64, 128, device="cuda")
    w = torch.randn(R, n_q, 64, device="cuda") * 0.1
    q8, wf = indexer.quantize_queries(q, w)
    page_table = torch.stack([torch.randperm(pages, device="cuda")[:max_pages] for _ in range(R)]).to(torch.int32)
    full = max_pages * 64 * ranks
    lengths = torch.randint(full // 2, full + 1, (R,), device="cuda", dtype=torch.int32)
    lengths[0] = full
    status = N.new_status("cuda")
    out = indexer.index_score(q8, wf, page_table, lengths, pool, ranks=ranks, rank=rank, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "index_score")
    ref = indexer.index_score_reference(q8, wf, page_table, lengths, pool, ranks=ranks, rank=rank)
    assert torch.equal(torch.isinf(out), torch.isinf(ref))
    fin = torch.isfinite(ref)
    err = (out[fin] - ref[fin]).abs().max().item()
    assert err < 2e-3 * ref[fin].abs().max().item() + 1e-3, err


def test_select_topk_ids(native):
    torch.manual_seed(5)
    pages, R, max_pages = 256, 3, 40
    pool = _index_pool(pages, 1)
    q8, wf = indexer.quantize_queries(torch.randn(R, 1, 64, 128, device="cuda"), torch.rand(R, 1, 64, device="cuda"))
    page_table = torch.stack([torch.randperm(pages, device="cuda")[:max_pages] for _ in range(R)]).to(torch.int32)
    lengths = torch.tensor([2560, 100, 1500], dtype=torch.int32, device="cuda")
    logits = indexer.index_score(q8, wf, page_table, lengths, pool)
    ids = indexer.select_topk(logits, 512, page_table, n_q=1)
    ref_logits = indexer.index_score_reference(q8, wf, page_table, lengths, pool)
    for r in range(R):
        n = min(512, int(lengths[r]))
        cols = torch.topk(ref_logits[r], n).indices
        want = ((page_table[r, cols >> 6].long() << 6) | (cols & 63)).tolist()
        got = [i for i in ids[r].tolist() if i >= 0]
        assert len(got) == n
        overlap = len(set(got) & set(want)) / n
        assert overlap > 0.995        # fp8 accumulation order may flip near-ties at the boundary


@pytest.mark.parametrize("R,n_q,max_pages,ranks,rank,k", [(3, 1, 40, 1, 0, 512), (4, 1, 300, 1, 0, 2048),
                                                         (2, 2, 64, 2, 1, 256), (2, 4, 40, 4, 2, 128)])
def test_fused_histogram_select_matches_separate_kernels(native, R, n_q, max_pages, ranks, rank, k):
    """The score kernel building the rows' histograms + the histogram-first select pick exactly the
    records the separate score and select kernels pick, call after call on one workspace."""
    from ulacache_b200.ops import topk as topk_op

    torch.manual_seed(R * 7 + max_pages)
    pages = 1024
    pool = _index_pool(pages, 3)
    q8, wf = indexer.quantize_queries(torch.randn(R, n_q, 64, 128, device="cuda"),
                                      torch.randn(R, n_q, 64, device="cuda"))
    page_table = torch.stack([torch.randperm(pages, device="cuda")[:max_pages] for _ in range(R)]).to(torch.int32)
    full = max_pages * 64 * ranks
    ws = topk_op.workspace(R * n_q, "cuda")
    status = N.new_status("cuda")
    for trial in range(3):
        lengths = torch.randint(1, full + 1, (R,), device="cuda", dtype=torch.int32)
        if trial == 0:
            lengths[0] = full
        if trial == 1:
            lengths[-1] = min(full, k // 2)            # a row shorter than k: everything is selected
        plain = indexer.index_score(q8, wf, page_table, lengths, pool, ranks=ranks, rank=rank, status=status)
        want = indexer.select_topk(plain, k, page_table, n_q=n_q, ranks=ranks, rank=rank)
        fused = indexer.index_score(q8, wf, page_table, lengths, pool, ranks=ranks, rank=rank, status=status,
                                    topk_workspace=ws)
        got = indexer.select_topk(fused, k, page_table, n_q=n_q, ranks=ranks, rank=rank, hist_workspace=ws)
        torch.cuda.synchronize()
        N.raise_on_status(status, "index_score")
        for r in range(R * n_q):
            assert sorted(got[r].tolist()) == sorted(want[r].tolist()), (trial, r)
        assert topk_op.workspace_is_clean(ws, R * n_q)         # the select leaves histograms and counters zero


def test_prefill_sized_selection_with_explicit_lengths_matches_the_fused_pair(native):
    """96 rows of growing context (a prefill chunk): plain scores + the row-parallel select given each row's
    length pick the records the score epilogue's histograms + the select that starts from them pick."""
    from ulacache_b200.ops import topk as topk_op

    torch.manual_seed(11)
    pages, R, max_pages, k = 2048, 96, 150, 2048
    pool = _index_pool(pages, 1)
    q8, wf = indexer.quantize_queries(torch.randn(R, 1, 64, 128, device="cuda"), torch.rand(R, 1, 64, device="cuda"))
    page_table = torch.stack([torch.randperm(pages, device="cuda")[:max_pages] for _ in range(R)]).to(torch.int32)
    lengths = (torch.arange(R, device="cuda", dtype=torch.int32) * 97 + 5).clamp(max=max_pages * 64)
    lengths[3], lengths[4], lengths[5] = 2048, 2049, 1
    ws = topk_op.workspace(R, "cuda")
    fused_logits = indexer.index_score(q8, wf, page_table, lengths, pool, topk_workspace=ws)
    fused = indexer.select_topk(fused_logits, k, page_table, n_q=1, hist_workspace=ws)
    plain_logits = indexer.index_score(q8, wf, page_table, lengths, pool)
    rows = indexer.select_topk(plain_logits, k, page_table, n_q=1, lengths=lengths)
    torch.cuda.synchronize()
    for r in range(R):
        a = sorted(i for i in fused[r].tolist() if i >= 0)
        b = sorted(i for i in rows[r].tolist() if i >= 0)
        assert a == b and len(a) == min(k, int(lengths[r])), r
