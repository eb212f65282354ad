"""Distributed Index on CPU: ownership arithmetic, rank-major layout, and two gloo ranks whose
striped scoring must select exactly what a replicated index selects."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from ulacache_b200.flashag import SlabLayout, local_columns
from ulacache_b200.indexer import IndexOwnership, IndexScorePlan, RankMajorScoreLayout


def test_ownership_round_trip_and_lengths():
    own = IndexOwnership(4, 64)
    tok = torch.arange(0, 5000)
    r, l = own.owner_of_token(tok), own.local_token(tok)
    assert torch.equal(own.logical_token(r, l), tok)
    for length in (0, 1, 63, 64, 65, 300, 4096, 4097):
        counts = [int(((tok < length) & (r == k)).sum()) for k in range(4)]
        assert counts == [int(own.local_length(length, k)) for k in range(4)]
    assert torch.equal(own.local_length(torch.tensor([65, 300]), 1), torch.tensor([1, 64]))
    assert local_columns(131072, 8) == 16384 and SlabLayout(8, 1000).bytes == 4 * 8 * 1000 * 8


def test_rank_major_layout_matches_logical_selection():
    torch.manual_seed(0)
    own = IndexOwnership(2, 64)
    lay = RankMajorScoreLayout(own, 256)
    logical = torch.randn(3, 512)
    gathered = torch.stack([logical[:, own.logical_token(r, torch.arange(256))] for r in range(2)])
    assert torch.equal(lay.to_logical(gathered), logical)
    lengths = torch.tensor([512, 100, 7])
    ids = lay.select(gathered, lengths, 16, always_first=2, always_recent=3)
    for row in range(3):
        got = [i for i in ids[row].tolist() if i >= 0]
        n = int(lengths[row])
        assert len(got) == min(16, n) and all(i < n for i in got)
        assert {0, 1} <= set(got) and {n - 1, n - 2, n - 3} <= set(got)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    from ulacache_b200.indexer import DistributedIndexScorer, OwnerIndexScorer
    from ulacache_b200.indexer.scorer import _merge

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(7)
    rows, width, k = 5, 1024, 32
    lengths = torch.tensor([1024, 700, 65, 64, 3])
    logical = torch.randn(rows, width)
    logical[:, 100] = logical[:, 200]                       # a tie: the lower token must win
    own = IndexOwnership(world, 64)
    cols = width // world
    local = logical[:, own.logical_token(rank, torch.arange(cols))]
    want = []
    for r in range(rows):
        n = int(lengths[r])
        order = torch.sort(logical[r, :n], descending=True, stable=True).indices[:k].tolist()
        want.append(sorted(order))
    for transport in ("candidates", "nccl"):
        plan = IndexScorePlan(rows=rows, max_length=width, topk=k, ranks=world, transport=transport)
        sc = DistributedIndexScorer(plan, rank=rank, group=dist.group.WORLD)
        ids = sc.select(local, lengths)
        got = [sorted(i for i in ids[r].tolist() if i >= 0) for r in range(rows)]
        assert got == want, (transport, rank)
    out[rank] = True
    dist.destroy_process_group()


def test_two_ranks_select_like_a_replicated_index():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def _owner_main(rank, world, port, out):
    """Independent queries per rank against an Index striped over both ranks."""
    import torch.distributed as dist
    from ulacache_b200.indexer import OwnerIndexScorer
    from ulacache_b200.ops import indexer, records

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows, k, max_pages = 2, 16, 3                          # contexts up to 2 * 3 * 64 tokens
    g = torch.Generator().manual_seed(11)                  # every rank builds the whole world, keeps its part
    lengths_all = torch.tensor([[300, 70], [129, 384]], dtype=torch.int32)          # [asker, row]
    keys = {(a, r): torch.randn(int(lengths_all[a, r]), 128, generator=g) for a in range(world) for r in range(rows)}
    queries = {a: (torch.randn(rows, 1, 64, 128, generator=g), torch.rand(rows, 1, 64, generator=g)) for a in range(world)}
    # owner-local pools: pages of (asker, row) striped by logical page over the owners
    pools = [[] for _ in range(world)]
    tables = torch.full((world, world, rows, max_pages), -1, dtype=torch.int32)      # [asker, owner, row, local page]
    for (a, r), kk in keys.items():
        q, sc = records.encode_index_key(kk)
        for p in range((kk.shape[0] + 63) // 64):
            owner, local = p % world, p // world
            page = torch.zeros(8448, dtype=torch.uint8)
            n = min(64, kk.shape[0] - p * 64)
            page[: n * 128] = q[p * 64: p * 64 + n].reshape(-1)
            page[8192: 8192 + n * 4] = sc[p * 64: p * 64 + n].contiguous().view(torch.uint8)
            tables[a, owner, r, local] = len(pools[owner])
            pools[owner].append(page)
    pool = torch.stack(pools[rank])
    q8, wf = indexer.quantize_queries(*queries[rank])
    from ulacache_b200.indexer import IndexScorePlan

    scorer = OwnerIndexScorer(IndexScorePlan(rows=rows, max_length=world * max_pages * 64, topk=k, ranks=world),
                              rank=rank, group=dist.group.WORLD)
    got = scorer.score(q8, wf, tables[rank].contiguous(), lengths_all[rank].contiguous(), pool)
    # dense reference on the dequantised keys
    for r in range(rows):
        kq, ks = records.encode_index_key(keys[(rank, r)])
        kd = kq.view(torch.float8_e4m3fn).float()
        s = torch.relu(torch.einsum("hd,td->ht", q8[r, 0].view(torch.float8_e4m3fn).float(), kd))
        logit = (s * wf[r, 0].unsqueeze(1)).sum(0) * ks
        want = sorted(torch.sort(logit, descending=True, stable=True).indices[:k].tolist())
        assert sorted(i for i in got[r].tolist() if i >= 0) == want, (rank, r)
    out[rank] = True
    dist.destroy_process_group()


def test_owner_scorer_serves_independent_queries():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_owner_main, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def _collective_owner_main(rank, world, port, out):
    import torch.distributed as dist
    from ulacache_b200.flashag import create_index_transport
    from ulacache_b200.indexer.nccl import CollectiveIndexOwner, local_score_columns

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    owner = create_index_transport("nccl", group=dist.group.WORLD, rank=rank, world=world, max_rows=6, cols=128,
                                   device="cpu")
    assert isinstance(owner, CollectiveIndexOwner) and owner.local_columns == local_score_columns(4, 2) == 128
    ws = owner.gathered_workspace.data_ptr()
    for q in (6, 3):                                         # a full and a partial prefix of the same workspace
        local = torch.full((q, 128), float(rank + 1)) + torch.arange(q)[:, None]
        got = owner.all_gather_scores(local)
        assert got.shape == (world, q, 128) and got.data_ptr() == ws
        for r in range(world):
            assert torch.equal(got[r], torch.full((q, 128), float(r + 1)) + torch.arange(q)[:, None])
    assert owner.calls == 2
    owner.validate_bounds(6, 4)
    errors = 0
    for bad in (lambda: owner.validate_bounds(6, 8),
                lambda: owner.all_gather_into_tensor(torch.zeros(7, 128)),               # beyond the bound
                lambda: owner.all_gather_into_tensor(torch.zeros(6, 128).t()),           # not contiguous
                lambda: owner.all_gather_into_tensor(torch.zeros(6, 128, dtype=torch.float64)),
                lambda: owner.all_gather_into_tensor(torch.zeros(2, 128), output=torch.zeros(4, 128))):
        try:
            bad()
        except ValueError:
            errors += 1
    with owner.graph_capture() as o:
        assert o is owner
    owner.close()
    owner.close()                                            # idempotent
    try:
        owner.all_gather_scores(torch.zeros(2, 128))
    except RuntimeError:
        errors += 1
    out[rank] = errors
    dist.destroy_process_group()


def test_collective_index_owner_gathers_into_its_own_workspace():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_collective_owner_main, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: 6, 1: 6}
