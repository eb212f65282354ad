"""Scorers of the distributed Index.

:class:`DistributedIndexScorer` - queries replicated on every rank (tensor-parallel attention).
Each rank scores only the index pages it owns, then either
  * ranks exchange their local top-k candidates and merge them (``candidates``: top-k of the union
    of per-rank top-k equals the global top-k), or
  * the score slices are all-gathered rank-major and selected in logical order (``tagged`` /
    ``nccl``; the baseline).
Both give the selection a replicated index would give, ties included (lower token first).

:class:`OwnerIndexScorer` - independent queries per rank (data-parallel attention) against an Index
that is still striped over all ranks: queries travel to the owners, every owner scores its shard
for every query, candidates travel back to the rank that asked.

Reference: ulacache/indexer/scorer.py:96-369 (CP scorer), native_owner.py:69-630 (owner scorer),
indexer/kernels/scoring.py:83-984 (query exchange / score restore).
"""
from __future__ import annotations

from .ownership import IndexOwnership
from .plan import IndexScorePlan
from .score_layout import RankMajorScoreLayout


def _all_gather(t, group, world):
    import torch
    import torch.distributed as dist

    t = t.contiguous()
    if world == 1:
        return t.unsqueeze(0)
    if t.is_cuda:
        out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=group)
        return out
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t, group=group)
    return torch.stack(parts)


def _local_candidates(scores, lengths_local, k, own: IndexOwnership, rank: int):
    """Per-row top-k of a local score slice -> (values fp32 [rows,k], logical tokens int32 [rows,k])."""
    import torch

    rows, cols = scores.shape
    pos = torch.arange(cols, device=scores.device).unsqueeze(0)
    s = torch.where(pos < lengths_local.long().unsqueeze(1), scores.float(), torch.full_like(scores, float("-inf")))
    kk = min(k, cols)
    if scores.is_cuda:
        val, idx = torch.topk(s, kk, dim=1)
    else:
        order = torch.sort(s, dim=1, descending=True, stable=True)
        val, idx = order.values[:, :kk], order.indices[:, :kk]
    tok = own.logical_token(rank, idx).to(torch.int32)
    tok = torch.where(val > float("-inf"), tok, torch.full_like(tok, -1))
    if kk < k:
        pad = k - kk
        val = torch.cat([val, torch.full((rows, pad), float("-inf"), device=val.device)], dim=1)
        tok = torch.cat([tok, torch.full((rows, pad), -1, dtype=torch.int32, device=tok.device)], dim=1)
    return val.contiguous(), tok.contiguous()


def _merge(cand_vals, cand_toks, k):
    """Global top-k from candidates [rows, n]: by value, ties to the lower token."""
    import torch

    big = cand_toks.long().clamp(min=0)
    # sort by token first, then stably by value: equal values keep token order
    by_tok = torch.sort(big, dim=1, stable=True)
    v = torch.gather(cand_vals, 1, by_tok.indices)
    t = torch.gather(cand_toks, 1, by_tok.indices)
    by_val = torch.sort(v, dim=1, descending=True, stable=True)
    t = torch.gather(t, 1, by_val.indices)[:, :k]
    return torch.where(by_val.values[:, :k] > float("-inf"), t, torch.full_like(t, -1)).to(torch.int32)


class DistributedIndexScorer:
    def __init__(self, plan: IndexScorePlan, *, rank: int = 0, group=None, transport=None):
        self.plan, self.rank, self.group = plan, rank, group
        self.own = IndexOwnership(plan.ranks, plan.page_tokens)
        self.layout = RankMajorScoreLayout(self.own, plan.local_columns)
        self.transport = transport

    def local_lengths(self, lengths):
        return self.own.local_length(lengths, self.rank)

    def score_local(self, q8, w, page_table, lengths, pool, *, status=None):
        """fp32 [rows, local_cols]: scores of the tokens this rank owns (other columns -inf)."""
        from ..ops import indexer

        return indexer.index_score(q8, w, page_table, lengths, pool, ranks=self.plan.ranks, rank=self.rank,
                                   status=status)

    def select(self, local_scores, lengths):
        """Logical token positions int32 [rows, topk] (-1 padded) of the global top-k."""
        p = self.plan
        if p.always_first or p.always_recent or p.transport != "candidates":
            if self.transport is None and p.transport == "nccl" and p.ranks > 1 and self.group is not None:
                # the library transport owns one workspace sized from the plan (no allocation per call)
                from .nccl import CollectiveIndexOwner

                self.transport = CollectiveIndexOwner(self.group, rank=self.rank, world=p.ranks, max_queries=p.rows,
                                                      max_page_width=p.local_columns // p.page_tokens * p.ranks,
                                                      device=local_scores.device)
            gathered = (self.transport.all_gather_scores(local_scores) if self.transport is not None
                        else _all_gather(local_scores, self.group, p.ranks))
            from .topk import topk_rank_major

            # (on GPUs: one radix-select launch over the rank-major scores with a shared index row)
            return topk_rank_major(gathered, lengths, p.topk, self.own, always_first=p.always_first,
                                   always_recent=p.always_recent)
        val, tok = _local_candidates(local_scores, self.local_lengths(lengths), p.topk, self.own, self.rank)
        if self.transport is not None and hasattr(self.transport, "exchange"):
            cv, ct = self.transport.exchange(tok, val)
        else:
            cv = _all_gather(val, self.group, p.ranks).permute(1, 0, 2).reshape(val.shape[0], -1)
            ct = _all_gather(tok, self.group, p.ranks).permute(1, 0, 2).reshape(tok.shape[0], -1)
        return _merge(cv, ct, p.topk)


class OwnerIndexScorer:
    """``rows`` of the plan = queries per rank; every rank contributes that many."""

    def __init__(self, plan: IndexScorePlan, *, rank: int = 0, group=None):
        self.plan, self.rank, self.group = plan, rank, group
        self.own = IndexOwnership(plan.ranks, plan.page_tokens)

    def score(self, q8, w, page_table, lengths, pool, *, status=None):
        """This rank's queries (``q8`` [rows,n_q,64,128] fp8, ``w`` [rows,n_q,64], ``page_table`` of
        OWNER-LOCAL index pages as every owner would see them: int32 [ranks, rows, max_pages], this
        rank's requests on every owner) -> logical token positions int32 [rows * n_q, topk]."""
        import torch
        from ..ops import indexer

        p = self.plan
        world = p.ranks
        # 1. queries to the owners
        all_q = _all_gather(q8, self.group, world)                         # [world, rows, n_q, 64, 128]
        all_w = _all_gather(w, self.group, world)
        all_len = _all_gather(lengths, self.group, world)                  # [world, rows]
        all_tab = _all_gather(page_table, self.group, world)               # [world(asker), ranks(owner), rows, pages]
        rows, n_q = q8.shape[0], q8.shape[1]
        # 2. score my shard for every asker's queries
        vals, toks = [], []
        for asker in range(world):
            sc = indexer.index_score(all_q[asker], all_w[asker], all_tab[asker, self.rank].contiguous(),
                                     all_len[asker].contiguous(), pool, ranks=world, rank=self.rank, status=status)
            ll = self.own.local_length(all_len[asker], self.rank).repeat_interleave(n_q)
            v, t = _local_candidates(sc, ll, p.topk, self.own, self.rank)
            vals.append(v)
            toks.append(t)
        # 3. candidates back to the askers (gathered everywhere, each rank keeps its own rows)
        cv = _all_gather(torch.stack(vals), self.group, world)             # [owner, asker, rows*n_q, k]
        ct = _all_gather(torch.stack(toks), self.group, world)
        mine_v = cv[:, self.rank].permute(1, 0, 2).reshape(rows * n_q, -1)
        mine_t = ct[:, self.rank].permute(1, 0, 2).reshape(rows * n_q, -1)
        # 4. merge
        return _merge(mine_v, mine_t, p.topk)
