"""Selection entry points over Index scores: which top-k form runs for which input layout.

Three inputs reach a selection:

* a rank's OWN slice ``[rows, local_cols]`` (``topk_local``) - the candidate path takes k per rank first;
* candidates ``[rows, ranks * k]`` gathered from all ranks with their token ids (``merge_candidates``);
* RANK-MAJOR gathered scores ``[ranks, rows, local_cols]`` as a score all-gather leaves them
  (``topk_rank_major``): element (r, row, c) is logical token ``ownership.logical_token(r, c)``.  The GPU form
  runs the radix-select kernel once per row over the ``ranks * local_cols`` scores with an explicit index row
  shared by all rows (stride 0), so nothing is permuted into logical order first; the optional page table turns
  the winning token positions into paged record ids inside the same launch (``xform``);
* COMPACT gathered scores (``topk_compact``): the ragged form of the line all-gather, where rank r sent only
  ``lengths[r, row]`` leading columns of each row and the rest of the slice is fill.

Ties go to the lower token in every form (the kernel's order inside a row is unspecified, the set is fixed).

Reference: ulacache/indexer/topk.py:11-50 (``rank_major_topk_module`` / ``compact_topk_module``: the dense and the
compact input specialisation of ``TopKRankMajorKernel::transform_paged``, csrc/indexer/topk_v2.cuh:1467).
"""
from __future__ import annotations


def topk_local(scores, k, lengths=None):
    """Per-row top-k of fp32 scores (ids int32 [rows, k], -1 padded)."""
    from ..ops import topk as T

    if scores.is_cuda:
        return T.topk(scores, k, lengths=lengths)
    return T.topk_reference(scores, k, lengths=lengths)


def merge_candidates(cand_vals, cand_ids, k):
    """Top-k over candidate (value, id) pairs gathered from all ranks -> ids int32 [rows, k]."""
    import torch
    from ..ops import topk as T

    if cand_vals.is_cuda:
        return T.topk(cand_vals, k, in_idx=cand_ids)
    order = torch.sort(cand_vals.float(), dim=1, descending=True, stable=True)
    ids = torch.gather(cand_ids, 1, order.indices[:, :k])
    return torch.where(order.values[:, :k] > float("-inf"), ids, torch.full_like(ids, -1)).to(torch.int32)


def paged_record_ids(tokens, page_table, page_tokens: int = 64):
    """Token positions int32 [rows, k] (-1 padded) -> record ids ``page_table[row, t // 64] * 64 + t % 64``."""
    import torch

    t = tokens.long().clamp(min=0)
    page = torch.gather(page_table.long(), 1, (t // page_tokens).clamp(max=page_table.shape[1] - 1))
    rec = page * page_tokens + t % page_tokens
    return torch.where(tokens >= 0, rec, torch.full_like(rec, -1)).to(torch.int32)


def _token_table(page_table, width: int, page_tokens: int):
    """int32 [rows, width]: record id of every token position (the kernel's ``xform`` table)."""
    import torch

    pos = torch.arange(width, device=page_table.device)
    page = page_table.long()[:, (pos // page_tokens).clamp(max=page_table.shape[1] - 1)]
    return (page * page_tokens + (pos % page_tokens)[None, :]).to(torch.int32).contiguous()


def topk_rank_major(gathered, lengths, k: int, ownership, *, page_table=None, always_first: int = 0,
                    always_recent: int = 0):
    """``gathered`` fp32 [ranks, rows, local_cols]; ``lengths`` [rows] logical context lengths.  Returns int32
    [rows, k] (-1 padded): logical token positions, or paged record ids when ``page_table`` int32
    [rows, max_pages] is given.  ``always_first`` / ``always_recent`` force the leading / trailing tokens in."""
    import torch
    from .score_layout import RankMajorScoreLayout

    ranks, rows, cols = gathered.shape
    layout = RankMajorScoreLayout(ownership, cols)
    pt = ownership.page_tokens
    if not gathered.is_cuda:
        tok = layout.select(gathered, lengths, k, always_first=always_first, always_recent=always_recent)
        return tok if page_table is None else paged_record_ids(tok, page_table, pt)
    from ..ops import topk as T

    token_of = layout.logical_index(gathered.device).reshape(1, -1).to(torch.int32)         # [1, ranks * cols]
    scores = gathered.permute(1, 0, 2).reshape(rows, ranks * cols).float()
    ln = lengths.to(gathered.device).long().reshape(-1, 1)
    valid = token_of < ln
    scores = torch.where(valid, scores, torch.full_like(scores, float("-inf")))
    if always_first or always_recent:
        forced = ((token_of < always_first) | (token_of >= ln - always_recent)) & valid
        scores = torch.where(forced, torch.full_like(scores, float("inf")), scores)
    xform = None if page_table is None else _token_table(page_table, ranks * cols, pt)
    vals = torch.empty((rows, k), dtype=torch.float32, device=gathered.device)
    out = T.topk(scores.contiguous(), k, in_idx=token_of.expand(rows, -1), xform=xform, out_val=vals)
    # a row with fewer than k valid tokens fills up with masked (-inf) positions: they are not winners
    return torch.where(vals > float("-inf"), out, torch.full_like(out, -1))


def topk_compact(gathered, sent_lengths, lengths, k: int, ownership, *, page_table=None):
    """The ragged all-gather's output: ``gathered`` fp32 [ranks, rows, local_cols] of which only the leading
    ``sent_lengths[r, row]`` columns of each (rank, row) carry scores (the rest is the transport's fill value).
    Columns beyond what a rank sent never win, whatever the fill value was."""
    import torch

    ranks, rows, cols = gathered.shape
    col = torch.arange(cols, device=gathered.device)[None, None, :]
    sent = sent_lengths.to(gathered.device).long().reshape(ranks, rows, 1)
    masked = torch.where(col < sent, gathered, torch.full_like(gathered, float("-inf")))
    return topk_rank_major(masked, lengths, k, ownership, page_table=page_table)
