"""Indexer scoring (block-scaled fp8 on tcgen05), local top-k and the cross-rank
candidate merge; plus the fp32 PyTorch reference of the score.

Scoring convention: ``logit[q, t] = key_scale[t] * sum_h w[q, h] * relu(q[q, h] . key[t])``
with ``q`` quantised to fp8 e4m3 per (query, head) and its scale folded into ``w``.
"""
from __future__ import annotations

import ctypes as C

from ..storage import layout as L
from . import _native as N
from . import records
from . import topk as topk_op


def quantize_queries(q, weights):
    """q [R, n_q, 64, 128] float, weights [R, n_q, 64] -> (uint8 fp8 tensor, fp32 weights
    with the per-(query, head) fp8 scale folded in)."""
    import torch

    x = q.float()
    amax = x.abs().amax(dim=-1)
    scale = records._exact_div(torch.clamp(amax, min=records.SCALE_FLOOR), records.FP8_MAX)
    q8 = (x * (1.0 / scale).unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q8.view(torch.uint8).contiguous(), (weights.float() * scale).contiguous()


def index_score_reference(q8, w, page_table, lengths, pool, *, ranks=1, rank=0):
    """fp32 statement of the score over this rank's shard.  Returns [R*n_q, max_pages*64]
    with -inf on columns the rank does not hold."""
    import torch

    R, n_q = q8.shape[0], q8.shape[1]
    max_pages = page_table.shape[1]
    keys, scales = records.decode_index_page(pool)
    qf = q8.view(torch.float8_e4m3fn).float()
    out = torch.full((R * n_q, max_pages * 64), float("-inf"), dtype=torch.float32, device=q8.device)
    for r in range(R):
        length = int(lengths[r])
        for a in range(max_pages):
            first = (a * ranks + rank) * 64
            n = max(0, min(64, length - first))
            phys = int(page_table[r, a])
            if n == 0 or phys < 0:
                continue
            k = keys[phys, :n]                                        # [n,128]
            s = torch.relu(torch.einsum("jhd,td->jht", qf[r], k))     # [n_q,64,n]
            logit = (s * w[r].unsqueeze(-1)).sum(dim=1) * scales[phys, :n]
            out[r * n_q:(r + 1) * n_q, a * 64:a * 64 + n] = logit
    return out


def index_score(q8, w, page_table, lengths, pool, *, ranks=1, rank=0, pages_per_cta=0, out=None, status=None,
                topk_workspace=None):
    """Score this rank's index shard.  ``pool`` uint8 [pages, 8448]; returns fp32
    ``[R*n_q, max_pages*64]`` (column = allocation page * 64 + offset).  ``topk_workspace``
    (``ops.topk.workspace(R * n_q, device)``): the kernel also leaves every row's histogram and
    valid length there for ``select_topk(..., hist_workspace=...)``; columns beyond a request's
    pages are then left unwritten."""
    import torch

    R, n_q = q8.shape[0], q8.shape[1]
    max_pages = page_table.shape[1]
    if not q8.is_cuda:
        return index_score_reference(q8, w, page_table, lengths, pool, ranks=ranks, rank=rank)
    if out is None:
        out = torch.empty((R * n_q, max_pages * 64), dtype=torch.float32, device=q8.device)
    code = N.cuda().ulc_index_score_hist(
        N.ptr(q8), N.ptr(w), N.ptr(page_table), N.ptr(lengths), N.ptr(pool), C.c_int(pool.shape[0]),
        C.c_int(R), C.c_int(n_q), C.c_int(max_pages), C.c_int(ranks), C.c_int(rank), C.c_int(pages_per_cta),
        N.ptr(out), N.ptr(topk_workspace), N.ptr(status), N.stream())
    N.check(code, "index_score")
    return out


def cols_to_ids(cols, page_table, *, n_q, ranks, rank, out=None):
    """Local score columns -> logical record IDs ((physical page * ranks + rank) * 64 + offset)."""
    import torch

    rows, k = cols.shape
    if not cols.is_cuda:
        c = cols.long()
        row_req = torch.arange(rows, device=cols.device) // n_q
        phys = page_table[row_req.unsqueeze(1), (c.clamp(min=0) >> 6)].long()
        ids = ((phys * ranks + rank) << 6) | (c & 63)
        return torch.where((c >= 0) & (phys >= 0), ids, torch.full_like(ids, -1)).to(torch.int32)
    if out is None:
        out = torch.empty_like(cols)
    N.check(N.cuda().ulc_index_cols_to_ids(N.ptr(cols), N.ptr(page_table), C.c_int(page_table.shape[1]),
                                           C.c_int(n_q), C.c_int(k), C.c_int(ranks), C.c_int(rank),
                                           C.c_int(rows), N.ptr(out), N.stream()), "index_cols_to_ids")
    return out


def select_topk(logits, k, page_table, *, n_q, ranks=1, rank=0, with_values=False, hist_workspace=None, lengths=None):
    """Local top-k of the score rows, translated to logical IDs (-1 where nothing valid).
    ``hist_workspace`` / ``lengths``: see ``ops.topk.topk_paged_ids``."""
    import torch

    if logits.is_cuda:
        vals = torch.empty((logits.shape[0], k), dtype=torch.float32, device=logits.device) if with_values else None
        ids = topk_op.topk_paged_ids(logits, k, page_table, rows_per_request=n_q, ranks=ranks, rank=rank, out_val=vals,
                                     hist_workspace=hist_workspace, lengths=lengths)
        return (ids, vals) if with_values else ids
    cols = topk_op.topk_reference(logits, k, lengths)
    vals = torch.gather(logits, 1, cols.clamp(min=0).long())
    vals[cols < 0] = float("-inf")
    ids = cols_to_ids(cols, page_table, n_q=n_q, ranks=ranks, rank=rank)
    ids = torch.where(torch.isfinite(vals), ids, torch.full_like(ids, -1))
    return (ids, vals) if with_values else ids


def index_ragged_gather_reference(pools, page_table, lengths):
    """PyTorch statement of :func:`index_ragged_gather`: ``pools`` = one uint8 [pages, 8448] tensor per owner."""
    import torch

    ranks = len(pools)
    keys, scales = [], []
    for q in range(page_table.shape[0]):
        n = int(lengths[q])
        t = torch.arange(n, device=page_table.device)
        col = t // 64
        page = torch.where(col < page_table.shape[1], page_table[q, col.clamp(max=page_table.shape[1] - 1)].long(),
                           torch.zeros_like(col))
        k = torch.zeros((n, 128), dtype=torch.uint8, device=page_table.device)
        s = torch.zeros(n, dtype=torch.float32, device=page_table.device)
        for r in range(ranks):
            m = (page > 0) & (page % ranks == r) & (page // ranks < pools[r].shape[0])
            if bool(m.any()):
                rows = pools[r][(page[m] // ranks)]
                off = (t[m] % 64)
                k[m] = torch.gather(rows, 1, (off * 128)[:, None] + torch.arange(128, device=rows.device))
                sb = torch.gather(rows, 1, (8192 + off * 4)[:, None] + torch.arange(4, device=rows.device))
                s[m] = sb.contiguous().view(torch.float32).reshape(-1)
        keys.append(k)
        scales.append(s)
    return torch.cat(keys), torch.cat(scales)


def index_ragged_gather(pool_ptrs, page_table, lengths, *, pool_pages: int, status=None):
    """Dense (keys uint8 [sum(lengths), 128], scales fp32 [sum(lengths)]) of every query's causal prefix, read from
    an Index striped over ``len(pool_ptrs)`` owners (logical page p on owner p % ranks, its page p // ranks).
    ``pool_ptrs``: base address of this layer's page pool on every owner (local or peer memory; tensors are
    accepted too); ``page_table`` int32 [queries, pages] logical page numbers (<= 0 = padding);
    ``lengths`` int32 [queries].  The prefix sums and the total are taken on the host (a prefill chunk is eager)."""
    import ctypes as C

    import torch

    ptrs = [int(p.data_ptr()) if hasattr(p, "data_ptr") else int(p) for p in pool_ptrs]
    lengths = lengths.to(torch.int32).contiguous()
    page_table = page_table.to(torch.int32)
    if page_table.stride(1) != 1:
        page_table = page_table.contiguous()
    offsets = (torch.cumsum(lengths, 0) - lengths).to(torch.int32)
    total = int(lengths.sum())
    longest = int(lengths.max()) if lengths.numel() else 0
    keys = torch.empty((total, 128), dtype=torch.uint8, device=page_table.device)
    scales = torch.empty(total, dtype=torch.float32, device=page_table.device)
    if total == 0:
        return keys, scales
    arr = (C.c_void_p * len(ptrs))(*ptrs)
    N.check(N.cuda().ulc_index_ragged_gather(arr, C.c_int(len(ptrs)), C.c_int(pool_pages), N.ptr(page_table),
                                             C.c_longlong(page_table.stride(0)), C.c_int(page_table.shape[1]),
                                             N.ptr(lengths), N.ptr(offsets), C.c_int(lengths.numel()), C.c_int(longest),
                                             C.c_int(total), N.ptr(keys), N.ptr(scales), N.ptr(status), N.stream()),
            "index_ragged_gather")
    return keys, scales
