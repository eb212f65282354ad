"""Radix-select top-k over score rows and its reference."""
from __future__ import annotations

import ctypes as C

from . import _native as N


def topk_reference(scores, k, lengths=None, in_idx=None, xform=None):
    """Set-valued reference: indices of the k largest scores per row (ties to the
    lowest position), -1 padding when a row has fewer than k valid entries."""
    import torch

    rows, L = scores.shape
    out = torch.full((rows, k), -1, dtype=torch.int32)
    s = scores.detach().float().cpu()
    for r in range(rows):
        n = L if lengths is None else int(min(max(int(lengths[r]), 0), L))
        row = s[r, :n].clone()
        row[row != row] = float("-inf")
        if n <= k:
            sel = torch.arange(n)
        else:
            order = torch.sort(row, descending=True, stable=True).indices
            sel = order[:k]
        vals = sel.to(torch.int64)
        if in_idx is not None:
            vals = in_idx[r].cpu().long()[vals]
        if xform is not None:
            t = xform[r].cpu().long()
            vals = torch.where(vals >= 0, t[vals.clamp(min=0)], torch.full_like(vals, -1))
        out[r, : vals.numel()] = vals.to(torch.int32)
    return out


_WORKSPACES = {}


def workspace(rows: int, device):
    """Zeroed scratch for the histogram-first selection of up to ``rows`` rows on ``device`` (one
    per device, grown on demand; every launch leaves it zero again, and launches that share it must
    be ordered on one stream).  Create it before capturing a CUDA graph that uses it."""
    import torch

    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    ws = _WORKSPACES.get(key)
    need = int(N.cuda().ulc_topk_workspace_bytes(C.c_int(rows)))
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def workspace_is_clean(ws, rows: int) -> bool:
    """True when the histograms and counters of the first ``rows`` rows are zero, i.e. the
    workspace is in the state every launch expects and leaves behind (synchronises)."""
    import torch

    per = int(N.cuda().ulc_topk_workspace_bytes(C.c_int(1)))
    head = ws[: rows * per].view(rows, per)[:, : 8192 + 16]
    return int(head.to(torch.int32).abs().sum()) == 0


def topk(scores, k, lengths=None, in_idx=None, xform=None, *, out=None, out_val=None, out_count=None,
         method="cluster"):
    """Top-k indices per row of an fp32 ``[rows, L]`` tensor (row stride free).

    ``method``: ``"cluster"`` = one launch, a cluster of CTAs per row exchanging histograms through
    distributed shared memory; ``"hist"`` = a histogram launch and a selection launch through a
    global-memory workspace, no clusters (better with many rows).

    ``lengths``: int32 per-row valid length.  ``in_idx``: int32 ``[rows, L]`` explicit
    index of each score (candidate-list mode).  ``xform``: int32 ``[rows, M]`` table
    applied to each emitted index.  Returns int32 ``[rows, k]``; the order within a
    row is unspecified, the set is deterministic.
    """
    import torch

    if not scores.is_cuda:
        return topk_reference(scores, k, lengths, in_idx, xform)
    assert scores.dtype == torch.float32 and scores.dim() == 2 and scores.stride(1) == 1
    rows, L = scores.shape
    if out is None:
        out = torch.empty((rows, k), dtype=torch.int32, device=scores.device)
    if method == "hist":
        ws = workspace(rows, scores.device)
        code = N.cuda().ulc_topk_ws(
            N.ptr(scores), C.c_longlong(scores.stride(0)), N.ptr(lengths), C.c_int(rows), C.c_int(L), C.c_int(k),
            N.ptr(in_idx), C.c_longlong(0 if in_idx is None else in_idx.stride(0)), N.ptr(xform),
            C.c_longlong(0 if xform is None else xform.stride(0)), C.c_void_p(0), C.c_longlong(0), C.c_int(1),
            C.c_int(1), C.c_int(0), C.c_int(0), N.ptr(out), N.ptr(out_val), N.ptr(out_count), N.ptr(ws), C.c_int(0),
            N.stream())
        N.check(code, "topk")
        return out
    code = N.cuda().ulc_topk(
        N.ptr(scores), C.c_longlong(scores.stride(0)), N.ptr(lengths), C.c_int(rows), C.c_int(L),
        C.c_int(k), N.ptr(in_idx), C.c_longlong(0 if in_idx is None else in_idx.stride(0)),
        N.ptr(xform), C.c_longlong(0 if xform is None else xform.stride(0)), N.ptr(out),
        N.ptr(out_val), N.ptr(out_count), N.stream())
    N.check(code, "topk")
    return out


def topk_paged_ids(scores, k, pages, *, rows_per_request=1, ranks=1, rank=0, out=None, out_val=None,
                   hist_workspace=None, lengths=None):
    """Top-k of score rows whose columns are (allocation page * 64 + offset): emits logical record
    IDs ``((pages[v >> 6] * ranks + rank) << 6) | (v & 63)`` directly and -1 for -inf scores.
    ``hist_workspace``: the workspace the scoring kernel left the rows' histograms and valid lengths
    in (``ops.indexer.index_score(..., topk_workspace=...)``): selection then takes one launch that
    reads each row's valid prefix only.  ``lengths`` (int32 per row, without a workspace): valid columns of each
    row, so that a short row is not searched over the whole table width."""
    import torch

    rows, L = scores.shape
    if out is None:
        out = torch.empty((rows, k), dtype=torch.int32, device=scores.device)
    if hist_workspace is not None:
        code = N.cuda().ulc_topk_ws(
            N.ptr(scores), C.c_longlong(scores.stride(0)), C.c_void_p(0), C.c_int(rows), C.c_int(L), C.c_int(k),
            C.c_void_p(0), C.c_longlong(0), C.c_void_p(0), C.c_longlong(0), N.ptr(pages), C.c_longlong(pages.stride(0)),
            C.c_int(rows_per_request), C.c_int(ranks), C.c_int(rank), C.c_int(1), N.ptr(out), N.ptr(out_val),
            C.c_void_p(0), N.ptr(hist_workspace), C.c_int(1), N.stream())
        N.check(code, "topk")
        return out
    code = N.cuda().ulc_topk_ex(
        N.ptr(scores), C.c_longlong(scores.stride(0)), N.ptr(lengths), C.c_int(rows), C.c_int(L), C.c_int(k),
        C.c_void_p(0), C.c_longlong(0), C.c_void_p(0), C.c_longlong(0), N.ptr(pages), C.c_longlong(pages.stride(0)),
        C.c_int(rows_per_request), C.c_int(ranks), C.c_int(rank), C.c_int(1), N.ptr(out), N.ptr(out_val),
        C.c_void_p(0), N.stream())
    N.check(code, "topk")
    return out


def set_launch_mode(mode="auto"):
    """Pin the launch shape of the CUDA top-k: ``"auto"`` (choose by rows and row length),
    ``"row"`` (one CTA per row), ``"cluster"`` (a cluster of eight CTAs per row) or ``"rows"`` / ``"rows_staged"`` (the
    many-rows throughput kernel: one CTA per row, sampled filter bin, block-scan compaction; streaming the row
    from global memory, or staging it whole in shared memory with asynchronous copies)."""
    N.cuda().ulc_topk_set_mode(C.c_int({"auto": 0, "row": 1, "cluster": 2, "rows": 3, "rows_staged": 4}[mode]))
