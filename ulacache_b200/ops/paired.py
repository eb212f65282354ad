"""Paired record planes (separate K and V pages) and receive-side slot ordering: launchers and references.

Kernels in ``csrc/paired_records.cu``; the torch functions are the CPU paths and the oracles of the GPU tests.

Reference: ulacache/storage/kernels/paired_records.py:8,37; ulacache/cache/kernels/local_cache.py:50-87.
"""
from __future__ import annotations

import ctypes as C

from . import _native as N


def compose_record_ids(table, requests, positions, lengths):
    """``table`` int32 [requests_total, context]: record of every token position of every request.  ``requests``
    int32 [rows], ``positions`` int32 [rows, width] (-1 padding; the row stride may exceed width), ``lengths`` int32
    [rows].  Returns int32 [rows, width]: the record of each position, -1 where the position is padding, at or
    beyond the row's length, or beyond the table's context."""
    import torch

    rows, width = positions.shape
    context = table.shape[1]
    if not positions.is_cuda:
        p = positions.long()
        valid = (p >= 0) & (p < lengths.long()[:, None]) & (p < context)
        rec = table[requests.long()[:, None], p.clamp(0, context - 1)]
        return torch.where(valid, rec, torch.full_like(rec, -1)).to(torch.int32)
    assert table.is_contiguous() and positions.stride(1) == 1
    out = torch.empty((rows, width), dtype=torch.int32, device=positions.device)
    N.check(N.cuda().ulc_compose_record_ids(N.ptr(table), C.c_longlong(table.stride(0)), C.c_int(context), N.ptr(requests),
                                            N.ptr(positions), C.c_longlong(positions.stride(0)), N.ptr(lengths),
                                            C.c_int(rows), C.c_int(width), N.ptr(out), N.stream()), "compose_record_ids")
    return out


def gather_pairs(key, value, records, positions, lengths, offsets, *, heads: int, total: int, padded: bool = False,
                 columns: int = 0):
    """``key`` / ``value``: planes [slots, heads * dim] (any dtype, unit inner stride).  ``records`` int32
    [rows, selected] slots (-1 = not resident), ``positions`` [rows, selected], ``lengths`` [rows], ``offsets`` int32
    [rows + 1].  Returns (out_key, out_value) [total, heads, dim]: output rows offsets[r] + c hold column c of row r.
    A valid position whose record is not resident gives zeros.  ``padded``: every column below ``columns`` is
    written (zeros where invalid); otherwise rows of invalid columns are left as they are (zero-initialised here)."""
    import torch

    rows, selected = records.shape
    dim = key.shape[1] // heads
    out_k = torch.zeros((total, heads, dim), dtype=key.dtype, device=key.device)
    out_v = torch.zeros((total, heads, dim), dtype=value.dtype, device=value.device)
    if not key.is_cuda:
        for r in range(rows):
            start, span = int(offsets[r]), int(offsets[r + 1] - offsets[r])
            for c in range(selected):
                p, slot = int(positions[r, c]), int(records[r, c])
                native_valid = c < span and 0 <= p < int(lengths[r])
                if not (c < columns if padded else native_valid):
                    continue
                if native_valid and slot >= 0:
                    out_k[start + c] = key[slot].view(heads, dim)
                    out_v[start + c] = value[slot].view(heads, dim)
                else:
                    out_k[start + c] = 0
                    out_v[start + c] = 0
        return out_k, out_v
    assert key.stride(1) == 1 and value.stride(1) == 1 and records.is_contiguous() and positions.stride(1) == 1
    eb = key.element_size()
    N.check(N.cuda().ulc_gather_pairs(N.ptr(key), N.ptr(value), C.c_longlong(key.stride(0) * eb),
                                      C.c_longlong(value.stride(0) * eb), N.ptr(records), N.ptr(positions),
                                      C.c_longlong(positions.stride(0)), N.ptr(lengths), N.ptr(offsets), N.ptr(out_k),
                                      N.ptr(out_v), C.c_int(rows), C.c_int(selected), C.c_int(heads), C.c_int(dim * eb),
                                      C.c_int(columns), C.c_int(1 if padded else 0), N.stream()), "gather_pairs")
    return out_k, out_v


def sort_free_tail(stack, count, records: int) -> bool:
    """Sort the top of a free-slot stack (``stack`` int32, ``count`` a one-element int32 tensor: entries below it
    are free, the top is popped first) descending over a bounded window, so that the next pops return ascending,
    mostly adjacent slots.  The window is 16384 entries for requests of up to 4096 records, else 32768; requests
    larger than 16384 records are left alone (returns False)."""
    import torch

    if records <= 0 or records > 16384:
        return False
    window = 16384 if records <= 4096 else 32768
    if not stack.is_cuda:
        n = int(count)
        start = max(0, n - window)
        stack[start:n] = torch.sort(stack[start:n], descending=True).values
        return True
    N.check(N.cuda().ulc_sort_free_tail(N.ptr(stack), N.ptr(count), C.c_int(window), N.stream()), "sort_free_tail")
    return True
