"""Memory budgets of the comparison arms, so that every method is given the same bytes.

Reference: ulacache/tools/benchmark_budget.py:1-45 (HiSparse buffer sizing).
"""
from __future__ import annotations


def hot_buffer_records(device_bytes: int, *, requests: int, record_bytes: int, layers: int, reserve_bytes: int = 0) -> int:
    """Records per request of a per-request hot buffer that fills ``device_bytes`` with ``requests``
    concurrent requests (every layer keeps its own buffer)."""
    usable = device_bytes - reserve_bytes
    if usable <= 0 or requests < 1:
        return 0
    return max(0, usable // (requests * record_bytes * layers))


def pooled_records(device_bytes: int, host_bytes: int, *, record_bytes: int, layers: int, metadata_per_record: int = 12):
    """(device records, host records) of a pooled cache under the same budget: the device tier also
    pays ``metadata_per_record`` bytes (directory, stamps, inverse map) per record of both tiers."""
    per_layer_rec = record_bytes * layers
    host = host_bytes // per_layer_rec
    dev = max(0, (device_bytes - host * metadata_per_record) // (per_layer_rec + metadata_per_record))
    return dev, host


def restored_cohort_metadata_tokens(*, requests: int, page_size: int = 64) -> int:
    """Token budget that admits a cohort restored from a snapshot, each request with ONE saved next token: the
    admission controller bills a whole page even for a one-token extension, and one spare page keeps the cohort
    off its strict remaining-budget boundary.  The budget covers metadata preparation only (no prefill forward
    runs for a restored request).

    Reference: ulacache/tools/benchmark_budget.py:5-15."""
    if any(type(v) is not int or v < 1 for v in (requests, page_size)):
        raise ValueError("cohort size and page size must be positive integers")
    return (requests + 1) * page_size


def hot_buffer_rows(*, physical_rows: int, requests: int, prefill_rows: int, page_size: int = 64, topk: int = 2048,
                    rank_limit: int = 32768) -> int:
    """Rows per request of the hot-buffer baseline's device buffer, as large as the pool allows: a complete
    request's prefill is held on the device until its host copy is finished (the reserve), every running request
    keeps its buffer plus one page for the current token, and the baseline's recency ranks are 16-bit
    (``rank_limit`` rows at most).  Refuses pools that cannot hold one full selection beside the reserve.

    Reference: ulacache/tools/benchmark_budget.py:18-45 (hisparse_buffer_rows)."""
    vals = (physical_rows, requests, prefill_rows, page_size, topk, rank_limit)
    if any(type(v) is not int or v < 1 for v in vals):
        raise ValueError("hot-buffer capacity inputs must be positive integers")
    reserve = -(-prefill_rows // page_size) * page_size
    rows = min((physical_rows - reserve) // (requests * page_size) * page_size - page_size, rank_limit // page_size * page_size)
    if rows < topk:
        raise ValueError("the pool cannot hold one full selection per request beside the prefill reserve")
    return rows
