"""Validators for recorded traces.

Reference: ulacache/telemetry/trace_coverage.py:4 (validate_bucket_rotation),
tp_trace_coverage.py:4 (validate_fused_begin_rotation).
"""
from __future__ import annotations

RECENT_BUCKETS = 255


def validate_bucket_rotation(bucket_epochs, epoch: int):
    """The recency ring after ``epoch`` steps: bucket ``e % 255`` must be labelled with the newest
    epoch ``e <= epoch`` congruent to it, or be empty (-1) when no such epoch has happened yet; no
    bucket may be older than 254 steps.  Returns the list of offending bucket ids."""
    bad = []
    for b, label in enumerate(int(x) for x in bucket_epochs):
        newest = epoch - ((epoch - b) % RECENT_BUCKETS)      # newest epoch <= `epoch` that maps to bucket b
        want = newest if newest >= 1 else -1
        if label != want:
            bad.append(b)
    return bad


def validate_trace_coverage(trace: dict, steps: int, layers: int):
    """Every (step, layer) of a replay window must be present in a loaded trace; returns the missing keys."""
    return [(s, l) for s in range(steps) for l in range(layers) if (s, l) not in trace]


def validate_fused_begin_rotation(observations, recent_count: int, valid_queries):
    """Check a run of ``begin_step`` observations taken AFTER the step's expiry and current-row pins:
    each row is (epoch, bucket, label before reuse, members before reuse, label after, current members,
    cold members before, cold members after).  Epochs must be consecutive, the bucket must be
    ``epoch % recent_count``, a non-empty reused bucket must have been old enough to expire, the cold
    bucket may only grow by what expired and shrink by current pins, and the run must visit every
    bucket.  Returns a summary dict; raises ``ValueError`` on the first violation."""
    if recent_count < 1:
        raise ValueError("a positive recent-bucket count is required")
    rows, limits = list(observations), list(valid_queries)
    if not rows or len(rows) != len(limits):
        raise ValueError("every observed begin needs its valid query bound")
    visited, previous = set(), None
    headers = members = nonempty = 0
    for row, queries in zip(rows, limits):
        if len(row) != 8:
            raise ValueError("an observation has eight fields")
        epoch, bucket, age, old_count, new_age, current_count, cold_before, cold_after = (int(v) for v in row)
        if epoch < 1 or bucket != epoch % recent_count or age < -1 or age > epoch:
            raise ValueError("invalid clock or bucket identity")
        if previous is not None and epoch != previous + 1:
            raise ValueError("the clock skipped or repeated an epoch")
        if min(old_count, current_count, cold_before, cold_after) < 0:
            raise ValueError("negative bucket membership")
        expired = age >= 0 and epoch - age >= recent_count
        if new_age != epoch or current_count > queries:
            raise ValueError("invalid current bucket after begin")
        if old_count and not expired:
            raise ValueError("a non-empty reused bucket was not old enough to expire")
        moved = old_count if expired else 0
        if not -queries <= cold_after - cold_before <= moved:
            raise ValueError("cold membership is not explained by expiry and current pins")
        headers += int(expired)
        members += moved
        nonempty += int(expired and old_count > 0)
        visited.add(bucket)
        previous = epoch
    if len(visited) != recent_count:
        raise ValueError("the run did not cover a full bucket rotation")
    return dict(steps=len(rows), first_epoch=int(rows[0][0]), last_epoch=int(rows[-1][0]), recent_buckets=recent_count,
                expired_headers=headers, expired_members=members, nonempty_expirations=nonempty, full_rotation=True)
