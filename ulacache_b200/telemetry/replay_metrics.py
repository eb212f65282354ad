"""Bytes moved between the tiers during a replay, from the residency counters.

:class:`DeviceReplayProbes` counts on the device, per management group and without touching cache
state: the step's unique historical lookups (deduplicated per request) split by where the record
lives, the bytes the step's plan moves in each direction, and the bytes of rows written straight to
the host tier.

Reference: ulacache/telemetry/replay_metrics.py:4-64 (ReplayMetrics: probes before the plan and
after each group), ulacache/csrc/telemetry/sparse_replay.cuh:11-112.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class ReplayMetrics:
    record_bytes: int
    layers_per_group: int = 1
    promoted: int = 0          # host -> device records
    demoted: int = 0           # device -> host records (victims of a swap)
    steps: int = 0
    history: list = field(default_factory=list)

    def add_step(self, promoted: int, demoted: int):
        self.promoted += int(promoted)
        self.demoted += int(demoted)
        self.steps += 1
        self.history.append((int(promoted), int(demoted)))

    def add_counters(self, before: dict, after: dict):
        """Difference of two ``residency counters`` snapshots (keys ``promotes``, ``swaps``)."""
        self.add_step(after.get("promotes", 0) - before.get("promotes", 0),
                      after.get("swaps", 0) - before.get("swaps", 0))

    @property
    def h2d_bytes(self) -> int:
        return self.promoted * self.record_bytes * self.layers_per_group

    @property
    def d2h_bytes(self) -> int:
        return self.demoted * self.record_bytes * self.layers_per_group

    def summary(self) -> dict:
        s = max(self.steps, 1)
        return {"steps": self.steps, "h2d_bytes": self.h2d_bytes, "d2h_bytes": self.d2h_bytes,
                "h2d_bytes_per_step": self.h2d_bytes / s, "d2h_bytes_per_step": self.d2h_bytes / s,
                "promoted_records": self.promoted, "demoted_records": self.demoted}


class DeviceReplayProbes:
    columns = ("lookup_tokens", "pool_hit_tokens", "cpu_miss_tokens", "unallocated_tokens", "errors",
               "history_h2d_bytes", "victim_d2h_bytes", "new_cpu_backup_bytes")

    def __init__(self, groups: int, queries: int, topk: int, *, device):
        import torch

        if min(groups, queries, topk) < 1:
            raise ValueError("groups, queries and topk must be positive")
        self.groups, self.queries, self.topk = groups, queries, topk
        self.counts = torch.zeros((groups, 8), dtype=torch.int64, device=device)
        size = 1 << (2 * queries * topk - 1).bit_length()
        self.keys = torch.full((size,), -1, dtype=torch.int64, device=device)

    def before_plan(self, group: int, selected, current, requests, directory, width: int = 1):
        """``selected`` int32 [queries, topk] (-1 padded), ``current`` int32 [queries] (the rows this
        step writes: not historical), ``requests`` int32 [queries / width] request ids (-1 = idle),
        ``directory`` int32 (slot encoding: >= 0 device, <= -2 host, -1 unallocated)."""
        import torch

        q, k = selected.shape
        self.keys.fill_(-1)
        if selected.is_cuda:
            import ctypes as C
            from ..ops import _native as N

            N.check(N.cuda().ulc_replay_unique_hits(
                N.ptr(selected.contiguous()), N.ptr(current.contiguous()), N.ptr(requests.contiguous()), N.ptr(directory),
                C.c_int(directory.numel()), N.ptr(self.keys), C.c_longlong(self.keys.numel()), N.ptr(self.counts[group]),
                C.c_int(q), C.c_int(width), C.c_int(k), N.stream()), "replay_unique_hits")
            return
        seen = set()
        c = self.counts[group]
        for qi in range(q):
            req = qi // width
            own = set(current[req * width:(req + 1) * width].tolist())
            for rid in selected[qi].tolist():
                if rid < 0 or rid in own:
                    continue
                if rid >= directory.numel() or int(requests[req]) < 0:
                    c[4] += 1
                    continue
                key = (int(requests[req]), rid)
                if key in seen:
                    continue
                seen.add(key)
                e = int(directory[rid])
                c[0] += 1
                c[1 if e >= 0 else 2 if e <= -2 else 3] += 1

    def after_group(self, group: int, plan, plan_count, current, directory, *, layers: int, row_bytes: int):
        """``plan`` int32 [5, capacity] (rows: record, device slot, host source, host destination,
        evicted record), ``plan_count`` int32 [1] on the device."""
        per = layers * row_bytes
        if plan.is_cuda:
            import ctypes as C
            from ..ops import _native as N

            N.check(N.cuda().ulc_replay_plan_bytes(N.ptr(plan), N.ptr(plan_count), C.c_int(plan.shape[1]),
                                                   C.c_longlong(per), N.ptr(self.counts[group]), N.stream()),
                    "replay_plan_bytes")
            N.check(N.cuda().ulc_replay_current_bytes(N.ptr(current.contiguous()), C.c_int(current.numel()),
                                                      N.ptr(directory), C.c_int(directory.numel()), C.c_longlong(per),
                                                      N.ptr(self.counts[group]), N.stream()), "replay_current_bytes")
            return
        n = min(int(plan_count.reshape(-1)[0]), plan.shape[1])
        c = self.counts[group]
        c[5] += int((plan[2, :n] >= 0).sum()) * per
        c[6] += int((plan[3, :n] >= 0).sum()) * per
        for rid in current.tolist():
            if 0 <= rid < directory.numel() and int(directory[rid]) <= -2:
                c[7] += per

    def snapshot(self) -> dict:
        rows = self.counts.cpu().tolist()
        for row in rows:
            if row[3] or row[4] or row[0] != row[1] + row[2]:
                raise RuntimeError("a replay looked up unallocated history or its lookup partition does not add up")
        return dict(columns=self.columns, groups=rows,
                    totals={key: sum(row[i] for row in rows) for i, key in enumerate(self.columns)})
